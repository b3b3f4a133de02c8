"""Interfaces of the parts a block is put together from, and their registries.

A part is built from the ``params`` of its ``PartSpec`` (sizes and constants),
the tensor-name prefix of its block, the operand dtype and the device.  It never
learns which model it is in.  Every part says which tensors it wants
(``weight_specs``), takes them (``load``) and runs on packed tokens.

====================  =====================================================
registry              interface beyond ``weight_specs`` / ``load``
====================  =====================================================
``NORMS``             ``forward(x_f32 [n, width], out [m, width], rows=None)``
``POSITIONS``         ``rotary_tables()`` -> (cos, sin) or None, and, for an
                      encoding with arithmetic of its own (``in_kernel = False``),
                      ``apply(qkv, ctx, heads, kv_heads, head_dim)``
``MIXERS``            ``cache_request()``; ``forward(x, ctx, residual, cache)``;
                      optionally ``fuses_norm``/``forward_normed`` and
                      ``shares_norm``/``forward_shared`` (see ``SharedNorm``)
``FEED_FORWARDS``     ``forward(x, ctx, residual)``; optionally the same
``BLOCKS``            ``forward(hidden_f32, ctx, cache)``; ``parts()``;
                      ``cache_request()``, ``check_shared_cache(view)``;
                      optionally ``first_shared_norm(ctx, n)``
``EMBEDDINGS``        ``forward(tokens, hidden_f32, status)``
``HEADS``             ``forward(x, logits_f32)``; optionally ``fuses_norm``,
                      ``forward_normed``, ``forward_pick`` (see ``LinearHead``)
====================  =====================================================

Mixers and feed-forwards read ``x`` (operand dtype, ``[n, width]``) and *add*
their result to ``residual`` (float32, ``[n, width]``): the residual sum is
float32 in every dtype, and a fused epilogue may add in place.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Mapping

import torch

from ..weights.loader import WeightSpec


@dataclass
class SharedNorm:
    """A norm of the residual rows begun by the part that wrote them last.

    In a decode step the kernel that adds a part's output to the residual has the new
    values in registers.  When the block tells it which norm reads them next
    (``ctx.emit_for``) and that norm is an RMSNorm, it can also write ``x`` = the rows times
    the norm's weights (bfloat16 [n, width]) and ``shares`` = every eight columns' sum of
    squares (float32 [n, width / 8]); the part after the norm then runs its first
    projection on ``x`` and multiplies its float32 sums by 1 / sqrt(mean of squares + eps):
    the same sum with one rounding moved.  Offered by a part through ``begin_norm`` when it
    runs its last projection as a decode kernel; taken by a part that has
    ``shares_norm(norm, ctx, n)`` and ``forward_shared(begun, residual, ctx[, cache])``.
    Nothing breaks if no part offers or takes it: the block falls back to the norm."""
    norm: Any
    x: torch.Tensor
    shares: torch.Tensor


def begin_norm(ctx, n: int, width: int):
    """For a part about to add ``[n, width]`` to the residual with a decode kernel: the
    ``emit`` argument of ``ops.gemv_bf16`` if the block named the norm that follows
    (``ctx.emit_for``), else None.  Leaves the ``SharedNorm`` in the context."""
    norm = getattr(ctx, "emit_for", None)
    if norm is None or getattr(norm, "kind", None) != "rmsnorm" or width % 8:
        return None
    x = ctx.workspace.get("normed_shared", (n, width), torch.bfloat16)
    shares = ctx.workspace.get("norm_shares", (n, width // 8), torch.float32)
    ctx.shared_norm = SharedNorm(norm, x, shares)
    return (x, norm.weight, shares)


class Part:
    # True: ``forward`` works from the device tensors of the step context alone,
    # so a step can be captured in a CUDA graph.  A part that reads the context's
    # host-side fields (``host_slots`` ...) sets this to False.
    device_only = True

    def __init__(self, params: Mapping[str, Any], prefix: str, dtype: torch.dtype,
                 device: torch.device):
        self.params = params
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    def tensor_name(self, stem: str, leaf: str = "weight") -> str:
        return f"{self.prefix}.{stem}.{leaf}" if self.prefix else f"{stem}.{leaf}"

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        pass

    def parameter_bytes(self) -> int:
        """Bytes of weights that one step reads."""
        return 0

    def step_flops(self, counts, starts) -> float:
        """Floating-point operations (a multiply-add counts two) of one step whose
        sequences bring ``counts`` tokens after ``starts`` cached ones: what a
        measurement divides by the step's time."""
        return 0.0

    def step_tables(self, counts, starts, have=()) -> Dict[str, Any]:
        """Integer tables (numpy int32 arrays by name) that this part wants on the
        device for a prompt step whose sequences bring ``counts`` tokens after
        ``starts`` cached ones: work lists of its kernels.  ``have``: names that
        another part has asked for already and need not be made again.  The engine uploads them
        with the step's other tables; ``ctx.tables[name]`` is the device copy and
        ``ctx.host_tables[name]`` the array.  A name spells out every size the table
        depends on, so parts with equal needs share one table.  Tables depend on
        ``counts`` and ``starts`` only, which a captured step fixes."""
        return {}


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: Dict[str, Callable[..., Part]] = {}

    def register(self, kind: str, factory: Callable[..., Part]) -> None:
        self._kinds[kind] = factory

    def build(self, kind: str, *args, **kwargs) -> Part:
        if kind not in self._kinds:
            raise KeyError(f"unknown {self.what} {kind!r}; known: {sorted(self._kinds)}")
        return self._kinds[kind](*args, **kwargs)

    def known(self):
        return sorted(self._kinds)


class PositionEncoding(Part):
    """How positions reach query and key heads.  Two ways to say it:

    * ``rotary_tables()`` returns float32 ``(cos, sin)`` of ``[positions, head_dim / 2]``
      for the rotate-half pairing over the whole head (or None: heads stay as they
      are); the mixer's kernels apply them, fused with the projection where they can;
    * an encoding with other arithmetic (interleaved pairs, a rotated fraction of the
      head, a learned table ...) sets ``in_kernel = False`` and implements ``apply``:
      it changes the q and k heads of the packed rows ``qkv`` ``[n, (heads + 2 *
      kv_heads) * head_dim]`` in place (v untouched; ``kv_heads`` is 0 when the rows
      hold q only), at the positions ``ctx.token_pos`` (-1: a padding row, to be left
      alone), before keys and values go to the cache.  The mixer then runs its
      projection unfused, calls ``apply`` and stores the heads as they come back."""
    in_kernel = True

    def rotary_tables(self):
        return None

    def apply(self, qkv: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError(f"{type(self).__name__} sets in_kernel = False but has no apply()")


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")
