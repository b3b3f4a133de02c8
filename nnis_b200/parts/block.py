"""Arrangements of the parts of a layer.

``Block`` is what the model needs of an arrangement: its parts (for weights and
work lists), what it wants of the cache, and ``forward``.  An arrangement reads
its parts from ``LayerSpec.parts`` by the roles it knows, so one with other or more
sub-layers (a post-norm, one norm for parallel branches, a third sub-layer) is a
class registered in ``BLOCKS``, not a change here.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) - the order of NNIS's
decoder (crates/nnis-model/src/runtime.rs:946-1097); roles mixer_norm, mixer,
ffn_norm, ffn.  In decode steps a norm may be shared out between the projections on
either side of it (``parts.base.SharedNorm``): the block tells the part before a norm
which norm follows, and hands what that part left to the part after it.
"""
from __future__ import annotations

from typing import Dict, Mapping, Sequence

import torch

from ..weights.loader import WeightSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part


class Block:
    """Base of the arrangements: subclasses build their parts in ``__init__`` (with
    ``build``), list them in ``parts()`` and run them in ``forward``.  ``mixer`` is
    the part that owns the layer's cache, if any."""
    mixer = None

    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        self.spec = layer_spec
        self.dtype = dtype
        self.device = device

    def build(self, registry, role: str) -> Part:
        part = self.spec.part(role)
        return registry.build(part.kind, part.params, self.spec.prefix, self.dtype, self.device)

    def parts(self) -> Sequence[Part]:
        raise NotImplementedError

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        raise NotImplementedError

    # -- what the model asks of every arrangement --------------------------------
    def cache_request(self):
        return self.mixer.cache_request() if self.mixer is not None else None

    def check_shared_cache(self, view) -> None:
        self.mixer.check_shared_cache(view)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for part in self.parts())

    def step_flops(self, counts, starts) -> float:
        return sum(part.step_flops(counts, starts) for part in self.parts())

    def step_tables(self, counts, starts, have=()) -> Dict[str, object]:
        tables: Dict[str, object] = {}
        for part in self.parts():
            wants = getattr(part, "step_tables", None)
            if wants is not None:
                for name, arr in wants(counts, starts, tuple(have) + tuple(tables)).items():
                    tables.setdefault(name, arr)
        return tables


class PreNormBlock(Block):
    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        super().__init__(layer_spec, dtype, device)
        self.mixer_norm = self.build(NORMS, "mixer_norm")
        self.mixer = self.build(MIXERS, "mixer")
        self.ffn_norm = self.build(NORMS, "ffn_norm")
        self.ffn = self.build(FEED_FORWARDS, "ffn")

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    @staticmethod
    def _shares(part, norm, ctx, n: int) -> bool:
        return bool(getattr(part, "shares_norm", None)) and part.shares_norm(norm, ctx, n)

    def first_shared_norm(self, ctx, n: int):
        """The norm this block applies first, if its mixer will take it begun by the part
        that runs before this block (asked by the model before that part runs)."""
        return self.mixer_norm if self._shares(self.mixer, self.mixer_norm, ctx, n) else None

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        normed = ctx.workspace.get("normed", (n, width), self.dtype)
        begun = ctx.take_shared_norm(self.mixer_norm)
        # the mixer's last projection may begin the norm before the feed-forward
        ctx.emit_for = self.ffn_norm if self._shares(self.ffn, self.ffn_norm, ctx, n) else None
        if begun is not None:
            self.mixer.forward_shared(begun, hidden, ctx, cache)
        # a part may fold the norm before it into its first kernel (decode steps)
        elif getattr(self.mixer, "fuses_norm", None) and self.mixer.fuses_norm(self.mixer_norm, ctx, n):
            self.mixer.forward_normed(hidden, self.mixer_norm, ctx, cache)
        else:
            self.mixer_norm.forward(hidden, normed)
            self.mixer.forward(normed, ctx, hidden, cache)
        begun = ctx.take_shared_norm(self.ffn_norm)
        # ... and the feed-forward's the first norm of the block that runs next
        ctx.emit_for = ctx.next_norm
        if begun is not None:
            self.ffn.forward_shared(begun, hidden, ctx)
        elif getattr(self.ffn, "fuses_norm", None) and self.ffn.fuses_norm(self.ffn_norm, ctx, n):
            self.ffn.forward_normed(hidden, self.ffn_norm, ctx)
        else:
            self.ffn_norm.forward(hidden, normed)
            self.ffn.forward(normed, ctx, hidden)
        ctx.emit_for = None


BLOCKS.register("prenorm", PreNormBlock)
