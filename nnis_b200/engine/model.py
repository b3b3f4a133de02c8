"""A decoder put together from a ``ModelSpec``: embedding, blocks in their run
order, final norm, head.  It holds weights and runs packed tokens; it owns no
cache and no batch logic.  NNIS's ``Model`` plays the same role with a fixed
decoder (crates/nnis-model/src/runtime.rs:109-128, :918-1120).
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Optional

import torch

from ..csrc import ops
from ..config.spec import ModelSpec
from ..parts import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..weights.loader import WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16; got {dtype}")
        self.spec, self.dtype, self.device = spec, dtype, torch.device(device)
        self.embedding = EMBEDDINGS.build(spec.embedding.kind, spec.embedding.params, "", dtype,
                                          self.device)
        self.blocks = [BLOCKS.build(layer.block, layer, dtype, self.device) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm.kind, spec.final_norm.params, "", dtype,
                                      self.device)
        self.head = HEADS.build(spec.head.kind, spec.head.params, "", dtype, self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        for i, entry in enumerate(spec.schedule):
            wants = self.blocks[entry.layer].cache_request()
            if entry.cache_of is not None and wants is not None:
                raise ValueError(f"schedule[{i}] reads the cache of entry {entry.cache_of} but its "
                                 f"mixer writes one of its own")

    # -- weights ------------------------------------------------------------
    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            for name, ws in part.weight_specs().items():
                if name in specs and specs[name].shape != ws.shape:
                    raise ValueError(f"tensor {name} is wanted with two shapes")
                specs.setdefault(name, ws)
        return specs

    @staticmethod
    def weight_specs_of(spec: ModelSpec) -> Dict[str, WeightSpec]:
        """Names and shapes without building device state (random-weights mode)."""
        return DecoderModel(spec, torch.float32, torch.device("cpu")).weight_specs()

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in (self.embedding, *self.blocks, self.final_norm, self.head):
            part.load(tensors)

    def parameter_bytes(self) -> int:
        """Bytes of weights one step reads: each scheduled block once per run,
        norms, the head; the embedding only through the head when tied."""
        total = self.final_norm.parameter_bytes() + self.head.parameter_bytes()
        for entry in self.spec.schedule:
            total += self.blocks[entry.layer].parameter_bytes()
        return total

    def step_flops(self, counts, starts, wanted: int) -> float:
        """Floating-point operations of one step (a multiply-add counts two): every
        scheduled block over the step's tokens, and the head on the wanted rows."""
        total = self.head.step_flops(counts, starts, wanted)
        for entry in self.spec.schedule:
            total += self.blocks[entry.layer].step_flops(counts, starts)
        return total

    # -- cache ----------------------------------------------------------------
    def cache_requests(self) -> List[Optional[object]]:
        return [None if e.cache_of is not None else self.blocks[e.layer].cache_request()
                for e in self.spec.schedule]

    def bind_cache(self, cache) -> None:
        self._views = []
        for i, entry in enumerate(self.spec.schedule):
            view = cache.view(entry.cache_of if entry.cache_of is not None else i)
            if entry.cache_of is not None:
                self.blocks[entry.layer].check_shared_cache(view)
            self._views.append(view)

    def step_tables(self, counts, starts) -> Dict[str, object]:
        """The work lists that the scheduled blocks want uploaded for a prompt step."""
        tables: Dict[str, object] = {}
        for layer in sorted({e.layer for e in self.spec.schedule}):
            for name, arr in self.blocks[layer].step_tables(counts, starts, tuple(tables)).items():
                tables.setdefault(name, arr)
        return tables

    # -- run ------------------------------------------------------------------
    def forward_and_pick(self, ctx, want_rows: torch.Tensor, picks: torch.Tensor,
                         logits: Optional[torch.Tensor], tokens: torch.Tensor,
                         pos: torch.Tensor) -> None:
        """A decode step that ends in the greedy pick: ``picks`` gets the token of
        each wanted row, ``tokens``/``pos`` (the step's own inputs) move on to the
        next step on live rows; ``logits`` is written too when it is given."""
        r = picks.numel()
        if getattr(self.head, "forward_pick", None) and self.head.fuses_norm(self.final_norm, r):
            self._run_blocks(ctx)
            ws = ctx.workspace
            hidden = ws.get("hidden", (ctx.n_tokens, self.spec.hidden_size), torch.float32)
            # zeroed once (the kernel leaves its ticket at zero) and kept with the step's
            # other buffers: steps that may run side by side have workspaces of their own
            scratch = ws.zeros("pick_scratch", (self.head.pick_scratch_ints(r),), torch.int32)
            self.head.forward_pick(hidden, self.final_norm, want_rows, picks, scratch, logits,
                                   tokens, pos)
            return
        if logits is None:
            logits = ctx.workspace.get("logits", (r, self.spec.vocab_size), torch.float32)
        self.forward(ctx, want_rows, logits)
        ops.argmax(logits, picks)
        ops.advance(tokens, pos, picks)

    def _run_blocks(self, ctx) -> torch.Tensor:
        hidden = ctx.workspace.get("hidden", (ctx.n_tokens, self.spec.hidden_size), torch.float32)
        self.embedding.forward(ctx.tokens, hidden, self.status)
        schedule = self.spec.schedule
        for i, entry in enumerate(schedule):
            # a block may begin the first norm of the block after it, if that one takes it
            ask = getattr(self.blocks[schedule[i + 1].layer], "first_shared_norm", None) \
                if i + 1 < len(schedule) else None
            ctx.next_norm = ask(ctx, ctx.n_tokens) if ask is not None else None
            self.blocks[entry.layer].forward(hidden, ctx, self._views[i])
        ctx.next_norm = ctx.shared_norm = None
        return hidden

    def forward(self, ctx, want_rows: torch.Tensor, logits: torch.Tensor) -> None:
        """Run ``ctx.n_tokens`` packed tokens; write the logits of the rows that
        ``want_rows`` (int32, indices into the packed tokens) names."""
        ws = ctx.workspace
        hidden = self._run_blocks(ctx)
        r = logits.shape[0]
        if r and getattr(self.head, "forward_normed", None) \
                and self.head.fuses_norm(self.final_norm, r):
            self.head.forward_normed(hidden, self.final_norm, want_rows, logits)
        elif r:
            final = ws.get("final", (r, self.spec.hidden_size), self.dtype)
            self.final_norm.forward(hidden, final, want_rows)
            self.head.forward(final, logits)
