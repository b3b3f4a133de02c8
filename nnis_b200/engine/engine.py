"""The step function: one batch of sequences, the tokens it brings, from the cache.

``Engine.step`` takes, for every sequence of the batch, its slot, its next
tokens and the places among them whose logits are wanted.  It reserves cache
pages, uploads the small integer tables of the step in one copy, runs the model
once over all packed tokens and returns float32 logits ``[wanted, vocab]`` on
the device.  A sequence may bring a whole prompt, a further chunk or a single
token; steps in which every sequence brings one token take the decode kernels.

NNIS exposes ``prefill`` (one sequence, token by token) and ``decode_one``
(crates/nnis-model/src/runtime.rs:756-790) and runs batches as sessions one
after another (crates/nnis-model/src/session_batch.rs:91-111); this is the
batched, ragged form of that surface.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence

import torch

from ..cache import PAGE_SIZE, CacheManager
from ..config import read_config
from ..csrc import ops
from ..config.spec import ModelSpec
from ..weights import load_weights
from .context import StepContext
from .model import DecoderModel
from .workspace import Workspace

QUERY_TILE = 64  # queries per CTA of the prompt attention kernel

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "f32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class StepError(ValueError):
    """The step's request is wrong; nothing was run and the cache is unchanged."""


@dataclass
class SequenceStep:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("nnis_b200 runs on a CUDA device only; there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; nnis_b200 has no CPU path")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"the kernels are built for sm_100a; device {device} is "
                           f"sm_{major}{minor}")
    return device


class Engine:
    def __init__(self, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype="bfloat16",
                 device="cuda:0", max_tokens: int = 1 << 16, max_slots: Optional[int] = None):
        self.device = require_cuda(device)
        self.dtype = _DTYPES[dtype]
        self.spec = spec
        torch.cuda.set_device(self.device)
        self.model = DecoderModel(spec, self.dtype, self.device)
        self.model.load(tensors)
        pages = -(-max_tokens // PAGE_SIZE)
        self.max_slots = max_slots if max_slots is not None else min(pages, 1024)
        self.cache = CacheManager(self.model.cache_requests(), self.dtype, self.device, max_tokens,
                                  self.max_slots, spec.max_positions)
        self.model.bind_cache(self.cache)
        self.workspace = Workspace(self.device)
        self._staging: Optional[torch.Tensor] = None  # pinned host ints of one step
        self.h2d_bytes = 0  # bytes of step tables copied so far (for measurements)

    # -- construction -------------------------------------------------------
    @classmethod
    def from_dir(cls, model_dir: str, dtype="bfloat16", device="cuda:0", **kwargs) -> "Engine":
        """The model class comes from config.json's architecture name."""
        device = require_cuda(device)
        spec = read_config(model_dir).to_spec()
        wanted = DecoderModel.weight_specs_of(spec)
        tensors = load_weights(model_dir, wanted, _DTYPES[dtype], device)
        return cls(spec, tensors, dtype, device, **kwargs)

    @classmethod
    def from_spec(cls, spec: ModelSpec, tensors: Mapping[str, torch.Tensor], dtype="bfloat16",
                  device="cuda:0", **kwargs) -> "Engine":
        """Tensors by name on any device, float32 or bfloat16; they are brought
        to the kept dtypes as the loader would."""
        device = require_cuda(device)
        wanted = DecoderModel.weight_specs_of(spec)
        compute = _DTYPES[dtype]
        kept = {}
        for name, ws in wanted.items():
            t = tensors[name]
            if tuple(t.shape) != tuple(ws.shape):
                raise ValueError(f"{name}: shape {list(t.shape)}, expected {list(ws.shape)}")
            kept[name] = t.to(torch.float32 if ws.role == "vector" else compute).to(device).contiguous()
        return cls(spec, kept, dtype, device, **kwargs)

    # -- slots ----------------------------------------------------------------
    def acquire_slot(self) -> int:
        return self.cache.acquire()

    def release_slot(self, slot: int) -> None:
        self.cache.release(slot)

    # -- the step -----------------------------------------------------------
    def _stage(self, ints: List[int]) -> torch.Tensor:
        """One pinned buffer -> one async copy -> int32 device tensor."""
        n = len(ints)
        if self._staging is None or self._staging.numel() < n:
            self._staging = torch.empty(max(n, 4096), dtype=torch.int32, pin_memory=True)
            self._staging_free = torch.cuda.Event()
            self._staging_free.record()
        # the previous copy out of the pinned buffer must be over before it is rewritten
        self._staging_free.synchronize()
        self._staging[:n] = torch.tensor(ints, dtype=torch.int32)
        dev = self.workspace.get("step_ints", (n,), torch.int32)
        dev.copy_(self._staging[:n], non_blocking=True)
        self.h2d_bytes += 4 * n
        self._staging_free.record()
        return dev

    def prepare(self, batch: Sequence[SequenceStep]):
        """Validate, reserve pages, upload the tables; returns (ctx, want_rows)."""
        if not batch:
            raise StepError("a step needs at least one sequence")
        vocab = self.spec.vocab_size
        slots = [s.slot for s in batch]
        counts, starts = [], []
        for s in batch:
            if len(s.tokens) == 0:
                raise StepError(f"slot {s.slot}: a sequence in a step brings at least one token")
            for t in s.tokens:
                if not 0 <= int(t) < vocab:
                    raise StepError(f"slot {s.slot}: token {t} is outside the vocabulary of {vocab}")
            for w in s.want:
                if not 0 <= int(w) < len(s.tokens):
                    raise StepError(f"slot {s.slot}: wanted place {w} is outside its "
                                    f"{len(s.tokens)} tokens")
            counts.append(len(s.tokens))
            starts.append(self.cache.length(s.slot))
        new_lengths = [a + b for a, b in zip(starts, counts)]
        self.cache.reserve(slots, new_lengths)

        tokens, pos, seq, want_rows = [], [], [], []
        base = 0
        for i, s in enumerate(batch):
            tokens.extend(int(t) for t in s.tokens)
            pos.extend(range(starts[i], new_lengths[i]))
            seq.extend([i] * counts[i])
            want_rows.extend(base + int(w) for w in s.want)
            base += counts[i]
        n, b = base, len(batch)
        tables, cols = [], []
        for g in range(len(self.cache.groups)):
            width = max(1, max(-(-L // PAGE_SIZE) for L in new_lengths))
            rows = []
            for s in slots:
                t = self.cache.page_table(g, s)
                rows.extend(t[:width] + [-1] * (width - len(t[:width])))
            tables.append(rows)
            cols.append(width)
        flat = tokens + pos + seq + slots + want_rows
        for rows in tables:
            flat += rows
        decode = all(c == 1 for c in counts)
        first_rows, tiles = [], []
        if not decode:
            row = 0
            for i, c in enumerate(counts):
                first_rows.append(row)
                row += c
                for q0 in range(0, c, QUERY_TILE):
                    tiles += [i, q0]
            flat += first_rows + starts + counts + tiles
        dev = self._stage(flat)
        o = 0

        def take(k):
            nonlocal o
            out = dev[o:o + k]
            o += k
            return out

        d_tokens, d_pos, d_seq, d_slots = take(n), take(n), take(n), take(b)
        d_want = take(len(want_rows))
        d_tables = [take(b * c).view(b, c) for c in cols]
        ctx = StepContext(
            n_tokens=n, n_seqs=b, tokens=d_tokens, token_pos=d_pos, token_seq=d_seq,
            seq_slots=d_slots, page_tables=d_tables, workspace=self.workspace,
            decode=decode, max_context=max(new_lengths),
            host_slots=slots, host_counts=counts, host_starts=starts)
        if not decode:
            ctx.seq_first_row, ctx.seq_start, ctx.seq_count = take(b), take(b), take(b)
            ctx.q_tiles = take(len(tiles)).view(-1, 2)
        return ctx, d_want, slots, new_lengths

    def step(self, batch: Sequence[SequenceStep]) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted places, vocab] in the
        order of the batch and of each sequence's ``want``."""
        ctx, d_want, slots, new_lengths = self.prepare(batch)
        logits = torch.empty((d_want.numel(), self.spec.vocab_size), dtype=torch.float32,
                             device=self.device)
        self.model.forward(ctx, d_want, logits)
        self.cache.commit(slots, new_lengths)
        return logits

    def check_status(self) -> None:
        """Raise if a kernel flagged bad input since the last check (syncs)."""
        if int(self.model.status.item()) != 0:
            self.model.status.zero_()
            raise StepError("a kernel met a token id outside the vocabulary")
        ops.check_status(self.device)

    # -- figures ----------------------------------------------------------------
    def memory(self) -> Dict[str, object]:
        return {"weights_bytes_per_step": self.model.parameter_bytes(),
                "workspace_bytes": self.workspace.bytes(), **self.cache.usage()}
