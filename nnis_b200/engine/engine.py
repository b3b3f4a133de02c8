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

import numpy as np
import torch

from ..cache import PAGE_SIZE, CacheManager
from ..config import read_config
from ..csrc import ops
from ..config.spec import ModelSpec
from ..weights import load_weights
from .context import StepContext
from .model import DecoderModel
from .workspace import Workspace

GRAPH_MIN_TOKENS = 256  # prompt steps at least this large are captured when they recur
MAX_STEP_GRAPHS = 4     # captured prompt steps kept (each holds buffers of its own)
MAX_SEEN_SHAPES = 64    # shapes seen once and remembered in case they come again

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
        self._step_graphs: Dict[object, dict] = {}  # captured prompt steps by shape, oldest use first
        self._seen_shapes: Dict[object, bool] = {}  # shapes of large prompt steps seen once
        parts = [p for blk in self.model.blocks for p in blk.parts()]
        self._graph_safe = all(getattr(p, "device_only", True) for p in parts)
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

    def truncate(self, slot: int, length: int) -> None:
        """The sequence of ``slot`` forgets its positions from ``length`` on; its next
        step goes on from there (see ``CacheManager.truncate`` for when that is refused)."""
        self.cache.truncate(slot, length)

    def snapshot(self, slot: int):
        """Keep what brings the sequence of ``slot`` back to where it is now (its
        length and its fixed-size state); ``restore`` goes back to it."""
        return self.cache.snapshot(slot)

    def restore(self, snapshot) -> None:
        self.cache.restore(snapshot)

    # -- the step -----------------------------------------------------------
    def _stage(self, parts: List[np.ndarray], workspace: Optional[Workspace] = None) -> torch.Tensor:
        """Int arrays -> one pinned buffer -> one async copy -> int32 device tensor."""
        workspace = workspace if workspace is not None else self.workspace
        n = int(sum(p.size for p in parts))
        if self._staging is None or self._staging.numel() < n:
            self._staging = torch.empty(max(2 * n, 4096), dtype=torch.int32, pin_memory=True)
            self._staging_np = self._staging.numpy()
            self._staging_free = torch.cuda.Event()
            self._staging_free.record()
        # the previous copy out of the pinned buffer must be over before it is rewritten
        self._staging_free.synchronize()
        o = 0
        for p in parts:
            self._staging_np[o:o + p.size] = p
            o += p.size
        dev = workspace.get("step_ints", (n,), torch.int32)
        dev.copy_(self._staging[:n], non_blocking=True)
        self.h2d_bytes += 4 * n
        self._staging_free.record()
        return dev

    def prepare(self, batch: Sequence[SequenceStep], workspace: Optional[Workspace] = None):
        """Validate, reserve pages, upload the tables; returns (ctx, want_rows,
        slots, new lengths).  ``workspace``: where the step's buffers live (the
        engine's own unless a captured graph has one of its own)."""
        workspace = workspace if workspace is not None else self.workspace
        if not batch:
            raise StepError("a step needs at least one sequence")
        vocab = self.spec.vocab_size
        slots = [s.slot for s in batch]
        counts, starts, token_arrays = [], [], []
        for s in batch:
            tok = np.asarray(s.tokens, dtype=np.int64).reshape(-1)
            if tok.size == 0:
                raise StepError(f"slot {s.slot}: a sequence in a step brings at least one token")
            if int(tok.min()) < 0 or int(tok.max()) >= vocab:
                bad = int(tok[(tok < 0) | (tok >= vocab)][0])
                raise StepError(f"slot {s.slot}: token {bad} is outside the vocabulary of {vocab}")
            for w in s.want:
                if not 0 <= int(w) < tok.size:
                    raise StepError(f"slot {s.slot}: wanted place {w} is outside its "
                                    f"{tok.size} tokens")
            token_arrays.append(tok.astype(np.int32))
            counts.append(int(tok.size))
            starts.append(self.cache.length(s.slot))
        new_lengths = [a + b for a, b in zip(starts, counts)]
        self.cache.reserve(slots, new_lengths)

        i32 = lambda x: np.asarray(x, dtype=np.int32).reshape(-1)
        n, b = int(sum(counts)), len(batch)
        pos = np.concatenate([np.arange(a, e, dtype=np.int32) for a, e in zip(starts, new_lengths)])
        seq = np.repeat(np.arange(b, dtype=np.int32), counts)
        first_rows = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.int32)
        want_rows = i32([first_rows[i] + int(w) for i, s in enumerate(batch) for w in s.want])
        parts = [np.concatenate(token_arrays), pos, seq, i32(slots), want_rows]
        cols = []
        for g in range(len(self.cache.groups)):
            width = max(1, max(-(-L // PAGE_SIZE) for L in new_lengths))
            table = np.full((b, width), -1, dtype=np.int32)
            for r, slot in enumerate(slots):
                t = self.cache.page_table(g, slot)[:width]
                table[r, :len(t)] = t
            parts.append(table.reshape(-1))
            cols.append(width)
        decode = all(c == 1 for c in counts)
        if not decode:
            parts += [first_rows, i32(starts), i32(counts)]
            # 16-byte alignment for the tables the parts asked for
            parts.append(np.zeros(-int(sum(p.size for p in parts)) % 4, dtype=np.int32))
            extra = self.model.step_tables(counts, starts)
            for name, arr in extra.items():
                flat = np.ascontiguousarray(arr, dtype=np.int32).reshape(-1)
                parts += [flat, np.zeros(-flat.size % 4, dtype=np.int32)]
        dev = self._stage(parts, workspace)
        o = 0

        def take(k):
            nonlocal o
            out = dev[o:o + k]
            o += k
            return out

        d_tokens, d_pos, d_seq, d_slots = take(n), take(n), take(n), take(b)
        d_want = take(want_rows.size)
        d_tables = [take(b * c).view(b, c) for c in cols]
        ctx = StepContext(
            n_tokens=n, n_seqs=b, tokens=d_tokens, token_pos=d_pos, token_seq=d_seq,
            seq_slots=d_slots, page_tables=d_tables, workspace=workspace,
            decode=decode, max_context=max(new_lengths),
            host_slots=slots, host_counts=counts, host_starts=starts)
        if not decode:
            ctx.seq_first_row, ctx.seq_start, ctx.seq_count = take(b), take(b), take(b)
            take(-o % 4)
            for name, arr in extra.items():
                ctx.tables[name] = take(arr.size).view(arr.shape)
                ctx.host_tables[name] = arr
                take(-arr.size % 4)
        return ctx, d_want, slots, new_lengths

    def step(self, batch: Sequence[SequenceStep]) -> torch.Tensor:
        """Run one step; returns float32 logits [wanted places, vocab] in the
        order of the batch and of each sequence's ``want``.

        Large prompt steps whose shape (token counts, start positions, number of
        wanted places) comes a second time are captured as a CUDA graph with buffers
        of their own and replayed from then on: such a step is a few hundred small
        launches, and the host is the slower side of them.  Shapes seen once are only
        remembered (they cost nothing and push no graph out); of the captured ones the
        least recently used goes when there are more than ``MAX_STEP_GRAPHS``."""
        key = None
        if sum(len(s.tokens) for s in batch) >= GRAPH_MIN_TOKENS and \
                any(len(s.tokens) > 1 for s in batch) and self._graph_safe:
            key = (tuple(len(s.tokens) for s in batch),
                   tuple(self.cache.length(s.slot) for s in batch),  # refuses slots that are not held
                   tuple(len(s.want) for s in batch))
        entry = self._step_graphs.get(key) if key is not None else None
        if entry is not None:
            self._step_graphs[key] = self._step_graphs.pop(key)  # most recently used last
            ctx, d_want, slots, new_lengths = self.prepare(batch, entry["workspace"])
            entry["graph"].replay()
            self.cache.commit(slots, new_lengths)
            return entry["logits"].clone()
        if key is not None and key in self._seen_shapes:
            return self._capture_step(batch, key)
        if key is not None:
            if len(self._seen_shapes) >= MAX_SEEN_SHAPES:
                self._seen_shapes.pop(next(iter(self._seen_shapes)))
            self._seen_shapes[key] = True
        ctx, d_want, slots, new_lengths = self.prepare(batch)
        logits = torch.empty((d_want.numel(), self.spec.vocab_size), dtype=torch.float32,
                             device=self.device)
        self.model.forward(ctx, d_want, logits)
        self.cache.commit(slots, new_lengths)
        return logits

    def _capture_step(self, batch: Sequence[SequenceStep], key) -> torch.Tensor:
        """Second time a prompt shape is seen: run it into buffers of its own (this
        run's logits are the step's result), then record the same launches as a graph
        for the next time."""
        workspace = Workspace(self.device)
        ctx, d_want, slots, new_lengths = self.prepare(batch, workspace)
        logits = torch.empty((d_want.numel(), self.spec.vocab_size), dtype=torch.float32,
                             device=self.device)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):  # allocates the workspace and computes the step
            self.model.forward(ctx, d_want, logits)
        torch.cuda.current_stream().wait_stream(side)
        result = logits.clone()
        workspace.frozen = True
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.model.forward(ctx, d_want, logits)
        self.cache.commit(slots, new_lengths)
        self._seen_shapes.pop(key, None)
        while len(self._step_graphs) >= MAX_STEP_GRAPHS:
            self._step_graphs.pop(next(iter(self._step_graphs)))  # the least recently used
        self._step_graphs[key] = {"graph": graph, "workspace": workspace, "logits": logits}
        return result

    def step_in_portions(self, batch: Sequence[SequenceStep], max_step_tokens: int) -> torch.Tensor:
        """The same result as ``step`` for prompts of any total length, run as several
        steps of at most ``max_step_tokens`` tokens each, so that the step's scratch
        (a few rows of the width and of the feed-forward's size per token) stays
        bounded: sequences are taken in order, one that does not fit is cut and goes
        on in the next portion (a later chunk starts from the cache like any other)."""
        if max_step_tokens <= 0:
            raise StepError("max_step_tokens must be positive")
        if sum(len(s.tokens) for s in batch) <= max_step_tokens:
            return self.step(batch)
        for s in batch:
            for w in s.want:
                if not 0 <= int(w) < len(s.tokens):
                    raise StepError(f"slot {s.slot}: wanted place {w} is outside its "
                                    f"{len(s.tokens)} tokens")
        portions, current, room = [], [], max_step_tokens
        keys = []  # (sequence, wanted place) of every row, in the order the portions give them
        for i, s in enumerate(batch):
            done = 0
            while done < len(s.tokens):
                take = min(room, len(s.tokens) - done)
                want = [int(w) - done for w in s.want if done <= int(w) < done + take]
                current.append((SequenceStep(s.slot, s.tokens[done:done + take], want), i, done))
                room -= take
                done += take
                if room == 0:
                    portions.append(current)
                    current, room = [], max_step_tokens
        if current:
            portions.append(current)
        rows = []
        for portion in portions:
            rows.append(self.step([p[0] for p in portion]))
            keys += [(i, done + w) for step, i, done in portion for w in step.want]
        logits = torch.cat(rows, dim=0)
        wanted = [(i, int(w)) for i, s in enumerate(batch) for w in s.want]
        if keys == wanted:
            return logits
        # wanted places that were not in ascending order within a sequence
        at = {}
        for r, k in enumerate(keys):
            at.setdefault(k, []).append(r)
        order = [at[k].pop(0) for k in wanted]
        return logits[torch.tensor(order, dtype=torch.long, device=logits.device)]

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
