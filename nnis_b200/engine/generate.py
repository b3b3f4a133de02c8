"""The generation loop above the step function.

Requests are taken in order into batches; the prompts of a batch run in one
step, then every live sequence gets one token per step; a sequence ends on a
stop token (which is emitted) or at its length, gives its slot back, and the
batch goes on without it; batches follow one another until no request is left.
A request that cannot run (bad token, too long, bad sampling policy) gets its
error in its own result and stops no other request
(NNIS: crates/nnis-model/src/session_batch.rs:82-111; stop rule
crates/nnis-model/src/runtime.rs:848-899; capacity rule :1143-1151).

Unlike NNIS the last token of a sequence is not run through the model: nothing
reads what that would compute.

The loop talks to a *backend* (``acquire_slot``, ``release_slot``, ``step``,
``greedy``, ``host_rows``), so its decisions can be tested without a GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache import PAGE_SIZE
from ..sampling import HostLogitSampler, SamplingConfig, SamplingError
from .engine import SequenceStep

DEFAULT_MAX_NEW_TOKENS = 16  # crates/nnis-cli/src/main.rs:22


@dataclass(frozen=True)
class GenerationConfig:
    """crates/nnis-model/src/config.rs:134-182, with a set of stop tokens."""
    max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS
    stop_token_ids: Tuple[int, ...] = ()

    def validate(self, vocab_size: int) -> None:
        if self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be positive; got {self.max_new_tokens}")
        for t in self.stop_token_ids:
            if not 0 <= t < vocab_size:
                raise ValueError(f"stop token {t} is outside the vocabulary of {vocab_size}")


@dataclass
class GenerationRequest:
    prompt: Sequence[int]
    generation: GenerationConfig = GenerationConfig()
    sampling: Optional[SamplingConfig] = None  # None: greedy


@dataclass
class GenerationResult:
    index: int
    token_ids: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None  # "stop" | "length" | "error"
    error: Optional[str] = None

    @property
    def ok(self) -> bool:
        return self.error is None


def pages_needed(request: GenerationRequest) -> int:
    # the last token is never run, so it needs no place in the cache
    return -(-(len(request.prompt) + request.generation.max_new_tokens - 1) // PAGE_SIZE)


def plan_batches(requests: Sequence[GenerationRequest], runnable: Sequence[bool], max_batch: int,
                 max_pages: int) -> List[List[int]]:
    """Request indices per batch, in order; a batch closes when it is full or
    the next request's pages would not fit beside it."""
    batches: List[List[int]] = []
    current: List[int] = []
    pages = 0
    for i, r in enumerate(requests):
        if not runnable[i]:
            continue
        need = pages_needed(r)
        if current and (len(current) >= max_batch or pages + need > max_pages):
            batches.append(current)
            current, pages = [], 0
        current.append(i)
        pages += need
    if current:
        batches.append(current)
    return batches


class Generator:
    def __init__(self, backend, vocab_size: int, max_positions: int, max_batch: int,
                 max_tokens: int, device_sampling: bool = False):
        if max_batch <= 0:
            raise ValueError("max_batch must be positive")
        self.backend = backend
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self.max_batch = max_batch
        self.max_pages = -(-max_tokens // PAGE_SIZE)
        self._device_rng = {}
        # True: requests that sample with a temperature only (no top-k, no top-p) draw
        # on the device, from SplitMix64 states kept there (same generator and seed as
        # the host sampler, candidates walked in token-id order instead of logit order)
        self.device_sampling = device_sampling and hasattr(backend, "sample_temperature")

    # -- checks made before any work -------------------------------------------
    def _refusal(self, r: GenerationRequest) -> Optional[str]:
        if len(r.prompt) == 0:
            return "the prompt is empty"
        for t in r.prompt:
            if not 0 <= int(t) < self.vocab_size:
                return f"prompt token {t} is outside the vocabulary of {self.vocab_size}"
        try:
            r.generation.validate(self.vocab_size)
            if r.sampling is not None:
                r.sampling.validate(self.vocab_size)
        except (ValueError, SamplingError) as e:
            return str(e)
        need = len(r.prompt) + r.generation.max_new_tokens
        if need > self.max_positions:
            return (f"prompt + generation requires {need} positions; the model has "
                    f"{self.max_positions}")
        if pages_needed(r) > self.max_pages:
            return (f"prompt + generation needs {pages_needed(r)} cache pages; the cache has "
                    f"{self.max_pages}")
        return None

    # -- picking -----------------------------------------------------------------
    def _pick(self, logits, rows: Sequence[int], requests, samplers) -> List[int]:
        """One token per row of ``logits``; row j belongs to request rows[j]."""
        sampled = [j for j, i in enumerate(rows) if requests[i].sampling is not None]
        if len(sampled) < len(rows):
            tokens = list(self.backend.greedy(logits))
        else:
            tokens = [0] * len(rows)
        on_device = [j for j in sampled if rows[j] in self._device_rng]
        if on_device:
            drawn = self.backend.sample_temperature(
                logits, on_device, [requests[rows[j]].sampling.temperature for j in on_device],
                [self._device_rng[rows[j]] for j in on_device])
            for j, t in zip(on_device, drawn):
                tokens[j] = t
            sampled = [j for j in sampled if rows[j] not in self._device_rng]
        if sampled:
            host = self.backend.host_rows(logits, sampled)
            for k, j in enumerate(sampled):
                tokens[j] = samplers[rows[j]].sample(host[k])
        return [int(t) for t in tokens]

    # -- the loop ------------------------------------------------------------------
    def generate(self, requests: Sequence[GenerationRequest],
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """``on_token(request index, token)`` is called as tokens are emitted."""
        results = [GenerationResult(i) for i in range(len(requests))]
        runnable = []
        for i, r in enumerate(requests):
            why = self._refusal(r)
            if why is not None:
                results[i].error, results[i].finish_reason = why, "error"
            runnable.append(why is None)
        self._device_rng = {}
        if self.device_sampling:
            self._device_rng = {i: self.backend.new_rng(r.sampling.seed) for i, r in enumerate(requests)
                                if runnable[i] and r.sampling is not None
                                and r.sampling.top_k is None and r.sampling.top_p is None}
        samplers = {i: HostLogitSampler(r.sampling, self.vocab_size)
                    for i, r in enumerate(requests)
                    if runnable[i] and r.sampling is not None and i not in self._device_rng}
        for batch in plan_batches(requests, runnable, self.max_batch, self.max_pages):
            self._run_batch(batch, requests, results, samplers, on_token)
        return results

    def _run_batch(self, batch, requests, results, samplers, on_token) -> None:
        slots = {}
        try:
            for i in batch:
                slots[i] = self.backend.acquire_slot()
            live = list(batch)
            logits = self.backend.step([SequenceStep(slots[i], list(requests[i].prompt),
                                                     [len(requests[i].prompt) - 1]) for i in live])
            if all(requests[i].sampling is None for i in batch) and \
                    getattr(self.backend, "decode_greedy", None) is not None and \
                    getattr(self.backend, "pipeline", True):
                self._run_greedy_on_device(batch, requests, results, slots, logits, on_token)
                return
            while True:
                tokens = self._pick(logits, live, requests, samplers)
                still = []
                for i, t in zip(live, tokens):
                    res, gen = results[i], requests[i].generation
                    res.token_ids.append(t)
                    if on_token is not None:
                        on_token(i, t)
                    if t in gen.stop_token_ids:
                        res.finish_reason = "stop"
                    elif len(res.token_ids) >= gen.max_new_tokens:
                        res.finish_reason = "length"
                    else:
                        still.append((i, t))
                        continue
                    self.backend.release_slot(slots.pop(i))
                if not still:
                    break
                live = [i for i, _ in still]
                logits = self.backend.step([SequenceStep(slots[i], [t], [0]) for i, t in still],
                                           need_logits=any(requests[i].sampling is not None
                                                           for i in live))
        except Exception as e:  # the batch's requests fail together, later batches still run
            for i in batch:
                if results[i].finish_reason is None:
                    results[i].error, results[i].finish_reason = f"{type(e).__name__}: {e}", "error"
        finally:
            for slot in slots.values():
                self.backend.release_slot(slot)

    def _run_greedy_on_device(self, batch, requests, results, slots, logits, on_token) -> None:
        """All-greedy batches: the backend keeps tokens and positions on the
        device and tells this loop each step's picks one step late.  The rules
        are the same: a stop token is emitted and ends its sequence, a sequence
        at its length ends, an ended sequence gives its slot back at once."""
        first = self.backend.greedy(logits)

        def emit(i: int, t: int) -> bool:
            """Record token t of request i; True if the sequence goes on."""
            res, gen = results[i], requests[i].generation
            res.token_ids.append(int(t))
            if on_token is not None:
                on_token(i, int(t))
            if t in gen.stop_token_ids:
                res.finish_reason = "stop"
            elif len(res.token_ids) >= gen.max_new_tokens:
                res.finish_reason = "length"
            else:
                return True
            self.backend.release_slot(slots.pop(i))
            return False

        rows = []
        for i, t in zip(batch, first):
            if emit(i, t):
                rows.append((i, slots[i], int(t), len(requests[i].prompt),
                             requests[i].generation.max_new_tokens - 1))
        if rows:
            self.backend.decode_greedy(rows, emit)
