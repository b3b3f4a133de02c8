"""The generation loop above the step function.

Requests are taken in order into batches; the prompts of a batch run in one
step, then every live sequence gets one token per step; a sequence ends on a
stop token (which is emitted), at its length, or when the caller's callback
says so, gives its slot back, and the batch goes on without it; batches follow
one another until no request is left.  A request that cannot run (bad token,
too long, bad sampling policy) gets its error in its own result and stops no
other request; when a step of a batch fails, its unfinished requests are run
again one by one, so that each request is a failure domain of its own
(NNIS: crates/nnis-model/src/session_batch.rs:82-111; stop rule
crates/nnis-model/src/runtime.rs:848-899; capacity rule :1143-1151).

A request normally gets a slot of the cache for as long as it runs and its last
token is not run through the model: nothing reads what that would compute.  A
request that names a slot of its caller (``GenerationRequest.slot``: a session)
runs on that slot, after what the slot holds, and keeps it; there every emitted
token is executed, the last one and a stop token too, so that the sequence can
go on where generation ended, as NNIS's sessions do
(crates/nnis-model/src/runtime.rs:814-846, :1264-1268;
crates/nnis-model/src/streaming.rs:14-20).

The loop talks to a *backend* (``acquire_slot``, ``release_slot``, ``step``,
``greedy``, ``host_rows``), so its decisions can be tested without a GPU.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

from ..cache import PAGE_SIZE
from ..sampling import HostLogitSampler, SamplingConfig, SamplingError
from .engine import SequenceStep

DEFAULT_MAX_NEW_TOKENS = 16  # crates/nnis-cli/src/main.rs:22


class StreamControl(enum.Enum):
    """What ``on_token`` may return (crates/nnis-model/src/streaming.rs:5-12):
    ``STOP`` ends that request cleanly after the token it was called for; anything
    else, ``None`` included, goes on."""
    CONTINUE = "continue"
    STOP = "stop"


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
    # a slot that the caller holds and keeps: the prompt follows what the slot holds,
    # and every emitted token is executed (see the module's docstring)
    slot: Optional[int] = None
    start: int = 0  # positions that ``slot`` holds already


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
    # the last token is not run (so it needs no place in the cache) unless the
    # request keeps its slot
    kept = 0 if request.slot is None else 1
    return -(-(request.start + len(request.prompt) + request.generation.max_new_tokens - 1 + kept)
             // PAGE_SIZE)


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
        need = r.start + len(r.prompt) + r.generation.max_new_tokens
        if need > self.max_positions:
            return (f"prompt + generation requires {need} positions; the model has "
                    f"{self.max_positions}")
        if pages_needed(r) > self.max_pages:
            return (f"prompt + generation needs {pages_needed(r)} cache pages; the cache has "
                    f"{self.max_pages}")
        return None

    # -- picking -----------------------------------------------------------------
    def _pick(self, logits, rows: Sequence[int], requests, samplers, results) -> List[Optional[int]]:
        """One token per row of ``logits``; row j belongs to request rows[j].  A row
        whose request has ended already, or whose sampler refuses its logits (that
        request then ends with the error), gets None."""
        alive = [j for j, i in enumerate(rows) if results[i].finish_reason is None]
        sampled = [j for j in alive if requests[rows[j]].sampling is not None]
        tokens: List[Optional[int]] = [None] * len(rows)
        if len(sampled) < len(alive):
            picked = list(self.backend.greedy(logits))
            for j in alive:
                tokens[j] = int(picked[j])
        on_device = [j for j in sampled if rows[j] in self._device_rng]
        if on_device:
            drawn = self.backend.sample_temperature(
                logits, on_device, [requests[rows[j]].sampling.temperature for j in on_device],
                [self._device_rng[rows[j]] for j in on_device])
            for j, t in zip(on_device, drawn):
                tokens[j] = int(t)
            sampled = [j for j in sampled if rows[j] not in self._device_rng]
        if sampled:
            host = self.backend.host_rows(logits, sampled)
            for k, j in enumerate(sampled):
                try:
                    tokens[j] = int(samplers[rows[j]].sample(host[k]))
                except SamplingError as e:  # this request alone
                    res = results[rows[j]]
                    res.error, res.finish_reason = f"{type(e).__name__}: {e}", "error"
                    tokens[j] = None
        return tokens

    def _samplers_for(self, indices, requests, samplers) -> None:
        """Fresh generators for these requests (at the start, and before a request
        is run again alone)."""
        for i in indices:
            r = requests[i]
            if r.sampling is None:
                continue
            if self.device_sampling and r.sampling.top_k is None and r.sampling.top_p is None:
                self._device_rng[i] = self.backend.new_rng(r.sampling.seed)
            else:
                samplers[i] = HostLogitSampler(r.sampling, self.vocab_size)

    # -- the loop ------------------------------------------------------------------
    def generate(self, requests: Sequence[GenerationRequest],
                 on_token: Optional[Callable[[int, int], Optional[StreamControl]]] = None
                 ) -> List[GenerationResult]:
        """``on_token(request index, token)`` is called as tokens are emitted; when it
        returns ``StreamControl.STOP`` that request ends there (``finish_reason``
        "stop") and the others go on."""
        results = [GenerationResult(i) for i in range(len(requests))]
        runnable = []
        for i, r in enumerate(requests):
            why = self._refusal(r)
            if why is not None:
                results[i].error, results[i].finish_reason = why, "error"
            runnable.append(why is None)
        self._device_rng = {}
        samplers: Dict[int, HostLogitSampler] = {}
        self._samplers_for([i for i in range(len(requests)) if runnable[i]], requests, samplers)
        shown: Dict[int, int] = {}  # tokens of each request that the callback has been shown
        for batch in plan_batches(requests, runnable, self.max_batch, self.max_pages):
            failed = self._run_batch(batch, requests, results, samplers, on_token, shown)
            if failed is not None and len(batch) > 1:
                # a step of the batch failed: each unfinished request again, alone;
                # tokens that the callback has seen already are not shown again
                again = [i for i in batch if results[i].finish_reason is None
                         and requests[i].slot is None]
                for i in again:
                    results[i].token_ids = []
                    self._samplers_for([i], requests, samplers)
                    failed_alone = self._run_batch([i], requests, results, samplers, on_token, shown)
                    self._fail([i], results, failed_alone)
            self._fail(batch, results, failed)
        return results

    @staticmethod
    def _fail(indices, results, error: Optional[BaseException]) -> None:
        if error is None:
            return
        for i in indices:
            if results[i].finish_reason is None:
                results[i].error = f"{type(error).__name__}: {error}"
                results[i].finish_reason = "error"

    def _run_batch(self, batch, requests, results, samplers, on_token, shown) -> Optional[BaseException]:
        """Runs the requests of ``batch`` together.  Returns the exception that ended
        the batch early, if any; requests it left unfinished have no finish reason.
        ``shown[i]``: how many tokens of request i the callback has been shown."""
        slots: Dict[int, int] = {}
        own = {i for i in batch if requests[i].slot is not None}

        def end(i: int) -> None:
            slot = slots.pop(i)
            if i not in own:
                self.backend.release_slot(slot)

        def tell(i: int, t: int) -> bool:
            """The callback for token t of request i; True when it asks to stop."""
            if on_token is None or len(results[i].token_ids) <= shown.get(i, 0):
                return False
            shown[i] = len(results[i].token_ids)
            return on_token(i, t) is StreamControl.STOP

        try:
            for i in batch:
                slots[i] = requests[i].slot if i in own else self.backend.acquire_slot()
            live = list(batch)
            logits = self.backend.step([SequenceStep(slots[i], list(requests[i].prompt),
                                                     [len(requests[i].prompt) - 1]) for i in live])
            if all(requests[i].sampling is None for i in batch) and \
                    getattr(self.backend, "decode_greedy", None) is not None and \
                    getattr(self.backend, "pipeline", True):
                self._run_greedy_on_device(batch, requests, results, slots, own, logits, tell, end)
                return None
            while True:
                tokens = self._pick(logits, live, requests, samplers, results)
                run, emitted = [], []  # (request, token, whether it goes on)
                for i, t in zip(live, tokens):
                    res, gen = results[i], requests[i].generation
                    if t is None:  # ended before this step, or its sampler refused
                        if i in slots:
                            end(i)
                        continue
                    res.token_ids.append(t)
                    emitted.append((i, t))
                    if t in gen.stop_token_ids:
                        res.finish_reason = "stop"
                    elif len(res.token_ids) >= gen.max_new_tokens:
                        res.finish_reason = "length"
                    if res.finish_reason is None:
                        run.append((i, t, True))
                    elif i in own:
                        run.append((i, t, False))  # executed all the same, no logits wanted
                        end(i)
                    else:
                        end(i)
                # the step first, the callback after it: a request on its caller's slot
                # has executed every token that its caller has been shown
                if run:
                    rows = [i for i, _, goes_on in run if goes_on]
                    logits = self.backend.step(
                        [SequenceStep(slots.get(i, requests[i].slot), [t], [0] if goes_on else [])
                         for i, t, goes_on in run],
                        need_logits=any(requests[i].sampling is not None for i in rows))
                    live = rows
                for i, t in emitted:
                    if tell(i, t) and results[i].finish_reason is None:
                        results[i].finish_reason = "stop"
                        end(i)
                if not any(results[i].finish_reason is None for i in live) or not run:
                    break
            return None
        except Exception as e:  # what is unfinished may run again alone; later batches still run
            return e
        finally:
            for i in list(slots):
                end(i)

    def _run_greedy_on_device(self, batch, requests, results, slots, own, logits, tell, end) -> None:
        """All-greedy batches: the backend keeps tokens and positions on the
        device and tells this loop each step's picks one step late.  The rules
        are the same: a stop token is emitted and ends its sequence, a sequence
        at its length ends, an ended sequence gives its slot back at once.  A row on
        its caller's slot gets one step more than it has tokens to pick, so that its
        last token is executed as well; a token that ended it early has been the input
        of the step launched before the pick was read."""
        first = self.backend.greedy(logits)

        def emit(i: int, t: int) -> bool:
            """Record token t of request i; True if the sequence goes on."""
            res, gen = results[i], requests[i].generation
            res.token_ids.append(int(t))
            if t in gen.stop_token_ids:
                res.finish_reason = "stop"
            elif len(res.token_ids) >= gen.max_new_tokens:
                res.finish_reason = "length"
            if tell(i, int(t)) and res.finish_reason is None:
                res.finish_reason = "stop"
            if res.finish_reason is None:
                return True
            end(i)
            return False

        rows = []
        for i, t in zip(batch, first):
            slot = slots[i]
            position = requests[i].start + len(requests[i].prompt)
            if emit(i, t):
                rows.append((i, slot, int(t), position,
                             requests[i].generation.max_new_tokens - 1 + (1 if i in own else 0)))
            elif i in own:  # ended with its first token: that token is executed here
                self.backend.step([SequenceStep(slot, [int(t)], [])], need_logits=False)
        if rows:
            self.backend.decode_greedy(rows, emit)
