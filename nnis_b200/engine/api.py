"""The Python entry point.

``LLM`` loads a model folder (the model class comes from config.json) and
generates for batches of prompts; ``InferenceSession`` is NNIS's one-sequence
surface - ``prefill``, ``decode_one``, ``generate``, ``generate_sampled``,
``reset`` (crates/nnis-model/src/runtime.rs:745-899,
crates/nnis-model/src/sampling.rs:216-255) - on a slot of the shared cache.
NNIS's own Python entry is a process wrapper around its binary with the options
``model_dir``, ``tokenizer_file``, ``prompt``, ``device_ordinal``,
``max_new_tokens`` (tools/nnis_hub_hf_generate.py:189-231); the same names are
used here in process.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Union

import numpy as np
import torch

from ..sampling import SamplingConfig
from ..sampling import device as device_sampling
from ..cache import PAGE_SIZE
from ..csrc import ops
from .decode import GraphDecoder
from .engine import Engine, SequenceStep, StepError
from .generate import (DEFAULT_MAX_NEW_TOKENS, GenerationConfig, GenerationRequest,
                       GenerationResult, Generator, StreamControl)

Prompt = Union[str, Sequence[int]]


class EngineBackend:
    """What the generation loop needs of an engine."""

    def __init__(self, engine: Engine, max_rows: int = 64, pipeline: bool = True,
                 max_step_tokens: int = 16384):
        self.engine = engine
        self.max_rows = max_rows
        # most tokens of one prompt step; longer batches of prompts run in portions
        self.max_step_tokens = max_step_tokens
        # True: all-greedy batches keep tokens on the device and the host reads
        # picks one step late.  False: every step's tokens come from the host.
        self.pipeline = pipeline
        self._decoders = {}
        self._views = {}
        self._pinned = None
        self._picked = None
        self._picked_for = None
        self._pick_host = None
        self._pick_np = None
        self.h2d_bytes = 0  # counted from the tensors copied, for measurements
        self.d2h_bytes = 0
        parts = [p for b in engine.model.blocks for p in b.parts()]
        if not all(getattr(p, "device_only", True) for p in parts):
            self.decode_greedy = None  # a part loops on the host: no graph

    def acquire_slot(self) -> int:
        return self.engine.acquire_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def step(self, batch, need_logits: bool = True):
        """Logits [len(batch) wanted rows, vocab] (or None when ``need_logits`` is
        false and the step could pick on the device: ``greedy`` then has the
        picks).  Steps in which every sequence brings one token and wants its
        logits run as a CUDA graph whose inputs (tokens, positions, page tables)
        come from the host in one copy."""
        single = True
        for s in batch:
            want = s.want
            if len(s.tokens) != 1 or len(want) != 1 or want[0] != 0:
                single = False
                break
        if not single or self.decode_greedy is None or len(batch) > self.max_rows:
            self._picked = None
            return self.engine.step_in_portions(batch, self.max_step_tokens)
        engine, cache = self.engine, self.engine.cache
        vocab = engine.spec.vocab_size
        slots, tokens = [], []
        for s in batch:
            token = int(s.tokens[0])
            if not 0 <= token < vocab:
                raise StepError(f"slot {s.slot}: token {s.tokens[0]} is outside the vocabulary")
            slots.append(s.slot)
            tokens.append(token)
        positions = [cache.length(s) for s in slots]
        new_lengths = [p + 1 for p in positions]
        cache.reserve(slots, new_lengths)
        dec = self._decoder(len(batch), max(new_lengths), need_logits)
        self.h2d_bytes += dec.upload(tokens, positions, slots)
        dec.launch()
        cache.commit(slots, new_lengths)
        n = len(batch)
        views = self._views.get((id(dec), n))
        if views is None:  # (slicing a tensor costs microseconds: once per decoder and row count)
            views = self._views[(id(dec), n)] = (dec.picked[:n], dec.logits[:n] if dec.logits is not None else None)
        self._picked = views[0]
        return views[1] if need_logits else None

    def greedy(self, logits: Optional[torch.Tensor]) -> List[int]:
        if self._picked is not None:  # the graph has picked already
            n = self._picked.numel()
            self.d2h_bytes += n * 4
            if self._pick_host is None or self._pick_host.numel() < n:
                self._pick_host = torch.empty(max(n, self.max_rows), dtype=torch.int32, pin_memory=True)
                self._pick_np = self._pick_host.numpy()
            ops.copy_async(self._pick_host[:n], self._picked)
            ops.stream_synchronize()
            return self._pick_np[:n].tolist()
        out = self.engine.workspace.get("picked", (logits.shape[0],), torch.int32)
        device_sampling.greedy(logits, out)
        self.d2h_bytes += out.numel() * 4
        return out.tolist()

    def new_rng(self, seed: int) -> torch.Tensor:
        """A SplitMix64 state on the device (int64 [1]) for one request."""
        return device_sampling.seed_states([seed], self.engine.device)

    def sample_temperature(self, logits: torch.Tensor, rows: Sequence[int],
                           temperatures: Sequence[float], states: Sequence[torch.Tensor]) -> List[int]:
        """One seeded draw per named row of ``logits`` on the device; each row's
        generator state advances in place."""
        index = torch.tensor(list(rows), dtype=torch.long, device=logits.device)
        picked_rows = logits if len(rows) == logits.shape[0] and list(rows) == list(range(len(rows))) \
            else logits[index].contiguous()
        temps = torch.tensor([float(t) for t in temperatures], dtype=torch.float32, device=logits.device)
        state = torch.cat(list(states))
        out = torch.empty(len(rows), dtype=torch.int32, device=logits.device)
        device_sampling.temperature(picked_rows, temps, state, out)
        for s, new in zip(states, state.split(1)):
            s.copy_(new)
        self.d2h_bytes += out.numel() * 4
        return out.tolist()

    def host_rows(self, logits: torch.Tensor, rows: Sequence[int]) -> np.ndarray:
        if len(rows) == logits.shape[0]:
            return logits.cpu().numpy()
        index = torch.tensor(list(rows), dtype=torch.long, device=logits.device)
        return logits[index].cpu().numpy()


    # -- greedy decoding with the batch's state on the device -------------------
    def _decoder(self, rows: int, max_context: int, want_logits: bool = False) -> GraphDecoder:
        bucket = 1
        while bucket < rows:
            bucket *= 2
        pages = 4
        while pages * PAGE_SIZE < max_context:
            pages *= 2
        context = min(pages * PAGE_SIZE, self.engine.spec.max_positions)
        key = (bucket, context, want_logits)
        if key not in self._decoders:
            self._decoders[key] = GraphDecoder(self.engine, bucket, context, want_logits)
        return self._decoders[key]

    def decode_greedy(self, rows, emit) -> None:
        """rows: (request, slot, next input token, its position, tokens still to
        pick).  Calls ``emit(request, token)`` for every pick in order; a False
        return means that sequence has ended (its slot is already given back)."""
        cache = self.engine.cache
        dec = self._decoder(len(rows), max(pos + left + 1 for _, _, _, pos, left in rows))
        live = {}
        for r, (i, slot, token, pos, left) in enumerate(rows):
            dec.set_row(r, slot, token, pos)
            live[r] = [i, slot, pos, left]
        for r in range(len(rows), dec.rows):
            dec.clear_row(r)
        if self._pinned is None or self._pinned.shape[1] < dec.rows:
            self._pinned = torch.empty((2, max(dec.rows, self.max_rows)), dtype=torch.int32,
                                       pin_memory=True)
        ended = set()
        pending = None
        turn = 0
        while live or pending is not None:
            launched = None
            if live:
                for r, (i, slot, pos, left) in live.items():
                    cache.reserve([slot], [pos + 1])
                    dec.sync_pages(r, slot)
                    cache.commit([slot], [pos + 1])
                dec.launch()
                buf = self._pinned[turn % 2]
                turn += 1
                launched = (dec.picks_to_host(buf[:dec.rows]), buf, {r: v[0] for r, v in live.items()})
                for r in list(live):
                    live[r][2] += 1
                    live[r][3] -= 1
                    if live[r][3] == 0:  # this step picked its last token
                        del live[r]
                        dec.clear_row(r)
            if pending is not None:
                event, buf, who = pending
                event.synchronize()
                for r, i in who.items():
                    if i in ended:
                        continue  # it had stopped before this step was read: the pick is dropped
                    if not emit(i, int(buf[r])):
                        ended.add(i)
                        if r in live:
                            del live[r]
                            dec.clear_row(r)
            pending = launched


def load_tokenizer(tokenizer_file: str):
    from tokenizers import Tokenizer
    return Tokenizer.from_file(tokenizer_file)


class LLM:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device_ordinal: int = 0,
                 device: Optional[str] = None, max_tokens: Optional[int] = None,
                 max_batch: int = 64, tokenizer_file: Optional[str] = None,
                 pipeline_decode: bool = True, device_sampling: bool = False,
                 max_step_tokens: int = 16384):
        device = device if device is not None else f"cuda:{int(device_ordinal)}"
        self.max_batch = max_batch
        if max_tokens is None:
            max_tokens = 1 << 17
        self.engine = Engine.from_dir(model_dir, dtype=dtype, device=device, max_tokens=max_tokens,
                                      max_slots=max(max_batch, 1))
        self.spec = self.engine.spec
        self.tokenizer = load_tokenizer(tokenizer_file) if tokenizer_file else None
        self.backend = EngineBackend(self.engine, max_batch, pipeline_decode, max_step_tokens)
        self._generator = Generator(self.backend, self.spec.vocab_size,
                                    self.spec.max_positions, max_batch, max_tokens, device_sampling)

    # -- text ---------------------------------------------------------------
    def encode(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer (tokenizer_file=...)")
        # special tokens on, as NNIS's command line does (crates/nnis-cli/src/main.rs:1075-1090)
        return list(self.tokenizer.encode(text, add_special_tokens=True).ids)

    def decode(self, ids: Sequence[int]) -> str:
        if self.tokenizer is None:
            raise ValueError("decoding to text needs a tokenizer (tokenizer_file=...)")
        return self.tokenizer.decode(list(ids), skip_special_tokens=True)

    # -- generation ---------------------------------------------------------
    def generate(self, prompts: Sequence[Prompt], max_new_tokens: int = DEFAULT_MAX_NEW_TOKENS,
                 sampling: Union[None, SamplingConfig, Sequence[Optional[SamplingConfig]]] = None,
                 stop_token_ids: Optional[Sequence[int]] = None,
                 on_token: Optional[Callable[[int, int], Optional[StreamControl]]] = None
                 ) -> List[GenerationResult]:
        """Greedy unless ``sampling`` is given (one policy for all prompts or one
        per prompt).  ``stop_token_ids=None`` takes config.json's eos ids.
        ``on_token(prompt index, token)`` sees tokens as they are emitted and may return
        ``StreamControl.STOP`` to end that prompt's generation; the others go on."""
        stops = tuple(self.spec.stop_token_ids if stop_token_ids is None else stop_token_ids)
        if sampling is None or isinstance(sampling, SamplingConfig):
            sampling = [sampling] * len(prompts)
        if len(sampling) != len(prompts):
            raise ValueError(f"{len(prompts)} prompts but {len(sampling)} sampling policies")
        gen = GenerationConfig(max_new_tokens=max_new_tokens, stop_token_ids=stops)
        requests = [GenerationRequest(self.encode(p) if isinstance(p, str) else list(p), gen, s)
                    for p, s in zip(prompts, sampling)]
        return self._generator.generate(requests, on_token)

    def new_session(self) -> "InferenceSession":
        return InferenceSession(self)


class InferenceSession:
    """One sequence on one slot; logits come back to the host as float32."""

    def __init__(self, llm: LLM):
        self.llm = llm
        self.engine = llm.engine
        self.slot = self.engine.acquire_slot()

    def position(self) -> int:
        return self.engine.cache.length(self.slot)

    def capacity(self) -> int:
        return self.engine.spec.max_positions

    def reset(self) -> None:
        self.engine.release_slot(self.slot)
        self.slot = self.engine.acquire_slot()

    def truncate(self, position: int) -> None:
        """Back to ``position`` tokens, as NNIS's sessions allow
        (crates/nnis-core/src/session.rs:430-445): the next ``decode_one`` follows them."""
        self.engine.truncate(self.slot, int(position))

    def snapshot(self):
        """Where the session is now, to come back to with ``restore`` after further
        tokens: the way back for a model whose layers keep state of fixed size, which
        cannot be truncated; for keys and values alone it is the same as ``truncate``."""
        return self.engine.snapshot(self.slot)

    def restore(self, snapshot) -> None:
        self.engine.restore(snapshot)

    def close(self) -> None:
        if self.slot is not None:
            self.engine.release_slot(self.slot)
            self.slot = None

    def prefill(self, input_ids: Sequence[int]) -> np.ndarray:
        """Resets, runs the prompt in one step, returns the last position's logits."""
        self.reset()
        ids = list(input_ids)
        if not ids:
            raise ValueError("the prompt is empty")
        logits = self.engine.step([SequenceStep(self.slot, ids, [len(ids) - 1])])
        return logits[0].cpu().numpy()

    def decode_one(self, token: int) -> np.ndarray:
        logits = self.engine.step([SequenceStep(self.slot, [int(token)], [0])])
        return logits[0].cpu().numpy()

    def generate(self, input_ids: Sequence[int], generation: GenerationConfig,
                 on_token: Optional[Callable[[int], Optional[StreamControl]]] = None,
                 keep_context: bool = False) -> List[int]:
        """Greedy generation on this session's own slot
        (crates/nnis-model/src/runtime.rs:796-899).  Like NNIS it starts from an empty
        session (``keep_context=True``: the prompt follows what the session holds) and
        executes every emitted token, the last one and a stop token too, so that
        afterwards ``position()`` is prompt + emitted tokens (runtime.rs:1264-1268) and
        ``decode_one`` goes on from there."""
        return self._generate(input_ids, generation, None, on_token, keep_context)

    def generate_sampled(self, input_ids: Sequence[int], generation: GenerationConfig,
                         sampling: SamplingConfig, keep_context: bool = False) -> List[int]:
        """crates/nnis-model/src/sampling.rs:216-255: seeded sampling on the host's
        policy, every emitted token executed."""
        return self._generate(input_ids, generation, sampling, None, keep_context)

    def generate_sampled_streaming(self, input_ids: Sequence[int], generation: GenerationConfig,
                                   sampling: SamplingConfig,
                                   on_token: Callable[[int], Optional[StreamControl]],
                                   keep_context: bool = False) -> List[int]:
        """crates/nnis-model/src/streaming.rs:25-72: ``on_token(token)`` is called for
        each emitted token once it has been executed; ``StreamControl.STOP`` ends the
        generation cleanly and leaves the session ready to go on."""
        return self._generate(input_ids, generation, sampling, on_token, keep_context)

    def _generate(self, input_ids, generation, sampling, on_token, keep_context) -> List[int]:
        if not keep_context:
            self.reset()
        request = GenerationRequest(list(input_ids), generation, sampling, slot=self.slot,
                                    start=self.position())
        callback = None if on_token is None else (lambda _i, t: on_token(t))
        res = self.llm._generator.generate([request], callback)[0]
        if res.error is not None:
            raise ValueError(res.error)
        return res.token_ids
