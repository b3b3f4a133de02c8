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
from .engine import Engine, SequenceStep
from .generate import (DEFAULT_MAX_NEW_TOKENS, GenerationConfig, GenerationRequest,
                       GenerationResult, Generator)

Prompt = Union[str, Sequence[int]]


class EngineBackend:
    """What the generation loop needs of an engine."""

    def __init__(self, engine: Engine):
        self.engine = engine

    def acquire_slot(self) -> int:
        return self.engine.acquire_slot()

    def release_slot(self, slot: int) -> None:
        self.engine.release_slot(slot)

    def step(self, batch):
        return self.engine.step(batch)

    def greedy(self, logits: torch.Tensor) -> List[int]:
        out = self.engine.workspace.get("picked", (logits.shape[0],), torch.int32)
        device_sampling.greedy(logits, out)
        return out.tolist()

    def host_rows(self, logits: torch.Tensor, rows: Sequence[int]) -> np.ndarray:
        if len(rows) == logits.shape[0]:
            return logits.cpu().numpy()
        index = torch.tensor(list(rows), dtype=torch.long, device=logits.device)
        return logits[index].cpu().numpy()


def load_tokenizer(tokenizer_file: str):
    from tokenizers import Tokenizer
    return Tokenizer.from_file(tokenizer_file)


class LLM:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device_ordinal: int = 0,
                 device: Optional[str] = None, max_tokens: Optional[int] = None,
                 max_batch: int = 64, tokenizer_file: Optional[str] = None):
        device = device if device is not None else f"cuda:{int(device_ordinal)}"
        self.max_batch = max_batch
        if max_tokens is None:
            max_tokens = 1 << 17
        self.engine = Engine.from_dir(model_dir, dtype=dtype, device=device, max_tokens=max_tokens,
                                      max_slots=max(max_batch, 1))
        self.spec = self.engine.spec
        self.tokenizer = load_tokenizer(tokenizer_file) if tokenizer_file else None
        self._generator = Generator(EngineBackend(self.engine), self.spec.vocab_size,
                                    self.spec.max_positions, max_batch, max_tokens)

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
                 on_token: Optional[Callable[[int, int], None]] = None) -> List[GenerationResult]:
        """Greedy unless ``sampling`` is given (one policy for all prompts or one
        per prompt).  ``stop_token_ids=None`` takes config.json's eos ids."""
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

    def generate(self, input_ids: Sequence[int], generation: GenerationConfig) -> List[int]:
        return self._generate(input_ids, generation, None)

    def generate_sampled(self, input_ids: Sequence[int], generation: GenerationConfig,
                         sampling: SamplingConfig) -> List[int]:
        return self._generate(input_ids, generation, sampling)

    def _generate(self, input_ids, generation, sampling) -> List[int]:
        self.close()
        try:
            res = self.llm._generator.generate([GenerationRequest(list(input_ids), generation,
                                                                  sampling)])[0]
        finally:
            self.slot = self.engine.acquire_slot()
        if res.error is not None:
            raise ValueError(res.error)
        return res.token_ids
