"""Sampling policy, with NNIS's names, defaults and rules
(crates/nnis-model/src/sampling.rs:20-81; policy version 1).

Greedy decoding is not a temperature of zero: it is the absence of a
``SamplingConfig``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Optional

SAMPLING_POLICY_VERSION = 1
_U64 = (1 << 64) - 1


class SamplingError(ValueError):
    pass


@dataclass(frozen=True)
class SamplingConfig:
    seed: int
    temperature: float = 1.0
    top_k: Optional[int] = None
    top_p: Optional[float] = None

    @classmethod
    def seeded(cls, seed: int) -> "SamplingConfig":
        return cls(seed=seed)

    def with_temperature(self, temperature: float) -> "SamplingConfig":
        return replace(self, temperature=temperature)

    def with_top_k(self, top_k: int) -> "SamplingConfig":
        return replace(self, top_k=top_k)

    def with_top_p(self, top_p: float) -> "SamplingConfig":
        return replace(self, top_p=top_p)

    def validate(self, vocab_size: int) -> None:
        if vocab_size <= 0:
            raise SamplingError("sampling requires a non-zero vocabulary")
        if isinstance(self.seed, bool) or not isinstance(self.seed, int) or not 0 <= self.seed <= _U64:
            raise SamplingError(f"sampling seed must be an unsigned 64-bit integer; got {self.seed!r}")
        t = self.temperature
        if not isinstance(t, (int, float)) or not math.isfinite(t) or t <= 0:
            raise SamplingError(f"sampling temperature must be finite and positive; got {t}")
        if self.top_k is not None and not 1 <= self.top_k <= vocab_size:
            raise SamplingError(f"sampling top_k must be in 1..={vocab_size}; got {self.top_k}")
        if self.top_p is not None:
            p = self.top_p
            if not math.isfinite(p) or p <= 0 or p > 1:
                raise SamplingError(f"sampling top_p must be finite and in (0, 1]; got {p}")
