"""The host sampler: NNIS's frozen policy, token for token.

Order of operations (crates/nnis-model/src/sampling.rs:113-202): sort by logit
descending with the lower id first among equals; keep the top k; weights
exp(logit / T - max) in float64; keep the shortest prefix whose weight reaches
top_p of the total (always at least one); one SplitMix64 draw times the kept
total; the first candidate whose running sum exceeds the draw.  Sums run in
candidate order, as the reference's loops do.
"""
from __future__ import annotations

import numpy as np

from .config import SamplingConfig, SamplingError

_MASK = (1 << 64) - 1


class SplitMix64:
    """crates/nnis-model/src/sampling.rs:261-284."""
    GAMMA = 0x9E3779B97F4A7C15

    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + self.GAMMA) & _MASK
        v = self.state
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & _MASK
        return v ^ (v >> 31)

    def next_unit_f64(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / float(1 << 53))


class HostLogitSampler:
    def __init__(self, config: SamplingConfig, vocab_size: int):
        config.validate(vocab_size)
        self.config = config
        self.vocab_size = vocab_size
        self.rng = SplitMix64(config.seed)

    def sample(self, logits) -> int:
        x = np.asarray(logits, dtype=np.float32).reshape(-1)
        if x.shape[0] != self.vocab_size:
            raise SamplingError(f"sampling expected {self.vocab_size} logits; got {x.shape[0]}")
        finite = np.isfinite(x)
        if not finite.all():
            i = int(np.argmin(finite))
            raise SamplingError(f"sampling logit {i} is non-finite: {x[i]}")
        order = np.argsort(-x.astype(np.float64), kind="stable")
        if self.config.top_k is not None:
            order = order[:self.config.top_k]
        inverse_temperature = 1.0 / float(np.float32(self.config.temperature))
        scaled = x[order].astype(np.float64) * inverse_temperature
        weights = np.exp(scaled - scaled[0])
        running = np.cumsum(weights)  # sequential, in candidate order
        total = float(running[-1])
        if not np.isfinite(total) or total <= 0.0:
            raise SamplingError("sampling softmax produced no positive finite probability mass")
        kept = len(order)
        if self.config.top_p is not None:
            threshold = float(np.float32(self.config.top_p)) * total
            hit = int(np.searchsorted(running, threshold, side="left"))  # first running >= threshold
            kept = max(min(hit + 1, kept), 1)
            total = float(running[kept - 1])
        draw = self.rng.next_unit_f64() * total
        pick = int(np.searchsorted(running[:kept], draw, side="right"))  # first running > draw
        return int(order[min(pick, kept - 1)])
