"""Picking tokens on the device: greedy argmax for any batch, and seeded
temperature sampling whose generator state lives beside the batch on the GPU.
The kernels are in ``csrc/sampling.cu``."""
from __future__ import annotations

import torch

from ..csrc import ops


def greedy(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """int32 ids of the largest logit per row; ties go to the lower id."""
    ops.argmax(logits, out)
    return out


def seed_states(seeds, device) -> torch.Tensor:
    """SplitMix64 states (the seeds themselves) as an int64 device tensor."""
    signed = [s - (1 << 64) if s >= (1 << 63) else s for s in seeds]
    return torch.tensor(signed, dtype=torch.int64, device=device)


def temperature(logits: torch.Tensor, temperatures: torch.Tensor, rng_state: torch.Tensor,
                out: torch.Tensor) -> torch.Tensor:
    ops.sample_temperature(logits, temperatures, rng_state, out)
    return out
