"""Position encodings that act on query and key heads.

``rope_half``: Llama's rotate-half RoPE over the whole head, unscaled.  The
cos/sin table is built once in float32 on the host from the reference's formula
(crates/nnis-model/src/runtime.rs:1166-1184): inv_f = 1 / theta^(2j/d),
angle = position * inv_f.  ``none`` leaves heads as they are.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .base import POSITIONS, Part


class RotaryHalf(Part):
    """params: head_dim, theta, max_positions."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        d = int(params["head_dim"])
        half = d // 2
        theta = torch.tensor(float(params["theta"]), dtype=torch.float32)
        exponent = (2 * torch.arange(half, dtype=torch.float32)) / float(d)
        inv_freq = 1.0 / torch.pow(theta, exponent)
        positions = torch.arange(int(params["max_positions"]), dtype=torch.float32)
        angle = positions[:, None] * inv_freq[None, :]
        self.cos = torch.cos(angle).to(device).contiguous()
        self.sin = torch.sin(angle).to(device).contiguous()

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        return self.cos, self.sin


class NoPosition(Part):
    def rotary_tables(self):
        return None


POSITIONS.register("rope_half", RotaryHalf)
POSITIONS.register("none", NoPosition)
