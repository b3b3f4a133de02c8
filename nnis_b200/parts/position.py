"""Position encodings that act on query and key heads.

``rope_half``: Llama's rotate-half RoPE over the whole head, unscaled.  The
cos/sin table is built once in float32 on the host from the reference's formula
(crates/nnis-model/src/runtime.rs:1166-1184): inv_f = 1 / theta^(2j/d),
angle = position * inv_f.  ``none`` leaves heads as they are.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from .base import POSITIONS, PositionEncoding

# one table per (head_dim, theta, max_positions, device): every layer of a model asks
# for the same one
_TABLES: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


class RotaryHalf(PositionEncoding):
    """params: head_dim, theta, max_positions.  The tables are made when first asked
    for (listing a model's tensor names needs none)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.key = (int(params["head_dim"]), float(params["theta"]), int(params["max_positions"]),
                    str(torch.device(device)))

    def rotary_tables(self) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if self.key not in _TABLES:
            d, theta, positions, _ = self.key
            half = d // 2
            exponent = (2 * torch.arange(half, dtype=torch.float32)) / float(d)
            inv_freq = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), exponent)
            angle = torch.arange(positions, dtype=torch.float32)[:, None] * inv_freq[None, :]
            _TABLES[self.key] = (torch.cos(angle).to(self.device).contiguous(),
                                 torch.sin(angle).to(self.device).contiguous())
        return _TABLES[self.key]


class NoPosition(PositionEncoding):
    def rotary_tables(self):
        return None


POSITIONS.register("rope_half", RotaryHalf)
POSITIONS.register("none", NoPosition)
