"""RMSNorm with a per-channel weight (NNIS: crates/nnis-model/src/kernels.rs:15-48)."""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import NORMS, Part


class RMSNorm(Part):
    """params: size, eps, name (tensor stem)."""
    kind = "rmsnorm"  # parts that can fold this norm into their first projection look for it

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = self.tensor_name(params["name"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.size,), "vector", init="ones")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def parameter_bytes(self) -> int:
        return self.size * 4

    def forward(self, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None) -> None:
        ops.rmsnorm(x, self.weight, self.eps, out, rows)


NORMS.register("rmsnorm", RMSNorm)
