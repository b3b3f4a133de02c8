"""Token embedding and the linear head that ends the model.

The head reads the embedding's table when the two are tied; there is no second
copy (NNIS keeps a transposed copy: crates/nnis-model/src/safetensors_loader.rs:755-786).
Logits are float32 in every dtype (crates/nnis-model/src/runtime.rs:1109-1116).
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import EMBEDDINGS, HEADS, Part
from .linear import STORE_F32, linear


class TokenEmbedding(Part):
    """params: vocab_size, hidden_size, name."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab = int(params["vocab_size"])
        self.width = int(params["hidden_size"])
        self.name = self.tensor_name(params["name"])
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.vocab, self.width), "matrix")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]

    def forward(self, tokens: torch.Tensor, hidden: torch.Tensor, status: torch.Tensor) -> None:
        ops.embed(self.table, tokens, hidden, status)


class LinearHead(Part):
    """params: vocab_size, hidden_size, name, tied_to (tensor stem or None)."""

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.vocab = int(params["vocab_size"])
        self.width = int(params["hidden_size"])
        tied = params.get("tied_to")
        self.tied = tied is not None
        self.name = self.tensor_name(tied if self.tied else params["name"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.name: WeightSpec((self.vocab, self.width), "matrix",
                                      fan_in=0 if self.tied else self.width)}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name]

    def parameter_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def step_flops(self, counts, starts, wanted: int = 0) -> float:
        return 2.0 * self.vocab * self.width * wanted

    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> None:
        linear(x, self.weight, None, logits, STORE_F32)

    def fuses_norm(self, norm, rows: int) -> bool:
        return (getattr(norm, "kind", None) == "rmsnorm" and self.dtype == torch.bfloat16
                and rows <= ops.GEMV_HEAD_ROWS
                and ops.gemv_takes(rows, self.vocab, self.width, ops.EPI_STORE_F32, self.device, True))

    def forward_pick(self, hidden: torch.Tensor, norm, rows: torch.Tensor, picks: torch.Tensor,
                     scratch: torch.Tensor, logits: Optional[torch.Tensor] = None,
                     next_tokens: Optional[torch.Tensor] = None,
                     next_pos: Optional[torch.Tensor] = None) -> None:
        """Final norm, head and greedy pick in one kernel; optionally the logits
        too, and the decode state moved on (tokens = picks, positions + 1)."""
        ops.gemv_bf16(self.weight, None, picks, ops.EPI_ARGMAX, hidden=hidden,
                      norm_weight=norm.weight, eps=norm.eps, rows=rows, m=picks.numel(),
                      logits=logits, scratch=scratch, next_tokens=next_tokens, next_pos=next_pos)

    def pick_scratch_ints(self, rows: int) -> int:
        return ops.argmax_scratch_ints(rows, self.vocab, self.width, self.device)

    def forward_normed(self, hidden: torch.Tensor, norm, rows: torch.Tensor,
                       logits: torch.Tensor) -> None:
        """Final norm of the wanted rows folded into the head (few rows)."""
        ops.gemv_bf16(self.weight, None, logits, ops.EPI_STORE_F32, hidden=hidden,
                      norm_weight=norm.weight, eps=norm.eps, rows=rows, m=logits.shape[0])


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("linear_head", LinearHead)
