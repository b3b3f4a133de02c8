"""Gated feed-forward: down( act(gate(x)) * up(x) ), added to the residual.

Gate and up are one projection (their matrices stacked along the output rows
at load) with float32 output; the activation kernel rounds once to the operand
dtype.  Steps 14-18 of NNIS's token pass
(crates/nnis-model/src/runtime.rs:1054-1093).

params: hidden_size, intermediate_size, activation ("silu"), bias,
names {gate, up, down}.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import FEED_FORWARDS, Part, begin_norm
from .linear import ADD_F32, STORE_F32, linear


class GatedMLP(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.bias = bool(params.get("bias", False))
        self.names = params["names"]
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} has no kernel")
        self.w_gu = self.b_gu = self.w_down = self.b_down = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        H, I = self.hidden, self.inter
        specs = {self.tensor_name(self.names["gate"]): WeightSpec((I, H), "matrix", fan_in=H),
                 self.tensor_name(self.names["up"]): WeightSpec((I, H), "matrix", fan_in=H),
                 self.tensor_name(self.names["down"]): WeightSpec((H, I), "matrix", fan_in=I)}
        if self.bias:
            specs[self.tensor_name(self.names["gate"], "bias")] = WeightSpec((I,), "vector")
            specs[self.tensor_name(self.names["up"], "bias")] = WeightSpec((I,), "vector")
            specs[self.tensor_name(self.names["down"], "bias")] = WeightSpec((H,), "vector")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        n = self.names
        self.w_gu = torch.cat([tensors[self.tensor_name(n["gate"])],
                               tensors[self.tensor_name(n["up"])]], 0).contiguous()
        self.w_down = tensors[self.tensor_name(n["down"])]
        if self.bias:
            self.b_gu = torch.cat([tensors[self.tensor_name(n["gate"], "bias")],
                                   tensors[self.tensor_name(n["up"], "bias")]], 0).contiguous()
            self.b_down = tensors[self.tensor_name(n["down"], "bias")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.w_gu, self.w_down, self.b_gu, self.b_down) if t is not None)

    def step_flops(self, counts, starts) -> float:
        return 2.0 * 3 * self.hidden * self.inter * sum(counts)

    def _fused_gate_up(self, ctx, n: int, normed: bool = False) -> bool:
        """The fused bfloat16 decode kernel for gate/up (few rows, one token each)."""
        return (self.dtype == torch.bfloat16 and ctx.decode
                and ops.gemv_pays(n, 2 * self.inter, self.hidden, ops.EPI_GATED, self.device, normed))

    def _fused_down(self, ctx, n: int) -> bool:
        return (self.dtype == torch.bfloat16 and ctx.decode
                and ops.gemv_pays(n, self.hidden, self.inter, ops.EPI_ADD_F32, self.device))

    def fuses_norm(self, norm, ctx, n: int) -> bool:
        return getattr(norm, "kind", None) == "rmsnorm" and self._fused_gate_up(ctx, n, normed=True)

    def shares_norm(self, norm, ctx, n: int) -> bool:
        """Whether gate/up can end a norm that the projection before it began."""
        return (getattr(norm, "kind", None) == "rmsnorm" and self.dtype == torch.bfloat16 and ctx.decode
                and ops.gemv_shares_norm(n, 2 * self.inter, self.hidden, ops.EPI_GATED, self.device))

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor) -> None:
        self._run(ctx, residual, x=x)

    def forward_shared(self, begun, residual: torch.Tensor, ctx) -> None:
        """The same on rows that the part before left weighted, with their sums of squares."""
        self._run(ctx, residual, begun=begun)

    def forward_normed(self, hidden: torch.Tensor, norm, ctx) -> None:
        """The same with the block's norm folded into the gate/up projection."""
        self._run(ctx, hidden, hidden=hidden, norm=norm)

    def _run(self, ctx, residual, x=None, hidden=None, norm=None, begun=None) -> None:
        n = residual.shape[0]
        ws = ctx.workspace
        act = ws.get("act", (n, self.inter), self.dtype)
        if begun is not None:
            ops.gemv_bf16(self.w_gu, self.b_gu, act, ops.EPI_GATED, x=begun.x, shares=begun.shares,
                          eps=begun.norm.eps, m=n)
        elif self._fused_gate_up(ctx, n, normed=hidden is not None):
            ops.gemv_bf16(self.w_gu, self.b_gu, act, ops.EPI_GATED, x=x, hidden=hidden,
                          norm_weight=norm.weight if norm is not None else None,
                          eps=norm.eps if norm is not None else 0.0, m=n)
        elif self.dtype == torch.bfloat16 and ops.gemm_tc_takes(n, 2 * self.inter, self.hidden):
            # tensor-core product with the activation in its epilogue
            ops.gemm_tc(x, self.w_gu, self.b_gu, act, ops.GEMM_GATED)
        else:
            gate_up = ws.get("gate_up", (n, 2 * self.inter), torch.float32)
            linear(x, self.w_gu, self.b_gu, gate_up, STORE_F32)
            ops.silu_mul(gate_up, act)
        if self._fused_down(ctx, n):
            ops.gemv_bf16(self.w_down, self.b_down, residual, ops.EPI_ADD_F32, x=act,
                          emit=begin_norm(ctx, n, self.hidden))
        else:
            linear(act, self.w_down, self.b_down, residual, ADD_F32, ws)


FEED_FORWARDS.register("gated_mlp", GatedMLP)
