"""y (op)= x . W^T + b: picks the kernel for a dtype and a shape.

float32 operands always run on the CUDA cores (no tensor-core mode exists that
keeps 32-bit products).  bfloat16 operands take the tcgen05 kernel where its
tile rules hold and the row count makes it worthwhile, else the CUDA-core
kernel.  NNIS makes the same kind of choice per projection family with its
projection plans (crates/nnis-model/src/projection_plan.rs:10-90).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops

STORE, STORE_F32, ADD_F32 = ops.STORE, ops.STORE_F32, ops.ADD_F32


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
           mode: int) -> None:
    if x.dtype == torch.bfloat16 and ops.gemm_tc_takes(x.shape[0], weight.shape[0], weight.shape[1]):
        ops.gemm_tc(x, weight, bias, out, mode)
    else:
        ops.gemm_simt(x, weight, bias, out, mode)
