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
           mode: int, workspace=None) -> None:
    """``workspace``: the step's buffers (``engine.workspace.Workspace``); with it the adding
    tensor-core product may cut a long K among several CTAs per tile (few rows, few tiles),
    which needs scratch for their partial sums."""
    m, (n, k) = x.shape[0], weight.shape
    if x.dtype == torch.bfloat16 and ops.gemm_tc_takes(m, n, k):
        scratch = tickets = None
        if mode == ADD_F32 and workspace is not None and ops.GEMM_SPLIT_K:
            splits, floats, tiles = ops.gemm_tc_splits(m, n, k, x.device)
            if splits > 1:
                scratch = workspace.get("gemm_split_sums", (floats,), torch.float32)
                tickets = workspace.zeros("gemm_split_tickets", (tiles,), torch.int32)
        ops.gemm_tc(x, weight, bias, out, mode, split_scratch=scratch, split_tickets=tickets)
    else:
        ops.gemm_simt(x, weight, bias, out, mode)
