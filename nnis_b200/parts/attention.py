"""Causal grouped-query attention over the paged cache.

One fused projection makes q, k and v (the three checkpoint matrices are
stacked along their output rows when they are loaded); the RoPE kernel rotates
q and k in place and stores k and v at each token's position; the attention
kernel reads every visible key from the cache; the output projection adds into
the residual stream.  Steps 4-12 of NNIS's token pass
(crates/nnis-model/src/runtime.rs:959-1044).

params: hidden_size, heads, kv_heads, head_dim, bias, window (0: all keys),
position (a PartSpec), names {q, k, v, o}, kv ("own" | "shared").  With
``kv == "shared"`` the part has no k/v projection and reads the cache that the
model hands it (another schedule entry's).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import numpy as np
import torch

from ..cache import PAGE_SIZE, KVRequest, KVView
from ..csrc import ops
from ..weights.loader import WeightSpec
from .base import MIXERS, POSITIONS, Part, begin_norm
from .linear import ADD_F32, STORE, linear


class Attention(Part):
    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params["kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.bias = bool(params.get("bias", False))
        self.window = int(params.get("window", 0))
        self.own_kv = params.get("kv", "own") == "own"
        self.names = params["names"]
        if self.heads % self.kv_heads:
            raise ValueError(f"heads={self.heads} is not a multiple of kv_heads={self.kv_heads}")
        if self.head_dim % 2 or not 2 <= self.head_dim <= 256:
            raise ValueError(f"attention kernels take even head sizes up to 256; got {self.head_dim}")
        pos = params["position"]
        self.position = POSITIONS.build(pos.kind, pos.params, prefix, dtype, device)
        # False: the encoding has arithmetic of its own (``apply``), so the
        # projection runs unfused and the kernels rotate nothing
        self.position_in_kernel = bool(getattr(self.position, "in_kernel", True))
        self.scale = 1.0 / math.sqrt(float(self.head_dim))
        self.stored_kv = self.kv_heads if self.own_kv else 0
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    # -- weights ----------------------------------------------------------
    def _proj_names(self):
        return ("q", "k", "v") if self.own_kv else ("q",)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        d, H = self.head_dim, self.hidden
        rows = {"q": self.heads * d, "k": self.kv_heads * d, "v": self.kv_heads * d}
        specs = {}
        for p in self._proj_names():
            specs[self.tensor_name(self.names[p])] = WeightSpec((rows[p], H), "matrix", fan_in=H)
            if self.bias:
                specs[self.tensor_name(self.names[p], "bias")] = WeightSpec((rows[p],), "vector")
        specs[self.tensor_name(self.names["o"])] = WeightSpec((H, self.heads * d), "matrix",
                                                              fan_in=self.heads * d)
        if self.bias:
            specs[self.tensor_name(self.names["o"], "bias")] = WeightSpec((H,), "vector")
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        ps = self._proj_names()
        self.w_qkv = torch.cat([tensors[self.tensor_name(self.names[p])] for p in ps], 0).contiguous()
        self.w_o = tensors[self.tensor_name(self.names["o"])]
        if self.bias:
            self.b_qkv = torch.cat([tensors[self.tensor_name(self.names[p], "bias")] for p in ps],
                                   0).contiguous()
            self.b_o = tensors[self.tensor_name(self.names["o"], "bias")]

    def parameter_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o, self.b_qkv, self.b_o)
                   if t is not None)

    # -- cache ------------------------------------------------------------
    def cache_request(self) -> Optional[KVRequest]:
        return KVRequest(self.kv_heads, self.head_dim, self.window) if self.own_kv else None

    def check_shared_cache(self, view: KVView) -> None:
        if not isinstance(view, KVView) or tuple(view.k.shape[1:]) != \
                (self.kv_heads, view.page_size, self.head_dim) or view.window != self.window:
            raise ValueError("the shared cache does not fit this attention's heads or window")

    def step_flops(self, counts, starts) -> float:
        d, nq, nkv, H = self.head_dim, self.heads, self.kv_heads, self.hidden
        tokens = sum(counts)
        flops = 2.0 * tokens * H * ((nq + 2 * self.stored_kv) * d + nq * d)
        for c, st in zip(counts, starts):  # scores and weighted values over the visible keys
            keys = sum(min(st + q + 1, self.window) if self.window > 0 else st + q + 1
                       for q in range(c)) if self.window > 0 else c * st + c * (c + 1) // 2
            flops += 4.0 * nq * d * keys
        return flops

    # -- work lists ---------------------------------------------------------
    def _tc_plan_name(self) -> str:
        return f"prefill_tc/window{self.window}/heads{self.heads}"

    TILES_64 = "prefill_mma/tiles64"  # (sequence, first query) per 64 queries of the step

    def step_tables(self, counts, starts, have=()):
        """Work lists of the bfloat16 prompt attention kernels: the units of the
        tcgen05 kernel (head size 64), shared by all layers with this window and
        number of heads, where that kernel pays; else the 64-query tiles of the
        mma.sync kernel (head sizes 64 and 128), the same for every layer."""
        if self.dtype != torch.bfloat16:
            return {}
        name = self._tc_plan_name()
        if ops.attention_prefill_tc_takes(self.head_dim, PAGE_SIZE, self.heads * self.head_dim) \
                and ops.prefill_tc_pays(counts, starts, self.window):
            if name + "/units" in have:
                return {}
            units, slots = ops.prefill_tc_plan(counts, starts, self.window, self.heads,
                                               ops.sm_count(self.device))
            return {name + "/units": units, name + "/slots": np.asarray([slots], dtype=np.int32)}
        if ops.attention_decode_mma_takes(self.head_dim, PAGE_SIZE) and self.TILES_64 not in have:
            tiles = [(i, q0) for i, c in enumerate(counts) for q0 in range(0, int(c), 64)]
            return {self.TILES_64: np.asarray(tiles, dtype=np.int32).reshape(-1, 2)}
        return {}

    # -- run --------------------------------------------------------------
    def _decode_kernels(self, ctx, n: int, normed: bool = False) -> bool:
        """The fused bfloat16 decode kernel for q, k, v: few rows, one token each."""
        return (self.dtype == torch.bfloat16 and ctx.decode
                and self.head_dim % 16 == 0 and self.position_in_kernel
                and ops.gemv_pays(n, self.w_qkv.shape[0], self.hidden, ops.EPI_QKV, self.device, normed))

    def _fused_out(self, ctx, n: int) -> bool:
        return (self.dtype == torch.bfloat16 and ctx.decode
                and ops.gemv_pays(n, self.hidden, self.heads * self.head_dim, ops.EPI_ADD_F32,
                                  self.device))

    def fuses_norm(self, norm, ctx, n: int) -> bool:
        return getattr(norm, "kind", None) == "rmsnorm" and self._decode_kernels(ctx, n, normed=True)

    def shares_norm(self, norm, ctx, n: int) -> bool:
        """Whether the q, k, v projection can end a norm that the projection before it began."""
        return (getattr(norm, "kind", None) == "rmsnorm" and self.dtype == torch.bfloat16 and ctx.decode
                and self.head_dim % 16 == 0 and self.position_in_kernel
                and ops.gemv_shares_norm(n, self.w_qkv.shape[0], self.hidden, ops.EPI_QKV, self.device))

    def forward(self, x: torch.Tensor, ctx, residual: torch.Tensor, cache: KVView) -> None:
        self._run(ctx, residual, cache, x=x)

    def forward_shared(self, begun, residual: torch.Tensor, ctx, cache: KVView) -> None:
        """The same on rows that the part before left weighted, with their sums of squares."""
        self._run(ctx, residual, cache, begun=begun)

    def forward_normed(self, hidden: torch.Tensor, norm, ctx, cache: KVView) -> None:
        """The same with the block's norm folded into the first projection."""
        self._run(ctx, hidden, cache, hidden=hidden, norm=norm)

    def _decode_shape(self, ctx, ctas: int, page_size: int):
        """(slices, stages) of the tensor-core decode kernel for a step with ``ctas``
        groups: the default stages, or one stage less (another CTA per SM) when that
        promises 10 % by the wave model; ``NNIS_DECODE_FILL`` keeps the default."""
        d = self.head_dim
        best = (ctx.decode_splits(ctas, ops.attention_decode_mma_resident(d, self.device), page_size), 0)
        if ops.DECODE_STAGE_CHOICE:
            base = ctx.decode_plan(ctas, ops.attention_decode_mma_resident(d, self.device), page_size)
            fewer = ops.attention_decode_mma_stages(d) - 1
            if fewer >= 2:
                other = ctx.decode_plan(ctas, ops.attention_decode_mma_resident(d, self.device, fewer),
                                        page_size)
                if other[1] < 0.9 * base[1]:
                    best = (other[0], fewer)
        return best

    def _run(self, ctx, residual, cache, x=None, hidden=None, norm=None, begun=None) -> None:
        n = residual.shape[0]
        d, nq, nkv = self.head_dim, self.heads, self.kv_heads
        ws = ctx.workspace
        table = ctx.page_tables[cache.group]
        tables = self.position.rotary_tables() if self.position_in_kernel else None
        cos, sin = tables if tables is not None else (None, None)
        attn = ws.get("attn", (n, nq * d), self.dtype)
        # the tensor-core decode attention: a CTA per (kv head, up to 16 query heads, slice)
        mma_decode = self.dtype == torch.bfloat16 and ctx.decode and n <= 65535 \
            and ops.attention_decode_mma_takes(d, cache.page_size)
        # ... or, with few sequences, short slices whose pages are all in shared memory at once
        tma_splits = ops.attention_decode_tma_plan(
            n, nq, nkv, d, cache.page_size, table.shape[1], self.device, ctx.share) if mma_decode else 0
        if begun is not None or self._decode_kernels(ctx, n, normed=hidden is not None):
            q = ws.get("q", (n, nq * d), self.dtype)
            if begun is not None:
                x, norm = begun.x, begun.norm
            ops.gemv_bf16(self.w_qkv, self.b_qkv, q, ops.EPI_QKV, x=x, hidden=hidden,
                          shares=begun.shares if begun is not None else None,
                          norm_weight=norm.weight if hidden is not None else None,
                          eps=norm.eps if norm is not None else 0.0, m=n,
                          token_pos=ctx.token_pos, token_seq=ctx.token_seq,
                          page_table=table if self.own_kv else None, cos=cos, sin=sin,
                          k_cache=cache.k if self.own_kv else None,
                          v_cache=cache.v if self.own_kv else None, heads=nq,
                          kv_heads=self.stored_kv, head_dim=d, page_size=cache.page_size,
                          # that attention kernel reads only positions, page ids and old
                          # pages before its wait: it may start together with this one
                          release_early=tma_splits > 0)
            q_buf, q_stride = q, nq * d
        elif self.dtype == torch.bfloat16 and ops.gemm_tc_qkv_takes(d) and self.position_in_kernel \
                and ops.gemm_tc_takes(n, self.w_qkv.shape[0], self.hidden):
            # tensor-core product with bias, RoPE and the cache store in its epilogue
            q = ws.get("q", (n, nq * d), self.dtype)
            ops.gemm_tc(x, self.w_qkv, self.b_qkv, q, ops.GEMM_QKV, token_pos=ctx.token_pos,
                        token_seq=ctx.token_seq, page_table=table if self.own_kv else None, cos=cos,
                        sin=sin, k_cache=cache.k if self.own_kv else None,
                        v_cache=cache.v if self.own_kv else None, heads=nq, kv_heads=self.stored_kv,
                        head_dim=d, page_size=cache.page_size)
            q_buf, q_stride = q, nq * d
        else:
            qkv = ws.get("qkv", (n, (nq + 2 * self.stored_kv) * d), self.dtype)
            linear(x, self.w_qkv, self.b_qkv, qkv, STORE)
            if not self.position_in_kernel:  # an encoding with arithmetic of its own
                self.position.apply(qkv, ctx, nq, self.stored_kv, d)
            ops.rope_store(qkv, ctx.token_pos, ctx.token_seq, table if self.own_kv else None, cos,
                           sin, cache.k if self.own_kv else None, cache.v if self.own_kv else None,
                           nq, self.stored_kv, d, cache.page_size)
            q_buf, q_stride = qkv, qkv.shape[1]
        if tma_splits:
            partial = tickets = None
            if tma_splits > 1:
                partial = ws.get("attn_partial", (n * nq * tma_splits * (d + 2),), torch.float32)
                tickets = ws.zeros("attn_tickets", (ops.mma_ticket_count(n, nq, nkv),), torch.int32)
            ops.attention_decode_tma(q_buf, q_stride, cache.k, cache.v, ctx.token_pos, ctx.token_seq,
                                     table, attn, nq, nkv, d, self.window, self.scale, tma_splits,
                                     partial, tickets,
                                     ahead=getattr(cache, "ahead", 0) if ops.KV_PREFETCH else 0)
        elif mma_decode:
            tiles = -(-(nq // nkv) // 16)
            splits, stages = self._decode_shape(ctx, n * nkv * tiles, cache.page_size)
            partial = tickets = None
            if splits > 1:
                partial = ws.get("attn_partial", (n * nq * splits * (d + 2),), torch.float32)
                tickets = ws.zeros("attn_tickets", (ops.mma_ticket_count(n, nq, nkv),), torch.int32)
            ops.attention_decode_mma(q_buf, q_stride, cache.k, cache.v, ctx.token_pos, ctx.token_seq,
                                     table, attn, nq, nkv, d, self.window, self.scale, splits,
                                     partial, tickets, stages)
        elif self.dtype == torch.bfloat16 and ctx.decode and n <= 65535 \
                and ops.attention_decode_takes(d):
            tiles = -(-(nq // nkv) // 4)
            splits = ctx.decode_splits(n * nkv * tiles)
            partial = ws.get("attn_partial", (n * nq * splits * (d + 2),), torch.float32) \
                if splits > 1 else None
            ops.attention_decode(q_buf, q_stride, cache.k, cache.v, ctx.token_pos, ctx.token_seq,
                                 table, attn, nq, nkv, d, self.window, self.scale, splits, partial)
        elif self.dtype == torch.bfloat16 and not ctx.decode \
                and self._tc_plan_name() + "/units" in ctx.tables \
                and ops.attention_prefill_tc_takes(d, cache.page_size, q_stride):
            # tcgen05 kernel: a CTA per (128 queries of a sequence, query head, chunk of pages)
            name = self._tc_plan_name()
            slots = int(ctx.host_tables[name + "/slots"][0])
            partial = tickets = None
            if slots:  # tiles were cut: scratch for the chunks, tickets that stay zero between launches
                partial = ws.get("attn_tc_partial", (slots * nq * ops.PREFILL_TC_PARTIAL,), torch.float32)
                tickets = ws.zeros("attn_tc_tickets", (slots * nq,), torch.int32)
            ops.attention_prefill_tc(q_buf, q_stride, cache.k, cache.v, ctx.tables[name + "/units"],
                                     partial, tickets, ctx.seq_first_row, ctx.seq_start, ctx.seq_count,
                                     table, attn, nq, nkv, d, self.window, self.scale)
        elif self.dtype == torch.bfloat16 and not ctx.decode and self.TILES_64 in ctx.tables \
                and ops.attention_decode_mma_takes(d, cache.page_size):
            ops.attention_prefill_mma(q_buf, q_stride, cache.k, cache.v, ctx.tables[self.TILES_64],
                                      ctx.seq_first_row, ctx.seq_start, ctx.seq_count, table, attn,
                                      nq, nkv, d, self.window, self.scale)
        else:
            splits = ctx.attention_splits(n * nq)
            partial = ws.get("attn_partial", (n * nq * splits * (d + 2),), torch.float32) \
                if splits > 1 else None
            ops.attention_generic(q_buf, q_stride, cache.k, cache.v, ctx.token_pos, ctx.token_seq,
                                  table, attn, nq, nkv, d, self.window, self.scale, splits, partial)
        if self._fused_out(ctx, n):
            ops.gemv_bf16(self.w_o, self.b_o, residual, ops.EPI_ADD_F32, x=attn,
                          emit=begin_norm(ctx, n, self.hidden))
        else:
            linear(attn, self.w_o, self.b_o, residual, ADD_F32, ws)


MIXERS.register("attention", Attention)
