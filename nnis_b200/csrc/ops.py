"""Python face of the CUDA entry points.

Each function checks dtypes, shapes, contiguity and device before it hands raw
pointers to the library, and turns a non-zero return code into an exception: a
size that a kernel does not take is refused with a message, never run.  Nothing
here computes; without the compiled library nothing works, on purpose.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}
_ARG_ERRORS = {-1: "bad argument", -2: "unsupported size or dtype", -3: "misaligned pointer",
               -4: "a kernel reported an error status"}


class KernelError(RuntimeError):
    pass


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched (or captured) so far in this process."""
    return _launches


def _lib() -> ctypes.CDLL:
    return _build.load()


def _check(code: int, what: str, kernels: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += kernels
        return
    if code < 0:
        raise KernelError(f"{what}: {_ARG_ERRORS.get(code, 'error')} (code {code})")
    raise KernelError(f"{what}: CUDA error {code} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream's handle (the raw getter is some ten microseconds
    cheaper than building a Stream object, and a decode step asks several times)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None:
            _need(t.is_cuda, "kernels take CUDA tensors only (there is no CPU path)")
            _need(t.is_contiguous(), "kernels take contiguous tensors")


def code_of(dtype: torch.dtype) -> int:
    _need(dtype in _DTYPE_CODE, f"dtype {dtype} is not supported (float32 or bfloat16)")
    return _DTYPE_CODE[dtype]


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, hidden: torch.Tensor,
          status: torch.Tensor) -> None:
    """hidden[n] = table[tokens[n]] widened to float32; an id outside the table
    sets ``status[0]`` and yields a zero row."""
    _cuda(table, tokens, hidden, status)
    n, width = hidden.shape
    _need(tokens.dtype == torch.int32 and tokens.numel() >= n, "tokens: int32 [n]")
    _need(hidden.dtype == torch.float32 and table.shape[1] == width, "hidden: float32 [n, width]")
    _need(status.dtype == torch.int32, "status: int32")
    _check(_lib().nnis_embed(_ptr(table), code_of(table.dtype), _ptr(tokens), _ptr(hidden), n, width,
                             table.shape[0], _ptr(status), _stream()), "embed")


def copy_async(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst <- src on the current stream, both contiguous and equally large; the host
    side of the pair must be pinned memory for the copy to be asynchronous."""
    _need(dst.is_contiguous() and src.is_contiguous(), "copy_async: contiguous tensors")
    nbytes = src.numel() * src.element_size()
    _need(nbytes == dst.numel() * dst.element_size(), "copy_async: sizes differ")
    code = _lib().nnis_copy_async(_ptr(dst), _ptr(src), ctypes.c_longlong(nbytes), _stream())
    if code != 0:
        raise KernelError(f"copy_async: CUDA error {code}")


def stream_synchronize() -> None:
    """Wait for the current stream (what ``Stream.synchronize`` does, without the object)."""
    code = _lib().nnis_stream_synchronize(_stream())
    if code != 0:
        raise KernelError(f"stream_synchronize: CUDA error {code}")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * weight, statistics in float32."""
    _cuda(x, weight, out, rows)
    n, width = out.shape
    _need(x.dtype == torch.float32 and x.shape[1] == width, "x: float32 [*, width]")
    _need(weight.dtype == torch.float32 and weight.numel() == width, "weight: float32 [width]")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() >= n, "rows: int32 [n]")
    else:
        _need(x.shape[0] >= n, "x has fewer rows than out")
    _check(_lib().nnis_rmsnorm(_ptr(x), _ptr(rows), _ptr(weight), _ptr(out), code_of(out.dtype), n,
                               width, ctypes.c_float(eps), PDL, _stream()), "rmsnorm")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:], gate_up float32 [n, 2I]."""
    _cuda(gate_up, out)
    n, inter = out.shape
    _need(gate_up.dtype == torch.float32 and tuple(gate_up.shape) == (n, 2 * inter),
          "gate_up: float32 [n, 2 * inter]")
    _check(_lib().nnis_silu_mul(_ptr(gate_up), _ptr(out), code_of(out.dtype),
                                ctypes.c_longlong(n), inter, _stream()), "silu_mul")


def rope_store(qkv: torch.Tensor, token_pos: torch.Tensor, token_seq: torch.Tensor,
               page_table: Optional[torch.Tensor], cos: Optional[torch.Tensor],
               sin: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
               v_cache: Optional[torch.Tensor], heads: int, kv_heads: int, head_dim: int,
               page_size: int) -> None:
    """Rotate q and k heads of packed rows in place, store k and v in the cache.
    ``kv_heads == 0``: the rows hold q only and nothing is stored."""
    _cuda(qkv, token_pos, token_seq, page_table, cos, sin, k_cache, v_cache)
    n = qkv.shape[0]
    _need(qkv.shape[1] == (heads + 2 * kv_heads) * head_dim, "qkv: [n, (heads + 2 kv_heads) * d]")
    _need(token_pos.dtype == torch.int32 and token_seq.dtype == torch.int32, "positions: int32")
    cols = 0
    if kv_heads > 0:
        _need(page_table is not None and page_table.dtype == torch.int32, "page_table: int32")
        _need(k_cache is not None and k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype,
              "cache dtype differs from qkv")
        _need(tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim), "cache: [pages, kv, page, d]")
        cols = page_table.shape[1]
    rotate = 0
    if cos is not None:
        _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "cos/sin: float32 [C, d/2]")
        rotate = 1
    _check(_lib().nnis_rope_store(_ptr(qkv), code_of(qkv.dtype), _ptr(token_pos), _ptr(token_seq),
                                  _ptr(page_table), cols, _ptr(cos), _ptr(sin), _ptr(k_cache),
                                  _ptr(v_cache), n, heads, kv_heads, head_dim, page_size, rotate,
                                  _stream()), "rope_store")


STORE, STORE_F32, ADD_F32 = 0, 1, 2


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
              mode: int) -> None:
    """out (op)= a . w^T + bias on the CUDA cores; float32 accumulation."""
    _cuda(a, w, bias, out)
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and a.dtype == w.dtype, "gemm: a [m, k], w [n, k] of one dtype")
    _need(tuple(out.shape) == (m, n), "gemm: out [m, n]")
    _need(out.dtype == (a.dtype if mode == STORE else torch.float32), "gemm: out dtype vs mode")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: bias float32 [n]")
    _check(_lib().nnis_gemm_simt(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, code_of(a.dtype),
                                 mode, _stream()), "gemm_simt")


def attention_generic(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                      out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                      scale: float, n_splits: int = 1,
                      partial: Optional[torch.Tensor] = None) -> None:
    """Causal attention of packed query tokens over the paged cache."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial)
    _need(q.is_cuda, "q: CUDA tensor")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim % 2 == 0 and 2 <= head_dim <= 256,
          f"attention: head_dim {head_dim} is not an even size in 2..256")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and out.dtype == k_cache.dtype == q.dtype,
          "attention: out [n, heads * d] in the cache dtype")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
    _check(_lib().nnis_attention_generic(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), n, heads, kv_heads, head_dim,
        page_size, window, ctypes.c_float(scale), n_splits, code_of(out.dtype), _stream()),
        "attention_generic", 2 if n_splits > 1 else 1)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(logits, out)
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32, "argmax: float32 -> int32")
    n, vocab = logits.shape
    _need(out.numel() >= n, "argmax: out too small")
    _check(_lib().nnis_argmax(_ptr(logits), _ptr(out), n, vocab, _stream()), "argmax")


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, rng_state: torch.Tensor,
                       out: torch.Tensor) -> None:
    """One seeded draw per row; ``rng_state`` (int64, SplitMix64) advances."""
    _cuda(logits, temperature, rng_state, out)
    n, vocab = logits.shape
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32, "sample: float32 -> int32")
    _need(temperature.dtype == torch.float32 and temperature.numel() >= n, "temperature: float32 [n]")
    _need(rng_state.dtype == torch.int64 and rng_state.numel() >= n, "rng_state: int64 [n]")
    _check(_lib().nnis_sample_temperature(_ptr(logits), _ptr(temperature), _ptr(rng_state),
                                          _ptr(out), n, vocab, _stream()), "sample_temperature")


EPI_STORE, EPI_STORE_F32, EPI_ADD_F32, EPI_GATED, EPI_QKV, EPI_ARGMAX = 0, 1, 2, 3, 4, 5
# programmatic dependent launch between the decode kernels (NNIS_PDL=0 turns it off)
PDL = 0 if os.environ.get("NNIS_PDL", "1") == "0" else 1
# The QKV projection of a decode step lets attention_decode_tma start with it instead of after
# its own wait, so that the copies of old pages run under it (NNIS_EARLY_RELEASE=0: off)
EARLY_RELEASE = 0 if os.environ.get("NNIS_EARLY_RELEASE", "1") == "0" else 1
_status = {}


def status_word(device) -> torch.Tensor:
    """One int32 per device that kernels set when a bounded wait runs out."""
    key = torch.device(device).index or 0
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[key]


def check_status(device) -> None:
    """Raise if a kernel gave up a wait since the last check (synchronises)."""
    word = status_word(device)
    if int(word.item()) != 0:
        word.zero_()
        raise KernelError("a kernel gave up waiting for an asynchronous copy; results are invalid")


def gemv_grid(m: int, n: int, k: int, device) -> int:
    return int(_lib().nnis_gemv_grid(m, n, k, sm_count(device)))
_sm_count = {}


def sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_count:
        _sm_count[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[key]


# The decode projections have two kernels: one whose CTAs hold all rows of x for eight
# output features each (at most 64 rows), and one that cuts the rows into tiles of 16
# (more than 16 rows, few output features, every CTA resident at once).  Where only the
# first applies, the parts choose it up to DECODE_GEMV_ROWS rows, and fold the norm before
# a projection into it up to GEMV_NORM_ROWS rows: every CTA of that kernel normalises all
# rows for itself, through registers, which with more than a tile of rows costs more than
# a norm kernel of its own.  Beyond that the general kernels (tcgen05) run.
DECODE_GEMV_ROWS = int(os.environ.get("NNIS_DECODE_GEMV_ROWS", "48"))
GEMV_NORM_ROWS = int(os.environ.get("NNIS_GEMV_NORM_ROWS", "16"))
# Most wanted rows for which the head runs as the decode projection kernel (with the final
# norm and the greedy pick folded in); with more, its products on mma.sync tiles cost more
# than the weights' way from memory, and the norm, the tcgen05 product and the pick run
# as kernels of their own.
GEMV_HEAD_ROWS = int(os.environ.get("NNIS_GEMV_HEAD_ROWS", "48"))


def gemv_kind(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False,
              rows_kernel: bool = True, shared_norm: bool = False) -> int:
    """Which decode projection kernel runs this product: 2 the one over tiles of rows, 1
    the one whose CTAs hold all rows, 0 neither (the general kernels must run).
    ``rows_kernel=False``: as if the first did not exist.  ``shared_norm``: with the norm
    before it begun by the projection before that (see ``gemv_bf16``'s ``emit``)."""
    sms = sm_count(device) if device is not None else 148
    if shared_norm:
        return int(_lib().nnis_gemv_kind(m, n, k, epilogue, 2, sms)) if rows_kernel else 0
    if not rows_kernel:
        return int(_lib().nnis_gemv_units_takes(m, n, k, epilogue, 1 if normed else 0, sms))
    return int(_lib().nnis_gemv_kind(m, n, k, epilogue, 1 if normed else 0, sms))


# A norm between two decode projections, shared out between them (both halves or neither).
# (bit 0: the norm before a gated feed-forward, bit 1: the norm before q, k, v)
SHARED_NORM = int(os.environ.get("NNIS_SHARED_NORM", "3"))


def gemv_shares_norm(m: int, n: int, k: int, epilogue: int, device=None) -> bool:
    """Whether the decode projection of these sizes can take its input from the epilogue of
    the projection before it (``gemv_bf16`` with ``emit`` there and ``shares`` here)."""
    return bool(SHARED_NORM & (2 if epilogue == EPI_QKV else 1)) \
        and gemv_kind(m, n, k, epilogue, device, shared_norm=True) == 2


def gemv_takes(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False) -> bool:
    """Whether a decode projection kernel can run this shape: K in steps of 16, N in
    steps of 8, operands that fit shared memory; at most 64 rows, or up to 128 where the
    kernel over tiles of rows applies."""
    return gemv_kind(m, n, k, epilogue, device, normed) > 0


def gemv_pays(m: int, n: int, k: int, epilogue: int = EPI_STORE, device=None, normed: bool = False) -> bool:
    """Whether the parts of a decode step should choose a decode projection kernel for
    this product (see the thresholds above)."""
    kind = gemv_kind(m, n, k, epilogue, device, normed)
    return kind == 2 or (kind == 1 and m <= DECODE_GEMV_ROWS and (not normed or m <= GEMV_NORM_ROWS))


def gemv_slices(m: int, n: int, k: int, device=None, rows_kernel: bool = True) -> int:
    """Launches that an ADD_F32 product of these sizes takes (slices of K, each
    adding its share in order); 0: not taken."""
    sms = sm_count(device) if device is not None else 148
    if not rows_kernel:
        return int(_lib().nnis_gemv_units_slices(m, n, k, sms))
    return int(_lib().nnis_gemv_slices(m, n, k, sms))


def gemv_bf16(w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, epilogue: int,
              x: Optional[torch.Tensor] = None, hidden: Optional[torch.Tensor] = None,
              norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
              rows: Optional[torch.Tensor] = None, m: Optional[int] = None,
              token_pos: Optional[torch.Tensor] = None, token_seq: Optional[torch.Tensor] = None,
              page_table: Optional[torch.Tensor] = None, cos: Optional[torch.Tensor] = None,
              sin: Optional[torch.Tensor] = None, k_cache: Optional[torch.Tensor] = None,
              v_cache: Optional[torch.Tensor] = None, heads: int = 0, kv_heads: int = 0,
              head_dim: int = 0, page_size: int = 0, logits: Optional[torch.Tensor] = None,
              scratch: Optional[torch.Tensor] = None, next_tokens: Optional[torch.Tensor] = None,
              next_pos: Optional[torch.Tensor] = None, release_early: bool = False,
              rows_kernel: bool = True, emit: Optional[tuple] = None,
              shares: Optional[torch.Tensor] = None) -> None:
    """A decode-step projection with its prologue and epilogue fused (at most 64
    rows).  The input is ``x`` (bfloat16 [m, k]) or ``hidden`` (float32 residual
    rows, normed with ``norm_weight``/``eps`` on the way in; ``rows`` picks them).
    EPI_ARGMAX writes
    int32 picks to ``out``; ``scratch`` (int32, ``argmax_scratch_ints``) is its
    workspace, ``logits`` optional, ``next_tokens``/``next_pos`` the decode state.
    ``release_early``: the kernel launched after this one may start together with it
    (only for a successor that reads, before its own wait, nothing that a kernel of
    the step writes: attention_decode_tma).  ``rows_kernel=False``: the kernel whose CTAs
    hold all rows even where the one over tiles of rows applies (for comparisons).

    A norm between two projections can be shared out between them.  ``emit`` (EPI_ADD_F32)
    is ``(x_next, norm_weight, shares)``: the epilogue also writes the rows it has summed,
    times ``norm_weight`` (float32 [n]), to ``x_next`` (bfloat16 [m, n]) and every eight
    columns' sum of squares to ``shares`` (float32 [m, n / 8]).  The projection after it
    takes ``x=x_next, shares=shares, eps=`` the norm's, and scales its sums by
    ``1 / sqrt(mean of squares + eps)`` (``gemv_shares_norm`` says whether it can)."""
    _cuda(w, bias, out, x, hidden, norm_weight, rows, token_pos, token_seq, page_table, cos, sin,
          k_cache, v_cache, logits, scratch, next_tokens, next_pos, shares, *(emit or ()))
    n, k = w.shape
    _need(w.dtype == torch.bfloat16, "gemv: bfloat16 weights")
    if hidden is not None:
        _need(hidden.dtype == torch.float32 and hidden.shape[1] == k, "gemv: hidden float32 [*, k]")
        _need(norm_weight is not None and norm_weight.dtype == torch.float32
              and norm_weight.numel() == k, "gemv: norm weight float32 [k]")
        rows_m = rows.numel() if rows is not None else hidden.shape[0]
        m = rows_m if m is None else m
        if rows is not None:
            _need(rows.dtype == torch.int32, "gemv: rows int32")
    else:
        _need(x is not None and x.dtype == torch.bfloat16 and x.shape[1] == k, "gemv: x bfloat16 [m, k]")
        m = x.shape[0] if m is None else m
    if shares is not None:
        _need(hidden is None and eps > 0.0, "gemv: shares come with x and the norm's eps")
        _need(shares.dtype == torch.float32 and tuple(shares.shape) == (m, k // 8) and shares.is_contiguous(),
              "gemv: shares float32 [m, k / 8]")
        _need(gemv_kind(m, n, k, epilogue, w.device, rows_kernel=rows_kernel, shared_norm=True) == 2,
              f"gemv: shape m={m} n={n} k={k} takes no shared norm")
    else:
        _need(gemv_kind(m, n, k, epilogue, w.device, hidden is not None, rows_kernel) > 0,
              f"gemv: shape m={m} n={n} k={k} is not taken")
    emit_x = emit_w = emit_ss = None
    if emit is not None:
        emit_x, emit_w, emit_ss = emit
        _need(epilogue == EPI_ADD_F32, "gemv: only the adding epilogue emits")
        _need(emit_x.dtype == torch.bfloat16 and tuple(emit_x.shape) == (m, n) and emit_x.is_contiguous(),
              "gemv: emit x bfloat16 [m, n]")
        _need(emit_w.dtype == torch.float32 and emit_w.numel() == n, "gemv: emit weight float32 [n]")
        _need(emit_ss.dtype == torch.float32 and tuple(emit_ss.shape) == (m, n // 8) and emit_ss.is_contiguous(),
              "gemv: emit shares float32 [m, n / 8]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemv: bias float32 [n]")
    if epilogue == EPI_STORE:
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n), "gemv: out bfloat16 [m, n]")
    elif epilogue in (EPI_STORE_F32, EPI_ADD_F32):
        _need(out.dtype == torch.float32 and tuple(out.shape) == (m, n), "gemv: out float32 [m, n]")
    elif epilogue == EPI_GATED:
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n // 2),
              "gemv: out bfloat16 [m, n / 2]")
    elif epilogue == EPI_QKV:
        _need(n == (heads + 2 * kv_heads) * head_dim and head_dim % 16 == 0, "gemv: qkv rows")
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, heads * head_dim),
              "gemv: q out bfloat16 [m, heads * d]")
        _need(token_pos is not None and token_pos.dtype == torch.int32 and token_pos.numel() >= m,
              "gemv: token_pos int32 [m]")
        if kv_heads > 0:
            _need(k_cache is not None and k_cache.dtype == torch.bfloat16
                  and tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim)
                  and page_table is not None and token_seq is not None, "gemv: cache [pages, kv, page, d]")
        if cos is not None:
            _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "gemv: cos/sin tables")
    elif epilogue == EPI_ARGMAX:
        _need(out.dtype == torch.int32 and out.numel() >= m, "gemv: picks int32 [m]")
        _need(scratch is not None and scratch.dtype == torch.int32
              and scratch.numel() >= argmax_scratch_ints(m, n, k, w.device), "gemv: argmax scratch")
        if logits is not None:
            _need(logits.dtype == torch.float32 and tuple(logits.shape) == (m, n), "gemv: logits [m, n]")
        if next_tokens is not None:
            _need(next_pos is not None and next_tokens.dtype == next_pos.dtype == torch.int32
                  and next_tokens.numel() >= m and next_pos.numel() >= m, "gemv: decode state int32")
    else:
        raise KernelError(f"gemv: unknown epilogue {epilogue}")
    cols = page_table.shape[1] if page_table is not None else 0
    best_val = best_idx = ticket = 0
    if epilogue == EPI_ARGMAX:
        grid = gemv_grid(m, n, k, w.device)
        base = scratch.data_ptr()
        ticket, best_val, best_idx = base, base + 16, base + 16 + 4 * m * grid
    _check(_lib().nnis_gemv_bf16(
        _ptr(x), _ptr(hidden), _ptr(rows), _ptr(norm_weight), ctypes.c_float(eps), _ptr(w), _ptr(bias), _ptr(out), m, n, k, epilogue, _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), cols, _ptr(cos), _ptr(sin), _ptr(k_cache), _ptr(v_cache), heads, kv_heads,
        head_dim, page_size, _ptr(logits), ctypes.c_void_p(best_val), ctypes.c_void_p(best_idx),
        ctypes.c_void_p(ticket), _ptr(next_tokens), _ptr(next_pos), _ptr(emit_x), _ptr(emit_w),
        _ptr(emit_ss), _ptr(shares), _ptr(status_word(w.device)),
        sm_count(w.device),
        PDL | (2 if release_early and PDL and EARLY_RELEASE else 0) | (0 if rows_kernel else 4), _stream()),
        "gemv_bf16",
        gemv_slices(m, n, k, w.device, rows_kernel) if epilogue == EPI_ADD_F32 and hidden is None else 1)


def argmax_scratch_ints(m: int, n: int, k: int, device) -> int:
    """int32 words of scratch for EPI_ARGMAX: a ticket, then per-CTA bests.  The
    buffer must be zero before its first use (the kernel re-zeroes the ticket)."""
    return 4 + 2 * m * gemv_grid(m, n, k, device)


def attention_decode(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                     out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                     scale: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                     merge: bool = True) -> None:
    """One query token per sequence over the paged bfloat16 cache.  With
    ``merge=False`` and several splits, ``partial`` is left for the consumer."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim % 16 == 0 and 16 <= head_dim <= 256,
          f"attention: head_dim {head_dim} is not a multiple of 16 in 16..256")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention_decode: out [n <= 65535, heads * d]")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
    _check(_lib().nnis_attention_decode(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), n, heads, kv_heads, head_dim,
        page_size, window, ctypes.c_float(scale), n_splits, 1 if merge else 0,
        _ptr(status_word(out.device)), PDL, _stream()),
        "attention_decode", 2 if n_splits > 1 and merge else 1)


def attention_decode_takes(head_dim: int) -> bool:
    """Head sizes of the CUDA-core decode kernel (whole 32-byte pieces of a row per lane)."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


# Whether the decode attention kernel for few sequences asks the same pages of the layer that
# runs next into L2 when it is through with its own (batch 8 of the 135M shape: +2 %).
KV_PREFETCH = os.environ.get("NNIS_KV_PREFETCH", "1") == "1"
PREFILL_SHORT_CHUNKS = os.environ.get("NNIS_PREFILL_SHORT_CHUNKS", "1") == "1"
TMA_SLICE_PAGES = int(os.environ.get("NNIS_TMA_SLICE_PAGES", "0"))  # 0: chosen by the plan
TMA_ATTENTION = 0 if os.environ.get("NNIS_TMA_ATTENTION", "1") == "0" else 1
_tma_ctas_per_sm: dict = {}


def attention_decode_tma_max_pages(head_dim: int) -> int:
    """Pages of one slice that attention_decode_tma holds (all at once, in shared memory)."""
    return int(_lib().nnis_attention_decode_tma_max_pages(int(head_dim)))


def tma_slices(groups: int, table_cols: int, sms: int, most_pages: int, fit, fixed_pages: int = 0) -> int:
    """The rule behind ``attention_decode_tma_plan``, free of the device: ``groups`` CTAs per
    slice (sequences x kv heads x tiles of query heads), ``table_cols`` pages to cut, ``sms``
    SMs, at most ``most_pages`` pages a slice, and ``fit(pages)`` the CTAs of that many pages
    that one SM holds at once.  Returns the number of slices, 0: not for this kernel."""
    def plan(pages: int):
        splits = min(128, -(-table_cols // pages))
        per = -(-table_cols // splits)
        if per > most_pages:
            return 0, 0, 0
        return splits, groups * splits, fit(per)

    if fixed_pages:
        splits, ctas, room = plan(fixed_pages)
        return splits if 0 < ctas <= room * sms else 0
    splits, ctas, room = plan(4)
    if splits > 16:
        # The slice that arrives last asks for 16 partial records a trip to L2: beyond 16 slices
        # (contexts beyond 4,096) the longest slices whose CTAs are still all resident, eight pages
        # one to an SM or six pages two to an SM (one sequence at context 16,384: 0.592 -> 0.512 ms
        # a step, two at 8,192: 0.540 -> 0.493)
        for pages in (8, 6):
            long_splits, long_ctas, long_room = plan(pages)
            if 0 < long_ctas <= min(long_room, 2) * sms:
                return long_splits
    if ctas > 2 * sms:
        wide, wide_ctas, wide_room = plan(6)
        if 0 < wide_ctas <= min(wide_room, 2) * sms:
            return wide
    return splits if 0 < ctas <= room * sms else 0


def attention_decode_tma_plan(n: int, heads: int, kv_heads: int, head_dim: int, page_size: int,
                              table_cols: int, device, share: int = 1) -> int:
    """Into how many slices attention_decode_tma cuts ``table_cols`` pages for a step of ``n``
    sequences, or 0 when the step is not for that kernel: it takes head sizes 64 and 128 and
    only steps whose CTAs are all resident together (few sequences, or short contexts);
    other steps stream their slices through the ring of attention_decode_mma.  Slices are of
    four pages (more for page tables beyond 128 x 4 columns, up to what fits; with more than 16
    slices of four pages, of eight or six pages where those CTAs are resident); when four pages make
    more CTAs than two per SM, of six pages if those CTAs are resident two to an SM: fewer
    partial records and fewer CTAs that wait for room beside the projection's (batch 8 of the
    135M shape: 0.637 -> 0.618 ms a step; at batch 1, where CTAs are few, four pages are
    4 % ahead).  ``share``: steps that run side by side on the device.
    ``NNIS_TMA_SLICE_PAGES`` fixes the pages of a slice."""
    if not TMA_ATTENTION or head_dim not in (64, 128) or page_size != 64 or n > 65535:
        return 0
    groups = n * kv_heads * (-(-(heads // kv_heads) // 16))
    sms = sm_count(device) // max(1, share)

    def fit(pages: int) -> int:
        key = (head_dim, pages, torch.device(device).index or 0)
        if key not in _tma_ctas_per_sm:
            _tma_ctas_per_sm[key] = int(_lib().nnis_attention_decode_tma_ctas_per_sm(head_dim, pages))
        return _tma_ctas_per_sm[key]

    return tma_slices(groups, table_cols, sms, attention_decode_tma_max_pages(head_dim), fit, TMA_SLICE_PAGES)


def attention_decode_tma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float, n_splits: int, partial: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None, ahead: int = 0) -> None:
    """Decode attention with every page of a slice in shared memory at once (``n_splits``
    from ``attention_decode_tma_plan``): pages by TMA, a warp per page.  Scratch as for
    ``attention_decode_mma``.  ``ahead``: elements from these caches to the ones read next
    (the next layer's), whose same pages the kernel asks into L2; 0: none."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial, tickets)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode_tma: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(head_dim in (64, 128) and page_size == 64, "attention_decode_tma: head size 64 or 128, pages of 64")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention: out [n <= 65535, heads * d]")
    most = attention_decode_tma_max_pages(head_dim)
    _need(1 <= n_splits <= 128 and -(-page_table.shape[1] // n_splits) <= most,
          f"attention_decode_tma: at most 128 slices of at most {most} pages")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
        _need(tickets is not None and tickets.dtype == torch.int32
              and tickets.numel() >= mma_ticket_count(n, heads, kv_heads), "attention: tickets")
    _check(_lib().nnis_attention_decode_tma(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), ctypes.c_longlong(pages * nkv * page_size),
        _ptr(token_pos), _ptr(token_seq), _ptr(page_table), page_table.shape[1], _ptr(out),
        _ptr(partial), _ptr(tickets), n, heads, kv_heads, head_dim, page_size, window,
        ctypes.c_float(scale), n_splits, ctypes.c_longlong(ahead), _ptr(status_word(out.device)), PDL,
        _stream()),
        "attention_decode_tma")


def attention_decode_mma_takes(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and page_size == 64


_decode_mma_resident: dict = {}
# 1: the decode attention may run with one stage less where the wave model favours it
DECODE_STAGE_CHOICE = int(os.environ.get("NNIS_DECODE_STAGE_CHOICE", "1")) \
    and os.environ.get("NNIS_DECODE_FILL") is None


def attention_decode_mma_stages(head_dim: int) -> int:
    """Pages of K and V that a CTA of the tensor-core decode kernel keeps in flight by default."""
    return int(_lib().nnis_attention_decode_mma_stages(int(head_dim)))


def attention_decode_mma_resident(head_dim: int, device, stages: int = 0) -> int:
    """How many CTAs of the tensor-core decode kernel the device holds at once
    (``stages`` pages in flight per CTA; 0: the default)."""
    key = (head_dim, torch.device(device).index or 0, stages)
    if key not in _decode_mma_resident:
        per_sm = int(_lib().nnis_attention_decode_mma_ctas_per_sm(int(head_dim), int(stages)))
        if per_sm <= 0:
            raise RuntimeError(f"decode attention kernel for head size {head_dim}: occupancy query failed")
        _decode_mma_resident[key] = per_sm * sm_count(device)
    return _decode_mma_resident[key]


def attention_decode_mma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         token_pos: torch.Tensor, token_seq: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float, n_splits: int = 1, partial: Optional[torch.Tensor] = None,
                         tickets: Optional[torch.Tensor] = None, stages: int = 0) -> None:
    """Decode attention on the tensor cores (head sizes 64 and 128).  With several
    splits the slice that finishes last merges them: ``out`` is always complete.
    ``tickets``: int32 zeros, ``mma_ticket_count`` of them, left zero.  ``stages``:
    pages in flight per CTA (0: the default; fewer let more CTAs share an SM)."""
    _cuda(k_cache, v_cache, token_pos, token_seq, page_table, out, partial, tickets)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_decode_mma: bfloat16 tensors")
    n = out.shape[0]
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_decode_mma_takes(head_dim, page_size),
          f"attention_decode_mma: head_dim {head_dim} / page {page_size} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and n <= 65535, "attention: out [n <= 65535, heads * d]")
    if n_splits > 1:
        _need(partial is not None and partial.dtype == torch.float32
              and partial.numel() >= n * heads * n_splits * (head_dim + 2),
              "attention: partial scratch too small")
        _need(tickets is not None and tickets.dtype == torch.int32
              and tickets.numel() >= mma_ticket_count(n, heads, kv_heads), "attention: tickets")
    _check(_lib().nnis_attention_decode_mma_staged(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(token_pos), _ptr(token_seq),
        _ptr(page_table), page_table.shape[1], _ptr(out), _ptr(partial), _ptr(tickets), n, heads,
        kv_heads, head_dim, page_size, window, ctypes.c_float(scale), n_splits, int(stages), PDL,
        _stream()), "attention_decode_mma")


def attention_prefill_mma(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                          tiles: torch.Tensor, seq_first_row: torch.Tensor, seq_start: torch.Tensor,
                          seq_count: torch.Tensor, page_table: torch.Tensor, out: torch.Tensor,
                          heads: int, kv_heads: int, head_dim: int, window: int, scale: float) -> None:
    """Prompt attention on the tensor cores (head sizes 64 and 128): packed query
    tokens, 64 per tile, each over its own sequence's keys in the paged cache."""
    _cuda(k_cache, v_cache, tiles, seq_first_row, seq_start, seq_count, page_table, out)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_prefill_mma: bfloat16 tensors")
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_decode_mma_takes(head_dim, page_size),
          f"attention_prefill_mma: head_dim {head_dim} / page {page_size} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim, "attention: out [n, heads * d]")
    for t in (tiles, seq_first_row, seq_start, seq_count):
        _need(t.dtype == torch.int32, "attention_prefill_mma: int32 tables")
    _need(tiles.dim() == 2 and tiles.shape[1] == 2 and tiles.shape[0] > 0, "tiles: int32 [n_tiles, 2]")
    _check(_lib().nnis_attention_prefill_mma(
        _ptr(q), q_stride, _ptr(k_cache), _ptr(v_cache), _ptr(tiles), tiles.shape[0],
        _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table), page_table.shape[1],
        _ptr(out), heads, kv_heads, head_dim, page_size, window, ctypes.c_float(scale), _stream()),
        "attention_prefill_mma")


WIDE_QUERY_TILE = 128  # queries per CTA of attention_prefill_tc
TC_ATTENTION = 0 if os.environ.get("NNIS_TC_ATTENTION", "1") == "0" else 1


def attention_prefill_tc_takes(head_dim: int, page_size: int, q_stride: int) -> bool:
    """Whether the tcgen05 prompt attention kernel runs these sizes."""
    return bool(TC_ATTENTION) and head_dim == 64 and page_size == 64 and q_stride % 8 == 0


def prefill_tc_plan(counts, starts, window: int, heads: int, sms: int):
    """Work list of attention_prefill_tc for a step whose sequences bring
    ``counts`` tokens after ``starts`` cached ones.

    A tile is 128 queries of one sequence; its keys are the pages from its first
    query's window start to its last query.  Two CTAs share an SM, so tiles are cut
    into chunks of pages while there would be fewer CTAs (units x heads) than 1.7
    per SM: the longest chunk of 32, 24, 16 or 12 pages that gives as many, else 8
    (a chunk costs a CTA's start and end, a trip of its rows through scratch and,
    for the last one of a tile, the merge; measured on one prompt of 1,024 / 2,048 /
    4,096 tokens and 9 heads the best lengths were 8 / 12 / none); then the shortest
    chunks from 8 pages on with which the CTAs still fit one wave of two to an SM (2,048
    tokens: 11 pages, 288 CTAs; a CTA walks its pages one after another).  Returns ``units`` int32 [n, 4] (sequence,
    first query, chunk | chunks << 16, first scratch slot), longest first, and the
    number of scratch slots.  ``prefill_tc_pays`` says whether the step is worth this
    kernel at all."""
    import numpy as np
    tiles = []
    for i, (c, st) in enumerate(zip(counts, starts)):
        for q0 in range(0, int(c), WIDE_QUERY_TILE):
            rows = min(WIDE_QUERY_TILE, int(c) - q0)
            pos0 = int(st) + q0
            lo = max(0, pos0 - window + 1) if window > 0 else 0
            tiles.append((i, q0, (pos0 + rows - 1) // 64 - lo // 64 + 1))
    chunk_pages = 8
    for cand in (1 << 30, 32, 24, 16, 12):
        if 10 * sum(-(-p // cand) for _, _, p in tiles) * heads >= 17 * sms:
            chunk_pages = cand
            break
    if PREFILL_SHORT_CHUNKS and chunk_pages > 8 and chunk_pages < (1 << 30):
        # A CTA walks its pages one after another (1.3 us a page): where the CTAs still fit
        # one wave of two to an SM with shorter chunks, the shortest such chunks end first.
        for cand in range(8, chunk_pages):
            if sum(-(-p // cand) for _, _, p in tiles) * heads <= 2 * sms:
                chunk_pages = cand
                break
    units, slot = [], 0
    for i, q0, pages in tiles:
        n = -(-pages // chunk_pages)
        while n > 1 and (n - 1) * (-(-pages // n)) >= pages:  # no chunk may be empty
            n -= 1
        per = -(-pages // n)
        for c in range(n):
            units.append((min(per, pages - c * per), i, q0, c | (n << 16), slot if n > 1 else 0))
        if n > 1:
            slot += n
    units.sort(key=lambda u: -u[0])
    return np.asarray([u[1:] for u in units], dtype=np.int32).reshape(-1, 4), slot


def prefill_tc_pays(counts, starts, window: int) -> bool:
    """Whether a step's tiles are long enough for attention_prefill_tc: with fewer
    than two and a half pages of keys per 128-query tile on average (many short
    prompts) the 64-query tiles of the mma.sync kernel waste less and run as fast
    or faster (8 x 128 tokens: 5.4 against 6.2 us; 8 x 256: 9.8 against 7.7 us)."""
    tiles = pages = 0
    for c, st in zip(counts, starts):
        for q0 in range(0, int(c), WIDE_QUERY_TILE):
            rows = min(WIDE_QUERY_TILE, int(c) - q0)
            pos0 = int(st) + q0
            lo = max(0, pos0 - window + 1) if window > 0 else 0
            tiles += 1
            pages += (pos0 + rows - 1) // 64 - lo // 64 + 1
    return tiles > 0 and 2 * pages >= 5 * tiles


PREFILL_TC_PARTIAL = 66 * WIDE_QUERY_TILE  # float32 per (scratch slot, head)


def attention_prefill_tc(q: torch.Tensor, q_stride: int, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         units: torch.Tensor, partial: Optional[torch.Tensor],
                         tickets: Optional[torch.Tensor], seq_first_row: torch.Tensor,
                         seq_start: torch.Tensor, seq_count: torch.Tensor, page_table: torch.Tensor,
                         out: torch.Tensor, heads: int, kv_heads: int, head_dim: int, window: int,
                         scale: float) -> None:
    """Prompt attention on tcgen05 (head size 64): packed query tokens, each over
    its own sequence's keys in the paged cache.  ``units`` comes from
    ``prefill_tc_plan``; when it cuts tiles, ``partial`` is float32 scratch of
    slots x heads x PREFILL_TC_PARTIAL values and ``tickets`` int32 [slots x heads],
    zero before the first launch (the kernel leaves them zero)."""
    _cuda(k_cache, v_cache, units, seq_first_row, seq_start, seq_count, page_table, out)
    _need(q.is_cuda and q.dtype == torch.bfloat16 == k_cache.dtype == out.dtype,
          "attention_prefill_tc: bfloat16 tensors")
    pages, nkv, page_size, d = k_cache.shape
    _need(nkv == kv_heads and d == head_dim, "cache shape differs from the heads given")
    _need(attention_prefill_tc_takes(head_dim, page_size, q_stride),
          f"attention_prefill_tc: head_dim {head_dim} / page {page_size} / stride {q_stride} is not taken")
    _need(heads % kv_heads == 0, "attention: heads is not a multiple of kv_heads")
    _need(pages * nkv * page_size < 2 ** 31, "attention: the cache has too many rows")
    _need(out.shape[1] == heads * head_dim and out.is_contiguous(), "attention: out [n, heads * d]")
    _need(k_cache.is_contiguous() and v_cache.is_contiguous(), "attention: contiguous cache")
    for t in (units, seq_first_row, seq_start, seq_count):
        _need(t.dtype == torch.int32, "attention_prefill_tc: int32 tables")
    _need(units.dim() == 2 and units.shape[1] == 4 and units.shape[0] > 0 and units.is_contiguous(),
          "units: int32 [n_units, 4]")
    if partial is not None:
        _cuda(partial, tickets)
        _need(partial.dtype == torch.float32 and tickets.dtype == torch.int32,
              "partial: float32 scratch, tickets: int32")
    _check(_lib().nnis_attention_prefill_tc(
        _ptr(q), q_stride, out.shape[0], _ptr(k_cache), _ptr(v_cache),
        ctypes.c_longlong(pages * nkv * page_size), _ptr(units), units.shape[0],
        _ptr(partial) if partial is not None else None, _ptr(tickets) if partial is not None else None,
        _ptr(seq_first_row), _ptr(seq_start), _ptr(seq_count), _ptr(page_table), page_table.shape[1],
        _ptr(out), heads, kv_heads, head_dim, page_size, window, ctypes.c_float(scale),
        _ptr(status_word(out.device)), PDL, _stream()),
        "attention_prefill_tc")


def mma_ticket_count(n: int, heads: int, kv_heads: int) -> int:
    return n * kv_heads * (-(-(heads // kv_heads) // 16))


TC_GEMM = 0 if os.environ.get("NNIS_TC_GEMM", "1") == "0" else 1


def gemm_tc_takes(m: int, n: int, k: int) -> bool:
    """Whether the tcgen05 kernel runs this bfloat16 product (else CUDA cores):
    K a multiple of 8 (rows of 16 bytes for TMA) and enough rows to fill a tile."""
    return bool(TC_GEMM) and m > 16 and k % 8 == 0 and -(-m // 128) <= 65535


GEMM_GATED, GEMM_QKV = 3, 4


def gemm_tc(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
            mode: int, token_pos: Optional[torch.Tensor] = None,
            token_seq: Optional[torch.Tensor] = None, page_table: Optional[torch.Tensor] = None,
            cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
            k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None,
            heads: int = 0, kv_heads: int = 0, head_dim: int = 0, page_size: int = 0,
            split_scratch: Optional[torch.Tensor] = None,
            split_tickets: Optional[torch.Tensor] = None) -> None:
    """out (op)= a . w^T + bias on the tensor cores (tcgen05, float32 accumulation
    in tensor memory); bfloat16 operands.  Modes: STORE, STORE_F32, ADD_F32,
    GEMM_GATED (w = [gate; up] rows, out bfloat16 [m, n / 2] = silu(gate) * up) and
    GEMM_QKV (bias, RoPE at each row's position, q to out [m, heads * d], k and v
    into the paged cache; head_dim 64 or 128).  ADD_F32 with ``split_scratch`` (float32)
    and ``split_tickets`` (int32, zero; left zero) of the sizes ``gemm_tc_splits`` names
    may cut K among several CTAs per tile; their sums are added in a fixed order."""
    _cuda(a, w, bias, out, token_pos, token_seq, page_table, cos, sin, k_cache, v_cache)
    m, k = a.shape
    n = w.shape[0]
    _need(a.dtype == w.dtype == torch.bfloat16 and w.shape[1] == k, "gemm_tc: bfloat16 a [m, k], w [n, k]")
    _need(gemm_tc_takes(m, n, k), f"gemm_tc: shape m={m} n={n} k={k} is not taken")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm_tc: bias float32 [n]")
    if mode == GEMM_GATED:
        _need(n % 2 == 0 and out.dtype == torch.bfloat16 and tuple(out.shape) == (m, n // 2),
              "gemm_tc: gated out bfloat16 [m, n / 2]")
    elif mode == GEMM_QKV:
        _need(gemm_tc_qkv_takes(head_dim) and n == (heads + 2 * kv_heads) * head_dim,
              "gemm_tc: qkv rows / head_dim not taken")
        _need(out.dtype == torch.bfloat16 and tuple(out.shape) == (m, heads * head_dim),
              "gemm_tc: q out bfloat16 [m, heads * d]")
        _need(token_pos is not None and token_pos.dtype == torch.int32 and token_pos.numel() >= m,
              "gemm_tc: token_pos int32 [m]")
        if kv_heads > 0:
            _need(k_cache is not None and k_cache.dtype == torch.bfloat16
                  and tuple(k_cache.shape[1:]) == (kv_heads, page_size, head_dim)
                  and page_table is not None and token_seq is not None, "gemm_tc: cache [pages, kv, page, d]")
        if cos is not None:
            _need(cos.dtype == torch.float32 and cos.shape[1] == head_dim // 2, "gemm_tc: cos/sin tables")
    else:
        _need(tuple(out.shape) == (m, n), "gemm_tc: out [m, n]")
        _need(out.dtype == (torch.bfloat16 if mode == STORE else torch.float32), "gemm_tc: out dtype vs mode")
    cols = page_table.shape[1] if page_table is not None else 0
    scratch, tickets = (split_scratch, split_tickets) if mode == ADD_F32 else (None, None)
    _cuda(scratch, tickets)
    _check(_lib().nnis_gemm_tc(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), m, n, k, mode, _ptr(token_pos),
                               _ptr(token_seq), _ptr(page_table), cols, _ptr(cos), _ptr(sin),
                               _ptr(k_cache), _ptr(v_cache), heads, kv_heads, head_dim, page_size,
                               _ptr(scratch), ctypes.c_longlong(scratch.numel() if scratch is not None else 0),
                               _ptr(tickets), tickets.numel() if tickets is not None else 0,
                               sm_count(a.device), _ptr(status_word(a.device)), PDL, _stream()),
           "gemm_tc")


# Whether the adding product may cut a long K among CTAs (few tiles): parts/linear.py asks.
GEMM_SPLIT_K = os.environ.get("NNIS_GEMM_SPLIT_K", "1") == "1"


def gemm_tc_splits(m: int, n: int, k: int, device=None):
    """(CTAs that share a tile of the adding product, float32 of scratch, tickets)."""
    floats, tiles = ctypes.c_longlong(0), ctypes.c_int(0)
    sms = sm_count(device) if device is not None else 148
    splits = int(_lib().nnis_gemm_tc_splits(m, n, k, sms, ctypes.byref(floats), ctypes.byref(tiles)))
    return splits, int(floats.value), int(tiles.value)


def gemm_tc_qkv_takes(head_dim: int) -> bool:
    return head_dim in (64, 128)


def advance(tokens: torch.Tensor, pos: torch.Tensor, picked: torch.Tensor) -> None:
    """tokens = picked; pos += 1, on live rows (pos >= 0) only."""
    _cuda(tokens, pos, picked)
    _need(tokens.dtype == pos.dtype == picked.dtype == torch.int32, "advance: int32")
    n = tokens.numel()
    _need(pos.numel() == n and picked.numel() >= n, "advance: sizes differ")
    _check(_lib().nnis_advance(_ptr(tokens), _ptr(pos), _ptr(picked), n, _stream()), "advance")


# ---------------------------------------------------------------------------
# The timeline of a step (trace.cu), for measurements.
_trace_buffer: Optional[torch.Tensor] = None


def trace_begin(capacity: int = 2048, device="cuda:0") -> torch.Tensor:
    """From now on every launch of an instrumented kernel (decode projections, decode
    attention) takes a slot of the returned buffer, int64 [capacity, 8]: first CTA's
    begin, last CTA's end, first and last CTA past the wait for the kernel before, and
    first and last CTA at two marks inside the kernel, in nanoseconds of the GPU's timer.  A graph captured meanwhile keeps its slots."""
    global _trace_buffer
    _trace_buffer = torch.zeros((capacity, 8), dtype=torch.int64, device=device)
    trace_clear()
    _lib().nnis_trace_set(_ptr(_trace_buffer), capacity)
    return _trace_buffer


def trace_clear() -> None:
    """Before the replay that is to be read: earliest words to the largest value, latest to zero."""
    _trace_buffer[:, 0::2] = torch.iinfo(torch.int64).max
    _trace_buffer[:, 1::2] = 0


def trace_end():
    """Stops handing out slots; returns the names of the launches that took one."""
    lib = _lib()
    lib.nnis_trace_name.restype = ctypes.c_char_p
    names = [lib.nnis_trace_name(i).decode() for i in range(int(lib.nnis_trace_count()))]
    lib.nnis_trace_set(None, 0)
    return names
