"""The entry point for callers that cannot allocate device memory
(nnis_b200/csrc/no_alloc.h), called through its exported C symbol and compared
with the ordinary entry point.  Collected last on purpose: it comes after every
other test in a run that stops at the first failure, and it passes alone in a
fresh process as well (it sets up nothing but its own inputs).

Who needs it: a program that gave all device memory to its own arena, code in
a latency-critical loop where cudaMalloc's implicit synchronisation is not
acceptable, or a plain-C / foreign-function caller with no allocator at hand.
Such a caller passes inputs and outputs only; the scratch of the split-KV merge
is a fixed array inside the library."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NNIS_ERR_NOALLOC_TOO_LARGE = -5


def _case(seed, nq, nkv, d, lengths):
    """A paged cache with shuffled pages and one query token per sequence."""
    g = torch.Generator().manual_seed(seed)
    page = 64
    n_pages = sum(-(-L // page) for L in lengths) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    cols = max(-(-L // page) for L in lengths)
    table = torch.full((len(lengths), cols), -1, dtype=torch.int32)
    for s, L in enumerate(lengths):
        for j in range(-(-L // page)):
            table[s, j] = order.pop()
    kc = torch.randn(n_pages, nkv, page, d, generator=g).bfloat16()
    vc = torch.randn(n_pages, nkv, page, d, generator=g).bfloat16()
    q = torch.randn(len(lengths), nq * d, generator=g).bfloat16()
    pos = torch.tensor([L - 1 for L in lengths], dtype=torch.int32)
    seq = torch.arange(len(lengths), dtype=torch.int32)
    return [t.to(DEV) for t in (q, kc, vc, pos, seq, table)]


def _call_noalloc(lib, q, kc, vc, pos, seq, table, out, nq, nkv, d, window, splits):
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.nnis_attention_decode_noalloc(
        ptr(q), nq * d, ptr(kc), ptr(vc), ptr(pos), ptr(seq), ptr(table), table.shape[1], ptr(out),
        out.shape[0], nq, nkv, d, 64, window, ctypes.c_float(1.0 / math.sqrt(d)), splits,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from nnis_b200.csrc import build, ops
    lib = build.load()
    for call, (seed, nq, nkv, d, lengths, window, splits) in enumerate([
            (1, 9, 3, 64, [700, 1, 130, 64], 0, 8),
            (2, 4, 2, 128, [33, 900], 200, 5)]):
        q, kc, vc, pos, seq, table = _case(seed, nq, nkv, d, lengths)
        n = len(lengths)
        want = torch.empty(n, nq * d, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(n * nq * splits * (d + 2), device=DEV)
        tickets = torch.zeros(ops.mma_ticket_count(n, nq, nkv), dtype=torch.int32, device=DEV)
        ops.attention_decode_mma(q, nq * d, kc, vc, pos, seq, table, want, nq, nkv, d, window,
                                 1.0 / math.sqrt(d), splits, partial, tickets)
        got = torch.full_like(want, 3.0)
        before = torch.cuda.memory_allocated()
        rc = _call_noalloc(lib, q, kc, vc, pos, seq, table, got, nq, nkv, d, window, splits)
        assert rc == 0, f"call {call}: return code {rc}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        diff = (got.float() - want.float()).abs().max().item()
        assert torch.isclose(got.float(), want.float(), rtol=1.6e-2, atol=1e-2).all(), \
            f"call {call}: max abs diff {diff}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from nnis_b200.csrc import build
    lib = build.load()
    q, kc, vc, pos, seq, table = _case(3, 32, 32, 128, [65] * 40)
    out = torch.empty(40, 32 * 128, dtype=torch.bfloat16, device=DEV)
    # 40 * 32 * 64 * 130 floats is far beyond the fixed scratch
    assert _call_noalloc(lib, q, kc, vc, pos, seq, table, out, 32, 32, 128, 0, 64) == \
        NNIS_ERR_NOALLOC_TOO_LARGE
    torch.cuda.synchronize()
