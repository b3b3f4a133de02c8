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


def _plain(q, kc, vc, table, lengths, nq, nkv, d, window):
    """The plain implementation's attention (tests/plain_llama.py) for the one query of
    each sequence: its keys and values gathered from the pages in order."""
    import plain_llama as P
    rows = []
    for s, L in enumerate(lengths):
        pages = table[s, :-(-L // 64)].tolist()
        k = torch.cat([kc[p] for p in pages], dim=1)[:, :L].transpose(0, 1).float().cpu()   # [L, nkv, d]
        v = torch.cat([vc[p] for p in pages], dim=1)[:, :L].transpose(0, 1).float().cpu()
        qs = torch.zeros(L, nq, d)
        qs[L - 1] = q[s].float().cpu().view(nq, d)
        rows.append(P.causal_attention(qs, k, v, window)[L - 1].reshape(nq * d))
    return torch.stack(rows)


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
        # ... and both against the plain implementation, which shares no code with them
        plain = _plain(q, kc, vc, table, lengths, nq, nkv, d, window)
        for name, t in (("no-alloc", got), ("ordinary", want)):
            assert torch.isclose(t.float().cpu().double(), plain, rtol=1.6e-2, atol=1e-2).all(), \
                f"call {call}: {name} entry point against the plain attention: max abs diff " \
                f"{(t.float().cpu().double() - plain).abs().max().item()}"


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from nnis_b200.csrc import build
    lib = build.load()
    q, kc, vc, pos, seq, table = _case(3, 32, 32, 128, [65] * 40)
    out = torch.empty(40, 32 * 128, dtype=torch.bfloat16, device=DEV)
    # 40 * 32 * 64 * 130 floats is far beyond the fixed scratch
    assert _call_noalloc(lib, q, kc, vc, pos, seq, table, out, 32, 32, 128, 0, 64) == \
        NNIS_ERR_NOALLOC_TOO_LARGE
    torch.cuda.synchronize()
    # sizes the kernel does not take are refused before anything is put on the stream
    assert _call_noalloc(lib, q, kc, vc, pos, seq, table, out, 32, 32, 96, 0, 2) == -2
    assert _call_noalloc(lib, q, kc, vc, pos, seq, table, out, 32, 32, 128, 0, 65) == -2


def test_no_alloc_entry_point_takes_exactly_what_fits():
    """The largest calls that the fixed array holds run and are right at their last
    rows, whose records and tickets lie at the array's end; the next larger ones are
    refused.  Records: a record is head_dim + 2 floats (66 or 130), so no call comes to
    2^20 floats exactly; 126 tokens x 8 heads x 8 slices x 130 = 1,048,320 is the
    largest of its shape and 127 tokens do not fit.  Tickets: 512 tokens x 8 kv heads
    are 4,096 exactly; 513 tokens are refused."""
    from nnis_b200.csrc import build, ops
    lib = build.load()
    for nq, nkv, d, splits, n, fits in ((8, 8, 128, 8, 126, True), (8, 8, 128, 8, 127, False),
                                        (8, 8, 64, 2, 512, True), (8, 8, 64, 2, 513, False)):
        lengths = [130 + (i % 5) for i in range(n)]
        q, kc, vc, pos, seq, table = _case(11, nq, nkv, d, lengths)
        got = torch.zeros(n, nq * d, dtype=torch.bfloat16, device=DEV)
        floats, tickets_needed = n * nq * splits * (d + 2), ops.mma_ticket_count(n, nq, nkv)
        assert (floats <= 1 << 20 and tickets_needed <= 4096) == fits
        rc = _call_noalloc(lib, q, kc, vc, pos, seq, table, got, nq, nkv, d, 0, splits)
        torch.cuda.synchronize()
        if not fits:
            assert rc == NNIS_ERR_NOALLOC_TOO_LARGE
            continue
        assert rc == 0
        want = torch.empty_like(got)
        partial = torch.empty(floats, device=DEV)
        tickets = torch.zeros(tickets_needed, dtype=torch.int32, device=DEV)
        ops.attention_decode_mma(q, nq * d, kc, vc, pos, seq, table, want, nq, nkv, d, 0,
                                 1.0 / math.sqrt(d), splits, partial, tickets)
        assert torch.isclose(got.float(), want.float(), rtol=1.6e-2, atol=1e-2).all()
        last = [n - 1]
        plain = _plain(q[last], kc, vc, table[last], [lengths[-1]], nq, nkv, d, 0)
        assert torch.isclose(got[last].float().cpu().double(), plain, rtol=1.6e-2, atol=1e-2).all()
