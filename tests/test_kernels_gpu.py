"""Each CUDA kernel alone against a plain float64 reference, at sizes other
than the engine's: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd numbers of heads and groups, windows, split key ranges."""
import math
import random

import numpy as np
import pytest
import torch

import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == "float32" else dict(rtol=1.6e-2, atol=1e-2)


def close(got, want, dtype, what=""):
    got, want = got.double().cpu(), want.double().cpu()
    t = tol(dtype)
    ok = torch.isclose(got, want, **t)
    assert ok.all(), (f"{what}: {int((~ok).sum())} of {ok.numel()} differ, max abs "
                      f"{float((got - want).abs().max()):.3e}")


def ops():
    from nnis_b200.csrc import ops as o
    return o


def away_from_bf16_ties(hidden, norm_weight, eps):
    """`hidden` with the few values moved whose normed value lies within 3e-6 (relative)
    of a bfloat16 rounding boundary: there the kernel's float32 norm and the float64
    reference may round to different bfloat16 values, and one such value shifts a whole
    row of products by more than the float32 bound.  With thousands of values per row
    some lie that close; the kernels are compared on inputs where rounding is decided."""
    hidden = hidden.clone()
    for _ in range(50):
        x = P.rms_norm(hidden, norm_weight, eps)
        risky = (x * (1 + 3e-6)).bfloat16() != (x * (1 - 3e-6)).bfloat16()
        if not bool(risky.any()):
            return hidden
        hidden[risky] *= 1.003
    raise AssertionError("could not move the values away from rounding boundaries")


@pytest.mark.parametrize("dtype", list(DT))
def test_embed_and_bad_ids(dtype):
    o = ops()
    table = torch.randn(301, 70).to(DT[dtype])
    tokens = torch.tensor([0, 300, 5, 17, 17], dtype=torch.int32)
    hidden = torch.empty(5, 70, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.embed(table.to(DEV), tokens.to(DEV), hidden, status)
    assert torch.equal(hidden.cpu(), P.embed(table, tokens.tolist()).float())
    assert int(status.item()) == 0
    o.embed(table.to(DEV), torch.tensor([3, 301, -1, 4, 2], dtype=torch.int32, device=DEV), hidden,
            status)
    assert int(status.item()) == 1
    assert float(hidden[1].abs().sum()) == 0 and float(hidden[2].abs().sum()) == 0
    assert torch.equal(hidden[0].cpu(), table[3].float())


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("width", [16, 100, 576, 2050])
def test_rmsnorm(dtype, width):
    o = ops()
    x = torch.randn(9, width) * 3
    w = 1 + 0.1 * torch.randn(width)
    out = torch.empty(9, width, dtype=DT[dtype], device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out)
    close(out, P.rms_norm(x, w, 1e-5), dtype, "rmsnorm")
    rows = torch.tensor([8, 0, 3], dtype=torch.int32)
    out2 = torch.empty(3, width, dtype=DT[dtype], device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, out2, rows.to(DEV))
    assert torch.equal(out2, out[rows.long().to(DEV)])


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("width", [72, 576, 1000, 1024, 1028, 578])
def test_rmsnorm_of_many_rows(dtype, width):
    """Enough rows for the warp-per-row kernel (widths that are multiples of 4 up to
    1,024) and widths beside it; rows picked through an index too."""
    o = ops()
    g = torch.Generator().manual_seed(width)
    x = torch.randn(301, width, generator=g) * 2
    w = 1 + 0.1 * torch.randn(width, generator=g)
    out = torch.full((301, width), 9.0, dtype=DT[dtype], device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, out)
    close(out, P.rms_norm(x, w, 1e-6), dtype, "rmsnorm many rows")
    rows = torch.randperm(301, generator=g)[:70].to(torch.int32)
    out2 = torch.empty(70, width, dtype=DT[dtype], device=DEV)
    o.rmsnorm(x.to(DEV), w.to(DEV), 1e-6, out2, rows.to(DEV))
    close(out2, P.rms_norm(x[rows.long()], w, 1e-6), dtype, "rmsnorm picked rows")


@pytest.mark.parametrize("dtype", list(DT))
def test_silu_mul(dtype):
    o = ops()
    gu = torch.randn(7, 2 * 45) * 4
    out = torch.empty(7, 45, dtype=DT[dtype], device=DEV)
    o.silu_mul(gu.to(DEV), out)
    close(out, P.swiglu(gu[:, :45], gu[:, 45:]), dtype, "silu_mul")


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("m", [1, 2, 3, 7, 16, 17, 100])
@pytest.mark.parametrize("n,k", [(5, 16), (64, 30), (130, 100), (257, 576)])
def test_gemm_simt(dtype, m, n, k):
    o = ops()
    g = torch.Generator().manual_seed(m * 1000 + n + k)
    a = torch.randn(m, k, generator=g).to(DT[dtype])
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(DT[dtype])
    bias = torch.randn(n, generator=g)
    want = P.linear(a, w, bias)
    for mode, out_dtype in ((o.STORE, DT[dtype]), (o.STORE_F32, torch.float32)):
        out = torch.empty(m, n, dtype=out_dtype, device=DEV)
        o.gemm_simt(a.to(DEV), w.to(DEV), bias.to(DEV), out, mode)
        close(out, want, dtype if mode == o.STORE else "float32", f"gemm mode {mode}")
    base = torch.randn(m, n, generator=g)
    acc = base.to(DEV).clone()
    o.gemm_simt(a.to(DEV), w.to(DEV), None, acc, o.ADD_F32)
    close(acc, base.double() + P.linear(a, w), "float32", "gemm add")


class PagedCase:
    """Sequences of unequal length in a paged cache whose pages are shuffled."""

    def __init__(self, lengths, new_counts, nq, nkv, d, dtype, seed=0, page=64, scale=1.0):
        rng = random.Random(seed)
        g = torch.Generator().manual_seed(seed)
        self.nq, self.nkv, self.d, self.page = nq, nkv, d, page
        self.lengths, self.new = lengths, new_counts
        n_pages = sum(-(-L // page) for L in lengths) + 3
        ids = list(range(n_pages))
        rng.shuffle(ids)
        cols = max(-(-L // page) for L in lengths)
        self.table = torch.full((len(lengths), cols), -1, dtype=torch.int32)
        self.q = [torch.randn(L, nq, d, generator=g) * scale for L in lengths]
        self.k = [torch.randn(L, nkv, d, generator=g) * scale for L in lengths]
        self.v = [torch.randn(L, nkv, d, generator=g) for L in lengths]
        if dtype == "bfloat16":
            self.q = [x.bfloat16().float() for x in self.q]
            self.k = [x.bfloat16().float() for x in self.k]
            self.v = [x.bfloat16().float() for x in self.v]
        # stale contents everywhere: a reused page is never clean
        self.k_cache = torch.randn(n_pages, nkv, page, d, generator=g) * 50
        self.v_cache = torch.randn(n_pages, nkv, page, d, generator=g) * 50
        for s, L in enumerate(lengths):
            for j in range(-(-L // page)):
                self.table[s, j] = ids.pop()

    def fill_cache(self, upto_new=True):
        """Write keys/values of the positions that precede this step's tokens."""
        for s, L in enumerate(self.lengths):
            old = L - self.new[s]
            for t in range(old):
                pg = int(self.table[s, t // self.page])
                self.k_cache[pg, :, t % self.page] = self.k[s][t]
                self.v_cache[pg, :, t % self.page] = self.v[s][t]

    def packed(self):
        pos, seq, rows_q, rows_k, rows_v = [], [], [], [], []
        for s, L in enumerate(self.lengths):
            for t in range(L - self.new[s], L):
                pos.append(t)
                seq.append(s)
                rows_q.append(self.q[s][t])
                rows_k.append(self.k[s][t])
                rows_v.append(self.v[s][t])
        return (torch.tensor(pos, dtype=torch.int32), torch.tensor(seq, dtype=torch.int32),
                torch.stack(rows_q), torch.stack(rows_k), torch.stack(rows_v))


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("nq,nkv,d", [(6, 2, 16), (5, 5, 48), (4, 1, 80), (3, 3, 128), (2, 1, 256)])
@pytest.mark.parametrize("window", [0, 37])
def test_rope_store_then_attention(dtype, nq, nkv, d, window):
    """Prompt chunks and single tokens in one packed batch: rotate, store, attend."""
    o = ops()
    lengths, new = [70, 1, 130, 64, 200], [70, 1, 5, 1, 1]
    case = PagedCase(lengths, new, nq, nkv, d, dtype, seed=d + nq)
    cos, sin = P.rope_tables(256, d, 10000.0)
    # the cache holds rotated keys of earlier positions
    rot_k = [P.rope_rotate_half(k, cos[:L], sin[:L]).float() for k, L in zip(case.k, lengths)]
    rot_q = [P.rope_rotate_half(q, cos[:L], sin[:L]).float() for q, L in zip(case.q, lengths)]
    if dtype == "bfloat16":
        rot_k = [x.bfloat16().float() for x in rot_k]
        rot_q = [x.bfloat16().float() for x in rot_q]
    plain_k, case.k = case.k, rot_k
    case.fill_cache()
    case.k = plain_k
    pos, seq, q, k, v = case.packed()
    n = pos.numel()
    qkv = torch.cat([q.reshape(n, -1), k.reshape(n, -1), v.reshape(n, -1)], 1).to(DT[dtype]).to(DEV)
    kc, vc = case.k_cache.to(DT[dtype]).to(DEV), case.v_cache.to(DT[dtype]).to(DEV)
    table = case.table.to(DEV)
    o.rope_store(qkv, pos.to(DEV), seq.to(DEV), table, cos.float().to(DEV), sin.float().to(DEV), kc,
                 vc, nq, nkv, d, 64)
    # the rotated rows, in place and in the cache
    want_q = torch.stack([rot_q[s][t] for t, s in zip(pos.tolist(), seq.tolist())]).reshape(n, -1)
    close(qkv[:, :nq * d], want_q, dtype, "rotated q")
    for i, (t, s) in enumerate(zip(pos.tolist(), seq.tolist())):
        pg = int(case.table[s, t // 64])
        close(kc[pg, :, t % 64], rot_k[s][t], dtype, "stored k")
        assert torch.equal(vc[pg, :, t % 64].float().cpu(), case.v[s][t].to(DT[dtype]).float())
    for splits in (1, 3):
        out = torch.empty(n, nq * d, dtype=DT[dtype], device=DEV)
        partial = torch.empty(n * nq * splits * (d + 2), device=DEV) if splits > 1 else None
        o.attention_generic(qkv, qkv.shape[1], kc, vc, pos.to(DEV), seq.to(DEV), table, out, nq, nkv,
                            d, window, 1.0 / math.sqrt(d), splits, partial)
        i = 0
        for s, L in enumerate(lengths):
            full = P.causal_attention(rot_q[s], rot_k[s], case.v[s].to(DT[dtype]).float(), window)
            want = full[L - new[s]:].reshape(new[s], -1)
            close(out[i:i + new[s]], want, dtype, f"attention seq {s} splits {splits}")
            i += new[s]


@pytest.mark.parametrize("dtype", list(DT))
def test_attention_finds_one_far_key_and_respects_the_window_edge(dtype):
    """One key far back is made to dominate; with a window that just excludes
    it, it must vanish, and with one that just includes it, it must win."""
    o = ops()
    nq, nkv, d, L, far = 4, 2, 32, 500, 123
    case = PagedCase([L], [1], nq, nkv, d, dtype, seed=3, scale=0.3)
    case.k[0][far] = case.q[0][L - 1][::2] * 40.0  # kv head h serves query heads 2h, 2h+1
    case.v[0][far] = 7.0
    if dtype == "bfloat16":
        case.k[0] = case.k[0].bfloat16().float()
    case.fill_cache()
    # the step's own token is written by hand here (no rotation in this test)
    pg = int(case.table[0, (L - 1) // 64])
    case.k_cache[pg, :, (L - 1) % 64] = case.k[0][L - 1]
    case.v_cache[pg, :, (L - 1) % 64] = case.v[0][L - 1]
    pos, seq, q, _, _ = case.packed()
    qd = q.reshape(1, -1).to(DT[dtype]).to(DEV)
    kc, vc = case.k_cache.to(DT[dtype]).to(DEV), case.v_cache.to(DT[dtype]).to(DEV)
    for window, sees in ((0, True), (L - far, True), (L - far - 1, False)):
        for splits in (1, 4):
            out = torch.empty(1, nq * d, dtype=DT[dtype], device=DEV)
            partial = torch.empty(nq * splits * (d + 2), device=DEV) if splits > 1 else None
            o.attention_generic(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                                nq, nkv, d, window, 1.0 / math.sqrt(d), splits, partial)
            want = P.causal_attention(case.q[0], case.k[0], case.v[0].to(DT[dtype]).float(),
                                      window)[L - 1:].reshape(1, -1)
            close(out, want, dtype, f"far key window {window} splits {splits}")
            even_heads = out.view(nq, d)[0::2].float()
            assert bool((even_heads > 6.5).all()) == sees


def test_padding_rows_store_nothing_and_come_out_zero():
    o = ops()
    nq, nkv, d = 2, 1, 16
    kc = torch.zeros(2, nkv, 64, d, device=DEV)
    vc = torch.zeros(2, nkv, 64, d, device=DEV)
    qkv = torch.ones(3, (nq + 2 * nkv) * d, device=DEV)
    pos = torch.tensor([0, -1, 1], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0, 0, 0], dtype=torch.int32, device=DEV)
    table = torch.tensor([[1]], dtype=torch.int32, device=DEV)
    o.rope_store(qkv, pos, seq, table, None, None, kc, vc, nq, nkv, d, 64)
    assert float(kc[1, 0, :2].sum()) == 2 * d and float(kc.sum()) == 2 * d
    out = torch.full((3, nq * d), 9.0, device=DEV)
    o.attention_generic(qkv, qkv.shape[1], kc, vc, pos, seq, table, out, nq, nkv, d, 0, 0.25)
    assert float(out[1].abs().sum()) == 0 and torch.allclose(out[0], torch.ones(nq * d, device=DEV))


def test_sizes_the_kernels_do_not_take_are_refused():
    o = ops()
    i = torch.zeros(1, dtype=torch.int32, device=DEV)
    for d in (23, 258):  # an odd head size, one beyond 256
        kc = torch.zeros(1, 1, 64, d, device=DEV)
        q = torch.zeros(1, d, device=DEV)
        with pytest.raises(o.KernelError, match="even size"):
            o.attention_generic(q, d, kc, kc, i, i, i.view(1, 1), q.clone(), 1, 1, d, 0, 1.0)
    with pytest.raises(o.KernelError):
        o.gemm_simt(torch.zeros(2, 4), torch.zeros(2, 4), None, torch.zeros(2, 2), 0)  # CPU tensors
    with pytest.raises(o.KernelError):
        o.rmsnorm(torch.zeros(2, 4, device=DEV), torch.zeros(5, device=DEV), 1e-5,
                  torch.zeros(2, 4, device=DEV))


def test_argmax_takes_the_lowest_index_among_equals():
    o = ops()
    rng = np.random.default_rng(0)
    logits = rng.normal(size=(6, 49157)).astype(np.float32)
    logits[0, [77, 40000]] = 9.0
    logits[1, :] = 0.0
    logits[2, 49156] = 12.0
    logits[3, :] = -np.inf
    logits[3, 5] = -1e30
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    o.argmax(torch.from_numpy(logits).to(DEV), out)
    want = [P.argmax_lowest(torch.from_numpy(r)) for r in logits]
    assert out.tolist() == want and want[:4] == [77, 0, 49156, 5]


def test_temperature_sampling_follows_the_seeded_draws():
    """Inverse CDF in id order with SplitMix64 draws, checked against a float64
    reference; the chosen id's interval must contain the draw."""
    o = ops()
    from nnis_b200.sampling.device import seed_states
    rng = np.random.default_rng(1)
    vocab, rows = 1003, 5
    logits = (rng.normal(size=(rows, vocab)) * 3).astype(np.float32)
    temps = np.array([1.0, 0.5, 2.0, 0.05, 1.3], dtype=np.float32)
    seeds = [42, 7, 2 ** 63 + 5, 0, 99]
    state = seed_states(seeds, DEV)
    plains = [P.PlainSplitMix64(s) for s in seeds]
    dl, dt = torch.from_numpy(logits).to(DEV), torch.from_numpy(temps).to(DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    counts = np.zeros(vocab)
    for _ in range(200):
        o.sample_temperature(dl, dt, state, out)
        got = out.tolist()
        for r in range(rows):
            u = plains[r].next_unit()
            w = np.exp((logits[r].astype(np.float64) - logits[r].max()) / float(temps[r]))
            cdf = np.cumsum(w)
            want = int(np.searchsorted(cdf, u * cdf[-1], side="right"))
            assert abs(got[r] - want) <= 0 or abs(cdf[got[r]] - u * cdf[-1]) < 1e-9 * cdf[-1]
        counts[got[0]] += 1
    assert counts.argmax() == logits[0].argmax() or counts.max() < 20


# ---------------------------------------------------------------------------
# the fused bfloat16 decode kernels
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 2, 3, 8, 11, 16, 17, 33, 40, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(8, 16), (104, 80), (960, 576), (1000, 1536), (3072, 576)])
def test_gemv_plain_epilogues_and_norm_prologue(m, n, k):
    """Both kernels of the decode projections: the one whose CTAs hold all rows (up to 64)
    and, from 17 rows on where every CTA is resident at once, the one over tiles of rows."""
    o = ops()
    kind = o.gemv_kind(m, n, k, o.EPI_STORE, DEV)
    if n == 3072 and m >= 64:
        # more CTAs over tiles of rows than are resident at once: the other kernel, up to its 64 rows
        assert kind == (1 if m == 64 else 0)
        if kind == 0:
            return
    else:
        assert kind == 2
    kernels = [True] if kind == 2 else []
    if o.gemv_kind(m, n, k, o.EPI_STORE, DEV, rows_kernel=False):
        kernels.append(False)
    assert kernels and (len(kernels) == 2 or m > 48)
    for rows_kernel in kernels:
        _gemv_plain_and_norm(o, m, n, k, rows_kernel)


def _gemv_plain_and_norm(o, m, n, k, rows_kernel):
    g = torch.Generator().manual_seed(m + n + k)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    want = P.linear(x, w, bias)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    o.gemv_bf16(w.to(DEV), bias.to(DEV), out, o.EPI_STORE, x=x.to(DEV), rows_kernel=rows_kernel)
    close(out, want, "bfloat16", "gemv store")
    out32 = torch.empty(m, n, device=DEV)
    o.gemv_bf16(w.to(DEV), None, out32, o.EPI_STORE_F32, x=x.to(DEV), rows_kernel=rows_kernel)
    close(out32, P.linear(x, w), "float32", "gemv store f32")
    base = torch.randn(m, n, generator=g)
    acc = base.to(DEV).clone()
    o.gemv_bf16(w.to(DEV), bias.to(DEV), acc, o.EPI_ADD_F32, x=x.to(DEV), rows_kernel=rows_kernel)
    close(acc, base.double() + want, "float32", "gemv add")
    # norm prologue with gathered rows
    if not o.gemv_kind(m, n, k, o.EPI_STORE_F32, DEV, True, rows_kernel):
        # with the normalised rows beside the weights only one CTA fits an SM, or (the
        # kernel whose CTAs hold all rows) x and the weight stages do not fit together
        assert m > 48
        return
    hidden = torch.randn(m + 5, k, generator=g) * 2
    nw = 1 + 0.1 * torch.randn(k, generator=g)
    rows = torch.randperm(m + 5, generator=g)[:m].to(torch.int32)
    # the inputs as drawn, rounding ties and all, held to the bound of a bfloat16 value ...
    o.gemv_bf16(w.to(DEV), None, out32, o.EPI_STORE_F32, hidden=hidden.to(DEV),
                norm_weight=nw.to(DEV), eps=1e-5, rows=rows.to(DEV), rows_kernel=rows_kernel)
    close(out32, P.linear(P.rms_norm(hidden[rows.long()], nw, 1e-5).bfloat16(), w), "bfloat16",
          "gemv norm prologue, inputs as drawn")
    # ... and, with the few values moved whose rounding is not decided, to the float32 bound
    hidden = away_from_bf16_ties(hidden, nw, 1e-5)
    normed = P.rms_norm(hidden[rows.long()], nw, 1e-5).bfloat16()
    o.gemv_bf16(w.to(DEV), None, out32, o.EPI_STORE_F32, hidden=hidden.to(DEV),
                norm_weight=nw.to(DEV), eps=1e-5, rows=rows.to(DEV), rows_kernel=rows_kernel)
    close(out32, P.linear(normed, w), "float32", "gemv norm prologue")


@pytest.mark.parametrize("m", [1, 8, 24])
@pytest.mark.parametrize("n,k", [(4096, 2048), (1544, 4096), (2048, 8192), (520, 6144), (2400, 2080)])
def test_gemv_long_rows_in_chunks_and_slices(m, n, k):
    """Rows of K too long for whole-row weight stages stream in chunks; rows of x
    too long for shared memory are taken by the adding epilogue alone, slice by slice."""
    o = ops()
    g = torch.Generator().manual_seed(m + n + k)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    # one far column of K matters: a chunk or a slice left out would show
    w[:, k - 3] = 1.0
    bias = torch.randn(n, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    x[:, k - 3] = 4.0
    want = P.linear(x, w, bias)
    base = torch.randn(m, n, generator=g)
    acc = base.to(DEV).clone()
    assert o.gemv_takes(m, n, k, o.EPI_ADD_F32, DEV)
    whole = o.gemv_takes(m, n, k, o.EPI_STORE_F32, DEV)
    assert whole or o.gemv_slices(m, n, k, DEV) > 1
    # all of x has to fit shared memory beside the weight stages
    assert whole or k * ((m + 15) // 16) > 4096
    assert not whole or k < 8192
    o.gemv_bf16(w.to(DEV), bias.to(DEV), acc, o.EPI_ADD_F32, x=x.to(DEV))
    close(acc, base.double() + want, "float32", "gemv add in slices")
    if not whole:
        with pytest.raises(o.KernelError, match="not taken"):
            o.gemv_bf16(w.to(DEV), None, torch.empty(m, n, device=DEV), o.EPI_STORE_F32, x=x.to(DEV))
        return
    out32 = torch.empty(m, n, device=DEV)
    o.gemv_bf16(w.to(DEV), bias.to(DEV), out32, o.EPI_STORE_F32, x=x.to(DEV))
    close(out32, want, "float32", "gemv store f32, chunks")
    hidden = torch.randn(m + 3, k, generator=g) * 2
    hidden[:, k - 3] = 9.0
    nw = 1 + 0.1 * torch.randn(k, generator=g)
    rows = torch.randperm(m + 3, generator=g)[:m].to(torch.int32)
    # the inputs as drawn, rounding ties and all, held to the bound of a bfloat16 value: a
    # normed value that rounds the other way moves its products by one bfloat16 step
    o.gemv_bf16(w.to(DEV), None, out32, o.EPI_STORE_F32, hidden=hidden.to(DEV),
                norm_weight=nw.to(DEV), eps=1e-5, rows=rows.to(DEV))
    close(out32, P.linear(P.rms_norm(hidden[rows.long()], nw, 1e-5).bfloat16(), w), "bfloat16",
          "gemv norm prologue, long rows, inputs as drawn")
    hidden = away_from_bf16_ties(hidden, nw, 1e-5)
    normed = P.rms_norm(hidden[rows.long()], nw, 1e-5).bfloat16()
    o.gemv_bf16(w.to(DEV), None, out32, o.EPI_STORE_F32, hidden=hidden.to(DEV),
                norm_weight=nw.to(DEV), eps=1e-5, rows=rows.to(DEV))
    close(out32, P.linear(normed, w), "float32", "gemv norm prologue, long rows")
    if n % 16 == 0:
        inter = n // 2
        out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
        o.gemv_bf16(w.to(DEV), bias.to(DEV), out, o.EPI_GATED, x=x.to(DEV))
        close(out, P.swiglu(want[:, :inter], want[:, inter:]), "bfloat16", "gemv gated, chunks")


@pytest.mark.parametrize("m", [1, 5, 16, 33, 64, 81])
@pytest.mark.parametrize("k,inter", [(80, 100), (576, 1536)])
def test_gemv_gated_epilogue(m, k, inter):
    o = ops()
    if not o.gemv_takes(m, 2 * inter, k, o.EPI_GATED, DEV):
        assert m > 64 and inter == 1536  # more CTAs over tiles of rows than are resident at once
        return
    g = torch.Generator().manual_seed(m)
    w = (torch.randn(2 * inter, k, generator=g) / math.sqrt(k) * 3).bfloat16()
    bias = torch.randn(2 * inter, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    y = P.linear(x, w, bias)
    for rows_kernel in (True, False):  # both kernels where both take the shape
        if not o.gemv_kind(m, 2 * inter, k, o.EPI_GATED, DEV, rows_kernel=rows_kernel):
            continue
        out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
        o.gemv_bf16(w.to(DEV), bias.to(DEV), out, o.EPI_GATED, x=x.to(DEV), rows_kernel=rows_kernel)
        close(out, P.swiglu(y[:, :inter], y[:, inter:]), "bfloat16", "gemv gated")


@pytest.mark.parametrize("nq,nkv,d,rotate", [(6, 2, 16, True), (3, 1, 48, True), (4, 4, 64, False),
                                             (2, 0, 32, True), (9, 3, 64, True)])
@pytest.mark.parametrize("copies", [1, 7, 20])
@pytest.mark.parametrize("rows_kernel", [True, False])
def test_gemv_qkv_epilogue_rotates_and_stores(nq, nkv, d, rotate, copies, rows_kernel):
    """Five rows (one of them padding), or several times these rows with a cache of their
    own each: more than a tile of rows goes to the kernel over tiles of rows."""
    o = ops()
    g = torch.Generator().manual_seed(nq * d)
    m, k, page = 5 * copies, 48, 64
    n = (nq + 2 * nkv) * d
    assert o.gemv_kind(m, n, k, o.EPI_QKV, DEV) == 2
    if not rows_kernel and m > 64:
        return  # the kernel whose CTAs hold all rows takes 64
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    pos = torch.tensor([0, 63, 64, -1, 130] * copies, dtype=torch.int32)
    seq = torch.cat([torch.tensor([0, 1, 2, 0, 3], dtype=torch.int32) + 4 * c for c in range(copies)])
    base = torch.tensor([[5, -1, -1], [2, -1, -1], [7, 1, -1], [0, 3, 4]], dtype=torch.int32)
    table = torch.cat([torch.where(base >= 0, base + 8 * c, base) for c in range(copies)])
    kc = torch.zeros(8 * copies, max(nkv, 1), page, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    cos, sin = P.rope_tables(200, d, 10000.0)
    q_out = torch.full((m, nq * d), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemv_bf16(w.to(DEV), bias.to(DEV), q_out, o.EPI_QKV, x=x.to(DEV), token_pos=pos.to(DEV),
                token_seq=seq.to(DEV), page_table=table.to(DEV) if nkv else None,
                cos=cos.float().to(DEV) if rotate else None, sin=sin.float().to(DEV) if rotate else None,
                k_cache=kc if nkv else None, v_cache=vc if nkv else None, heads=nq, kv_heads=nkv,
                head_dim=d, page_size=page, rows_kernel=rows_kernel)
    _qkv_matches(P.linear(x, w, bias), q_out, kc, vc, pos, seq, table, nq, nkv, d, page, rotate, copies)


def _qkv_matches(y, q_out, kc, vc, pos, seq, table, nq, nkv, d, page, rotate, copies):
    """`y` [m, (nq + 2 nkv) d], the projection's output before rounding and rotation,
    against what the QKV epilogue left in `q_out` and the caches."""
    cos, sin = P.rope_tables(200, d, 10000.0)
    y = y.bfloat16().double()
    for i in range(y.shape[0]):
        p = int(pos[i])
        if p < 0:
            assert float((q_out[i].float() - 9.0).abs().max()) == 0  # padding row untouched
            continue
        c, s = (cos[p:p + 1], sin[p:p + 1]) if rotate else (torch.ones(1, d // 2).double(),
                                                            torch.zeros(1, d // 2).double())
        heads = y[i].view(nq + 2 * nkv, d)
        rq = P.rope_rotate_half(heads[:nq][None], c, s)[0]
        close(q_out[i].view(nq, d), rq, "bfloat16", "q")
        if nkv:
            rk = P.rope_rotate_half(heads[nq:nq + nkv][None], c, s)[0]
            pg = int(table[int(seq[i]), p // page])
            close(kc[pg, :, p % page], rk, "bfloat16", "k")
            close(vc[pg, :, p % page], heads[nq + nkv:], "bfloat16", "v")
    if nkv:
        assert int((kc.float().abs().sum(-1) > 0).sum()) == 4 * nkv * copies  # nothing else was written


@pytest.mark.parametrize("m", [1, 8, 11, 16, 40, 100])
@pytest.mark.parametrize("width,inter", [(576, 1536), (80, 112), (1536, 3072), (960, 2560)])
def test_gemv_shares_a_norm_between_two_projections(m, width, inter):
    """The adding epilogue begins the norm that follows it (rows times the norm's weights,
    shares of the sums of squares); the gated and the QKV projection end it on their sums.
    The rows differ in size by factors up to 13, so that a row scaled by another row's
    factor would show."""
    o = ops()
    g = torch.Generator().manual_seed(m + width)
    eps = 1e-5
    w_down = (torch.randn(width, inter, generator=g) / math.sqrt(inter)).bfloat16()
    x = torch.randn(m, inter, generator=g).bfloat16()
    size = 1.0 + 3.0 * (torch.arange(m) % 5).double()
    x = (x.double() * size[:, None]).bfloat16()
    base = torch.randn(m, width, generator=g) * size[:, None].float()
    nw = 1 + 0.1 * torch.randn(width, generator=g)
    want = base.double() + P.linear(x, w_down)
    took = 0
    for rows_kernel in (True, False):
        if not o.gemv_kind(m, width, inter, o.EPI_ADD_F32, DEV, rows_kernel=rows_kernel):
            continue
        took += 1
        acc = base.to(DEV).clone()
        x_next = torch.full((m, width), 7.0, dtype=torch.bfloat16, device=DEV)
        shares = torch.full((m, width // 8), -1.0, device=DEV)
        o.gemv_bf16(w_down.to(DEV), None, acc, o.EPI_ADD_F32, x=x.to(DEV), rows_kernel=rows_kernel,
                    emit=(x_next, nw.to(DEV), shares))
        close(acc, want, "float32", "gemv add that emits")
        # of the sums as the kernel has them: the weighted rows to the bit, the squares to rounding
        assert torch.equal(x_next, (acc * nw.to(DEV)).bfloat16())
        close(shares, acc.double().view(m, width // 8, 8).square().sum(-1), "float32", "shares of the squares")
    if not took:
        assert m > 64 and inter > 1536  # neither kernel: the general product runs, which shares no norm
        return
    if not o.gemv_shares_norm(m, 2 * inter, width, o.EPI_GATED, DEV):
        # more CTAs over tiles of rows than are resident at once
        assert (m > 64 or inter > 1536) and width != 80
        return
    # the norm with its one rounding where the kernels have it: on the weighted rows, before the scale
    hidden = acc.cpu().double()
    normed = x_next.cpu().double() / torch.sqrt(hidden.square().mean(-1, keepdim=True) + eps)
    close(normed, P.rms_norm(acc.cpu(), nw, eps), "bfloat16", "the rows normed in two halves")
    w_gu = (torch.randn(2 * inter, width, generator=g) / math.sqrt(width) * 3).bfloat16()
    bias = torch.randn(2 * inter, generator=g)
    out = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    o.gemv_bf16(w_gu.to(DEV), bias.to(DEV), out, o.EPI_GATED, x=x_next, shares=shares, eps=eps)
    y = P.linear(normed, w_gu, bias)
    close(out, P.swiglu(y[:, :inter], y[:, inter:]), "bfloat16", "gemv gated after a shared norm")
    # the QKV projection: rows at positions of their own, one of five a padding row
    nq, nkv, d, page = 3, 1, 32, 64
    n = (nq + 2 * nkv) * d
    assert o.gemv_shares_norm(m, n, width, o.EPI_QKV, DEV)
    copies = (m + 4) // 5
    pos = torch.tensor([0, 63, 64, -1, 130] * copies, dtype=torch.int32)[:m]
    seq = torch.cat([torch.tensor([0, 1, 2, 0, 3], dtype=torch.int32) + 4 * c for c in range(copies)])[:m]
    tbl = torch.tensor([[5, -1, -1], [2, -1, -1], [7, 1, -1], [0, 3, 4]], dtype=torch.int32)
    table = torch.cat([torch.where(tbl >= 0, tbl + 8 * c, tbl) for c in range(copies)])
    kc = torch.zeros(8 * copies, nkv, page, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    cos, sin = P.rope_tables(200, d, 10000.0)
    w_qkv = (torch.randn(n, width, generator=g) / math.sqrt(width)).bfloat16()
    bias = torch.randn(n, generator=g)
    q_out = torch.full((m, nq * d), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemv_bf16(w_qkv.to(DEV), bias.to(DEV), q_out, o.EPI_QKV, x=x_next, shares=shares, eps=eps,
                token_pos=pos.to(DEV), token_seq=seq.to(DEV), page_table=table.to(DEV),
                cos=cos.float().to(DEV), sin=sin.float().to(DEV), k_cache=kc, v_cache=vc, heads=nq,
                kv_heads=nkv, head_dim=d, page_size=page)
    y = P.linear(normed, w_qkv, bias)
    live = int((pos >= 0).sum())
    for i in range(m):
        p = int(pos[i])
        if p < 0:
            assert float((q_out[i].float() - 9.0).abs().max()) == 0
            continue
        heads = y[i].bfloat16().double().view(nq + 2 * nkv, d)
        close(q_out[i].view(nq, d), P.rope_rotate_half(heads[:nq][None], cos[p:p + 1], sin[p:p + 1])[0],
              "bfloat16", "q after a shared norm")
        pg = int(table[int(seq[i]), p // page])
        close(kc[pg, :, p % page], P.rope_rotate_half(heads[nq:nq + nkv][None], cos[p:p + 1], sin[p:p + 1])[0],
              "bfloat16", "k after a shared norm")
        close(vc[pg, :, p % page], heads[nq + nkv:], "bfloat16", "v after a shared norm")
    assert int((kc.float().abs().sum(-1) > 0).sum()) == live * nkv


def test_gemv_refuses_what_it_does_not_take():
    o = ops()
    assert not o.gemv_takes(129, 64, 64) and not o.gemv_takes(4, 64, 56) and not o.gemv_takes(4, 68, 64)
    assert o.gemv_takes(64, 64, 64) and o.gemv_takes(128, 64, 64) and not o.gemv_takes(64, 64, 4096)
    # more than 64 rows: only the kernel over tiles of rows, which wants every CTA resident
    # (and has no picking epilogue)
    assert not o.gemv_takes(80, 49152, 576) and not o.gemv_takes(80, 64, 64, o.EPI_ARGMAX)
    assert o.gemv_kind(64, 49152, 576) == 1 and o.gemv_kind(17, 64, 64, o.EPI_ARGMAX) == 1
    assert o.gemv_kind(8, 960, 576) == 2 and o.gemv_kind(8, 960, 576, rows_kernel=False) == 1
    with pytest.raises(o.KernelError, match="not taken"):
        o.gemv_bf16(torch.zeros(68, 64, dtype=torch.bfloat16, device=DEV), None,
                    torch.zeros(2, 68, dtype=torch.bfloat16, device=DEV), o.EPI_STORE,
                    x=torch.zeros(2, 64, dtype=torch.bfloat16, device=DEV))


@pytest.mark.parametrize("nq,nkv,d", [(6, 2, 16), (5, 5, 48), (4, 1, 80), (9, 3, 64), (16, 2, 128),
                                      (2, 1, 256)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_kernel(nq, nkv, d, window):
    """One token per sequence, contexts from 1 to many pages, with padding rows."""
    o = ops()
    lengths = [1, 64, 65, 300, 1000, 7]
    case = PagedCase(lengths, [1] * len(lengths), nq, nkv, d, "bfloat16", seed=nq + d)
    case.fill_cache()
    for s, L in enumerate(lengths):  # the step's own key and value
        pg = int(case.table[s, (L - 1) // 64])
        case.k_cache[pg, :, (L - 1) % 64] = case.k[s][L - 1]
        case.v_cache[pg, :, (L - 1) % 64] = case.v[s][L - 1]
    pos, seq, q, _, _ = case.packed()
    pos = torch.cat([pos, torch.tensor([-1], dtype=torch.int32)])  # a padding row at the end
    seq = torch.cat([seq, torch.tensor([0], dtype=torch.int32)])
    n = pos.numel()
    qd = torch.cat([q.reshape(n - 1, -1), torch.ones(1, nq * d)]).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    want = torch.cat([P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(),
                                         window)[L - 1:].reshape(1, -1)
                      for s, L in enumerate(lengths)])
    for splits in (1, 2, 7):
        out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(n * nq * splits * (d + 2), device=DEV) if splits > 1 else None
        o.attention_decode(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out, nq,
                           nkv, d, window, 1.0 / math.sqrt(d), splits, partial)
        close(out[:n - 1], want, "bfloat16", f"decode attention splits {splits}")
        assert float(out[n - 1].float().abs().max()) == 0


@pytest.mark.parametrize("m", [1, 6, 16, 50])
@pytest.mark.parametrize("n,k", [(8, 16), (1000, 80), (49152, 576), (3000, 2048)])
def test_gemv_argmax_epilogue_picks_moves_on_and_can_write_logits(m, n, k):
    o = ops()
    if not o.gemv_takes(m, n, k, o.EPI_ARGMAX, DEV):
        assert m > 32 and k == 2048  # 64 rows of x of this length do not fit shared memory
        return
    g = torch.Generator().manual_seed(m + n)
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    w[n // 2] = w[3]  # two equal logits in every row: the lower index must win when they lead
    hidden = torch.randn(m, k, generator=g)
    hidden[0] = w[3].float() * 4  # row 0 is led by index 3 (and its twin)
    nw = torch.ones(k)
    # the inputs as drawn, held to the bound of a bfloat16 value (see away_from_bf16_ties)
    raw_logits = torch.zeros(m, n, device=DEV)
    o.gemv_bf16(w.to(DEV), None, torch.empty(m, dtype=torch.int32, device=DEV), o.EPI_ARGMAX,
                hidden=hidden.to(DEV), norm_weight=nw.to(DEV), eps=1e-5,
                rows=torch.arange(m, dtype=torch.int32, device=DEV), m=m, logits=raw_logits,
                scratch=torch.zeros(o.argmax_scratch_ints(m, n, k, DEV), dtype=torch.int32, device=DEV))
    close(raw_logits, P.linear(P.rms_norm(hidden, nw, 1e-5).bfloat16(), w), "bfloat16",
          "argmax logits, inputs as drawn")
    hidden = away_from_bf16_ties(hidden, nw, 1e-5)
    want_logits = P.linear(P.rms_norm(hidden, nw, 1e-5).bfloat16(), w)
    want = [P.argmax_lowest(r) for r in want_logits]
    assert want[0] == 3
    rows = torch.arange(m, dtype=torch.int32, device=DEV)
    scratch = torch.zeros(o.argmax_scratch_ints(m, n, k, DEV), dtype=torch.int32, device=DEV)
    tokens = torch.full((m,), 7, dtype=torch.int32, device=DEV)
    pos = torch.arange(10, 10 + m, dtype=torch.int32, device=DEV)
    pos[m - 1] = -1  # a padding row keeps its state
    for with_logits in (False, True, False):  # the scratch is reused across launches
        picks = torch.full((m,), -5, dtype=torch.int32, device=DEV)
        logits = torch.zeros(m, n, device=DEV) if with_logits else None
        t, p = tokens.clone(), pos.clone()
        o.gemv_bf16(w.to(DEV), None, picks, o.EPI_ARGMAX, hidden=hidden.to(DEV), norm_weight=nw.to(DEV),
                    eps=1e-5, rows=rows, m=m, logits=logits, scratch=scratch, next_tokens=t, next_pos=p)
        got = picks.tolist()
        for r in range(m):  # equal up to rounding: accept any index whose logit ties the best
            assert got[r] == want[r] or abs(float(want_logits[r, got[r]] - want_logits[r, want[r]])) < 1e-3
        assert got[0] == 3
        assert t.tolist()[:m - 1] == got[:m - 1] and p.tolist()[:m - 1] == list(range(11, 10 + m))
        if m > 1:
            assert int(t[m - 1]) == 7 and int(p[m - 1]) == -1
        if with_logits:
            close(logits, want_logits, "float32", "argmax logits")
    o.check_status(DEV)


@pytest.mark.parametrize("nq,nkv,d", [(9, 3, 64), (4, 4, 64), (32, 1, 64), (20, 1, 128), (6, 2, 128)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_on_tensor_cores(nq, nkv, d, window):
    """Head sizes 64 and 128, groups below, at and above 16 heads, contexts from
    one key to many pages, a padding row, one slice and many."""
    o = ops()
    lengths = [1, 64, 65, 300, 1000, 7, 129]
    case = PagedCase(lengths, [1] * len(lengths), nq, nkv, d, "bfloat16", seed=nq + d)
    case.fill_cache()
    for s, L in enumerate(lengths):
        pg = int(case.table[s, (L - 1) // 64])
        case.k_cache[pg, :, (L - 1) % 64] = case.k[s][L - 1]
        case.v_cache[pg, :, (L - 1) % 64] = case.v[s][L - 1]
    pos, seq, q, _, _ = case.packed()
    pos = torch.cat([pos, torch.tensor([-1], dtype=torch.int32)])
    seq = torch.cat([seq, torch.tensor([0], dtype=torch.int32)])
    n = pos.numel()
    qd = torch.cat([q.reshape(n - 1, -1), torch.ones(1, nq * d)]).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    want = torch.cat([P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(),
                                         window)[L - 1:].reshape(1, -1)
                      for s, L in enumerate(lengths)])
    tickets = torch.zeros(o.mma_ticket_count(n, nq, nkv), dtype=torch.int32, device=DEV)
    # slices, and pages in flight per CTA (0: the default; fewer let more CTAs share an SM)
    assert o.attention_decode_mma_resident(d, DEV, o.attention_decode_mma_stages(d) - 1) \
        > o.attention_decode_mma_resident(d, DEV)
    for splits, stages in ((1, 0), (2, 0), (7, 0), (1, 2), (16, 0), (3, 3), (5, 2)):
        out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(n * nq * splits * (d + 2), device=DEV) if splits > 1 else None
        o.attention_decode_mma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                               nq, nkv, d, window, 1.0 / math.sqrt(d), splits, partial, tickets, stages)
        close(out[:n - 1], want, "bfloat16", f"tensor-core decode attention splits {splits} stages {stages}")
        assert float(out[n - 1].float().abs().max()) == 0
        assert int(tickets.abs().sum()) == 0
    assert not o.attention_decode_mma_takes(48, 64) and not o.attention_decode_mma_takes(64, 32)


@pytest.mark.parametrize("nq,nkv,d", [(9, 3, 64), (4, 4, 64), (32, 1, 64), (20, 1, 128), (6, 2, 128)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_fed_by_tma(nq, nkv, d, window):
    """Every page of a slice in shared memory at once (pages by TMA, a warp per page): head
    sizes 64 and 128, groups below, at and above 16 heads, contexts from one key to many
    pages, a padding row, one slice to sixteen, stale values in pages beyond each length."""
    o = ops()
    lengths = [1, 64, 65, 300, 1000, 7, 129]
    case = PagedCase(lengths, [1] * len(lengths), nq, nkv, d, "bfloat16", seed=nq + d)
    case.fill_cache()
    for s, L in enumerate(lengths):
        pg = int(case.table[s, (L - 1) // 64])
        case.k_cache[pg, :, (L - 1) % 64] = case.k[s][L - 1]
        case.v_cache[pg, :, (L - 1) % 64] = case.v[s][L - 1]
    pos, seq, q, _, _ = case.packed()
    pos = torch.cat([pos, torch.tensor([-1], dtype=torch.int32)])
    seq = torch.cat([seq, torch.tensor([0], dtype=torch.int32)])
    n = pos.numel()
    qd = torch.cat([q.reshape(n - 1, -1), torch.ones(1, nq * d)]).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    want = torch.cat([P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(),
                                         window)[L - 1:].reshape(1, -1)
                      for s, L in enumerate(lengths)])
    cols = case.table.shape[1]
    assert cols == 16
    most = o.attention_decode_tma_max_pages(d)
    assert most == (8 if d == 64 else 6)
    tickets = torch.zeros(o.mma_ticket_count(n, nq, nkv), dtype=torch.int32, device=DEV)
    for splits in (2, 3, 4, 7, 16):
        if -(-cols // splits) > most:
            continue  # eight pages of head size 128 do not fit a CTA's shared memory
        out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        partial = torch.full((n * nq * splits * (d + 2),), float("nan"), device=DEV)
        o.attention_decode_tma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                               nq, nkv, d, window, 1.0 / math.sqrt(d), splits, partial, tickets)
        close(out[:n - 1], want, "bfloat16", f"decode attention by TMA, {splits} slices")
        assert float(out[n - 1].float().abs().max()) == 0
        assert int(tickets.abs().sum()) == 0
    with pytest.raises(o.KernelError, match="slices of at most"):
        o.attention_decode_tma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                               nq, nkv, d, window, 1.0 / math.sqrt(d), 1)  # 16 pages in one slice
    # the same while it asks the pages of a cache that lies further on (or back) into L2: the
    # layer of its group that runs next; nothing of the result may change
    both_k, both_v = torch.stack([kc, kc]), torch.stack([vc, vc])
    for layer, ahead in ((0, kc.numel()), (1, -kc.numel())):
        out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        partial = torch.full((n * nq * 4 * (d + 2),), float("nan"), device=DEV)
        o.attention_decode_tma(qd, nq * d, both_k[layer], both_v[layer], pos.to(DEV), seq.to(DEV),
                               case.table.to(DEV), out, nq, nkv, d, window, 1.0 / math.sqrt(d), 4, partial,
                               tickets, ahead=ahead)
        close(out[:n - 1], want, "bfloat16", f"decode attention by TMA, asking pages {ahead} elements on")
    # one slice: a context of up to four pages needs no scratch
    short = PagedCase([200, 3], [1, 1], nq, nkv, d, "bfloat16", seed=5)
    short.fill_cache()
    for s, L in enumerate(short.lengths):
        pg = int(short.table[s, (L - 1) // 64])
        short.k_cache[pg, :, (L - 1) % 64] = short.k[s][L - 1]
        short.v_cache[pg, :, (L - 1) % 64] = short.v[s][L - 1]
    spos, sseq, sq, _, _ = short.packed()
    out = torch.empty(2, nq * d, dtype=torch.bfloat16, device=DEV)
    o.attention_decode_tma(sq.reshape(2, -1).bfloat16().to(DEV), nq * d, short.k_cache.bfloat16().to(DEV),
                           short.v_cache.bfloat16().to(DEV), spos.to(DEV), sseq.to(DEV), short.table.to(DEV),
                           out, nq, nkv, d, window, 1.0 / math.sqrt(d), 1)
    want = torch.cat([P.causal_attention(short.q[s], short.k[s], short.v[s].bfloat16().float(),
                                         window)[L - 1:].reshape(1, -1) for s, L in enumerate(short.lengths)])
    close(out, want, "bfloat16", "decode attention by TMA, one slice")
    o.check_status(DEV)
    # the plan: few sequences take it, many do not; short contexts need one slice
    assert o.attention_decode_tma_plan(2, nq, nkv, d, 64, 64, DEV) == 16
    assert o.attention_decode_tma_plan(1, nq, nkv, d, 64, 1, DEV) == 1
    assert o.attention_decode_tma_plan(4000, nq, nkv, d, 64, 64, DEV) == 0
    assert o.attention_decode_tma_plan(2, nq, nkv, d, 64, 1000, DEV) == 0  # slices would be too long
    assert o.attention_decode_tma_plan(2, nq, nkv, 48, 64, 8, DEV) == 0


def test_attention_decode_fed_by_tma_long_contexts_in_many_slices():
    """Contexts of thousands of keys in 16 to 64 slices (eight pages down to two a slice): the
    slice that arrives last merges more records than it asks for in one trip.  In every
    sequence one far key (a few hundred keys in) is made to stand out for one head, so that a
    slice left out of a merge would change the result; the same for the newest key."""
    o = ops()
    nq, nkv, d = 9, 3, 64
    lengths = [8192, 5003, 4097]
    case = PagedCase(lengths, [1] * len(lengths), nq, nkv, d, "bfloat16", seed=21)
    for s, L in enumerate(lengths):
        far = 300 + 700 * s
        q_far = case.q[s][L - 1, (s % nkv) * 3]
        # (a score two above the logarithm of the sum of all others: some nine tenths of the weight)
        score = math.log(1.65 * L) + 2.0
        case.k[s][far, s % nkv] = (q_far * (score * math.sqrt(d) / float(q_far.square().sum()))).bfloat16().float()
        case.v[s][far] = 7.0
    case.fill_cache()
    for s, L in enumerate(lengths):
        pg = int(case.table[s, (L - 1) // 64])
        case.k_cache[pg, :, (L - 1) % 64] = case.k[s][L - 1]
        case.v_cache[pg, :, (L - 1) % 64] = case.v[s][L - 1]
    pos, seq, q, _, _ = case.packed()
    n = pos.numel()
    qd = q.reshape(n, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)

    def newest_query(q_last, k, v):
        """The plain function's last row alone (it is quadratic in the length): every key is
        visible to the newest query."""
        out = torch.empty(nq, d, dtype=torch.float64)
        for hq in range(nq):
            hk = hq // (nq // nkv)
            p = torch.softmax((k[:, hk].double() @ q_last[hq].double()) / math.sqrt(d), dim=0)
            out[hq] = p @ v[:, hk].double()
        return out

    short = slice(0, 130)
    close(newest_query(case.q[0][129], case.k[0][short], case.v[0][short]),
          P.causal_attention(case.q[0][short], case.k[0][short], case.v[0][short])[-1], "float32", "the last row")
    want = torch.cat([newest_query(case.q[s][L - 1], case.k[s], case.v[s].bfloat16().float()).reshape(1, -1)
                      for s, L in enumerate(lengths)])
    # the far key decides its head's output: most of the weight lies on it
    assert all(float(want[s, (s % nkv) * 3 * d:(s % nkv) * 3 * d + d].mean()) > 4.5 for s in range(len(lengths)))
    cols = case.table.shape[1]
    assert cols == 128
    tickets = torch.zeros(o.mma_ticket_count(n, nq, nkv), dtype=torch.int32, device=DEV)
    for splits in (16, 22, 32, 43, 64, 86, 128):
        out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
        partial = torch.full((n * nq * splits * (d + 2),), float("nan"), device=DEV)
        for _ in range(2):  # (the tickets come back to zero: a second launch finds them so)
            o.attention_decode_tma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                                   nq, nkv, d, 0, 1.0 / math.sqrt(d), splits, partial, tickets)
        close(out, want, "bfloat16", f"decode attention by TMA, {splits} slices of a long context")
        assert int(tickets.abs().sum()) == 0
    o.check_status(DEV)
    # the plan: beyond 16 slices of four pages, the longest slices whose CTAs are all resident
    assert o.attention_decode_tma_plan(1, nq, nkv, d, 64, 128, DEV) == 16   # eight pages, 48 CTAs
    assert o.attention_decode_tma_plan(3, nq, nkv, d, 64, 128, DEV) == 16   # 144 CTAs, one to an SM
    assert o.attention_decode_tma_plan(4, nq, nkv, d, 64, 128, DEV) == 22   # six pages, two to an SM
    assert o.attention_decode_tma_plan(1, nq, nkv, d, 64, 256, DEV) == 32
    assert o.attention_decode_tma_plan(2, nq, nkv, d, 64, 256, DEV) == 43
    assert o.attention_decode_tma_plan(3, nq, nkv, d, 64, 256, DEV) == 0    # the ring kernel's
    assert o.attention_decode_tma_plan(1, nq, nkv, d, 64, 384, DEV) == 48   # 24,576 keys: eight pages
    assert o.attention_decode_tma_plan(1, nq, nkv, d, 64, 512, DEV) == 86   # 32,768 keys: six pages
    assert o.attention_decode_tma_plan(2, nq, nkv, d, 64, 512, DEV) == 0
    assert o.attention_decode_tma_plan(8, nq, nkv, d, 64, 64, DEV) == 11    # (as before at 4,096)


def test_attention_decode_fed_by_tma_with_more_ctas_than_two_per_sm():
    """Many sequences: more CTAs than two per SM (three fill an SM's registers, so the last
    of them start when the first have left); the same results."""
    o = ops()
    nq, nkv, d = 9, 3, 64
    rng = np.random.default_rng(3)
    lengths = [int(x) for x in rng.integers(1, 1000, size=40)] + [1000, 64, 65]
    case = PagedCase(lengths, [1] * len(lengths), nq, nkv, d, "bfloat16", seed=11)
    case.fill_cache()
    for s, L in enumerate(lengths):
        pg = int(case.table[s, (L - 1) // 64])
        case.k_cache[pg, :, (L - 1) % 64] = case.k[s][L - 1]
        case.v_cache[pg, :, (L - 1) % 64] = case.v[s][L - 1]
    pos, seq, q, _, _ = case.packed()
    n = pos.numel()
    splits = 4
    assert n * nkv * splits > 2 * o.sm_count(DEV)
    qd = q.reshape(n, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    want = torch.cat([P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(), 0)[L - 1:].reshape(1, -1)
                      for s, L in enumerate(lengths)])
    tickets = torch.zeros(o.mma_ticket_count(n, nq, nkv), dtype=torch.int32, device=DEV)
    out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    partial = torch.full((n * nq * splits * (d + 2),), float("nan"), device=DEV)
    o.attention_decode_tma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV), out,
                           nq, nkv, d, 0, 1.0 / math.sqrt(d), splits, partial, tickets)
    close(out, want, "bfloat16", "decode attention by TMA, 43 sequences")
    assert int(tickets.abs().sum()) == 0


def test_decode_attention_by_tma_finds_one_far_key():
    o = ops()
    nq, nkv, d, L, far = 8, 2, 64, 900, 77
    case = PagedCase([L], [1], nq, nkv, d, "bfloat16", seed=9, scale=0.3)
    for h in range(nkv):
        case.k[0][far, h] = case.q[0][L - 1, h * 4] * 30.0
    case.k[0] = case.k[0].bfloat16().float()
    case.v[0][far] = 7.0
    case.fill_cache()
    pg = int(case.table[0, (L - 1) // 64])
    case.k_cache[pg, :, (L - 1) % 64] = case.k[0][L - 1]
    case.v_cache[pg, :, (L - 1) % 64] = case.v[0][L - 1]
    pos, seq, q, _, _ = case.packed()
    qd = q.reshape(1, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    tickets = torch.zeros(o.mma_ticket_count(1, nq, nkv), dtype=torch.int32, device=DEV)
    for window, sees in ((0, True), (L - far, True), (L - far - 1, False)):
        for splits in (2, 5, 15):
            out = torch.empty(1, nq * d, dtype=torch.bfloat16, device=DEV)
            partial = torch.full((nq * splits * (d + 2),), float("nan"), device=DEV)
            o.attention_decode_tma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV),
                                   out, nq, nkv, d, window, 1.0 / math.sqrt(d), splits, partial, tickets)
            want = P.causal_attention(case.q[0], case.k[0], case.v[0].bfloat16().float(),
                                      window)[L - 1:].reshape(1, -1)
            close(out, want, "bfloat16", f"far key window {window} slices {splits}")
            lead = out.view(nq, d)[0::4].float()
            assert bool((lead > 6.5).all()) == sees


def test_tensor_core_decode_attention_finds_one_far_key():
    o = ops()
    nq, nkv, d, L, far = 8, 2, 64, 900, 77
    case = PagedCase([L], [1], nq, nkv, d, "bfloat16", seed=9, scale=0.3)
    for h in range(nkv):
        case.k[0][far, h] = case.q[0][L - 1, h * 4] * 30.0
    case.k[0] = case.k[0].bfloat16().float()
    case.v[0][far] = 7.0
    case.fill_cache()
    pg = int(case.table[0, (L - 1) // 64])
    case.k_cache[pg, :, (L - 1) % 64] = case.k[0][L - 1]
    case.v_cache[pg, :, (L - 1) % 64] = case.v[0][L - 1]
    pos, seq, q, _, _ = case.packed()
    qd = q.reshape(1, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    tickets = torch.zeros(o.mma_ticket_count(1, nq, nkv), dtype=torch.int32, device=DEV)
    for window, sees in ((0, True), (L - far, True), (L - far - 1, False)):
        for splits in (1, 5):
            out = torch.empty(1, nq * d, dtype=torch.bfloat16, device=DEV)
            partial = torch.empty(nq * splits * (d + 2), device=DEV)
            o.attention_decode_mma(qd, nq * d, kc, vc, pos.to(DEV), seq.to(DEV), case.table.to(DEV),
                                   out, nq, nkv, d, window, 1.0 / math.sqrt(d), splits, partial, tickets)
            want = P.causal_attention(case.q[0], case.k[0], case.v[0].bfloat16().float(),
                                      window)[L - 1:].reshape(1, -1)
            close(out, want, "bfloat16", f"far key window {window} splits {splits}")
            lead = out.view(nq, d)[0::4].float()
            assert bool((lead > 6.5).all()) == sees


@pytest.mark.parametrize("m", [17, 64, 128, 129, 300, 2048])
@pytest.mark.parametrize("n,k", [(8, 16), (64, 72), (130, 200), (576, 576), (960, 576), (515, 1536)])
def test_gemm_on_tcgen05(m, n, k):
    """Any M and N, K in steps of 8: tails are zero-filled on the way in and
    masked on the way out; bias, and the three output modes."""
    o = ops()
    assert o.gemm_tc_takes(m, n, k) and not o.gemm_tc_takes(m, n, k + 4) and not o.gemm_tc_takes(16, n, k)
    g = torch.Generator().manual_seed(m * 7 + n + k)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, generator=g)
    want = P.linear(a, w, bias)
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), out, o.STORE)
    close(out, want, "bfloat16", "tcgen05 store")
    out32 = torch.full((m, n), 7.0, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), None, out32, o.STORE_F32)
    close(out32, P.linear(a, w), "float32", "tcgen05 store f32")
    base = torch.randn(m, n, generator=g)
    acc = base.to(DEV).clone()
    o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), acc, o.ADD_F32)
    close(acc, base.double() + want, "float32", "tcgen05 add")
    o.check_status(DEV)


@pytest.mark.parametrize("m,n,k", [(2048, 1536, 64), (1500, 1290, 72), (2100, 1288, 136)])
def test_gemm_on_tcgen05_wide_tiles(m, n, k):
    """Enough 128-column tiles for every SM: the 128 x 128 tile shape, with outputs
    that leave by TMA (rows on 16-byte boundaries) and one that cannot."""
    o = ops()
    g = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, generator=g)
    want = P.linear(a, w, bias)
    out = torch.full((m, n), 7.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), out, o.STORE)
    close(out, want, "bfloat16", "tcgen05 wide store")
    base = torch.randn(m, n, generator=g)
    acc = base.to(DEV).clone()
    for _ in range(2):
        o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), acc, o.ADD_F32)
    close(acc, base.double() + 2 * want, "float32", "tcgen05 wide add twice")
    o.check_status(DEV)


@pytest.mark.parametrize("m,n,k", [(64, 2048, 8192), (33, 192, 2048 + 72), (130, 320, 4096), (17, 64, 2048)])
def test_gemm_on_tcgen05_adds_with_k_cut_among_ctas(m, n, k):
    """Few tiles and a long K: several CTAs share a tile, each a run of k-blocks; their sums
    meet in scratch and the one that arrives last adds them in the order of the runs, so two
    launches give the same bits.  One far column of K matters: a run left out would show."""
    o = ops()
    splits, floats, tiles = o.gemm_tc_splits(m, n, k, DEV)
    assert splits > 1 and floats == tiles * splits * 128 * 64 and tiles == -(-m // 128) * -(-n // 64)
    assert o.gemm_tc_splits(2048, n, k, DEV)[0] == 1 or n < 512  # many tiles: no split
    g = torch.Generator().manual_seed(m + n)
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    a[:, k - 5] = 3.0
    w[:, k - 5] = 1.0
    bias = torch.randn(n, generator=g)
    want = P.linear(a, w, bias)
    base = torch.randn(m, n, generator=g)
    scratch = torch.full((floats,), float("nan"), device=DEV)
    tickets = torch.zeros(tiles, dtype=torch.int32, device=DEV)
    outs = []
    for _ in range(2):
        acc = base.to(DEV).clone()
        o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), acc, o.ADD_F32, split_scratch=scratch, split_tickets=tickets)
        close(acc, base.double() + want, "float32", "tcgen05 add, K cut among CTAs")
        outs.append(acc)
    assert torch.equal(outs[0], outs[1]) and int(tickets.abs().sum()) == 0
    whole = base.to(DEV).clone()  # the same without scratch: one CTA a tile, one long float32 sum
    o.gemm_tc(a.to(DEV), w.to(DEV), bias.to(DEV), whole, o.ADD_F32)
    assert float((whole - outs[0]).abs().max()) < 2e-4
    o.check_status(DEV)


def test_gemm_on_tcgen05_many_k_blocks_reuse_every_stage():
    o = ops()
    g = torch.Generator().manual_seed(0)
    m, n, k = 256, 256, 64 * 23 + 8
    a = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    out = torch.empty(m, n, device=DEV)
    for _ in range(3):
        o.gemm_tc(a.to(DEV), w.to(DEV), None, out, o.STORE_F32)
    close(out, P.linear(a, w), "float32", "tcgen05 long k")
    o.check_status(DEV)


@pytest.mark.parametrize("nq,nkv,d", [(9, 3, 64), (2, 2, 64), (4, 1, 128)])
@pytest.mark.parametrize("window", [0, 70])
def test_prompt_attention_on_tensor_cores(nq, nkv, d, window):
    """Whole prompts and later chunks of unequal length in one packed batch."""
    o = ops()
    lengths, new = [70, 1, 200, 64, 333, 129], [70, 1, 5, 64, 200, 65]
    case = PagedCase(lengths, new, nq, nkv, d, "bfloat16", seed=d + nq)
    case.fill_cache()
    for s, L in enumerate(lengths):  # the step's own keys and values are stored already
        for t in range(L - new[s], L):
            pg = int(case.table[s, t // 64])
            case.k_cache[pg, :, t % 64] = case.k[s][t]
            case.v_cache[pg, :, t % 64] = case.v[s][t]
    pos, seq, q, _, _ = case.packed()
    n = pos.numel()
    qd = q.reshape(n, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    first, tiles, row = [], [], 0
    for i, c in enumerate(new):
        first.append(row)
        row += c
        tiles += [[i, q0] for q0 in range(0, c, 64)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    o.attention_prefill_mma(qd, nq * d, kc, vc, i32(tiles), i32(first),
                            i32([L - c for L, c in zip(lengths, new)]), i32(new), case.table.to(DEV),
                            out, nq, nkv, d, window, 1.0 / math.sqrt(d))
    r = 0
    for s, L in enumerate(lengths):
        full = P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(), window)
        close(out[r:r + new[s]], full[L - new[s]:].reshape(new[s], -1), "bfloat16", f"prompt attention seq {s}")
        r += new[s]


@pytest.mark.parametrize("nq,nkv", [(9, 3), (2, 2), (4, 1)])
@pytest.mark.parametrize("window", [0, 70])
@pytest.mark.parametrize("pad,sms", [(0, 1000), (24, 2), (0, 0)])
def test_prompt_attention_on_tcgen05(nq, nkv, window, pad, sms):
    """Head size 64 on the fifth-generation tensor cores: whole prompts and later
    chunks of unequal length in one packed batch, 128 queries per tile, more pages
    than the ring of stages holds, queries inside wider rows (``pad``); tiles cut
    into chunks of pages, merged by the last chunk to arrive (planned as for very many SMs), or whole (as for few)."""
    o = ops()
    d = 64
    lengths, new = [70, 1, 200, 64, 333, 129, 1500], [70, 1, 5, 64, 200, 65, 1500]
    case = PagedCase(lengths, new, nq, nkv, d, "bfloat16", seed=3 * nq + window)
    case.fill_cache()
    for s, L in enumerate(lengths):  # the step's own keys and values are stored already
        for t in range(L - new[s], L):
            pg = int(case.table[s, t // 64])
            case.k_cache[pg, :, t % 64] = case.k[s][t]
            case.v_cache[pg, :, t % 64] = case.v[s][t]
    pos, seq, q, _, _ = case.packed()
    n = pos.numel()
    stride = nq * d + pad
    assert o.attention_prefill_tc_takes(d, 64, stride) and not o.attention_prefill_tc_takes(128, 64, stride)
    qd = torch.full((n, stride), 3.0, dtype=torch.bfloat16, device=DEV)
    qd[:, :nq * d] = q.reshape(n, -1).bfloat16().to(DEV)
    kc, vc = case.k_cache.bfloat16().to(DEV), case.v_cache.bfloat16().to(DEV)
    starts = [L - c for L, c in zip(lengths, new)]
    first = [sum(new[:i]) for i in range(len(new))]
    units, slots = o.prefill_tc_plan(new, starts, window, nq, sms)
    assert (slots > 0) == (sms == 1000 and window == 0)  # the long prompt is cut only when SMs would idle
    covered = sorted((int(u[0]), int(u[1]), int(u[2]) & 0xffff) for u in units)
    assert len(set(covered)) == len(covered)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    partial = torch.full((max(slots, 1) * nq * o.PREFILL_TC_PARTIAL,), float("nan"), device=DEV)
    tickets = torch.zeros(max(slots, 1) * nq, dtype=torch.int32, device=DEV)
    out = torch.full((n, nq * d), 5.0, dtype=torch.bfloat16, device=DEV)
    for _ in range(2):  # the second launch finds the tickets as the first left them
        o.attention_prefill_tc(qd, stride, kc, vc, i32(units), partial if slots else None,
                               tickets if slots else None, i32(first), i32(starts), i32(new),
                               case.table.to(DEV), out, nq, nkv, d, window, 1.0 / math.sqrt(d))
    o.check_status(DEV)
    assert int(tickets.abs().sum()) == 0
    r = 0
    for s, L in enumerate(lengths):
        full = P.causal_attention(case.q[s], case.k[s], case.v[s].bfloat16().float(), window)
        close(out[r:r + new[s]], full[L - new[s]:].reshape(new[s], -1), "bfloat16", f"prompt attention seq {s}")
        r += new[s]


@pytest.mark.parametrize("m", [17, 128, 200])
@pytest.mark.parametrize("inter,k", [(100, 72), (1536, 576), (64, 64), (196, 136), (200, 64), (392, 72)])
def test_gemm_on_tcgen05_gated_epilogue(m, inter, k):
    o = ops()
    g = torch.Generator().manual_seed(m + inter)
    w = (torch.randn(2 * inter, k, generator=g) / math.sqrt(k) * 3).bfloat16()
    bias = torch.randn(2 * inter, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    y = P.linear(x, w, bias)
    out = torch.full((m, inter), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x.to(DEV), w.to(DEV), bias.to(DEV), out, o.GEMM_GATED)
    close(out, P.swiglu(y[:, :inter], y[:, inter:]), "bfloat16", "tcgen05 gated")
    o.check_status(DEV)


@pytest.mark.parametrize("nq,nkv,d,rotate", [(9, 3, 64, True), (2, 2, 128, True), (3, 1, 64, False),
                                             (4, 0, 128, True)])
def test_gemm_on_tcgen05_qkv_epilogue_rotates_and_stores(nq, nkv, d, rotate):
    o = ops()
    g = torch.Generator().manual_seed(nq * d)
    m, k, page = 150, 72, 64
    n = (nq + 2 * nkv) * d
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, generator=g)
    x = torch.randn(m, k, generator=g).bfloat16()
    # two sequences: positions 0..99 and 30..78, one padding row
    pos = torch.tensor(list(range(100)) + list(range(30, 79)) + [-1], dtype=torch.int32)
    seq = torch.tensor([0] * 100 + [1] * 49 + [0], dtype=torch.int32)
    table = torch.tensor([[5, 2], [7, 1]], dtype=torch.int32)
    kc = torch.zeros(8, max(nkv, 1), page, d, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    cos, sin = P.rope_tables(200, d, 10000.0)
    q_out = torch.full((m, nq * d), 9.0, dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(x.to(DEV), w.to(DEV), bias.to(DEV), q_out, o.GEMM_QKV, token_pos=pos.to(DEV),
              token_seq=seq.to(DEV), page_table=table.to(DEV) if nkv else None,
              cos=cos.float().to(DEV) if rotate else None, sin=sin.float().to(DEV) if rotate else None,
              k_cache=kc if nkv else None, v_cache=vc if nkv else None, heads=nq, kv_heads=nkv,
              head_dim=d, page_size=page)
    y = P.linear(x, w, bias).bfloat16().double()
    assert float((q_out[m - 1].float() - 9.0).abs().max()) == 0  # padding row untouched
    valid = pos >= 0
    p_idx = pos[valid].long()
    c, s = (cos[p_idx], sin[p_idx]) if rotate else (torch.ones(len(p_idx), d // 2).double(),
                                                    torch.zeros(len(p_idx), d // 2).double())
    heads = y[valid].view(-1, nq + 2 * nkv, d)
    close(q_out[:m - 1].view(-1, nq, d), P.rope_rotate_half(heads[:, :nq], c, s), "bfloat16", "q")
    if nkv:
        rk = P.rope_rotate_half(heads[:, nq:nq + nkv], c, s)
        for i in (0, 63, 64, 99, 100, 148):
            pg = int(table[int(seq[i]), int(pos[i]) // page])
            close(kc[pg, :, int(pos[i]) % page], rk[i], "bfloat16", "k")
            close(vc[pg, :, int(pos[i]) % page], heads[i, nq + nkv:], "bfloat16", "v")
        assert int((kc.float().abs().sum(-1) > 0).sum()) == 149 * nkv
    o.check_status(DEV)
