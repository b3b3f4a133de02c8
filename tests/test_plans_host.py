"""Work lists that the host makes for kernels: checked without a GPU."""


def test_prompt_attention_plan_cuts_tiles_without_empty_chunks():
    from nnis_b200.csrc import ops as o
    for counts, starts, window in [([2048], [0], 0), ([700, 3], [100, 0], 0), ([5000], [0], 300),
                                   ([129], [64 * 37 + 5], 0)]:
        for sms in (1, 148, 10 ** 6):
            units, slots = o.prefill_tc_plan(counts, starts, window, 9, sms)
            per_tile = {}
            for s, q0, z, slot in units.tolist():
                per_tile.setdefault((s, q0), []).append((z & 0xffff, z >> 16, slot))
            assert sorted(per_tile) == sorted((i, q0) for i, c in enumerate(counts) for q0 in range(0, c, 128))
            used = 0
            for (s, q0), chunks in per_tile.items():
                n = chunks[0][1]
                assert sorted(c for c, _, _ in chunks) == list(range(n)) and all(k == n for _, k, _ in chunks)
                rows = min(128, counts[s] - q0)
                pos0 = starts[s] + q0
                lo = max(0, pos0 - window + 1) if window else 0
                pages = (pos0 + rows - 1) // 64 - lo // 64 + 1
                assert (n - 1) * (-(-pages // n)) < pages
                used += n if n > 1 else 0
                if n > 1:  # the chunks of a tile share its first scratch slot; tiles do not overlap
                    assert len({slot for _, _, slot in chunks}) == 1
            assert used == slots
            firsts = sorted((chunks[0][2], chunks[0][1]) for chunks in per_tile.values() if chunks[0][1] > 1)
            assert all(a[0] + a[1] <= b[0] for a, b in zip(firsts, firsts[1:]))


def test_decode_attention_slices_fill_waves():
    """The slices of a decode step's key range: as many CTAs as run together, fewer
    waves before shorter slices, never below 256 keys a slice."""
    import torch
    from nnis_b200.engine.context import StepContext
    empty = torch.zeros(0, dtype=torch.int32)

    def pick(ctas, context, resident=444):
        ctx = StepContext(n_tokens=0, n_seqs=0, tokens=empty, token_pos=empty, token_seq=empty,
                          seq_slots=empty, page_tables=[], workspace=None, decode=True, max_context=context)
        return ctx.decode_splits(ctas, resident, 64)

    # one wave where the groups divide the resident CTAs: batch 8, 16, 32, 64 of three kv heads
    assert [pick(c, 4096) for c in (24, 48, 96, 192)] == [16, 9, 4, 2]
    # a wave that would stay 42 % empty is cut further: 256 groups take three slices, two waves
    assert pick(256, 4096) == 3
    # more groups than resident CTAs: no slices at all
    assert pick(2048, 4096) == 1
    for ctas in (1, 3, 40, 100, 443, 445, 5000):
        for context in (1, 64, 300, 4096, 8192, 100000):
            s = pick(ctas, context)
            assert 1 <= s <= 64 and (s - 1) * 256 < max(context, 1)
    # short contexts are not cut
    assert pick(3, 200) == 1 and pick(3, 512) == 2


def test_prompt_attention_plan_takes_the_shortest_chunks_that_fit_one_wave():
    """One prompt of 2,048 tokens, nine heads, 148 SMs: chunks of 12 pages are the longest
    that give enough CTAs, chunks of 11 the shortest with which two CTAs to an SM still hold
    them all (a CTA walks its pages one after another: the longest chunk ends last)."""
    from nnis_b200.csrc import ops as o
    units, _ = o.prefill_tc_plan([2048], [0], 0, 9, 148)
    chunks = {}
    for s, q0, z, slot in units.tolist():
        chunks[q0] = z >> 16
    assert len(units) * 9 <= 2 * 148 and len(units) == 32
    assert chunks[2048 - 128] == 3 and chunks[0] == 1 and chunks[128 * 10] == 2  # 32, 2 and 22 pages
    # 4,096 tokens: a tile a CTA fills a wave; 1,024: chunks of eight pages as before
    assert len(o.prefill_tc_plan([4096], [0], 0, 9, 148)[0]) == 32
    assert max(z >> 16 for _, _, z, _ in o.prefill_tc_plan([1024], [0], 0, 9, 148)[0].tolist()) == 2


def test_bench_sums_a_traced_step_per_kernel():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    big = 1 << 62
    # per launch: begin, end, first and last past the wait, marks
    rows = [[1000, 4000, 1500, 2000, big, 0, big, 0], [3500, 9000, 4500, 5000, big, 0, big, 0],
            [8000, 9500, big, 0, big, 0, big, 0]]
    got = bench.kernel_times(["a", "b", "a"], rows)
    assert got["a"] == {"launches": 2, "us": 3.5} and got["b"] == {"launches": 1, "us": 4.0}
    assert got["step"] == {"launches": 3, "us": 8.5}


def test_a_begun_norm_is_handed_on_once_and_only_to_the_block_that_owns_it():
    """What a part leaves of a norm in the step's context: taken by the norm it names,
    dropped when another norm asks first, never seen twice; and the prenorm arrangement
    offers a norm only where the part after it says it takes it."""
    import torch
    from nnis_b200.engine.context import StepContext
    from nnis_b200.parts.base import SharedNorm, begin_norm
    from nnis_b200.parts.block import PreNormBlock
    empty = torch.zeros(0, dtype=torch.int32)

    class Space:
        def get(self, name, shape, dtype):
            return torch.zeros(shape, dtype=dtype)

    ctx = StepContext(n_tokens=0, n_seqs=0, tokens=empty, token_pos=empty, token_seq=empty,
                      seq_slots=empty, page_tables=[], workspace=Space(), decode=True, max_context=1)

    class Norm:
        kind = "rmsnorm"
        weight = torch.ones(16)
        eps = 1e-5

    a, b = Norm(), Norm()
    assert begin_norm(ctx, 3, 16) is None and ctx.shared_norm is None  # no block asked for it
    ctx.emit_for = a
    x, weight, shares = begin_norm(ctx, 3, 16)
    assert x.shape == (3, 16) and x.dtype == torch.bfloat16 and shares.shape == (3, 2) and weight is a.weight
    assert isinstance(ctx.shared_norm, SharedNorm)
    assert ctx.take_shared_norm(a).x is x and ctx.take_shared_norm(a) is None
    begin_norm(ctx, 3, 16)
    assert ctx.take_shared_norm(b) is None and ctx.take_shared_norm(a) is None  # dropped, not kept
    assert begin_norm(ctx, 3, 12) is None  # a width that is no multiple of eight
    other = Norm()
    other.kind = "layernorm"
    ctx.emit_for = other
    assert begin_norm(ctx, 3, 16) is None

    # the arrangement: which norm each part is told about, and what reaches the parts
    calls = []

    class Mixer:
        def forward(self, x, ctx, residual, cache):
            calls.append(("mixer", ctx.emit_for))

    class SharingFfn:
        def shares_norm(self, norm, ctx, n):
            return True

        def forward(self, x, ctx, residual):
            calls.append(("ffn", ctx.emit_for))

        def forward_shared(self, begun, residual, ctx):
            calls.append(("ffn shared", begun.norm))

    class PlainNorm(Norm):
        def forward(self, hidden, out, rows=None):
            pass

    block = PreNormBlock.__new__(PreNormBlock)
    block.dtype = torch.bfloat16
    block.mixer_norm, block.ffn_norm = PlainNorm(), PlainNorm()
    block.mixer, block.ffn = Mixer(), SharingFfn()
    ctx.emit_for = None
    ctx.next_norm = a
    hidden = torch.zeros(3, 16)
    assert block.first_shared_norm(ctx, 3) is None  # this mixer takes no begun norm
    block.forward(hidden, ctx, None)
    # the mixer was told of the feed-forward's norm and left nothing: the norm ran whole;
    # the feed-forward was told of the next block's first norm
    assert calls == [("mixer", block.ffn_norm), ("ffn", a)] and ctx.emit_for is None

    class EmittingMixer(Mixer):
        def forward(self, x, ctx, residual, cache):
            begin_norm(ctx, 3, 16)

    calls.clear()
    block.mixer = EmittingMixer()
    block.forward(hidden, ctx, None)
    assert calls == [("ffn shared", block.ffn_norm)] and ctx.shared_norm is None


def test_decode_attention_by_tma_takes_the_longest_slices_that_stay_resident():
    """The slices of the decode attention whose pages are all in shared memory at once, on a
    device of 148 SMs that holds three CTAs of four pages, two of five or six, one of seven or
    eight to an SM (head size 64): four pages; six where four make more CTAs than two to an
    SM; beyond 16 slices, eight or six where those CTAs are all resident; else not this kernel."""
    from nnis_b200.csrc.ops import tma_slices
    fit = lambda pages: 3 if pages <= 4 else 2 if pages <= 6 else 1

    def slices(sequences, pages, kv_heads=3, fixed=0):
        return tma_slices(sequences * kv_heads, pages, 148, 8, fit, fixed)

    # context 4,096 (64 pages): one to six sequences 16 slices of four pages, seven and eight
    # 11 slices of six (two CTAs to an SM), nine 16 of four again (297 CTAs of six pages are one too
    # many for two to an SM; 432 of four fit three to an SM), ten and more none
    assert [slices(n, 64) for n in (1, 2, 6, 7, 8, 9)] == [16, 16, 16, 11, 11, 16]
    assert slices(10, 64) == 0 and slices(64, 64) == 0
    # short contexts: one slice, many sequences
    assert slices(1, 1) == 1 and slices(40, 4) == 1 and slices(200, 4) == 0
    # beyond 16 slices of four pages: eight pages one to an SM, six pages two to an SM
    assert slices(1, 128) == 16 and slices(3, 128) == 16 and slices(4, 128) == 22
    assert slices(1, 256) == 32 and slices(2, 256) == 43 and slices(3, 256) == 0
    assert slices(1, 384) == 48 and slices(1, 512) == 86 and slices(2, 512) == 0
    # never more than 128 slices, never more than eight pages a slice
    assert slices(1, 1024) == 0 and slices(1, 1000, kv_heads=1) == 125 and slices(1, 1025, kv_heads=1) == 0
    # a fixed slice length is taken if its CTAs are resident
    assert slices(8, 64, fixed=4) == 16 and slices(8, 64, fixed=8) == 0 and slices(2, 64, fixed=8) == 8
    for n in (1, 2, 3, 5, 8, 13, 40):
        for pages in (1, 3, 16, 17, 63, 64, 65, 100, 128, 129, 255, 256, 400, 512, 700):
            s = slices(n, pages)
            if s:
                per = -(-pages // s)
                assert 1 <= s <= 128 and per <= 8 and s * per >= pages
                assert n * 3 * s <= 148 * fit(per)


def _ops_with_the_library():
    """The kernels' library holds the rules of which kernel takes which product as plain host
    functions; they need no GPU, only the library (built with nvcc at first use)."""
    import pytest
    from nnis_b200.csrc import ops
    try:
        ops._lib()
    except Exception as e:  # no compiler here
        pytest.skip(f"the kernels' library is not built here: {e}")
    return ops


def test_which_kernel_takes_the_projections_of_a_decode_step():
    """On 148 SMs, for the SmolLM2 shapes: 2 the kernel over tiles of rows, 1 the kernel whose
    CTAs hold all rows, 0 neither (norm kernel and tensor-core product); and where the norm
    before QKV and before gate/up can be shared out between the projections around it."""
    o = _ops_with_the_library()

    def plans(H, inter, nq, nkv, d, m):
        qkv = (nq + 2 * nkv) * d
        return dict(qkv=o.gemv_kind(m, qkv, H, o.EPI_QKV, None, True),
                    qkv_shares=o.gemv_kind(m, qkv, H, o.EPI_QKV, shared_norm=True) == 2,
                    out=o.gemv_kind(m, H, nq * d, o.EPI_ADD_F32),
                    gate_up=o.gemv_kind(m, 2 * inter, H, o.EPI_GATED, None, True),
                    gate_up_shares=o.gemv_kind(m, 2 * inter, H, o.EPI_GATED, shared_norm=True) == 2,
                    down=o.gemv_kind(m, H, inter, o.EPI_ADD_F32), down_slices=o.gemv_slices(m, H, inter))

    small, middle, large = (576, 1536, 9, 3, 64), (960, 2560, 15, 5, 64), (2048, 8192, 32, 32, 64)
    # the benchmark's shape: everything over tiles of rows up to 64 rows, both norms shared
    for m in (1, 8, 16, 48, 64):
        assert plans(*small, m) == dict(qkv=2, qkv_shares=True, out=2, gate_up=2, gate_up_shares=True,
                                        down=2, down_slices=1), m
    # at 128 rows gate/up has more CTAs than are resident at once
    p = plans(*small, 128)
    assert (p["qkv"], p["out"], p["down"], p["gate_up"], p["gate_up_shares"]) == (2, 2, 2, 0, False)
    # the 360M shape: the same up to 16 rows, its down projection in two slices of K;
    # from 48 rows on gate/up (640 units) leaves the kernel over tiles of rows and shares no norm
    for m in (1, 8, 16):
        assert plans(*middle, m) == dict(qkv=2, qkv_shares=True, out=2, gate_up=2, gate_up_shares=True,
                                         down=2, down_slices=2), m
    for m in (48, 64):
        p = plans(*middle, m)
        assert (p["qkv"], p["qkv_shares"], p["gate_up"], p["gate_up_shares"]) == (2, True, 1, False), m
    # the 1.7B shape: rows of 2,048 are longer than a warp's share of x in registers, so the
    # norm stays in the prologue of the kernel whose CTAs hold all rows, and nothing is shared;
    # the down projection (K = 8,192) runs in four slices of K
    for m in (1, 8, 16):
        p = plans(*large, m)
        assert (p["qkv"], p["qkv_shares"], p["gate_up"], p["gate_up_shares"]) == (1, False, 1, False), m
        assert (p["out"], p["down"], p["down_slices"]) == (2, 1, 4), m
    # what no decode kernel takes: more than 128 rows, K off a multiple of 16, N off a multiple of 8
    assert o.gemv_kind(129, 576, 576, o.EPI_ADD_F32) == 0 and o.gemv_kind(8, 576, 568, o.EPI_ADD_F32) == 0
    assert o.gemv_kind(8, 572, 576, o.EPI_ADD_F32) == 0
    # a shared norm ends only in the QKV and the gated epilogue
    assert o.gemv_kind(8, 576, 576, o.EPI_STORE, shared_norm=True) == 0
    # the adding tensor-core product cuts a long K among CTAs only where tiles are few
    assert o.gemm_tc_splits(64, 2048, 8192)[0] == 4 and o.gemm_tc_splits(2048, 576, 1536)[0] == 1
