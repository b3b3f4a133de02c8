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
