"""The schedules that the benchmark times, held to the plain implementation logit by
logit: decoding through ``GraphDecoder`` (the captured step with programmatic dependent
launches, the fused head and pick, the tensor-core decode attention with its slices)
at contexts that end at 4,096, with 8 rows (11 slices of up to 384 keys) and with 64 rows of
unequal contexts (few slices, the launch shape with three pages in flight).

The model is narrow (width 128, two layers) so that the float64 oracle stays cheap,
but its attention has the benchmark's own shape - 9 query heads on 3 key/value heads of
64 - so that the slice and stage choices are the benchmark's.  Query and key
projections are scaled up so that a few far keys carry each softmax: a slice that was
lost or read from a wrong page would move the logits far beyond the bound."""
import random

import pytest
import torch

import plain_llama as P
from helpers import check_logits

pytestmark = pytest.mark.gpu
CFG = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=512, hidden_size=128,
           intermediate_size=256, num_hidden_layers=2, num_attention_heads=9, num_key_value_heads=3,
           head_dim=64, max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=100000.0,
           hidden_act="silu", tie_word_embeddings=True, attention_bias=False, torch_dtype="bfloat16")
CONTEXT = 4096
STEPS = 5


def build(dtype, max_rows):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    spec = config_from_dict(CFG).to_spec()
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=4096, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    for name in tensors:
        if name.endswith(("q_proj.weight", "k_proj.weight")):
            tensors[name] = tensors[name] * 3.0  # scores nine times as wide: peaked softmax
    bf = dtype == "bfloat16"
    plain = {k: (v.to(torch.bfloat16).float() if bf else v.float()) for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype=dtype, max_tokens=max_rows * (CONTEXT + 64),
                              max_slots=max_rows)
    return engine, plain


def decode_rows(engine, ends, rng, chains=None):
    """Fill the cache up to ``end - STEPS`` tokens per row, then STEPS graph launches as
    bench.py makes them.  Returns per row the whole sequence (the picks appended) and
    the logits of each launch."""
    from nnis_b200.engine import SequenceStep
    from nnis_b200.engine.decode import GraphDecoder
    rows = len(ends)
    slots = [engine.acquire_slot() for _ in range(rows)]
    seqs = [[rng.randrange(CFG["vocab_size"]) for _ in range(end - STEPS + 1)] for end in ends]
    fed = [0] * rows
    while any(fed[r] < len(seqs[r]) - 1 for r in range(rows)):
        batch, budget = [], 16384
        for r in range(rows):
            n = min(2048, len(seqs[r]) - 1 - fed[r], budget)
            if n > 0:
                batch.append(SequenceStep(slots[r], seqs[r][fed[r]:fed[r] + n], []))
                fed[r] += n
                budget -= n
        engine.step(batch)
    dec = GraphDecoder(engine, rows, CONTEXT, want_logits=True, chains=chains)
    engine.cache.reserve(slots, list(ends))
    for r in range(rows):
        dec.set_row(r, slots[r], seqs[r][-1], len(seqs[r]) - 1)
    dec.capture()
    logits = []
    for _ in range(STEPS):
        dec.launch()
        logits.append(dec.logits.clone())
        for r, t in enumerate(dec.picked.tolist()):
            seqs[r].append(t)
    torch.cuda.synchronize()
    engine.check_status()
    engine.cache.commit(slots, list(ends))
    for s in slots:
        engine.release_slot(s)
    return seqs, torch.stack(logits).cpu(), dec


def check_rows(seqs, logits, ends, plain, dtype, which, what):
    bf = dtype == "bfloat16"
    for r in which:
        want = P.forward(CFG, plain, seqs[r][:ends[r]], emulate_bf16=bf)[ends[r] - STEPS:ends[r]]
        check_logits(logits[:, r].numpy(), want, dtype, f"{what} row {r} (context {ends[r]})")
        # the picks that the graph fed itself are the oracle's greedy tokens wherever
        # the oracle's own margin is clear
        for t in range(STEPS):
            top = torch.topk(want[t], 2).values
            if float(top[0] - top[1]) > 0.05 * max(1.0, float(want[t].abs().max())):
                assert seqs[r][ends[r] - STEPS + 1 + t] == int(torch.argmax(want[t])), (what, r, t)


@pytest.mark.parametrize("dtype,chains", [("bfloat16", None), ("bfloat16", 2), ("float32", None)])
def test_eight_rows_decode_to_context_4096_through_the_graph(dtype, chains):
    """``chains``: None is what the benchmark launches (one chain of all rows); 2 deals
    the rows to two chains that run side by side in the graph."""
    engine, plain = build(dtype, 8)
    ends = [4096, 4090, 3000, 2049, 300, 64 + STEPS, 70, 4096]
    seqs, logits, dec = decode_rows(engine, ends, random.Random(8), chains)
    if dtype == "bfloat16":  # 11 slices of up to 384 keys, every page of a slice in shared memory at once
        from nnis_b200.csrc import ops
        rows = dec.chains[0][1] - dec.chains[0][0]
        assert ops.attention_decode_tma_plan(rows, 9, 3, 64, 64, dec.cols, engine.device, len(dec.chains)) == 11
        # (with few enough sequences: 16 slices of 256 keys)
        assert ops.attention_decode_tma_plan(2, 9, 3, 64, 64, dec.cols, engine.device) == 16
    check_rows(seqs, logits, ends, plain, dtype, [0, 3, 5, 7], f"8 rows {dtype}")
    assert engine.cache.usage()["pages_held"] == [0]


@pytest.mark.parametrize("chains", [None, 4])
def test_sixty_four_rows_of_unequal_context_decode_through_the_graph(chains):
    engine, plain = build("bfloat16", 64)
    rng = random.Random(64)
    ends = [4096, 2500, 6 + STEPS, 4096] + [rng.randrange(STEPS + 1, 4097) for _ in range(59)] + [4095]
    seqs, logits, dec = decode_rows(engine, ends, rng, chains)
    from nnis_b200.csrc import ops
    mixer = engine.model.blocks[0].mixer
    rows = dec.chains[0][1] - dec.chains[0][0]
    # too many CTAs to be resident together: the slices stream through the ring
    assert ops.attention_decode_tma_plan(rows, 9, 3, 64, 64, dec.cols, engine.device, len(dec.chains)) == 0
    splits, stages = mixer._decode_shape(dec.ctx, rows * 3, 64)
    assert 1 < splits <= 4, (splits, stages)  # few long slices
    if len(dec.chains) == 1:
        assert stages == 3  # the launch shape with three pages in flight, one wave of 576 CTAs
    check_rows(seqs, logits, ends, plain, "bfloat16", [0, 1, 2, 63], "64 rows")
    assert engine.cache.usage()["pages_held"] == [0]


def test_eighty_rows_decode_through_the_graph():
    """More rows than the kernel whose CTAs hold all rows takes (64): five tiles of rows in the
    kernel over tiles of rows, and the head as norm, tcgen05 product and pick."""
    engine, plain = build("bfloat16", 80)
    from nnis_b200.csrc import ops
    hidden, inter = CFG["hidden_size"], CFG["intermediate_size"]
    for n, k, epi, normed in [((9 + 6) * 64, hidden, ops.EPI_QKV, True), (hidden, 9 * 64, ops.EPI_ADD_F32, False),
                              (2 * inter, hidden, ops.EPI_GATED, True), (hidden, inter, ops.EPI_ADD_F32, False)]:
        assert ops.gemv_kind(80, n, k, epi, engine.device, normed) == 2
        assert ops.gemv_kind(80, n, k, epi, engine.device, normed, rows_kernel=False) == 0
    rng = random.Random(80)
    ends = [1500, 6 + STEPS, 1499] + [rng.randrange(STEPS + 1, 1501) for _ in range(76)] + [777]
    seqs, logits, dec = decode_rows(engine, ends, rng)
    check_rows(seqs, logits, ends, plain, "bfloat16", [0, 1, 2, 40, 79], "80 rows")
    assert engine.cache.usage()["pages_held"] == [0]
