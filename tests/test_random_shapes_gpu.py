"""Seeded random Llama shapes with head sizes 64 and 128 (the sizes the tensor-core
kernels take) through the engine against the plain implementation: odd widths,
grouped / multi-head / multi-query attention, biases, tied and separate heads,
prompts of unequal length in one step, then single tokens."""
import random

import pytest
import torch

import plain_llama as P
from helpers import check_logits

pytestmark = pytest.mark.gpu


def random_config(rng):
    d = rng.choice([64, 64, 128])
    nkv = rng.choice([1, 2, 3, 5])
    nq = nkv * rng.choice([1, 2, 3])
    return dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=rng.choice([300, 515, 1000]),
                hidden_size=rng.choice([72, 200, 256, 328, 576]), intermediate_size=rng.choice([96, 200, 392, 1000]),
                num_hidden_layers=2, num_attention_heads=nq, num_key_value_heads=nkv, head_dim=d,
                max_position_embeddings=2048, rms_norm_eps=rng.choice([1e-5, 1e-6]),
                rope_theta=rng.choice([10000.0, 100000.0]), hidden_act="silu",
                tie_word_embeddings=rng.choice([True, False]), attention_bias=rng.choice([True, False]),
                torch_dtype="float32")


@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_shape(seed, dtype):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    rng = random.Random(seed)
    cfg = random_config(rng)
    spec = config_from_dict(cfg).to_spec()
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=seed, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    bf = dtype == "bfloat16"
    w = {k: (v.to(torch.bfloat16).float() if bf else v.float()) for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype=dtype, max_tokens=64 * 40, max_slots=4)
    lens = [rng.choice([3, 64, 129, 300, 700]), rng.choice([1, 65, 200])]
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n + 3)] for n in lens]
    want = [P.forward(cfg, w, t, bf) for t in seqs]
    slots = [engine.acquire_slot() for _ in seqs]
    picks = [[0, n - 1] for n in lens]
    got = engine.step([SequenceStep(s, t[:n], p) for s, t, n, p in zip(slots, seqs, lens, picks)])
    check_logits(got.cpu().numpy(), torch.cat([x[p] for x, p in zip(want, picks)]), dtype, f"prompts of {cfg}")
    for k in range(3):
        got = engine.step([SequenceStep(s, [t[n + k]], [0]) for s, t, n in zip(slots, seqs, lens)])
        check_logits(got.cpu().numpy(), torch.stack([x[n + k] for x, n in zip(want, lens)]), dtype,
                     f"token {k} of {cfg}")
    engine.check_status()
    engine.cache.check()


@pytest.mark.parametrize("batch", [1, 8, 24, 64])
def test_wide_layers_decode_with_long_rows_of_k(batch):
    """A layer as wide as the 1.7B shape (hidden 2,048, intermediate 8,192, 32 heads of 64):
    the decode projections stream K in chunks there, and the down projection adds slice by
    slice; with 64 rows the tcgen05 products run, the down projection with K cut among the
    CTAs of a tile; prompts, then single tokens of a batch, against the plain implementation."""
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=520, hidden_size=2048,
               intermediate_size=8192, num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=32,
               max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=130000.0, hidden_act="silu",
               tie_word_embeddings=True, attention_bias=False, torch_dtype="bfloat16")
    spec = config_from_dict(cfg).to_spec()
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=5, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    w = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype="bfloat16", max_tokens=64 * batch * 2, max_slots=batch)
    if batch == 64:
        from nnis_b200.csrc import ops
        assert ops.gemm_tc_splits(batch, 2048, 8192, engine.device)[0] == 4
        assert not ops.gemv_pays(batch, 2048, 8192, ops.EPI_ADD_F32, engine.device)
    rng = random.Random(batch)
    lens = [rng.choice([2, 5, 9]) for _ in range(batch)]
    seqs = [[rng.randrange(cfg["vocab_size"]) for _ in range(n + 2)] for n in lens]
    checked = seqs[:3]  # the plain implementation is slow at this width
    want = [P.forward(cfg, w, t, True) for t in checked]
    slots = [engine.acquire_slot() for _ in seqs]
    got = engine.step([SequenceStep(s, t[:n], [n - 1]) for s, t, n in zip(slots, seqs, lens)])
    check_logits(got.cpu().numpy()[:len(checked)], torch.stack([x[n - 1] for x, n in zip(want, lens)]),
                 "bfloat16", "wide prompts")
    for k in range(2):
        got = engine.step([SequenceStep(s, [t[n + k]], [0]) for s, t, n in zip(slots, seqs, lens)])
        check_logits(got.cpu().numpy()[:len(checked)], torch.stack([x[n + k] for x, n in zip(want, lens)]),
                     "bfloat16", f"wide token {k}")
    engine.check_status()
    engine.cache.check()
