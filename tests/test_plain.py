"""The plain implementation itself: closed forms and fixed points taken from
NNIS's own tests (no GPU)."""
import math

import torch

import plain_llama as P
from helpers import TINY_A, TINY_B, load_plain_weights, make_model, read_config_json


def test_attention_closed_forms():
    # crates/nnis-model/src/kernels.rs:525-558: two keys, scores 0 and 1 -> e/(e+1)
    d = 16
    q = torch.zeros(2, 1, d, dtype=torch.float64)
    q[1, 0, 0] = math.sqrt(d)
    k = torch.zeros(2, 1, d)
    k[1, 0, 0] = 1.0
    v = torch.zeros(2, 1, d)
    v[0, 0, 0], v[1, 0, 0] = 0.0, 10.0
    out = P.causal_attention(q, k, v)
    assert abs(float(out[1, 0, 0]) - 10 * math.e / (math.e + 1)) < 1e-5
    assert float(out[0, 0, 0]) == 0.0  # the first query sees only the first key


def test_window_hides_old_keys():
    T, d = 6, 16
    q = torch.zeros(T, 1, d)
    k = torch.zeros(T, 1, d)
    v = torch.arange(T, dtype=torch.float32)[:, None, None].expand(T, 1, d).clone()
    out = P.causal_attention(q, k, v, window=2)
    assert torch.allclose(out[:, 0, 0].float(), torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5, 4.5]))


def test_gqa_maps_query_heads_to_kv_heads():
    T, d = 1, 16
    q = torch.zeros(T, 4, d)
    k = torch.zeros(T, 2, d)
    v = torch.zeros(T, 2, d)
    v[0, 0, :], v[0, 1, :] = 1.0, 2.0
    out = P.causal_attention(q, k, v)
    assert out[0, :, 0].tolist() == [1.0, 1.0, 2.0, 2.0]


def test_rope_is_a_rotation_and_identity_at_zero():
    cos, sin = P.rope_tables(5, 16, 10000.0)
    x = torch.randn(5, 3, 16)
    y = P.rope_rotate_half(x, cos, sin)
    assert torch.allclose(y[0].float(), x[0])
    assert torch.allclose(y.norm(dim=-1).float(), x.norm(dim=-1), atol=1e-5)
    assert abs(float(cos[1, 0]) - math.cos(1.0)) < 1e-6


def test_rmsnorm_and_swiglu_values():
    x = torch.tensor([[3.0, 4.0]])
    y = P.rms_norm(x, torch.tensor([1.0, 2.0]), 1e-6)
    assert torch.allclose(y.float(), torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5), atol=1e-5)
    g = torch.tensor([0.0, 1.0])
    assert torch.allclose(P.swiglu(g, torch.tensor([5.0, 2.0])).float(),
                          torch.tensor([0.0, 2.0 / (1 + math.exp(-1.0))]))


def test_zero_projections_give_zero_logits_and_token_zero(tmp_path):
    # crates/nnis-model/src/runtime.rs:1262-1274
    d = make_model(str(tmp_path / "m"), TINY_A, 0)
    w = {k: torch.zeros_like(v) for k, v in load_plain_weights(d, False).items()}
    cfg = read_config_json(d)
    logits = P.forward(cfg, w, [1, 2, 3])
    assert float(logits.abs().max()) == 0.0
    assert P.greedy_generate(cfg, w, [1, 2, 3], 2) == [0, 0]


def test_argmax_ties_go_to_the_lower_index():
    assert P.argmax_lowest(torch.tensor([1.0, 4.0, 4.0, -2.0])) == 1


def test_splitmix_frozen_sequence():
    # crates/nnis-model/src/sampling.rs:326-333
    rng = P.PlainSplitMix64(42)
    assert [P.plain_sample([0.0] * 4, rng) for _ in range(10)] == [2, 0, 1, 1, 0, 3, 0, 3, 1, 2]


def test_prefix_of_a_sequence_has_the_same_logits(tmp_path):
    d = make_model(str(tmp_path / "m"), TINY_B, 3)
    w, cfg = load_plain_weights(d, False), read_config_json(d)
    tokens = [5, 9, 400, 3, 77, 12, 300]
    full = P.forward(cfg, w, tokens)
    part = P.forward(cfg, w, tokens[:4])
    assert torch.allclose(full[:4], part, atol=1e-9)
    assert float(full.abs().max()) > 0.1  # healthy weights give logits of some size
    rounded = P.forward(cfg, load_plain_weights(d, True), tokens, emulate_bf16=True)
    assert 0 < float((rounded - full).abs().max()) < 0.2 * float(full.abs().max())


def test_bfloat16_rounding_is_to_nearest_even():
    """The cases NNIS pins for its float32 -> bfloat16 conversion
    (crates/nnis-rt/src/bf16.rs:32-49), for the conversion that the loader, the
    random-weights mode and this file's bfloat16 emulation use."""
    import numpy as np

    def rounded(bits=None, value=None):
        x = torch.tensor(np.array([bits], dtype=np.uint32).view(np.float32)) if bits is not None \
            else torch.tensor([value], dtype=torch.float32)
        return float(x.bfloat16().float())

    one = int(np.array([1.0], dtype=np.float32).view(np.uint32)[0])
    assert rounded(value=1.0) == 1.0 and rounded(value=0.0) == 0.0 and rounded(value=-2.5) == -2.5
    assert rounded(bits=one + 0x8000) == 1.0            # an exact tie keeps the even mantissa
    assert rounded(bits=one + 0x8001) == 1.0 + 2.0 ** -7  # just past the tie goes up
    assert rounded(bits=one + 0x10000 + 0x8000) == 1.0 + 2.0 ** -6  # a tie above an odd mantissa goes up
    assert rounded(value=float("inf")) == float("inf")
    assert math.isnan(rounded(value=float("nan")))
