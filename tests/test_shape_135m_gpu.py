"""The SmolLM2-135M shape with random weights: the engine's float32 and bfloat16
logits against the plain float64 implementation, a prompt in one step and its
last tokens one by one.  The shape comes from a config.json like any other; only
this file knows its numbers."""
import random

import pytest
import torch

import plain_llama as P
from helpers import TraceBuilder, check_logits, load_plain_weights, make_model, read_config_json, read_step

pytestmark = pytest.mark.gpu

SHAPE_135M = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=49152,
                  hidden_size=576, intermediate_size=1536, num_hidden_layers=30,
                  num_attention_heads=9, num_key_value_heads=3, max_position_embeddings=8192,
                  rms_norm_eps=1e-5, rope_theta=100000.0, hidden_act="silu",
                  tie_word_embeddings=True, attention_bias=False, torch_dtype="float32")


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    return make_model(str(tmp_path_factory.mktemp("shape135m")), SHAPE_135M, seed=135)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_135m_shape_matches_the_plain_implementation(model_dir, dtype, tmp_path):
    from nnis_b200.engine import Engine
    from nnis_b200.engine.replay import replay
    rng = random.Random(7)
    tokens = [rng.randrange(49152) for _ in range(40)]
    bf = dtype == "bfloat16"
    want = P.forward(read_config_json(model_dir), load_plain_weights(model_dir, as_bf16=bf), tokens,
                     emulate_bf16=bf)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=256)
    trace = TraceBuilder()
    trace.step([("r", tokens[:32], range(32))])
    for t in range(32, 40):
        trace.step([("r", tokens[t:t + 1], [0])], end=["r"] if t == 39 else [])
    out = str(tmp_path / "out")
    replay(engine, trace.lines, out)
    check_logits(read_step(out, 0, 49152), want[:32], dtype, f"135M {dtype} prompt")
    for t in range(32, 40):
        check_logits(read_step(out, t - 31, 49152), want[t:t + 1], dtype, f"135M {dtype} token {t}")
    # greedy tokens agree wherever the plain logits have a clear winner
    got_last = torch.from_numpy(read_step(out, 8, 49152))[0]
    top2 = torch.topk(want[39], 2).values
    if float(top2[0] - top2[1]) > 0.05 * float(want[39].abs().max()):
        assert int(got_last.argmax()) == int(want[39].argmax())
