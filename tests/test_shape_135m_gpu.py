"""The SmolLM2-135M shape with all its 30 layers and random weights: the engine's
float32 and bfloat16 logits against the plain float64 implementation, through the three
cuts of work (whole, last tokens one by one, unequal batches one after another with
slots and pages used again, prompts that cross a page), and its greedy tokens.  The
shape comes from a config.json like any other; only this file knows its numbers."""
import random

import pytest
import torch

import plain_llama as P
from helpers import (load_plain_weights, make_model, read_config_json, read_step, replay_against_plain,
                     three_cuts)

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
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=64 * 16)
    trace, sequences = three_cuts(
        random.Random(7), 49152, whole=(40,), last32=(70,),
        batches=([(5, 9), (66, 69), (17, 18)], [(1, 4), (64, 66), (2, 3), (31, 33)]))
    out = str(tmp_path / "out")
    replay_against_plain(engine, model_dir, dtype, trace, sequences, out, "135M")
    # greedy tokens: at every position of the whole request where the plain logits have
    # a clear winner the engine picks it (and such positions exist)
    bf = dtype == "bfloat16"
    want = P.forward(read_config_json(model_dir), load_plain_weights(model_dir, as_bf16=bf),
                     sequences["w0"], emulate_bf16=bf)
    got = torch.from_numpy(read_step(out, 0, 49152))
    top2 = torch.topk(want, 2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.05 * want.abs().amax(dim=-1)
    assert int(clear.sum()) >= 5, "the prompt has too few positions with a clear winner"
    assert torch.equal(got.argmax(dim=-1)[clear], want.argmax(dim=-1)[clear])
