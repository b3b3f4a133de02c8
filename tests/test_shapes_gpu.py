"""Further configurations through the three cuts of work, against the plain
implementation, in float32 and in bfloat16: every kind of head size that a
configuration may name (NNIS asks for an even one: crates/nnis-model/src/config.rs:38-105),
and the layer sizes of SmolLM2-135M, 360M and 1.7B with two layers instead of their
30, 32 and 24 (the oracle is a float64 program on the CPU; the sizes of a layer, the
vocabulary and the head are the full ones)."""
import random

import pytest

from helpers import make_model, replay_against_plain, three_cuts

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def llama(**sizes):
    base = dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu",
                rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=True,
                attention_bias=False, torch_dtype="bfloat16", max_position_embeddings=512)
    base.update(sizes)
    return base


# head sizes that are no multiple of 16 (8, 24, 40, 72) beside heads and widths of all kinds
HEAD_SIZES = {
    "d8": llama(vocab_size=300, hidden_size=40, intermediate_size=72, num_hidden_layers=2,
                num_attention_heads=5, num_key_value_heads=5),
    "d24": llama(vocab_size=259, hidden_size=96, intermediate_size=136, num_hidden_layers=2,
                 num_attention_heads=4, num_key_value_heads=2, attention_bias=True),
    "d40": llama(vocab_size=410, hidden_size=100, intermediate_size=88, num_hidden_layers=3,
                 num_attention_heads=3, num_key_value_heads=1, head_dim=40, rope_theta=500000.0,
                 tie_word_embeddings=False),
    "d72": llama(vocab_size=333, hidden_size=144, intermediate_size=160, num_hidden_layers=2,
                 num_attention_heads=2, num_key_value_heads=1, rms_norm_eps=1e-6),
    "d2": llama(vocab_size=64, hidden_size=12, intermediate_size=20, num_hidden_layers=1,
                num_attention_heads=6, num_key_value_heads=3),
    "d250": llama(vocab_size=70, hidden_size=64, intermediate_size=48, num_hidden_layers=1,
                  num_attention_heads=2, num_key_value_heads=1, head_dim=250),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(HEAD_SIZES))
def test_every_even_head_size_runs_the_three_cuts(name, dtype, tmp_path):
    from nnis_b200.engine import Engine
    cfg = HEAD_SIZES[name]
    model_dir = make_model(str(tmp_path / "model"), cfg, seed=300 + len(name))
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=64 * 64)
    trace, sequences = three_cuts(random.Random(17), cfg["vocab_size"])
    replay_against_plain(engine, model_dir, dtype, trace, sequences, str(tmp_path / "out"), name)


def smollm2(**sizes):
    return llama(**{**dict(vocab_size=49152, rope_theta=100000.0, max_position_embeddings=8192,
                           num_hidden_layers=2), **sizes})


# layer sizes of the three checkpoints of the family; two layers each (30, 32 and 24 in full)
FAMILY = {
    "135m": smollm2(hidden_size=576, intermediate_size=1536, num_attention_heads=9,
                    num_key_value_heads=3),
    "360m": smollm2(hidden_size=960, intermediate_size=2560, num_attention_heads=15,
                    num_key_value_heads=5),
    "1.7b": smollm2(hidden_size=2048, intermediate_size=8192, num_attention_heads=32,
                    num_key_value_heads=32, rope_theta=130000.0),
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(FAMILY))
def test_the_family_shapes_run_the_three_cuts(name, dtype, tmp_path):
    """Two of the shape's layers; prompts that cross a page, decode steps of one to
    five rows, a prompt step of several sequences; slots and pages used again."""
    from nnis_b200.engine import Engine
    cfg = FAMILY[name]
    model_dir = make_model(str(tmp_path / "model"), cfg, seed=7)
    engine = Engine.from_dir(model_dir, dtype=dtype, max_tokens=64 * 32)
    trace, sequences = three_cuts(
        random.Random(23), cfg["vocab_size"], whole=(3, 70), last32=(97,),
        batches=([(5, 9), (66, 70), (17, 19)], [(1, 6), (40, 41), (64, 66), (2, 5), (31, 33)]))
    replay_against_plain(engine, model_dir, dtype, trace, sequences, str(tmp_path / "out"), name)
