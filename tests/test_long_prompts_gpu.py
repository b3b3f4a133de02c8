"""Long prompts through the engine with head size 64 (the size the tcgen05 prompt
attention takes): prompts of many pages and several 128-query tiles, a prompt
continued by a second chunk, single tokens after it, a layer with a window beside
a layer without (two groups of the cache), in float32 and bfloat16 against the
plain implementation."""
import random
from dataclasses import replace

import pytest
import torch

import plain_llama as P
from helpers import check_logits
from nnis_b200.config.spec import PartSpec

pytestmark = pytest.mark.gpu

CFG = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=300, hidden_size=128,
           intermediate_size=200, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
           head_dim=64, max_position_embeddings=2048, rms_norm_eps=1e-5, rope_theta=10000.0,
           hidden_act="silu", tie_word_embeddings=True, attention_bias=False, torch_dtype="float32")
WINDOWS = [0, 150]


def plain_forward(w, tokens, bf):
    """plain_llama.forward with a window on the second layer."""
    eps, T = CFG["rms_norm_eps"], len(tokens)
    cos, sin = P.rope_tables(T, CFG["head_dim"], CFG["rope_theta"])
    h = P.embed(w["model.embed_tokens.weight"], tokens)
    for layer, window in enumerate(WINDOWS):
        p = f"model.layers.{layer}."
        n = P._round(P.rms_norm(h, w[p + "input_layernorm.weight"], eps), bf)
        h = h + P.attention_layer(CFG, w, p + "self_attn.", n, cos, sin, bf, window)
        n = P._round(P.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), bf)
        h = h + P.mlp_layer(CFG, w, p + "mlp.", n, bf)
    return P.linear(P._round(P.rms_norm(h, w["model.norm.weight"], eps), bf), w["model.embed_tokens.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_in_chunks_with_and_without_a_window(dtype):
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    spec = config_from_dict(CFG).to_spec()
    layers = list(spec.layers)
    mixer = layers[1].part("mixer")
    layers[1] = replace(layers[1], parts={**layers[1].parts, "mixer": PartSpec(
        mixer.kind, {**mixer.params, "window": WINDOWS[1]})})
    spec = replace(spec, layers=tuple(layers))
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=64, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    bf = dtype == "bfloat16"
    w = {k: (v.to(torch.bfloat16).float() if bf else v.float()) for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype=dtype, max_tokens=64 * 40, max_slots=3)
    assert len(engine.cache.groups) == 2  # the windowed layer keeps pages of its own
    rng = random.Random(5)
    seqs = {"a": [rng.randrange(300) for _ in range(700)], "b": [rng.randrange(300) for _ in range(131)],
            "c": [rng.randrange(300) for _ in range(64)]}
    want = {k: plain_forward(w, v, bf) for k, v in seqs.items()}
    slot = {k: engine.acquire_slot() for k in seqs}
    # whole prompts of unequal length in one step (a: first chunk only)
    picks = {"a": [0, 127, 128, 399], "b": [0, 63, 64, 130], "c": [63]}
    got = engine.step([SequenceStep(slot["a"], seqs["a"][:400], picks["a"]),
                       SequenceStep(slot["b"], seqs["b"], picks["b"]),
                       SequenceStep(slot["c"], seqs["c"], picks["c"])])
    rows = torch.cat([want[k][picks[k]] for k in ("a", "b", "c")])
    check_logits(got.cpu().numpy(), rows, dtype, "first chunks")
    engine.release_slot(slot["b"])
    engine.release_slot(slot["c"])
    # the second chunk of a starts inside a page and a tile, beyond the window of layer 1
    got = engine.step([SequenceStep(slot["a"], seqs["a"][400:690], [0, 100, 289])])
    check_logits(got.cpu().numpy(), want["a"][[400, 500, 689]], dtype, "second chunk")
    for t in range(690, 700):
        got = engine.step([SequenceStep(slot["a"], [seqs["a"][t]], [0])])
        check_logits(got.cpu().numpy(), want["a"][t:t + 1], dtype, f"token {t}")
    engine.release_slot(slot["a"])
    engine.check_status()
    engine.cache.check()


def test_a_recurring_long_prompt_is_replayed_from_a_graph_with_cut_tiles():
    """The same prompt shape three times on fresh slots: run as it comes, captured,
    replayed.  With one 1,500-token prompt the tcgen05 attention cuts its tiles into
    chunks, whose scratch and tickets live in the captured step's own buffers."""
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    spec = config_from_dict(CFG).to_spec()
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=65, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    w = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype="bfloat16", max_tokens=64 * 60, max_slots=2)
    rng = random.Random(9)
    picks = [0, 700, 1499]
    for round_ in range(4):
        tokens = [rng.randrange(300) for _ in range(1500)]
        want = P.forward(CFG, w, tokens, True)
        slot = engine.acquire_slot()
        got = engine.step([SequenceStep(slot, tokens, picks)])
        check_logits(got.cpu().numpy(), want[picks], "bfloat16", f"round {round_}")
        engine.release_slot(slot)
    assert any(e["graph"] is not None for e in engine._step_graphs.values())
    engine.check_status()


def test_a_decode_step_of_fifty_sequences_takes_the_product_kernels_and_matches():
    """More than 48 rows in a decode step: norm kernel and tcgen05 products instead of
    the decode projection kernel (bfloat16, head size 64), rows of unequal context."""
    from nnis_b200.config import config_from_dict
    from nnis_b200.engine import Engine, SequenceStep
    from nnis_b200.engine.model import DecoderModel
    from nnis_b200.weights import random_tensors
    spec = config_from_dict(CFG).to_spec()
    tensors = random_tensors(DecoderModel.weight_specs_of(spec), seed=66, std=1.0, norm_std=0.1,
                             std_by_fan_in=True)
    w = {k: v.to(torch.bfloat16).float() for k, v in tensors.items()}
    engine = Engine.from_spec(spec, tensors, dtype="bfloat16", max_tokens=64 * 120, max_slots=50)
    rng = random.Random(11)
    seqs = [[rng.randrange(300) for _ in range(rng.choice([2, 5, 17, 64, 65, 130]) + 2)] for _ in range(50)]
    slots = [engine.acquire_slot() for _ in seqs]
    engine.step([SequenceStep(s, t[:-2], []) for s, t in zip(slots, seqs)])
    want = [P.forward(CFG, w, t, True) for t in seqs]
    for back in (2, 1):  # two decode steps of all fifty
        got = engine.step([SequenceStep(s, [t[-back]], [0]) for s, t in zip(slots, seqs)])
        check_logits(got.cpu().numpy(), torch.stack([x[len(t) - back] for x, t in zip(want, seqs)]),
                     "bfloat16", f"decode step {3 - back} of fifty")
    for s in slots:
        engine.release_slot(s)
    engine.check_status()


def test_generation_of_fifty_prompts_agrees_with_stepping_the_engine():
    """Through LLM.generate the fifty rows run in the 64-row decode graph (padding rows
    beside them); the tokens must be those of plain greedy stepping with the same kernels."""
    import tempfile
    from nnis_b200 import LLM
    from nnis_b200.engine import SequenceStep
    from nnis_b200.weights import write_random_model
    with tempfile.TemporaryDirectory() as d:
        write_random_model(CFG, 67, d, std=1.0, norm_std=0.1, std_by_fan_in=True)
        llm = LLM(d, dtype="bfloat16", max_tokens=64 * 120, max_batch=64)
        rng = random.Random(12)
        prompts = [[rng.randrange(300) for _ in range(rng.choice([1, 3, 8, 40]))] for _ in range(50)]
        out = llm.generate(prompts, max_new_tokens=5, stop_token_ids=())
        engine = llm.engine
        for i in (0, 7, 23, 49):
            slot = engine.acquire_slot()
            logits = engine.step([SequenceStep(slot, prompts[i], [len(prompts[i]) - 1])])
            toks = []
            for _ in range(5):
                toks.append(int(logits[0].argmax()))
                logits = engine.step([SequenceStep(slot, [toks[-1]], [0])])
            engine.release_slot(slot)
            assert out[i].ok and list(out[i].token_ids) == toks, (i, out[i].token_ids, toks)
