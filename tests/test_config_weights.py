"""Configuration, registry, safetensors and weight errors (no GPU)."""
import json
import os

import pytest
import torch

from helpers import TINY_A, TINY_B, make_model
from nnis_b200.config import (ConfigError, LlamaConfig, config_from_dict, known_architectures,
                              read_config)
from nnis_b200.engine.model import DecoderModel
from nnis_b200.weights import SafetensorsFile, WeightError, load_weights, write_safetensors


def test_llama_config_reads_every_key():
    c = config_from_dict(TINY_B)
    assert isinstance(c, LlamaConfig)
    assert (c.vocab_size, c.hidden_size, c.intermediate_size) == (515, 96, 272)
    assert (c.num_hidden_layers, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == \
        (3, 3, 1, 32)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 500000.0
    assert c.attention_bias and c.mlp_bias and not c.tie_word_embeddings
    assert c.stop_token_ids == (3, 11) and c.stored_dtype == "bfloat16"
    assert config_from_dict(c.to_dict()) == c


def test_head_dim_is_derived_and_kv_heads_default():
    raw = dict(TINY_A)
    del raw["num_key_value_heads"]
    c = config_from_dict(raw)
    assert c.head_dim == 16 and c.num_key_value_heads == 4


def test_smollm2_shape_needs_no_constant_in_code():
    raw = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=49152,
               hidden_size=576, intermediate_size=1536, num_hidden_layers=30,
               num_attention_heads=9, num_key_value_heads=3, max_position_embeddings=8192,
               rms_norm_eps=1e-5, rope_theta=100000, hidden_act="silu", tie_word_embeddings=True,
               torch_dtype="bfloat16", eos_token_id=0, bos_token_id=0, use_cache=True)
    spec = config_from_dict(raw).to_spec()
    assert len(spec.layers) == 30 and len(spec.schedule) == 30
    assert spec.layers[0].part("mixer")["head_dim"] == 64
    assert spec.head["tied_to"] == "model.embed_tokens"


@pytest.mark.parametrize("change, word", [
    ({"architectures": ["MistralForCausalLM"]}, "unknown architecture"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope scaling"),
    ({"rope_interleaved": True}, "rope_interleaved"),
    ({"torch_dtype": "float16"}, "torch_dtype"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": float("inf")}, "rope_theta"),
    ({"vocab_size": 0}, "vocab_size"),
    ({"eos_token_id": 999}, "eos_token_id"),
    ({"hidden_size": 66}, "hidden_size"),
])
def test_bad_configs_are_refused_by_key(change, word):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_missing_keys_are_listed():
    raw = {k: v for k, v in TINY_A.items() if k not in ("vocab_size", "rms_norm_eps")}
    with pytest.raises(ConfigError) as e:
        config_from_dict(raw)
    assert "vocab_size" in str(e.value) and "rms_norm_eps" in str(e.value)


def test_registry_names_known_architectures():
    assert "LlamaForCausalLM" in known_architectures()


def test_dtype_key_of_newer_exporters():
    raw = dict(TINY_A)
    del raw["torch_dtype"]
    raw["dtype"] = "bfloat16"
    raw["rope_parameters"] = {"rope_theta": 12345.0, "rope_type": "default"}
    del raw["rope_theta"]
    c = config_from_dict(raw)
    assert c.stored_dtype == "bfloat16" and c.rope_theta == 12345.0


def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors)
    from safetensors.torch import load_file
    theirs = load_file(path)
    with SafetensorsFile(path) as f:
        for k, v in tensors.items():
            assert torch.equal(f.tensor(k), v) and torch.equal(theirs[k], v)


def test_random_model_folder_loads_and_is_seeded(tmp_path):
    d1 = make_model(str(tmp_path / "m1"), TINY_B, seed=5)
    d2 = make_model(str(tmp_path / "m2"), TINY_B, seed=5)
    d3 = make_model(str(tmp_path / "m3"), TINY_B, seed=6)
    spec = read_config(d1).to_spec()
    wanted = DecoderModel.weight_specs_of(spec)
    w1 = load_weights(d1, wanted, torch.bfloat16, torch.device("cpu"))
    w2 = load_weights(d2, wanted, torch.bfloat16, torch.device("cpu"))
    w3 = load_weights(d3, wanted, torch.bfloat16, torch.device("cpu"))
    assert set(w1) == set(wanted)
    assert all(torch.equal(w1[k], w2[k]) for k in w1)
    assert any(not torch.equal(w1[k], w3[k]) for k in w1)
    # matrices keep bfloat16, vectors are float32, shapes as wanted
    assert w1["model.layers.0.self_attn.q_proj.weight"].dtype == torch.bfloat16
    assert w1["model.layers.0.input_layernorm.weight"].dtype == torch.float32
    assert w1["model.layers.0.self_attn.q_proj.bias"].dtype == torch.float32
    assert "lm_head.weight" in w1


def test_float32_run_widens_bfloat16_exactly(tmp_path):
    d = make_model(str(tmp_path / "m"), TINY_B, seed=1)
    wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
    bf = load_weights(d, wanted, torch.bfloat16, torch.device("cpu"))
    f32 = load_weights(d, wanted, torch.float32, torch.device("cpu"))
    for k in bf:
        assert f32[k].dtype == torch.float32
        assert torch.equal(bf[k].float(), f32[k])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = make_model(str(tmp_path / "m"), TINY_A, seed=1)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(64, 32)
    tensors["model.layers.7.extra.weight"] = torch.zeros(2)
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)  # ignored buffer
    write_safetensors(path, tensors)
    wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
    with pytest.raises(WeightError) as e:
        load_weights(d, wanted, torch.float32, torch.device("cpu"))
    msg = str(e.value)
    assert "missing (2)" in msg and "model.layers.1.mlp.up_proj.weight" in msg \
        and "model.norm.weight" in msg
    assert "unexpected (1)" in msg and "model.layers.7.extra.weight" in msg
    assert "inv_freq" not in msg
    assert "wrong shape or dtype (1)" in msg and "[64, 32]" in msg and "[64, 64]" in msg


def test_lm_head_beside_tied_embedding_is_unexpected(tmp_path):
    d = make_model(str(tmp_path / "m"), TINY_A, seed=1)
    path = os.path.join(d, "model.safetensors")
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    tensors["lm_head.weight"] = torch.zeros(256, 64)
    write_safetensors(path, tensors)
    wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
    with pytest.raises(WeightError, match="unexpected"):
        load_weights(d, wanted, torch.float32, torch.device("cpu"))


def test_missing_files_and_both_files(tmp_path):
    d = str(tmp_path / "empty")
    os.makedirs(d)
    with pytest.raises(WeightError, match="neither"):
        load_weights(d, {}, torch.float32, torch.device("cpu"))
    m = make_model(str(tmp_path / "m"), TINY_A, seed=1)
    with open(os.path.join(m, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {}}, f)
    with pytest.raises(WeightError, match="both"):
        load_weights(m, {}, torch.float32, torch.device("cpu"))


def test_sharded_folder_and_float16_refusal(tmp_path):
    d = make_model(str(tmp_path / "m"), TINY_A, seed=2)
    single = os.path.join(d, "model.safetensors")
    with SafetensorsFile(single) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    names = sorted(tensors)
    half = len(names) // 2
    write_safetensors(os.path.join(d, "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    write_safetensors(os.path.join(d, "s2.safetensors"), {n: tensors[n] for n in names[half:]})
    os.remove(single)
    with open(os.path.join(d, "model.safetensors.index.json"), "w") as f:
        json.dump({"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors")
                                  for i, n in enumerate(names)}}, f)
    wanted = DecoderModel.weight_specs_of(read_config(d).to_spec())
    w = load_weights(d, wanted, torch.float32, torch.device("cpu"))
    assert all(torch.equal(w[n], tensors[n]) for n in names)
    tensors[names[0]] = tensors[names[0]].to(torch.float16)
    write_safetensors(os.path.join(d, "s1.safetensors"), {n: tensors[n] for n in names[:half]})
    with pytest.raises(WeightError, match="float16"):
        load_weights(d, wanted, torch.float32, torch.device("cpu"))


def _tiny_a_as_nnis_directory(tmp_path):
    from nnis_b200.weights import write_nnis_directory
    d = make_model(str(tmp_path / "hf"), TINY_A, seed=2)
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    cfg = json.load(open(os.path.join(d, "config.json")))
    return d, cfg, tensors, write_nnis_directory(cfg, tensors, str(tmp_path / "nnis"))


def test_nnis_model_folder_reads_as_the_same_model(tmp_path):
    """model.json + raw files (NNIS's own folder): its names and transposed projections come
    out as the tensors of the Hugging Face folder it was written from; the tied head is a
    tensor of its own there."""
    hf_dir, cfg, tensors, nnis_dir = _tiny_a_as_nnis_directory(tmp_path)
    manifest = json.load(open(os.path.join(nnis_dir, "model.json")))
    assert manifest["format"] == "nnis-model" and manifest["version"] == 1
    by_name = {e["name"]: e for e in manifest["tensors"]}
    H, V = TINY_A["hidden_size"], TINY_A["vocab_size"]
    kvw = H // TINY_A["num_attention_heads"] * TINY_A["num_key_value_heads"]
    assert by_name["layers.0.k_proj"]["shape"] == [H, kvw]  # [in, out]
    assert by_name["token_embedding"]["shape"] == [V, H] and by_name["lm_head"]["shape"] == [H, V]
    config = read_config(nnis_dir)
    assert not config.tie_word_embeddings and config.hidden_size == H and config.vocab_size == V
    assert config.rms_norm_eps == pytest.approx(TINY_A["rms_norm_eps"])
    wanted = DecoderModel.weight_specs_of(config.to_spec())
    got = load_weights(nnis_dir, wanted, torch.float32, torch.device("cpu"))
    for name, t in tensors.items():
        assert torch.equal(got[name], t.float()), name
    assert torch.equal(got["lm_head.weight"], tensors["model.embed_tokens.weight"].float())
    from nnis_b200.weights import check_weights
    assert check_weights(nnis_dir, wanted)["weight_files"] == ["model.json"]


def test_nnis_model_folder_faults(tmp_path):
    from nnis_b200.weights import NnisDirectoryError, write_nnis_directory
    hf_dir, cfg, tensors, nnis_dir = _tiny_a_as_nnis_directory(tmp_path)
    path = os.path.join(nnis_dir, "model.json")
    good = json.load(open(path))

    def with_change(change):
        m = json.loads(json.dumps(good))
        change(m)
        json.dump(m, open(path, "w"))

    for change, word in ((lambda m: m.update(format="other"), "is not 'nnis-model'"),
                         (lambda m: m.update(version=2), "supported version is 1"),
                         (lambda m: m["tensors"][0].update(file="../x.bin"), "parent traversal"),
                         (lambda m: m["tensors"][0].update(file="/abs.bin"), "parent traversal"),
                         (lambda m: m["tensors"].append(dict(m["tensors"][0])), "duplicate tensor name"),
                         (lambda m: m["tensors"][0].update(shape=[0, 3]), "non-zero dimensions"),
                         (lambda m: m["tensors"][0].update(dtype="f16"), "not f32 or bf16"),
                         (lambda m: m["config"].pop("rope_theta"), "config lacks rope_theta")):
        with_change(change)
        with pytest.raises(ConfigError, match=word):
            read_config(nnis_dir)
    # a file of the wrong length, an unknown tensor and a missing one: the loader's one error
    with_change(lambda m: m["tensors"][0].update(shape=[m["tensors"][0]["shape"][0] + 1] + m["tensors"][0]["shape"][1:]))
    wanted = DecoderModel.weight_specs_of(config_from_dict({**cfg, "tie_word_embeddings": False}).to_spec())
    with pytest.raises(WeightError, match="requires"):
        load_weights(nnis_dir, wanted, torch.float32, torch.device("cpu"))

    def rename(m):
        entry = next(e for e in m["tensors"] if e["name"] == "layers.1.up_proj")
        entry["name"] = "layers.1.sideways_proj"
    with_change(rename)
    with pytest.raises(WeightError) as e:
        load_weights(nnis_dir, wanted, torch.float32, torch.device("cpu"))
    assert "missing (1): model.layers.1.mlp.up_proj.weight" in str(e.value)
    assert "unexpected (1): layers.1.sideways_proj" in str(e.value)
    # biases have no place in the format
    d = make_model(str(tmp_path / "b"), TINY_B, seed=2)
    with SafetensorsFile(os.path.join(d, "model.safetensors")) as f:
        with_bias = {n: f.tensor(n) for n in f.names()}
    with pytest.raises(NnisDirectoryError, match="no place"):
        write_nnis_directory(json.load(open(os.path.join(d, "config.json"))), with_bias, str(tmp_path / "nb"))
