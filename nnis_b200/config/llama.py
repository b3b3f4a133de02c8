"""Typed configuration of the Llama dense decoder, read from config.json.

Keys and rules follow NNIS's reader of Hugging Face folders
(crates/nnis-model/src/safetensors_loader.rs:66-93 keys, :136-189 rules;
crates/nnis-model/src/config.rs:38-101 shape validation).  Differences, all
additions: ``attention_bias`` and ``mlp_bias`` are accepted (NNIS rejects
them), ``head_dim`` may be given, ``eos_token_id`` may be a list, and both the
``torch_dtype`` and the ``dtype`` spelling of the stored dtype are read.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Tuple

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


class ConfigError(ValueError):
    """config.json cannot be used; the message names the key."""


_DTYPES = {"float32": "float32", "f32": "float32", "bfloat16": "bfloat16", "bf16": "bfloat16"}
_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
             "num_attention_heads", "max_position_embeddings", "rms_norm_eps")


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    value = raw[key]
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key} must be a positive integer; got {value!r}")
    return value


def _positive_float(value: Any, key: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) \
            or not math.isfinite(value) or value <= 0:
        raise ConfigError(f"config.json: {key} must be finite and positive; got {value!r}")
    return float(value)


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    attention_bias: bool
    mlp_bias: bool
    stored_dtype: str
    stop_token_ids: Tuple[int, ...]

    architecture = "LlamaForCausalLM"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        archs = raw.get("architectures")
        if archs != [cls.architecture]:
            raise ConfigError(f"config.json: architectures must be [{cls.architecture!r}]; "
                              f"got {archs!r}")
        if raw.get("model_type", "llama") != "llama":
            raise ConfigError(f"config.json: model_type must be 'llama'; got {raw['model_type']!r}")
        missing = [k for k in _REQUIRED if k not in raw]
        if missing:
            raise ConfigError(f"config.json: missing keys {missing}")
        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = raw.get("num_key_value_heads")
        kv_heads = heads if kv_heads is None else _positive_int(raw, "num_key_value_heads")
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads={heads} is not a multiple of "
                              f"num_key_value_heads={kv_heads}")
        if raw.get("head_dim") is not None:
            head_dim = _positive_int(raw, "head_dim")
        else:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size={hidden} is not a multiple of "
                                  f"num_attention_heads={heads} and no head_dim is given")
            head_dim = hidden // heads
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim={head_dim} must be even for rotate-half RoPE")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act must be 'silu'; got {act!r}")
        if raw.get("rope_interleaved", False):
            raise ConfigError("config.json: rope_interleaved=true is not supported")
        theta = raw.get("rope_theta")
        scaling = raw.get("rope_scaling")
        rope_parameters = raw.get("rope_parameters")
        if isinstance(rope_parameters, Mapping):
            theta = rope_parameters.get("rope_theta", theta)
            if rope_parameters.get("rope_type", "default") != "default":
                scaling = rope_parameters
        if scaling is not None:
            raise ConfigError(f"config.json: rope scaling is not supported; got {scaling!r}")
        if theta is None:
            raise ConfigError("config.json: missing keys ['rope_theta']")
        dtype_key = raw.get("torch_dtype", raw.get("dtype"))
        if dtype_key is None:
            raise ConfigError("config.json: missing keys ['torch_dtype']")
        if dtype_key not in _DTYPES:
            raise ConfigError(f"config.json: torch_dtype must be one of {sorted(_DTYPES)}; "
                              f"got {dtype_key!r}")
        vocab = _positive_int(raw, "vocab_size")
        eos = raw.get("eos_token_id")
        if eos is None:
            stops: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            stops = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(t, int) for t in eos):
            stops = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of "
                              f"integers; got {eos!r}")
        for t in stops:
            if not 0 <= t < vocab:
                raise ConfigError(f"config.json: eos_token_id {t} is outside vocab_size={vocab}")
        return cls(
            vocab_size=vocab,
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=_positive_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=_positive_int(raw, "max_position_embeddings"),
            rms_norm_eps=_positive_float(raw["rms_norm_eps"], "rms_norm_eps"),
            rope_theta=_positive_float(theta, "rope_theta"),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            mlp_bias=bool(raw.get("mlp_bias", False)),
            stored_dtype=_DTYPES[dtype_key],
            stop_token_ids=stops,
        )

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "torch_dtype": self.stored_dtype,
        }
        if len(self.stop_token_ids) == 1:
            out["eos_token_id"] = self.stop_token_ids[0]
        elif self.stop_token_ids:
            out["eos_token_id"] = list(self.stop_token_ids)
        return out

    # ------------------------------------------------------------------
    def to_spec(self) -> ModelSpec:
        """Pre-norm blocks of attention and a gated MLP, one after another
        (crates/nnis-model/src/runtime.rs:946-1097)."""
        norm = PartSpec("rmsnorm", {"size": self.hidden_size, "eps": self.rms_norm_eps})
        position = PartSpec("rope_half", {
            "head_dim": self.head_dim, "theta": self.rope_theta,
            "max_positions": self.max_position_embeddings})
        layers = []
        for i in range(self.num_hidden_layers):
            mixer = PartSpec("attention", {
                "hidden_size": self.hidden_size, "heads": self.num_attention_heads,
                "kv_heads": self.num_key_value_heads, "head_dim": self.head_dim,
                "bias": self.attention_bias, "window": 0, "position": position,
                "names": {"q": "self_attn.q_proj", "k": "self_attn.k_proj",
                          "v": "self_attn.v_proj", "o": "self_attn.o_proj"}})
            ffn = PartSpec("gated_mlp", {
                "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "activation": "silu", "bias": self.mlp_bias,
                "names": {"gate": "mlp.gate_proj", "up": "mlp.up_proj",
                          "down": "mlp.down_proj"}})
            layers.append(LayerSpec(prefix=f"model.layers.{i}", block="prenorm", parts={
                "mixer_norm": PartSpec("rmsnorm", {**norm.params, "name": "input_layernorm"}),
                "mixer": mixer,
                "ffn_norm": PartSpec("rmsnorm", {**norm.params, "name": "post_attention_layernorm"}),
                "ffn": ffn}))
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=self.hidden_size,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "name": "model.embed_tokens"}),
            layers=tuple(layers),
            schedule=tuple(ScheduleEntry(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rmsnorm", {**norm.params, "name": "model.norm"}),
            head=PartSpec("linear_head", {
                "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "name": "lm_head",
                "tied_to": "model.embed_tokens" if self.tie_word_embeddings else None}),
            stop_token_ids=self.stop_token_ids,
            stored_dtype=self.stored_dtype,
        )
        spec.validate()
        return spec
