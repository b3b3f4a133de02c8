"""NNIS's own model folder: ``model.json`` plus one raw little-endian file per tensor.

``model.json`` is ``{"format": "nnis-model", "version": 1, "config": {...},
"tensors": [{"name", "dtype": "f32"|"bf16", "shape", "file"}, ...]}``
(crates/nnis-model/src/format.rs:12-30 the manifest, :43-134 loading, :136-190
its checks; the configuration's fields crates/nnis-model/src/config.rs:21-35).
Its tensors carry NNIS's names (``token_embedding``, ``layers.N.q_proj``,
``final_norm``, ``lm_head``; format.rs:192-233) and its projections are stored
transposed, ``[in, out]`` (crates/nnis-model/src/weights.rs:296-302).

Here such a folder is read as what the rest of the library knows: a
configuration in config.json's keys and tensors under Hugging Face names in
``[out, in]`` layout, behind the interface of ``SafetensorsFile`` so that the
loader's checks and its one error apply unchanged.  ``write_nnis_directory``
writes one (tests; moving a model between the two forms).
"""
from __future__ import annotations

import json
import os
import re
from typing import Any, Dict, List, Mapping, Optional, Tuple

import numpy as np
import torch

MANIFEST = "model.json"
FORMAT = "nnis-model"
VERSION = 1
_DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}
_TORCH_DTYPE_KEY = {"f32": "float32", "bf16": "bfloat16"}

# NNIS name -> (Hugging Face name, stored transposed)
_GLOBAL = {"token_embedding": ("model.embed_tokens.weight", False),
           "final_norm": ("model.norm.weight", False),
           "lm_head": ("lm_head.weight", True)}
_PER_LAYER = {"input_norm": ("input_layernorm.weight", False),
              "post_attention_norm": ("post_attention_layernorm.weight", False),
              "q_proj": ("self_attn.q_proj.weight", True), "k_proj": ("self_attn.k_proj.weight", True),
              "v_proj": ("self_attn.v_proj.weight", True), "o_proj": ("self_attn.o_proj.weight", True),
              "gate_proj": ("mlp.gate_proj.weight", True), "up_proj": ("mlp.up_proj.weight", True),
              "down_proj": ("mlp.down_proj.weight", True)}
_LAYER_NAME = re.compile(r"^layers\.(\d+)\.([a-z_]+)$")


class NnisDirectoryError(ValueError):
    pass


def is_nnis_directory(model_dir: str) -> bool:
    return os.path.isfile(os.path.join(model_dir, MANIFEST))


def hf_name(name: str) -> Optional[Tuple[str, bool]]:
    """(Hugging Face name, transposed) of an NNIS tensor name; None if it is not one."""
    if name in _GLOBAL:
        return _GLOBAL[name]
    m = _LAYER_NAME.match(name)
    if m and m.group(2) in _PER_LAYER:
        tail, transposed = _PER_LAYER[m.group(2)]
        return f"model.layers.{int(m.group(1))}.{tail}", transposed
    return None


def nnis_name(name: str) -> Optional[Tuple[str, bool]]:
    """The inverse of ``hf_name``."""
    for own, (theirs, transposed) in _GLOBAL.items():
        if name == theirs:
            return own, transposed
    m = re.match(r"^model\.layers\.(\d+)\.(.+)$", name)
    if m:
        for own, (tail, transposed) in _PER_LAYER.items():
            if m.group(2) == tail:
                return f"layers.{int(m.group(1))}.{own}", transposed
    return None


def _relative_file(model_dir: str, file: str, name: str) -> str:
    parts = file.split("/") if isinstance(file, str) else []
    if not file or os.path.isabs(file) or "\\" in file or any(p in ("", "..") for p in parts if p != "."):
        raise NnisDirectoryError(f"tensor {name!r}: file path {file!r} must be a relative path without "
                                 f"parent traversal")
    return os.path.join(model_dir, *[p for p in parts if p != "."])


def read_manifest(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, MANIFEST)
    try:
        with open(path, "r", encoding="utf-8") as f:
            manifest = json.load(f)
    except FileNotFoundError:
        raise NnisDirectoryError(f"{path}: no such file") from None
    except json.JSONDecodeError as e:
        raise NnisDirectoryError(f"{path}: not valid JSON: {e}") from None
    if not isinstance(manifest, dict) or manifest.get("format") != FORMAT:
        raise NnisDirectoryError(f"{path}: model format {manifest.get('format') if isinstance(manifest, dict) else None!r} "
                                 f"is not {FORMAT!r}")
    if manifest.get("version") != VERSION:
        raise NnisDirectoryError(f"{path}: format version {manifest.get('version')!r}; supported version is {VERSION}")
    if not isinstance(manifest.get("config"), dict) or not isinstance(manifest.get("tensors"), list):
        raise NnisDirectoryError(f"{path}: config must be an object and tensors a list")
    seen = set()
    for entry in manifest["tensors"]:
        if not isinstance(entry, dict) or not isinstance(entry.get("name"), str) or not entry["name"]:
            raise NnisDirectoryError(f"{path}: every tensor needs a non-empty name")
        name = entry["name"]
        if name in seen:
            raise NnisDirectoryError(f"{path}: duplicate tensor name {name} in model manifest")
        seen.add(name)
        shape = entry.get("shape")
        if not isinstance(shape, list) or not shape or any(type(s) is not int or s <= 0 for s in shape):
            raise NnisDirectoryError(f"{path}: tensor {name} shape must contain only non-zero dimensions; "
                                     f"got {shape!r}")
        if entry.get("dtype") not in _DTYPES:
            raise NnisDirectoryError(f"{path}: tensor {name} dtype {entry.get('dtype')!r} is not f32 or bf16")
        _relative_file(model_dir, entry.get("file"), name)
    return manifest


def config_of_manifest(manifest: Mapping[str, Any]) -> Dict[str, Any]:
    """The manifest's configuration in config.json's keys.  The folder always has a
    head of its own and no biases; its one architecture is the Llama decoder."""
    c = manifest["config"]
    required = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                "num_key_value_heads", "max_position_embeddings", "rms_norm_eps", "rope_theta", "activation",
                "weight_dtype")
    missing = [k for k in required if k not in c]
    if missing:
        raise NnisDirectoryError(f"{MANIFEST}: config lacks {', '.join(missing)}")
    if c["weight_dtype"] not in _TORCH_DTYPE_KEY:
        raise NnisDirectoryError(f"{MANIFEST}: weight_dtype {c['weight_dtype']!r} is not f32 or bf16")
    out = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_act": c["activation"],
           "torch_dtype": _TORCH_DTYPE_KEY[c["weight_dtype"]], "tie_word_embeddings": False,
           "attention_bias": False, "mlp_bias": False}
    for key in required[:9]:
        out[key] = c[key]
    if c.get("eos_token_id") is not None:
        out["eos_token_id"] = c["eos_token_id"]
    return out


class NnisDirectorySource:
    """The folder's tensors under Hugging Face names and layout, with the interface
    of ``SafetensorsFile``.  Names that are not NNIS's keep their own name, so that
    the loader reports them as unexpected."""

    def __init__(self, model_dir: str):
        self.path = os.path.join(model_dir, MANIFEST)
        manifest = read_manifest(model_dir)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], str, bool]] = {}
        for entry in manifest["tensors"]:
            mapped = hf_name(entry["name"])
            name, transposed = mapped if mapped is not None else (entry["name"], False)
            shape = tuple(entry["shape"])
            if transposed and len(shape) == 2:
                shape = (shape[1], shape[0])
            dtype = _DTYPES[entry["dtype"]]
            file = _relative_file(model_dir, entry["file"], entry["name"])
            if os.path.islink(file):
                raise NnisDirectoryError(f"{file}: symbolic links are not followed")
            count = int(np.prod(entry["shape"], dtype=np.int64))
            try:
                size = os.path.getsize(file)
            except OSError:
                raise NnisDirectoryError(f"tensor {entry['name']}: file {entry['file']!r} is missing") from None
            if size != count * dtype.itemsize:
                raise NnisDirectoryError(f"tensor {entry['name']} file has {size} bytes; shape {entry['shape']} "
                                         f"{entry['dtype']} requires {count * dtype.itemsize}")
            self.entries[name] = (dtype, shape, file, transposed and len(shape) == 2)

    def names(self) -> List[str]:
        return list(self.entries)

    def meta(self, name: str):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, file, transposed = self.entries[name]
        raw = np.fromfile(file, dtype=np.uint8)
        t = torch.from_numpy(raw).view(dtype)
        if transposed:
            return t.reshape(shape[1], shape[0]).t().contiguous()
        return t.reshape(shape)

    def close(self) -> None:
        pass


def write_nnis_directory(config: Mapping[str, Any], tensors: Mapping[str, torch.Tensor], out_dir: str) -> str:
    """Writes ``model.json`` and the raw files from a configuration in config.json's
    keys and tensors under Hugging Face names.  A tied head is written out as a
    tensor of its own, as the format wants; biases have no place in it."""
    os.makedirs(out_dir, exist_ok=True)
    stored = str(config.get("torch_dtype", config.get("dtype", "float32")))
    weight_dtype = "bf16" if stored in ("bfloat16", "bf16") else "f32"
    manifest_config = {k: config[k] for k in ("vocab_size", "hidden_size", "intermediate_size",
                                              "num_hidden_layers", "num_attention_heads",
                                              "max_position_embeddings", "rms_norm_eps", "rope_theta")}
    manifest_config["num_key_value_heads"] = config.get("num_key_value_heads", config["num_attention_heads"])
    manifest_config["activation"] = config.get("hidden_act", "silu")
    manifest_config["weight_dtype"] = weight_dtype
    if isinstance(config.get("eos_token_id"), int):
        manifest_config["eos_token_id"] = config["eos_token_id"]
    items = dict(tensors)
    if "lm_head.weight" not in items and "model.embed_tokens.weight" in items:
        items["lm_head.weight"] = items["model.embed_tokens.weight"]
    entries = []
    for name in sorted(items):
        mapped = nnis_name(name)
        if mapped is None:
            raise NnisDirectoryError(f"tensor {name!r} has no place in an NNIS model folder")
        own, transposed = mapped
        t = items[name].detach().cpu().to(_DTYPES[weight_dtype])
        if transposed:
            t = t.t()
        t = t.contiguous()
        file = own + ".bin"
        t.view(torch.uint8).numpy().tofile(os.path.join(out_dir, file))
        entries.append({"name": own, "dtype": weight_dtype, "shape": list(t.shape), "file": file})
    with open(os.path.join(out_dir, MANIFEST), "w", encoding="utf-8") as f:
        json.dump({"format": FORMAT, "version": VERSION, "config": manifest_config, "tensors": entries}, f,
                  indent=1)
        f.write("\n")
    return out_dir
