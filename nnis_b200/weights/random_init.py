"""Random-weights mode: a model folder from a configuration and a seed.

Writes ``config.json`` and ``model.safetensors`` so that every other part of
the framework (loader, engine, replay, command line) meets random models the
same way as real ones.  NNIS has no such mode; its tests build weights by hand
(crates/nnis-model/src/runtime.rs:1192-1261).

Values: matrices N(0, std^2), norm weights 1 + N(0, norm_std^2) (or N(0,std^2)
around zero when ``norm_center`` is 0), biases N(0, std^2); each tensor is drawn
in float32 from a CPU generator of its own, seeded with the seed and a hash of
the tensor's name, so that a tensor's values depend on nothing but the seed, its
name and its shape; then stored in the configuration's dtype.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Mapping

import torch

from ..config import config_from_dict
from .loader import SINGLE_FILE, WeightSpec
from .safetensors_io import write_safetensors

_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tensor_seed(seed: int, name: str) -> int:
    """The generator seed of one tensor: the model's seed xor the first eight bytes
    of SHA-256 of the tensor's name (63 bits)."""
    digest = hashlib.sha256(name.encode("utf-8")).digest()
    return ((int(seed) & (2 ** 63 - 1)) ^ int.from_bytes(digest[:8], "little")) & (2 ** 63 - 1)


def random_tensors(wanted: Mapping[str, WeightSpec], seed: int, std: float = 0.02,
                   norm_std: float = 0.01, norm_center: float = 1.0,
                   std_by_fan_in: bool = False) -> Dict[str, torch.Tensor]:
    """``std_by_fan_in`` draws projections with std / sqrt(fan_in): with std 1
    activations keep their size through the layers and attention scores are of
    order one, which tests of attention need."""
    out: Dict[str, torch.Tensor] = {}
    for name in sorted(wanted):
        spec = wanted[name]
        if spec.role == "table":
            raise ValueError(f"{name}: integer tables have no random mode")
        gen = torch.Generator(device="cpu")
        gen.manual_seed(tensor_seed(seed, name))
        x = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if spec.init == "ones":
            out[name] = norm_center + x * norm_std
        elif std_by_fan_in and spec.fan_in > 0:
            out[name] = x * (std / spec.fan_in ** 0.5)
        else:
            out[name] = x * std
    return out


def write_random_model(config: Mapping, seed: int, out_dir: str, std: float = 0.02,
                       norm_std: float = 0.01, norm_center: float = 1.0,
                       std_by_fan_in: bool = False) -> str:
    """``config`` is the content of config.json.  Returns ``out_dir``."""
    from ..engine.model import DecoderModel  # the model names its tensors
    typed = config_from_dict(config)
    spec = typed.to_spec()
    wanted = DecoderModel.weight_specs_of(spec)
    tensors = random_tensors(wanted, seed, std, norm_std, norm_center, std_by_fan_in)
    dtype = _DTYPE[spec.stored_dtype]
    os.makedirs(out_dir, exist_ok=True)
    write_safetensors(os.path.join(out_dir, SINGLE_FILE),
                      {k: v.to(dtype) for k, v in tensors.items()})
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(typed.to_dict(), f, indent=1)
    return out_dir
