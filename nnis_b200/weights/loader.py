"""Weights by tensor name, with one error that tells everything wrong at once.

The model says which tensors it wants (``WeightSpec`` by full name); the loader
finds them in ``model.safetensors`` or in the shards that
``model.safetensors.index.json`` names (or, in a folder without those, in NNIS's
own ``model.json`` with its raw tensor files: ``nnis_directory.py``), and raises a single ``WeightError``
listing missing tensors, unexpected tensors and wrong shapes or dtypes.  NNIS
reports the same faults one at a time
(crates/nnis-model/src/safetensors_loader.rs:389-438 files, :711-724 shape and
dtype, :831-856 missing and unconsumed).

Kept dtypes: matrices and tables of the model take the compute dtype (bfloat16
stays bfloat16; float32 runs widen bfloat16 exactly); vectors (norm weights,
biases) are held in float32, which is exact for either stored dtype, so a tensor
stored in 32-bit stays 32-bit; integer tensors become int32.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from .nnis_directory import MANIFEST, NnisDirectoryError, NnisDirectorySource
from .safetensors_io import SafetensorsError, SafetensorsFile

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"
# Buffers that exporters store although they are no parameters.
_IGNORED = (re.compile(r".*\.rotary_emb\.inv_freq$"),)


class WeightError(ValueError):
    pass


@dataclass(frozen=True)
class WeightSpec:
    shape: Tuple[int, ...]
    role: str  # "matrix" | "vector" | "table" (integer)
    init: str = "normal"  # random mode: "normal" around 0, "ones" around 1
    fan_in: int = 0  # random mode: inputs summed per output (0: not a projection)


def _discover(model_dir: str) -> List[str]:
    single = os.path.join(model_dir, SINGLE_FILE)
    index = os.path.join(model_dir, INDEX_FILE)
    has_single, has_index = os.path.isfile(single), os.path.isfile(index)
    if has_single and has_index:
        raise WeightError(f"{model_dir}: both {SINGLE_FILE} and {INDEX_FILE} are present")
    if has_single:
        return [single]
    if not has_index:
        raise WeightError(f"{model_dir}: neither {SINGLE_FILE} nor {INDEX_FILE} found")
    with open(index, "r", encoding="utf-8") as f:
        weight_map = json.load(f).get("weight_map")
    if not isinstance(weight_map, dict) or not weight_map:
        raise WeightError(f"{index}: weight_map is missing or empty")
    shards = []
    for shard in sorted(set(weight_map.values())):
        if os.path.basename(shard) != shard or shard in (".", ".."):
            raise WeightError(f"{index}: shard {shard!r} is not a plain file name")
        shards.append(os.path.join(model_dir, shard))
    return shards


def _has_safetensors(model_dir: str) -> bool:
    return os.path.isfile(os.path.join(model_dir, SINGLE_FILE)) or \
        os.path.isfile(os.path.join(model_dir, INDEX_FILE))


def _kept_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if role == "table":
        return torch.int32
    if role == "vector":
        return torch.float32
    return compute


def _open_and_check(model_dir: str, wanted: Mapping[str, WeightSpec]):
    """Opens the weight files and checks names, shapes and dtypes against what the
    model wants: (open files, file of each tensor, ignored names) or one WeightError."""
    files = []
    try:
        if not _has_safetensors(model_dir) and os.path.isfile(os.path.join(model_dir, MANIFEST)):
            files.append(NnisDirectorySource(model_dir))  # NNIS's own folder: model.json + raw files
        else:
            for path in _discover(model_dir):
                if os.path.islink(path):
                    raise WeightError(f"{path}: symbolic links are not followed")
                files.append(SafetensorsFile(path))
    except (SafetensorsError, NnisDirectoryError) as e:
        for f in files:
            f.close()
        raise WeightError(str(e)) from None
    except WeightError:
        for f in files:
            f.close()
        raise
    try:
        where: Dict[str, SafetensorsFile] = {}
        duplicate: List[str] = []
        for f in files:
            for name in f.names():
                if name in where:
                    duplicate.append(name)
                where[name] = f
        missing = sorted(n for n in wanted if n not in where)
        ignored = sorted(n for n in where if n not in wanted and any(p.match(n) for p in _IGNORED))
        unexpected = sorted(n for n in where if n not in wanted and n not in ignored)
        wrong: List[str] = []
        for name, spec in wanted.items():
            if name not in where:
                continue
            dtype, shape = where[name].meta(name)
            if tuple(shape) != tuple(spec.shape):
                wrong.append(f"{name}: shape {list(shape)}, expected {list(spec.shape)}")
            elif spec.role == "table" and dtype.is_floating_point:
                wrong.append(f"{name}: dtype {dtype}, expected an integer type")
            elif spec.role != "table" and dtype not in (torch.float32, torch.bfloat16):
                wrong.append(f"{name}: dtype {dtype}, expected float32 or bfloat16")
        if missing or unexpected or wrong or duplicate:
            lines = [f"{model_dir}: the weights do not fit the model"]
            if missing:
                lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
            if unexpected:
                lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
            if wrong:
                lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
            if duplicate:
                lines.append(f"  stored twice ({len(duplicate)}): " + ", ".join(sorted(duplicate)))
            raise WeightError("\n".join(lines))
        return files, where, ignored
    except Exception:
        for f in files:
            f.close()
        raise


def check_weights(model_dir: str, wanted: Mapping[str, WeightSpec]) -> Dict[str, object]:
    """The loader's checks without reading a tensor: raises the same WeightError,
    else says what it found (files, tensors taken and ignored, stored dtypes and
    bytes).  NNIS's preflight of a model folder does the same on the CPU
    (crates/nnis-cli/src/bin/nnis-hf.rs:345-478)."""
    files, where, ignored = _open_and_check(model_dir, wanted)
    try:
        dtypes, stored_bytes = set(), 0
        for name in wanted:
            dtype, shape = where[name].meta(name)
            dtypes.add(str(dtype).replace("torch.", ""))
            count = 1
            for extent in shape:
                count *= int(extent)
            stored_bytes += count * dtype.itemsize
        return {"weight_files": [os.path.basename(f.path) for f in files],
                "recognized_tensors": len(wanted), "ignored_tensors": len(ignored),
                "stored_dtypes": sorted(dtypes), "stored_bytes": stored_bytes}
    finally:
        for f in files:
            f.close()


def load_weights(model_dir: str, wanted: Mapping[str, WeightSpec], compute_dtype: torch.dtype,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    files, where, _ = _open_and_check(model_dir, wanted)
    try:
        out: Dict[str, torch.Tensor] = {}
        for name, spec in wanted.items():
            t = where[name].tensor(name)
            out[name] = t.to(_kept_dtype(spec.role, t.dtype, compute_dtype)).to(device).contiguous()
        return out
    finally:
        for f in files:
            f.close()
