"""Reader and writer of the safetensors container.

The format is an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets"}}`` and the raw little-endian tensor
bytes.  NNIS reads the same files through the safetensors crate
(crates/nnis-model/src/safetensors_loader.rs:689-753); here the container is
parsed directly so that loading needs nothing beyond torch and numpy.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Tuple

import numpy as np
import torch

_TORCH = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
          "I32": torch.int32, "I64": torch.int64, "U8": torch.uint8, "F64": torch.float64}
_NAMES = {v: k for k, v in _TORCH.items()}
_MAX_HEADER = 100 << 20


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """Memory-mapped view; ``tensor(name)`` copies one tensor out."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        self._file = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._file.read(8))
        if header_len > min(size - 8, _MAX_HEADER):
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._file.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from None
        header.pop("__metadata__", None)
        self._base = 8 + header_len
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, info in header.items():
            dtype = _TORCH.get(info.get("dtype"))
            if dtype is None:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype "
                                       f"{info.get('dtype')!r}")
            shape = tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            count = int(np.prod(shape, dtype=np.int64)) if shape else 1
            if end - begin != count * dtype.itemsize or self._base + end > size or begin < 0:
                raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self):
        return list(self.entries)

    def meta(self, name: str):
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        dtype, shape, begin, end = self.entries[name]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin,
                            offset=self._base + begin).copy()
        return torch.from_numpy(raw).view(dtype).reshape(shape)

    def close(self):
        self._map.close()
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    header, offset, blobs = {}, 0, []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        blob = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)
    os.replace(tmp, path)
