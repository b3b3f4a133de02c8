"""Scratch tensors of a step, kept between steps and grown on demand.

Buffers are looked up by name; a request larger than the buffer on hand
replaces it.  Once a CUDA graph has been captured over the workspace it is
frozen: a request that would move a buffer is an error then, because the graph
holds the old address.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class Workspace:
    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self.frozen = False

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        count = 1
        for s in shape:
            count *= int(s)
        key = (name, dtype)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would move after graph capture")
            # grow with headroom so a slowly growing batch does not reallocate each step
            buf = torch.empty(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def zeros(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that is zero when first handed out and that its users leave
        zero (tickets of kernels that reset them); never moved once made."""
        count = 1
        for s in shape:
            count *= int(s)
        key = (name + "#zeros", dtype, count)
        buf = self._buffers.get(key)
        if buf is None:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would be made after graph capture")
            buf = torch.zeros(max(count, 1), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:count].view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())
