"""Arrangements of the four parts of a layer.

``prenorm``: h += mixer(norm1(h)); h += ffn(norm2(h)) - the order of NNIS's
decoder (crates/nnis-model/src/runtime.rs:946-1097).  Another arrangement
(post-norm, parallel attention and MLP) is another class registered here.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..weights.loader import WeightSpec
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Part


class PreNormBlock:
    def __init__(self, layer_spec, dtype: torch.dtype, device: torch.device):
        p = layer_spec.prefix
        self.mixer_norm = NORMS.build(layer_spec.mixer_norm.kind, layer_spec.mixer_norm.params, p,
                                      dtype, device)
        self.mixer = MIXERS.build(layer_spec.mixer.kind, layer_spec.mixer.params, p, dtype, device)
        self.ffn_norm = NORMS.build(layer_spec.ffn_norm.kind, layer_spec.ffn_norm.params, p, dtype,
                                    device)
        self.ffn = FEED_FORWARDS.build(layer_spec.ffn.kind, layer_spec.ffn.params, p, dtype, device)
        self.dtype = dtype

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs: Dict[str, WeightSpec] = {}
        for part in self.parts():
            specs.update(part.weight_specs())
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)

    def parameter_bytes(self) -> int:
        return sum(part.parameter_bytes() for part in self.parts())

    def step_tables(self, counts, starts, have=()) -> Dict[str, object]:
        tables: Dict[str, object] = {}
        for part in self.parts():
            wants = getattr(part, "step_tables", None)
            if wants is not None:
                for name, arr in wants(counts, starts, tuple(have) + tuple(tables)).items():
                    tables.setdefault(name, arr)
        return tables

    def forward(self, hidden: torch.Tensor, ctx, cache) -> None:
        n, width = hidden.shape
        normed = ctx.workspace.get("normed", (n, width), self.dtype)
        # a part may fold the norm before it into its first kernel (decode steps)
        if getattr(self.mixer, "fuses_norm", None) and self.mixer.fuses_norm(self.mixer_norm, ctx, n):
            self.mixer.forward_normed(hidden, self.mixer_norm, ctx, cache)
        else:
            self.mixer_norm.forward(hidden, normed)
            self.mixer.forward(normed, ctx, hidden, cache)
        if getattr(self.ffn, "fuses_norm", None) and self.ffn.fuses_norm(self.ffn_norm, ctx, n):
            self.ffn.forward_normed(hidden, self.ffn_norm, ctx)
        else:
            self.ffn_norm.forward(hidden, normed)
            self.ffn.forward(normed, ctx, hidden)


BLOCKS.register("prenorm", PreNormBlock)
