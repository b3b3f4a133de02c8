"""Architecture-neutral description of a decoder: parts, layers, run order.

A typed architecture configuration (``LlamaConfig`` for instance) is turned
into a ``ModelSpec``.  Everything below the registry works from the spec only:
no part and no engine file names an architecture.  The spec is plain data:

* a ``PartSpec`` is a kind (a key of one of the part registries in
  ``nnis_b200.parts``) and the sizes and constants of that part;
* a ``LayerSpec`` names the arrangement of a block and, by role, the parts that
  this arrangement is made of (``parts``: role -> ``PartSpec``; the arrangement's
  class says which roles it knows), chosen layer by layer, so two layers of one
  model may differ in every part and in how many they have;
* ``schedule`` is the order in which layers run.  An entry may name a layer a
  second time (its weights are shared, its cache is its own), and
  ``cache_of`` lets an entry read the cache that an earlier entry wrote.

NNIS keeps the same facts as a capability record next to a fixed decoder
(crates/nnis-model/src/decoder_capabilities.rs:8-75); here they drive the build.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """One block: ``prefix`` is the tensor-name prefix of its weights, ``block`` the
    arrangement (a key of ``parts.BLOCKS``) and ``parts`` what it is made of, by the
    roles that this arrangement knows (``prenorm``: mixer_norm, mixer, ffn_norm, ffn)."""
    prefix: str
    block: str
    parts: Mapping[str, PartSpec]

    def part(self, role: str) -> PartSpec:
        if role not in self.parts:
            raise KeyError(f"layer {self.prefix!r} ({self.block}) has no part {role!r}; "
                           f"it has {sorted(self.parts)}")
        return self.parts[role]


@dataclass(frozen=True)
class ScheduleEntry:
    """Run ``layer``; read the cache of schedule entry ``cache_of`` instead of
    writing one of its own when that is set (it must come earlier)."""
    layer: int
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the run order (schedule) is empty")
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {entry.layer}; the model has "
                                 f"{len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < i:
                    raise ValueError(f"schedule[{i}].cache_of={entry.cache_of} must name an "
                                     f"earlier schedule entry")
                if self.schedule[entry.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of={entry.cache_of} names an entry "
                                     f"that owns no cache itself")
        for t in self.stop_token_ids:
            if not 0 <= t < self.vocab_size:
                raise ValueError(f"stop token {t} is outside the vocabulary of {self.vocab_size}")
