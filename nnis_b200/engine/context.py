"""What a step tells the parts: where each packed token sits.

All tensors are int32 on the device.  ``token_pos[n]`` is the position of token
n in its sequence (-1 marks a padding row, which no kernel stores or reads);
``token_seq[n]`` is the row of its sequence in this step's batch, which indexes
``page_tables[g]`` (one table per cache group) and ``seq_slots``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .workspace import Workspace

_SM_COUNT = {}
# tuning of the decode attention split: CTAs per SM to aim for, fewest keys per slice
_FILL_ENV = os.environ.get("NNIS_DECODE_FILL")
_FILL = int(_FILL_ENV or "8")
_SLICE_KEYS = int(os.environ.get("NNIS_DECODE_SLICE_KEYS", "256"))


def sm_count(device: torch.device) -> int:
    key = torch.device(device).index or 0
    if key not in _SM_COUNT:
        _SM_COUNT[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _SM_COUNT[key]


@dataclass
class StepContext:
    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor
    token_pos: torch.Tensor
    token_seq: torch.Tensor
    seq_slots: torch.Tensor
    page_tables: List[torch.Tensor]
    workspace: Workspace
    decode: bool
    max_context: int  # longest sequence after this step (host knowledge)
    # host-side copies, for parts that loop on the host (toy mixers in tests)
    host_slots: Sequence[int] = field(default_factory=list)
    host_counts: Sequence[int] = field(default_factory=list)
    host_starts: Sequence[int] = field(default_factory=list)
    fixed_splits: int = 0  # > 0: a captured graph fixed the split count
    share: int = 1  # steps that run side by side on the device (chains of a decode graph)
    # per sequence of the batch (device int32 [n_seqs]): the packed row of its
    # first token in this step, that token's position, its number of tokens.
    # None in decode steps and in contexts built without them.
    seq_first_row: Optional[torch.Tensor] = None
    seq_start: Optional[torch.Tensor] = None
    seq_count: Optional[torch.Tensor] = None
    # what the parts asked for with ``step_tables``: device copies and the arrays
    tables: Dict[str, torch.Tensor] = field(default_factory=dict)
    host_tables: Dict[str, object] = field(default_factory=dict)
    # A norm shared out between the projection before it and the one after it (decode
    # steps; see ``parts.base.SharedNorm``).  ``next_norm``: set by the model while a block
    # runs, the norm that the block after it applies first if that block will take it begun.
    # ``emit_for``: set by a block while one of its parts runs, the norm that reads the
    # residual after that part.  ``shared_norm``: what the part left, until the block that
    # owns the norm takes it.
    next_norm: object = None
    emit_for: object = None
    shared_norm: object = None

    def take_shared_norm(self, norm):
        """What the part before left of ``norm``'s work, or None; nothing is kept."""
        begun, self.shared_norm = self.shared_norm, None
        return begun if begun is not None and begun.norm is norm else None

    def attention_splits(self, query_rows: int) -> int:
        """How many ways to cut each query's key range so the GPU is full when
        there are few queries and many keys (decoding)."""
        if self.fixed_splits > 0:
            return self.fixed_splits
        if not self.decode:
            return 1
        warps_wanted = sm_count(self.tokens.device) * 16
        by_rows = max(1, warps_wanted // max(1, query_rows))
        by_keys = max(1, -(-self.max_context // 128))
        return int(min(by_rows, by_keys, 64))

    def decode_splits(self, ctas: int, resident: int = 0, page_size: int = 64) -> int:
        """The same for the decode kernels, whose CTAs (4 warps) each own a kv head
        of a sequence, at least 256 keys a slice.  ``resident``: how many CTAs of the
        kernel the device holds at once (see ``decode_plan``).  Without it: fill the
        SMs a few times over."""
        if resident > 0 and _FILL_ENV is None:
            return self.decode_plan(ctas, resident, page_size)[0]
        by_keys = max(1, -(-self.max_context // _SLICE_KEYS))
        by_ctas = max(1, sm_count(self.tokens.device) * _FILL // max(1, ctas))
        return int(min(by_ctas, by_keys, 64))

    def decode_plan(self, ctas: int, resident: int, page_size: int = 64):
        """(slices, cost) for a decode kernel of which ``resident`` CTAs run together.
        The CTAs run in waves, a wave lasts as long as one slice, and a slice costs
        its pages plus about four pages' time of start and merge: the number of
        slices with the least waves x (pages per slice + 4) is taken, more slices only
        for a gain of 3 %.  Measured on the 135M, 360M and 1.7B shapes at batch 8 to
        64 this picks the fastest or second fastest of all choices (at batch 64 of
        the 135M shape two slices, one wave; three slices, a wave and a third, cost
        12 % of the step).  The cost serves to compare launch shapes of one kernel."""
        by_keys = max(1, -(-self.max_context // _SLICE_KEYS))
        pages = max(1, -(-self.max_context // page_size))
        resident = max(1, resident // max(1, self.share))  # its share of the device
        best, best_cost = 1, None
        for s in range(1, int(min(by_keys, 64)) + 1):
            waves = -(-ctas * s // max(1, resident))
            cost = waves * (pages / s + 4.0)
            if best_cost is None or cost < 0.97 * best_cost:  # more slices only for a clear gain
                best, best_cost = s, cost
        return best, best_cost
