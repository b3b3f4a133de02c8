"""The cache: per-sequence slots over paged key/value storage, and state.

Each schedule entry of a model may ask for one of two things:

* ``KVRequest`` - keys and values of every position (``window == 0``) or of the
  last ``window`` positions.  Entries with the same (kv_heads, head_dim, window)
  form a *group* with storage and a page pool of its own:
  ``k, v: [entries, pages, kv_heads, page_size, head_dim]``.  A page id is
  valid for every entry of its group, so one page table per group and sequence
  serves all its layers.  A windowed group gives pages back as soon as they fall
  wholly out of the window.
* ``StateRequest`` - a fixed-size tensor per sequence, ``[slots, *shape]``,
  zeroed when a slot is taken.  The Llama decoder asks for none; the area
  exists so that a recurrent mixer needs no change here.

Lengths are per slot (all layers advance together inside a step).  Positions at
or beyond a slot's length are never read, so a reused slot cannot see what its
last owner left (NNIS relies on the same rule:
crates/nnis-rt/src/kv_cache.rs:368-395).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple, Union

import torch

from .slots import CacheFull, FreeList, SlotError

PAGE_SIZE = 64


@dataclass(frozen=True)
class KVRequest:
    kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class CacheSnapshot:
    """What ``CacheManager.snapshot`` keeps of one sequence: its length and a copy of
    its fixed-size state (keys and values need no copy: going back only forgets)."""
    slot: int
    owner: int
    length: int
    states: List[torch.Tensor]


@dataclass
class KVView:
    """What an attention-like part gets: its own layer of a group's storage."""
    group: int
    k: torch.Tensor  # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    page_size: int
    window: int
    ahead: int = 0  # elements from k (and v) to those of the group's layer that runs next; 0: none


@dataclass
class StateView:
    state: torch.Tensor  # [slots, *shape]


class _KVGroup:
    def __init__(self, key: Tuple[int, int, int], entries: List[int], pages: int,
                 dtype: torch.dtype, device: torch.device):
        self.kv_heads, self.head_dim, self.window = key
        self.entries = entries
        self.pool = FreeList(pages, "page")
        shape = (len(entries), pages, self.kv_heads, PAGE_SIZE, self.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        # per slot: logical page index -> page id, -1 where given back
        self.tables: Dict[int, List[int]] = {}

    def first_needed_page(self, length: int) -> int:
        """Pages before this one hold no key that a later position may read."""
        if self.window <= 0:
            return 0
        return max(0, length - self.window + 1) // PAGE_SIZE if length > 0 else 0


class CacheManager:
    def __init__(self, requests: Sequence[Optional[Union[KVRequest, StateRequest]]],
                 dtype: torch.dtype, device: torch.device, max_tokens: int, max_slots: int,
                 max_positions: int):
        if max_tokens <= 0 or max_slots <= 0:
            raise ValueError("max_tokens and max_slots must be positive")
        self.dtype, self.device = dtype, torch.device(device)
        self.max_positions = max_positions
        self.pages_total = -(-max_tokens // PAGE_SIZE)
        self.slots = FreeList(max_slots, "slot")
        self.lengths: List[int] = [0] * max_slots
        # counts what happened to a slot's page tables other than growth at their end
        # (taken, given back, truncated): a copy of a table kept elsewhere is good only
        # for the version it was made at
        self.versions: List[int] = [0] * max_slots
        # counts every change of any page table, growth included: while it stands still a
        # copy of the tables of the same slots needs no look
        self.epoch = 0
        self.owners: List[int] = [0] * max_slots  # how many sequences have held each slot
        self.groups: List[_KVGroup] = []
        self._views: List[Optional[Union[KVView, StateView]]] = []
        by_key: Dict[Tuple[int, int, int], List[int]] = {}
        for i, r in enumerate(requests):
            if isinstance(r, KVRequest):
                by_key.setdefault((r.kv_heads, r.head_dim, r.window), []).append(i)
        group_of: Dict[int, Tuple[int, int]] = {}
        for key, entries in by_key.items():
            g = _KVGroup(key, entries, self.pages_total, dtype, self.device)
            for j, e in enumerate(entries):
                group_of[e] = (len(self.groups), j)
            self.groups.append(g)
        self._states: List[torch.Tensor] = []
        for i, r in enumerate(requests):
            if isinstance(r, KVRequest):
                gi, j = group_of[i]
                g = self.groups[gi]
                nxt = (j + 1) % len(g.entries)  # (after the last layer: the first, in the next step)
                self._views.append(KVView(gi, g.k[j], g.v[j], PAGE_SIZE, g.window,
                                          (nxt - j) * g.k[0].numel()))
            elif isinstance(r, StateRequest):
                t = torch.zeros((max_slots, *r.shape), dtype=r.dtype, device=self.device)
                self._states.append(t)
                self._views.append(StateView(t))
            elif r is None:
                self._views.append(None)
            else:
                raise TypeError(f"schedule entry {i}: unknown cache request {r!r}")

    # -- what parts see ---------------------------------------------------
    def view(self, entry: int):
        return self._views[entry]

    # -- slots --------------------------------------------------------------
    def acquire(self) -> int:
        slot = self.slots.take()
        self.lengths[slot] = 0
        self.versions[slot] += 1
        self.epoch += 1
        self.owners[slot] += 1
        for g in self.groups:
            g.tables[slot] = []
        for t in self._states:
            t[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        if not self.slots.is_held(slot):
            raise SlotError(f"slot {slot} is not held (freed twice?)")
        for g in self.groups:
            for page in g.tables.pop(slot):
                if page >= 0:
                    g.pool.give(page)
        self.lengths[slot] = 0
        self.versions[slot] += 1
        self.epoch += 1
        self.slots.give(slot)

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise SlotError(f"slot {slot} is not held")
        return self.lengths[slot]

    # -- growth -------------------------------------------------------------
    def reserve(self, slots: Sequence[int], new_lengths: Sequence[int]) -> None:
        """Make room for positions below ``new_lengths``; all or nothing."""
        if len(set(slots)) != len(slots):
            raise SlotError(f"a slot appears twice in one step: {list(slots)}")
        need = [0] * len(self.groups)
        for slot, n in zip(slots, new_lengths):
            if not self.slots.is_held(slot):
                raise SlotError(f"slot {slot} is not held")
            if n < self.lengths[slot]:
                raise SlotError(f"slot {slot}: length cannot shrink ({self.lengths[slot]} -> {n})")
            if n > self.max_positions:
                raise CacheFull(f"slot {slot}: {n} positions exceed the model's "
                                f"{self.max_positions}")
            for gi, g in enumerate(self.groups):
                need[gi] += max(0, -(-n // PAGE_SIZE) - len(g.tables[slot]))
        for gi, g in enumerate(self.groups):
            if need[gi] > g.pool.free:
                raise CacheFull(f"{need[gi]} pages wanted, {g.pool.free} of {g.pool.count} free "
                                f"(group {gi}); raise max_tokens")
        for slot, n in zip(slots, new_lengths):
            for g in self.groups:
                table = g.tables[slot]
                more = -(-n // PAGE_SIZE) - len(table)
                if more > 0:
                    table.extend(g.pool.take_many(more))
                    self.epoch += 1

    def commit(self, slots: Sequence[int], new_lengths: Sequence[int]) -> None:
        """The step has been issued: lengths advance, windowed groups give back
        the pages that no later position can read."""
        for slot, n in zip(slots, new_lengths):
            self.lengths[slot] = n
            for g in self.groups:
                if g.window > 0:
                    table = g.tables[slot]
                    for i in range(min(g.first_needed_page(n), len(table))):
                        if table[i] >= 0:
                            g.pool.give(table[i])
                            table[i] = -1
                            self.epoch += 1

    def truncate(self, slot: int, length: int) -> None:
        """Forget the positions from ``length`` on (NNIS: crates/nnis-rt/src/kv_cache.rs:181-183):
        the pages beyond go back to their pools; what a kept page holds beyond the
        length is never read and is written over by the next tokens.  Refused, with
        nothing changed, where going back is not possible: fixed-size state has no
        earlier value (``snapshot`` and ``restore`` are the way back for such a model),
        and a windowed group may have given back pages that the positions after
        ``length`` would read again."""
        if not self.slots.is_held(slot):
            raise SlotError(f"slot {slot} is not held")
        if not 0 <= length <= self.lengths[slot]:
            raise SlotError(f"slot {slot}: cannot truncate {self.lengths[slot]} positions to {length}")
        if length == self.lengths[slot]:
            return
        if self._states:
            raise SlotError("a sequence with fixed-size state cannot go back to an earlier length "
                            "(take a snapshot before the tokens that may be taken back, and restore it)")
        self._forget_from(slot, length)

    def _forget_from(self, slot: int, length: int) -> None:
        keep = -(-length // PAGE_SIZE)
        for gi, g in enumerate(self.groups):
            table = g.tables[slot]
            if any(page < 0 for page in table[g.first_needed_page(length):keep]):
                raise SlotError(f"slot {slot}: group {gi} (window {g.window}) has given back pages that "
                                f"position {length} would read")
        for g in self.groups:
            table = g.tables[slot]
            for page in table[keep:]:
                if page >= 0:
                    g.pool.give(page)
            del table[keep:]
        self.lengths[slot] = length
        self.versions[slot] += 1
        self.epoch += 1

    def snapshot(self, slot: int) -> CacheSnapshot:
        """What is needed to bring this sequence back to where it is now after further
        steps: its length and a copy of its fixed-size state.  The way back for models
        with state of fixed size, which ``truncate`` cannot serve; it works for any
        model (with keys and values alone it is a truncation)."""
        if not self.slots.is_held(slot):
            raise SlotError(f"slot {slot} is not held")
        return CacheSnapshot(slot, self.owners[slot], self.lengths[slot],
                             [t[slot].clone() for t in self._states])

    def restore(self, snapshot: CacheSnapshot) -> None:
        """Back to the snapshot: later positions are forgotten, the state is what it
        was.  Refused, with nothing changed, if the slot has been given back since, is
        shorter than the snapshot, or a windowed group has dropped pages it would need."""
        slot = snapshot.slot
        if not self.slots.is_held(slot) or self.owners[slot] != snapshot.owner:
            raise SlotError(f"slot {slot} is not held by the sequence of this snapshot any more")
        if snapshot.length > self.lengths[slot]:
            raise SlotError(f"slot {slot}: the snapshot holds {snapshot.length} positions, the "
                            f"sequence only {self.lengths[slot]}")
        if snapshot.length < self.lengths[slot]:
            self._forget_from(slot, snapshot.length)
        for t, kept in zip(self._states, snapshot.states):
            t[slot].copy_(kept)

    def page_table(self, group: int, slot: int) -> List[int]:
        return self.groups[group].tables[slot]

    def kv_bytes_per_token(self) -> int:
        """Bytes of keys and values that one position of one sequence holds over all
        layers (a windowed group counted like a full one)."""
        return sum(2 * len(g.entries) * g.kv_heads * g.head_dim * g.k.element_size()
                   for g in self.groups)

    # -- telemetry (crates/nnis-rt/src/kv_telemetry.rs:42-80) ----------------
    def usage(self) -> Dict[str, object]:
        return {
            "slots_held": self.slots.held, "slots_total": self.slots.count,
            "pages_held": [g.pool.held for g in self.groups], "pages_total": self.pages_total,
            "live_tokens": sum(self.lengths[s] for s in range(self.slots.count)
                               if self.slots.is_held(s)),
            "kv_bytes": sum(g.k.numel() * g.k.element_size() * 2 for g in self.groups),
        }

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            held = [p for t in g.tables.values() for p in t if p >= 0]
            if len(set(held)) != len(held):
                raise SlotError("a page is in two page tables")
            if len(held) != g.pool.held:
                raise SlotError(f"{g.pool.held} pages held, {len(held)} in page tables")
