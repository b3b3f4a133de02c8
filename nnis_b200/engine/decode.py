"""Decoding as one CUDA graph per step, with the batch's state on the device.

The rows of a step are dealt to a few *chains*: each chain runs the whole model over
its own rows on a stream of its own, and the graph holds the chains side by side.  A
decode step of a small model is a chain of some hundred short kernels, each waiting
for the one before it; what bounds it is the latency of that chain, not the bytes.
Rows do not depend on one another, so two or four chains of fewer rows each overlap
their latencies, while the weights that the chains read one shortly after the other
come from DRAM once and from L2 afterwards.

A ``GraphDecoder`` holds, for a fixed number of rows, the current token and
position of each row, its slot's page tables and the picked tokens.  One graph
runs embedding, every block, final norm, head and the pick, then moves each live
row on by one; the host launches it once per step, copies the picks to pinned
memory and reads them one step late, so the GPU never waits for the host.  Rows
without a sequence carry position -1: no kernel stores or reads for them, which
is how padding changes no result.

NNIS enqueues its fixed-length greedy loop once and synchronises at the end
(crates/nnis-model/src/runtime.rs:814-846); with a stop token it reads one id
per step (:848-899).  The graph with a one-step lag gives the first form's
overlap with the second form's stops.
"""
from __future__ import annotations

import os
from typing import Optional, Sequence

import torch

from ..cache import PAGE_SIZE
from ..csrc import ops
from .context import StepContext, sm_count
from .workspace import Workspace


def chains_for(rows: int) -> int:
    """How many chains the rows of a decode step are dealt to (``NNIS_DECODE_CHAINS``
    sets it; measured on the SmolLM2-135M shape, see the decode step's notes)."""
    forced = os.environ.get("NNIS_DECODE_CHAINS")
    if forced:
        return max(1, min(int(forced), rows))
    # Measured at context 4,096: on the SmolLM2-135M shape two chains of four rows take
    # 0.84 ms a step against 0.75 ms for one chain of eight (the kernels of one chain keep
    # the other's off the SMs they hold), and two chains of 32 rows gain 3 % over one of 64;
    # on the 360M and 1.7B shapes two chains of 32 lose a quarter (rows beyond 48 take the
    # tcgen05 products, two chains of 32 the decode projections with long rows of K).  One
    # chain is the rule; the switch is for measurements.
    return 1


class GraphDecoder:
    def __init__(self, engine, rows: int, max_context: int, want_logits: bool = False,
                 chains: Optional[int] = None):
        self.engine = engine
        self.want_logits = want_logits
        self.rows = rows
        self.device = engine.device
        self.max_context = min(max_context, engine.spec.max_positions)
        self.cols = max(1, -(-self.max_context // PAGE_SIZE))
        n_groups = len(engine.cache.groups)
        dev = self.device
        # tokens | positions | slots | one page table per group: one buffer, so
        # that the host can replace the whole state with one copy
        self.state_ints = rows * (3 + n_groups * self.cols)
        self.state = torch.full((self.state_ints,), -1, dtype=torch.int32, device=dev)
        self.tokens = self.state[0:rows]
        self.pos = self.state[rows:2 * rows]
        self.slots = self.state[2 * rows:3 * rows]
        self.tables = [self.state[3 * rows + g * rows * self.cols:
                                  3 * rows + (g + 1) * rows * self.cols].view(rows, self.cols)
                       for g in range(n_groups)]
        self.tokens.zero_()
        self.slots.zero_()
        self.seq = torch.arange(rows, dtype=torch.int32, device=dev)
        self.want = torch.arange(rows, dtype=torch.int32, device=dev)
        self.host_state = torch.empty(self.state_ints, dtype=torch.int32, pin_memory=True)
        self._host_np = self.host_state.numpy()
        self._host_state_free = torch.cuda.Event()
        self._host_state_free.record()
        # what the pinned copy holds per (group, row): the slot's table (a new list
        # with every acquisition) and its version in the cache (a truncation shortens
        # the list in place and later pages may differ), how many of its pages, how
        # many dropped in front; None: unknown (rows that were set one by one on the device)
        self._mirror = None
        # the cache's epoch and the slots at the last look at the tables (see upload)
        self._tables_seen = None
        self._windowed = any(g.window > 0 for g in engine.cache.groups)
        self.logits = torch.empty((rows, engine.spec.vocab_size), dtype=torch.float32, device=dev) \
            if want_logits else None
        self.picked = torch.zeros(rows, dtype=torch.int32, device=dev)
        # the chains: consecutive runs of rows, each with a context, buffers and a
        # stream of its own
        n_chains = max(1, min(chains if chains is not None else chains_for(rows), rows))
        per = -(-rows // n_chains)
        self.chains = []
        for a in range(0, rows, per):
            b = min(rows, a + per)
            self.chains.append((a, b, self._context(a, b), torch.cuda.Stream(device=dev) if a else None))
        for _, _, ctx, _ in self.chains:
            ctx.share = len(self.chains)
        self.ctx = self.chains[0][2]          # what a step with one chain runs
        self.workspace = self.ctx.workspace
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0
        # host side of the rows
        self.host_tables = [[[-1] * self.cols for _ in range(rows)] for _ in range(n_groups)]
        self._host_tables_unknown = False  # True: every entry of host_tables is None
        self._pinned_out: Optional[torch.Tensor] = None

    def _context(self, a: int, b: int) -> StepContext:
        """The step context of rows a..b-1 as a batch of their own."""
        n = b - a
        warps_wanted = sm_count(self.device) * 16
        n_heads = max(1, n * self._query_heads())
        splits = int(min(max(1, warps_wanted // n_heads), max(1, -(-self.max_context // 128)), 64))
        return StepContext(
            n_tokens=n, n_seqs=n, tokens=self.tokens[a:b], token_pos=self.pos[a:b],
            token_seq=self.seq[:n], seq_slots=self.slots[a:b],
            page_tables=[t[a:b] for t in self.tables], workspace=Workspace(self.device), decode=True,
            max_context=self.max_context, fixed_splits=splits)

    def _query_heads(self) -> int:
        heads = [getattr(part, "heads", 1) for b in self.engine.model.blocks for part in b.parts()]
        return max(heads) if heads else 1

    # -- the captured step ----------------------------------------------------
    def _run_chain(self, a: int, b: int, ctx: StepContext) -> None:
        self.engine.model.forward_and_pick(
            ctx, self.want[:b - a], self.picked[a:b], self.logits[a:b] if self.logits is not None else None,
            self.tokens[a:b], self.pos[a:b])

    def _body(self) -> None:
        """Every chain on its stream: the first on the current one, the others forked
        from it and joined to it again (inside a capture that makes parallel branches)."""
        main = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(main)
        joins = []
        for a, b, ctx, stream in self.chains[1:]:
            stream.wait_event(fork)
            with torch.cuda.stream(stream):
                self._run_chain(a, b, ctx)
                done = torch.cuda.Event()
                done.record(stream)
                joins.append(done)
        a, b, ctx, _ = self.chains[0]
        self._run_chain(a, b, ctx)
        for done in joins:
            main.wait_event(done)

    def capture(self) -> None:
        if self.graph is not None:
            return
        side = torch.cuda.Stream(device=self.device)
        saved = self.pos.clone()
        self.pos.fill_(-1)  # the warm-up run must not touch the cache, tokens or positions
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._body()
        torch.cuda.current_stream().wait_stream(side)
        for _, _, ctx, _ in self.chains:
            ctx.workspace.frozen = True
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            self._body()
        self.launches_per_step = ops.launch_count() - before
        self.graph = graph
        self.pos.copy_(saved)

    # -- rows ---------------------------------------------------------------------
    def set_row(self, row: int, slot: int, token: int, position: int) -> None:
        """Put a sequence on a row: its next input token and that token's position."""
        cache = self.engine.cache
        self._mirror = None  # the device copy now differs from the pinned one
        update = torch.tensor([token, position, slot], dtype=torch.int32).pin_memory()
        self.tokens[row:row + 1].copy_(update[0:1], non_blocking=True)
        self.pos[row:row + 1].copy_(update[1:2], non_blocking=True)
        self.slots[row:row + 1].copy_(update[2:3], non_blocking=True)
        for g in range(len(self.tables)):
            pages = cache.page_table(g, slot)[:self.cols]
            line = pages + [-1] * (self.cols - len(pages))
            self.host_tables[g][row] = line
            self._host_tables_unknown = False
            self.tables[g][row].copy_(torch.tensor(line, dtype=torch.int32).pin_memory(),
                                      non_blocking=True)

    def clear_row(self, row: int) -> None:
        self._mirror = None
        self.pos[row:row + 1].fill_(-1)

    def sync_pages(self, row: int, slot: int) -> None:
        """After the cache reserved more room for ``slot``: send new page ids."""
        cache = self.engine.cache
        self._mirror = None
        for g in range(len(self.tables)):
            pages = cache.page_table(g, slot)[:self.cols]
            line = self.host_tables[g][row]
            for j, page in enumerate(pages):
                if line[j] != page:
                    line[j] = page
                    self._host_tables_unknown = False
                    self.tables[g][row, j:j + 1].fill_(page)

    def upload(self, tokens: Sequence[int], positions: Sequence[int], slots: Sequence[int]) -> int:
        """Replace the state of all rows from the host in one copy: row r gets
        the r-th sequence; rows beyond them are padding.  Returns the bytes sent.
        The pinned copy is kept between calls, so a step rewrites the tokens and
        positions and only those page-table entries that changed."""
        cache = self.engine.cache
        rows, cols, n = self.rows, self.cols, len(tokens)
        self._host_state_free.synchronize()  # the copy out of the pinned buffer is over
        st = self._host_np
        fresh = self._mirror is None
        if fresh:
            st[:] = -1
            self._mirror = [[None] * rows for _ in self.tables]
        st[0:n] = tokens
        st[rows:rows + n] = positions
        same_rows = not fresh and self._tables_seen is not None and self._tables_seen[1] == tuple(slots)
        if not same_rows:  # (else the padding rows and the slots stand as they were written)
            st[n:rows] = 0
            st[rows + n:2 * rows] = -1
            st[2 * rows:2 * rows + n] = slots
            st[2 * rows + n:3 * rows] = 0
        # (no page table has changed since these slots' tables were last looked at, and no
        # windowed group drops pages by length alone: nothing to look at)
        seen = (cache.epoch, tuple(slots))
        groups = () if not fresh and seen == self._tables_seen and not self._windowed else enumerate(cache.groups)
        self._tables_seen = seen
        for g, group in groups:
            base = 3 * rows + g * rows * cols
            mirror = self._mirror[g]
            for r, slot in enumerate(slots):
                table = cache.page_table(g, slot)
                count = min(len(table), cols)
                dropped = min(group.first_needed_page(cache.lengths[slot]), count) if group.window > 0 else 0
                known = mirror[r]
                version = cache.versions[slot]
                same = known is not None and known[0] is table and known[3] == version
                if same and known[1] == count and known[2] == dropped:
                    continue
                line = st[base + r * cols:base + (r + 1) * cols]
                if same and known[1] <= count and known[2] <= dropped:
                    line[known[1]:count] = table[known[1]:count]
                    line[known[2]:dropped] = -1
                else:
                    line[:count] = table[:count]
                    line[count:] = -1
                mirror[r] = (table, count, dropped, version)
        ops.copy_async(self.state, self.host_state)
        self._host_state_free.record()
        if not self._host_tables_unknown:  # the partial-update path starts from scratch next time
            for g in range(len(self.tables)):
                self.host_tables[g] = [[None] * cols for _ in range(rows)]
            self._host_tables_unknown = True
        return self.state_ints * 4

    # -- stepping -------------------------------------------------------------------
    def launch(self) -> None:
        self.capture()
        self.graph.replay()

    def picks_to_host(self, into: torch.Tensor) -> torch.cuda.Event:
        """Copy this step's picks into pinned ``into``; the event says when."""
        into.copy_(self.picked, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return event
