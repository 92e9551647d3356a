"""Cache manager: paged keys/values per group of runs, block tables, state slots.

What the reference does (somi_inference/core/paged_attention.py:112-296): one
allocator shared by all layers, one tensor per layer of shape
[num_blocks, 2, block_size, kv_heads, head_dim], a dict from sequence id to its
block list and token count, two-phase use (`allocate_slots` before the forward,
`advance_tokens` after it), and `free_sequence` when a sequence ends.

What this manager does differently:

* Runs of the schedule are put into *groups* by what they need (kv heads, key
  width, value width, window).  Each group has its own page pool, its own device
  storage and its own block table per request.  Where keys and values have the
  same width the storage is one tensor `[runs_in_group, 2, num_pages, kv_heads,
  page_size, head_dim]` (a page of one kv head is contiguous, and one tensor map
  covers keys and values); where they differ, keys and values are two tensors
  `[runs_in_group, num_pages, kv_heads, page_size, width]`.  Runs that attend over all keys and runs that only
  ever read a window therefore never compete for, or waste, each other's pages.
* A window group gives pages back as soon as every position in them has fallen
  out of the window (`commit`); the block table keeps -1 in their place.
* Every request also gets a *state slot*: an index into per-run tensors of fixed
  size `[num_slots, ...]` for mixers whose memory does not grow with length.
  The slot's tensors are zeroed when the request registers.
* `reserve` is all-or-nothing across groups: either every group has the pages
  for the new tokens or `OutOfPages` is raised and nothing changed.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import CacheNeeds, PagedKVNeeds
from .pages import OutOfPages, PagePool

FREED = -1   # block-table entry of a page that was given back (or never taken)


@dataclass
class PagedView:
    """What a mixer gets for one run that keeps paged keys and values."""

    group: int                 # index into StepBatch.groups
    keys: torch.Tensor         # [num_pages, kv_heads, page_size, head_dim]
    values: torch.Tensor       # [num_pages, kv_heads, page_size, value width]
    page_size: int
    window: int | None
    # the group's whole tensor, for tensor maps over keys and values at once; None where keys
    # and values differ in width and are stored apart
    storage: torch.Tensor | None = None


@dataclass
class CacheView:
    paged: PagedView | None = None
    state: dict[str, torch.Tensor] = field(default_factory=dict)   # name -> [num_slots, ...]


class _Group:
    def __init__(self, needs: PagedKVNeeds, runs: list[int], num_pages: int, page_size: int,
                 max_requests: int, max_blocks: int, dtype: torch.dtype,
                 device: torch.device) -> None:
        self.needs = needs
        self.runs = runs
        self.pool = PagePool(num_pages)
        self.page_size = page_size
        if needs.value_width == needs.head_dim:
            self.storage = torch.zeros(
                (len(runs), 2, num_pages, needs.num_kv_heads, page_size, needs.head_dim),
                dtype=dtype, device=device)
            self.keys, self.values = self.storage[:, 0], self.storage[:, 1]
        else:
            self.storage = None
            self.keys = torch.zeros((len(runs), num_pages, needs.num_kv_heads, page_size,
                                     needs.head_dim), dtype=dtype, device=device)
            self.values = torch.zeros((len(runs), num_pages, needs.num_kv_heads, page_size,
                                       needs.value_width), dtype=dtype, device=device)
        # host block tables, one row per state slot (= per live request)
        self.tables = np.full((max_requests, max_blocks), FREED, dtype=np.int32)
        self.first_live = np.zeros(max_requests, dtype=np.int64)  # first block not yet given back
        self.num_blocks = np.zeros(max_requests, dtype=np.int64)  # blocks ever taken

    def blocks_needed(self, slot: int, new_len: int) -> int:
        want = -(-new_len // self.page_size)
        return max(0, want - int(self.num_blocks[slot]))


class CacheManager:
    def __init__(self, needs_per_run: list[CacheNeeds | None], owner_of_run: list[int | None],
                 *, num_pages: int, page_size: int, max_requests: int, max_positions: int,
                 dtype: torch.dtype, device: torch.device | str) -> None:
        """`needs_per_run[i]` is what run i's mixer asked for (None: nothing);
        `owner_of_run[i]` is the run whose cache run i reads (None: its own)."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.max_requests = max_requests
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_blocks = -(-max_positions // page_size)
        self._slots = PagePool(max_requests)          # state slots reuse the pool logic
        self._slot_of: dict[object, int] = {}
        self._len: dict[object, int] = {}
        self._reserved: dict[object, int] = {}
        self.groups: list[_Group] = []
        self._views: list[CacheView | None] = [None] * len(needs_per_run)

        by_key: dict[tuple, list[int]] = {}
        for run, (needs, owner) in enumerate(zip(needs_per_run, owner_of_run)):
            if owner is None and needs is not None and needs.paged is not None:
                p = needs.paged
                by_key.setdefault((p.num_kv_heads, p.head_dim, p.window, p.value_width),
                                  []).append(run)
        for key, runs in by_key.items():
            needs = PagedKVNeeds(*key)
            self.groups.append(_Group(needs, runs, num_pages, page_size, max_requests,
                                      self.max_blocks, dtype, self.device))
        for run, (needs, owner) in enumerate(zip(needs_per_run, owner_of_run)):
            if owner is not None or needs is None:
                continue
            view = CacheView()
            if needs.paged is not None:
                for gi, g in enumerate(self.groups):
                    if run in g.runs:
                        r = g.runs.index(run)
                        view.paged = PagedView(gi, g.keys[r], g.values[r], page_size,
                                               g.needs.window, g.storage)
            if needs.state is not None:
                for name, (shape, sdtype) in needs.state.tensors.items():
                    view.state[name] = torch.zeros((max_requests, *shape), dtype=sdtype,
                                                   device=self.device)
            self._views[run] = view
        for run, owner in enumerate(owner_of_run):
            if owner is not None:
                self._views[run] = self._views[owner]

    # ------------------------------------------------------------------ views
    def view(self, run: int) -> CacheView | None:
        return self._views[run]

    # --------------------------------------------------------------- requests
    def is_registered(self, req: object) -> bool:
        return req in self._slot_of

    def register(self, req: object) -> int:
        """Admit a request: give it a state slot (zeroed).  Returns the slot."""
        if req in self._slot_of:
            raise ValueError(f"request {req!r} is already registered")
        try:
            (slot,) = self._slots.take(1)
        except OutOfPages:
            raise OutOfPages(f"all {self.max_requests} request slots are in use") from None
        self._slot_of[req] = slot
        self._len[req] = 0
        self._reserved[req] = 0
        for g in self.groups:
            g.tables[slot, :] = FREED
            g.first_live[slot] = 0
            g.num_blocks[slot] = 0
        for view in {id(v): v for v in self._views if v is not None}.values():
            for t in view.state.values():
                t[slot].zero_()
        return slot

    def slot(self, req: object) -> int:
        return self._slot_of[req]

    def length(self, req: object) -> int:
        """Tokens of `req` whose keys/values (or state) are in the cache."""
        return self._len[req]

    def live_requests(self) -> list[object]:
        return list(self._slot_of)

    def pages_needed(self, req: object, n_tokens: int) -> list[int]:
        """Pages each group would have to take to hold `n_tokens` more tokens."""
        slot = self._slot_of[req]
        new_len = self._len[req] + n_tokens
        return [g.blocks_needed(slot, new_len) for g in self.groups]

    def free_pages(self) -> list[int]:
        return [g.pool.num_free for g in self.groups]

    def reserve(self, req: object, n_tokens: int) -> None:
        """Take the pages that positions [length, length + n_tokens) need, in every group."""
        if n_tokens <= 0:
            raise ValueError("reserve needs a positive token count")
        if self._reserved[req]:
            raise RuntimeError(f"request {req!r} has an uncommitted reservation")
        slot = self._slot_of[req]
        new_len = self._len[req] + n_tokens
        if -(-new_len // self.page_size) > self.max_blocks:
            raise ValueError(f"request {req!r} would reach {new_len} tokens; the cache is laid "
                             f"out for {self.max_blocks * self.page_size}")
        needed = [g.blocks_needed(slot, new_len) for g in self.groups]
        for g, n in zip(self.groups, needed):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {req!r} needs {n} pages, {g.pool.num_free} free "
                                 f"(window={g.needs.window})")
        for g, n in zip(self.groups, needed):
            if n:
                first = int(g.num_blocks[slot])
                g.tables[slot, first:first + n] = g.pool.take(n)
                g.num_blocks[slot] = first + n
        self._reserved[req] = n_tokens

    def cancel(self, req: object) -> None:
        """Undo an uncommitted reservation: pages beyond the committed length go back."""
        if not self._reserved[req]:
            return
        self._reserved[req] = 0
        slot = self._slot_of[req]
        keep = -(-self._len[req] // self.page_size)
        for g in self.groups:
            last = int(g.num_blocks[slot])
            if last > keep:
                g.pool.give_back([int(p) for p in g.tables[slot, keep:last]])
                g.tables[slot, keep:last] = FREED
                g.num_blocks[slot] = keep

    def commit(self, req: object) -> None:
        """The reserved tokens were written: advance the length, drop pages out of window."""
        n = self._reserved[req]
        if not n:
            raise RuntimeError(f"request {req!r} has nothing reserved")
        self._reserved[req] = 0
        self._len[req] += n
        slot = self._slot_of[req]
        for g in self.groups:
            if g.needs.window is None:
                continue
            # the next query sits at position `length` and reads keys > length - window
            first_needed = max(0, self._len[req] - g.needs.window + 1) // self.page_size
            first = int(g.first_live[slot])
            if first_needed > first:
                g.pool.give_back([int(p) for p in g.tables[slot, first:first_needed]])
                g.tables[slot, first:first_needed] = FREED
                g.first_live[slot] = first_needed

    def release(self, req: object) -> None:
        """The request ended (or was preempted): everything it holds goes back."""
        slot = self._slot_of.pop(req)
        del self._len[req]
        del self._reserved[req]
        for g in self.groups:
            first, last = int(g.first_live[slot]), int(g.num_blocks[slot])
            g.pool.give_back([int(p) for p in g.tables[slot, first:last]])
            g.tables[slot, :last] = FREED
            g.first_live[slot] = 0
            g.num_blocks[slot] = 0
        self._slots.give_back([slot])

    # ------------------------------------------------------------ batch views
    def block_tables(self, group: int, slots: np.ndarray, width: int) -> np.ndarray:
        """Rows of the group's block table for `slots`, cut to `width` columns."""
        return self.groups[group].tables[slots, :width]

    def blocks_in_use(self, group: int, slot: int) -> int:
        return int(self.groups[group].num_blocks[slot])

    def held_pages(self, req: object, group: int) -> list[int]:
        slot = self._slot_of[req]
        g = self.groups[group]
        return [int(p) for p in g.tables[slot, int(g.first_live[slot]):int(g.num_blocks[slot])]]

    def check_consistency(self) -> None:
        """Every page is either free or held by exactly one live request (used by tests)."""
        for gi, g in enumerate(self.groups):
            seen: set[int] = set()
            for req in self._slot_of:
                for p in self.held_pages(req, gi):
                    if p in seen:
                        raise AssertionError(f"page {p} of group {gi} is held twice")
                    if not g.pool.is_held(p):
                        raise AssertionError(f"page {p} of group {gi} is in a table but free")
                    seen.add(p)
            if len(seen) != g.pool.num_held:
                raise AssertionError(f"group {gi}: {g.pool.num_held} pages held by the pool, "
                                     f"{len(seen)} found in tables (a page was lost)")
