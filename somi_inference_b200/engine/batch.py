"""The batch of one step: flat tokens of several requests and where their cache lies.

The reference has two separate forward entry points, one whole prompt or B
single tokens, described by `ForwardContext(mode, attn_fn, posi_idx)`
(somi_inference/models/qwen2.py:27-43; somi_inference/models/qwen2_adapter.py:64-146)
and rebuilds block tables in every layer (qwen2_adapter.py:117).  Here one
descriptor serves any mixture: each request contributes `q_len >= 1` consecutive
tokens that continue from its cached length.  Everything is laid out once per
step in one pinned int32 buffer and copied to the device in one transfer.

Requests with more than one token come first ("prefill" range), single-token
requests after them ("decode" range), so that kernels specialised for either
find a contiguous range; `logit_rows` keeps the caller's order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager


@dataclass
class StepEntry:
    """One request's share of a step."""

    request: object                 # any hashable id
    tokens: Sequence[int]           # its next tokens (>= 1)
    want: Sequence[int] = ()        # indices into `tokens` whose logits are wanted


@dataclass
class GroupBatch:
    block_table: torch.Tensor       # int32 [R, width] page ids, -1 where none
    slot_map: torch.Tensor          # int32 [T] page * page_size + offset of every token
    width: int


@dataclass
class HostBatch:
    """Host copies of the small arrays, for parts that plan on the host."""

    cu_q: np.ndarray
    ctx_len: np.ndarray
    state_slot: np.ndarray
    requests: list


@dataclass
class StepBatch:
    num_tokens: int
    num_requests: int
    num_prefill_requests: int       # requests [0, this) have q_len > 1
    num_prefill_tokens: int         # their tokens are rows [0, this)
    max_q_len: int
    max_kv_len: int
    token_ids: torch.Tensor         # int32 [T]
    positions: torch.Tensor         # int32 [T]
    token_request: torch.Tensor     # int32 [T] index of the token's request in this batch
    cu_q: torch.Tensor              # int32 [R+1]
    ctx_len: torch.Tensor           # int32 [R] tokens cached before this step
    state_slot: torch.Tensor        # int32 [R]
    logit_rows: torch.Tensor        # int32 [K] rows whose logits are returned, caller's order
    tiles: dict[int, torch.Tensor]  # q-tile size -> int32 [n_tiles, 3] (request, first row, rows)
    groups: list[GroupBatch]
    host: HostBatch
    # the sizes that fix every offset in the buffer, then the multi-token requests and their tokens:
    # two steps with equal keys launch the same kernels with the same arguments
    layout_key: tuple = field(default_factory=tuple)


_NO_TILES = np.zeros((0, 3), dtype=np.int64)


def _align(n: int, a: int = 4) -> int:
    return -(-n // a) * a


class BatchBuilder:
    """Fills pinned host memory and issues one host-to-device copy per step."""

    def __init__(self, cache: CacheManager, *, device: torch.device | str,
                 q_tile_sizes: Sequence[int], capacity_ints: int = 1 << 20,
                 vocab_size: int | None = None, max_positions: int | None = None) -> None:
        self.cache = cache
        self.device = torch.device(device)
        self.q_tile_sizes = tuple(q_tile_sizes)
        self.vocab_size = vocab_size
        self.max_positions = max_positions
        self.width_step = max(1, 512 // cache.page_size)     # table columns come in steps of 512 tokens
        self._capacity = 0
        self._turn = 0
        self.uploads = 0
        self._decode_views: dict = {}
        self._alloc(capacity_ints)

    def _alloc(self, capacity: int) -> None:
        pin = self.device.type == "cuda"
        self._host = [torch.empty(capacity, dtype=torch.int32, pin_memory=pin) for _ in range(2)]
        self._events = [None, None]
        self._event_pool = [torch.cuda.Event(), torch.cuda.Event()] if pin else [None, None]
        self._stream_raw, self._stream_obj = None, None
        self._device_index = (self.device.index if self.device.index is not None
                              else torch.cuda.current_device()) if self.device.type == "cuda" else -1
        self._dev = torch.empty(capacity, dtype=torch.int32, device=self.device)
        self._capacity = capacity
        self.generation = getattr(self, "generation", 0) + 1    # device addresses changed

    @property
    def h2d_bytes_last(self) -> int:
        return self._last_bytes

    def build(self, entries: Sequence[StepEntry]) -> tuple[StepBatch, list[int]]:
        """Lay out the batch.  Pages for the new tokens must already be reserved.

        Returns the batch and, for each wanted logit in the caller's order
        (entries in order, `want` in order), nothing more: `logit_rows` already
        holds them in that order.  The second value is the order in which the
        entries were placed (indices into `entries`).
        """
        if not entries:
            raise ValueError("a step needs at least one entry")
        if all(len(e.tokens) == 1 for e in entries):
            return self._build_decode(entries)
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) <= 1, i))
        R = len(entries)
        q_lens = np.array([len(entries[i].tokens) for i in order], dtype=np.int64)
        if (q_lens < 1).any():
            raise ValueError("every entry of a step needs at least one token")
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
        T = int(q_lens.sum())
        cu_q = np.zeros(R + 1, dtype=np.int64)
        np.cumsum(q_lens, out=cu_q[1:])
        ctx = np.array([self.cache.length(entries[i].request) for i in order], dtype=np.int64)
        slots = np.array([self.cache.slot(entries[i].request) for i in order], dtype=np.int64)
        n_prefill = int((q_lens > 1).sum())
        n_prefill_tokens = int(cu_q[n_prefill])

        token_ids = np.empty(T, dtype=np.int64)
        for j, i in enumerate(order):
            token_ids[cu_q[j]:cu_q[j + 1]] = entries[i].tokens
        if self.vocab_size is not None and ((token_ids < 0) | (token_ids >= self.vocab_size)).any():
            bad = token_ids[(token_ids < 0) | (token_ids >= self.vocab_size)][0]
            raise ValueError(f"token id {int(bad)} is outside the vocabulary of {self.vocab_size}")
        token_req = np.repeat(np.arange(R, dtype=np.int64), q_lens)
        positions = np.arange(T, dtype=np.int64) - cu_q[token_req] + ctx[token_req]
        kv_len = ctx + q_lens
        if self.max_positions is not None and int(kv_len.max()) > self.max_positions:
            raise ValueError(f"a request would reach {int(kv_len.max())} positions; the model "
                             f"has {self.max_positions}")

        # wanted rows in the caller's order
        place = {i: j for j, i in enumerate(order)}
        rows: list[int] = []
        for i, e in enumerate(entries):
            j = place[i]
            for w in e.want:
                if not 0 <= w < len(e.tokens):
                    raise ValueError(f"request {e.request!r}: wanted index {w} is outside its "
                                     f"{len(e.tokens)} tokens")
                rows.append(int(cu_q[j]) + int(w))
        K = len(rows)

        # q tiles over the prefill range
        tiles_np: dict[int, np.ndarray] = {}
        for bm in self.q_tile_sizes:
            parts = []
            for j in range(n_prefill):
                starts = np.arange(0, q_lens[j], bm, dtype=np.int64)
                t = np.empty((len(starts), 3), dtype=np.int64)
                t[:, 0] = j
                t[:, 1] = cu_q[j] + starts
                t[:, 2] = np.minimum(bm, q_lens[j] - starts)
                parts.append(t)
            tiles_np[bm] = (np.concatenate(parts) if parts else np.zeros((0, 3), dtype=np.int64))

        ps = self.cache.page_size
        widths = []
        tables = []
        slot_maps = []
        for gi in range(len(self.cache.groups)):
            # the width is rounded up so that the layout, and with it a captured graph, stays
            # the same while requests grow by a few hundred tokens
            width = int(max(-(-int(kv_len.max()) // ps), 1))
            width = min(-(-width // self.width_step) * self.width_step, self.cache.max_blocks)
            table = self.cache.block_tables(gi, slots, width)
            page = table[token_req, positions // ps].astype(np.int64)
            if (page < 0).any():
                raise RuntimeError("a token of this step has no page (reserve was not called, "
                                   "or the page fell out of its window)")
            widths.append(width)
            tables.append(table)
            slot_maps.append(page * ps + positions % ps)

        # ---- layout
        sizes = [T, T, T, R + 1, R, R, K] + [3 * len(tiles_np[bm]) for bm in self.q_tile_sizes]
        for gi in range(len(tables)):
            sizes += [R * widths[gi], T]
        arrays = [token_ids, positions, token_req, cu_q, ctx, slots, np.array(rows, dtype=np.int64)]
        arrays += [tiles_np[bm].reshape(-1) for bm in self.q_tile_sizes]
        for gi in range(len(tables)):
            arrays += [tables[gi].reshape(-1), slot_maps[gi]]
        offsets, total = self._upload(sizes, arrays)

        def dv(k: int) -> torch.Tensor:
            return self._dev[offsets[k]:offsets[k] + sizes[k]]

        n_fixed = 7
        tiles = {bm: dv(n_fixed + t).view(-1, 3) for t, bm in enumerate(self.q_tile_sizes)}
        g0 = n_fixed + len(self.q_tile_sizes)
        groups = [GroupBatch(dv(g0 + 2 * gi).view(R, widths[gi]), dv(g0 + 2 * gi + 1), widths[gi])
                  for gi in range(len(tables))]
        batch = StepBatch(
            num_tokens=T, num_requests=R, num_prefill_requests=n_prefill,
            num_prefill_tokens=n_prefill_tokens, max_q_len=int(q_lens.max()),
            max_kv_len=int(kv_len.max()),
            token_ids=dv(0), positions=dv(1), token_request=dv(2), cu_q=dv(3), ctx_len=dv(4),
            state_slot=dv(5), logit_rows=dv(6), tiles=tiles, groups=groups,
            host=HostBatch(cu_q=cu_q, ctx_len=ctx, state_slot=slots,
                           requests=[entries[i].request for i in order]),
            layout_key=tuple(sizes) + (n_prefill, n_prefill_tokens),
        )
        return batch, order

    # ------------------------------------------------------------ decode-only steps
    def _build_decode(self, entries: Sequence[StepEntry]) -> tuple[StepBatch, list[int]]:
        """The same layout for a step of single-token requests only, with plain lists where the
        general path uses array operations: such steps are short, so the host's share counts."""
        cache = self.cache
        R = len(entries)
        reqs = [e.request for e in entries]
        if len(set(reqs)) != R:
            raise ValueError("a request appears twice in one step")
        toks = [int(e.tokens[0]) for e in entries]
        if self.vocab_size is not None and not (0 <= min(toks) and max(toks) < self.vocab_size):
            bad = next(t for t in toks if not 0 <= t < self.vocab_size)
            raise ValueError(f"token id {bad} is outside the vocabulary of {self.vocab_size}")
        ctx = [cache.length(r) for r in reqs]
        slots = [cache.slot(r) for r in reqs]
        max_kv = max(ctx) + 1
        if self.max_positions is not None and max_kv > self.max_positions:
            raise ValueError(f"a request would reach {max_kv} positions; the model has "
                             f"{self.max_positions}")
        rows: list[int] = []
        for j, e in enumerate(entries):
            for w in e.want:
                if w != 0:
                    raise ValueError(f"request {e.request!r}: wanted index {w} is outside its 1 token")
                rows.append(j)
        K = len(rows)
        ps = cache.page_size
        slots_np = np.asarray(slots, dtype=np.int64)
        pos_np = np.asarray(ctx, dtype=np.int64)
        widths, tables, slot_maps = [], [], []
        ar = np.arange(R)
        for gi in range(len(cache.groups)):
            width = max(-(-max_kv // ps), 1)
            width = min(-(-width // self.width_step) * self.width_step, cache.max_blocks)
            table = cache.block_tables(gi, slots_np, width)
            page = table[ar, pos_np // ps].astype(np.int64)
            if (page < 0).any():
                raise RuntimeError("a token of this step has no page (reserve was not called, "
                                   "or the page fell out of its window)")
            widths.append(width)
            tables.append(table)
            slot_maps.append(page * ps + pos_np % ps)
        sizes = [R, R, R, R + 1, R, R, K] + [0] * len(self.q_tile_sizes)
        for gi in range(len(tables)):
            sizes += [R * widths[gi], R]
        arrays = [toks, ctx, range(R), range(R + 1), ctx, slots, rows]
        arrays += [() for _ in self.q_tile_sizes]
        for gi in range(len(tables)):
            arrays += [tables[gi].reshape(-1), slot_maps[gi]]
        offsets, total = self._upload(sizes, arrays)
        key = tuple(sizes)
        views = self._decode_views.get(key)
        if views is None or views[0] is not self._dev:
            # the device views depend on the sizes only: made once per layout
            def dv(k: int) -> torch.Tensor:
                return self._dev[offsets[k]:offsets[k] + sizes[k]]

            n_fixed = 7
            tiles = {bm: dv(n_fixed + t).view(-1, 3) for t, bm in enumerate(self.q_tile_sizes)}
            g0 = n_fixed + len(self.q_tile_sizes)
            groups = [GroupBatch(dv(g0 + 2 * gi).view(R, widths[gi]), dv(g0 + 2 * gi + 1), widths[gi])
                      for gi in range(len(tables))]
            views = (self._dev, [dv(k) for k in range(7)], tiles, groups)
            if len(self._decode_views) > 256:
                self._decode_views.clear()
            self._decode_views[key] = views
        _, fixed, tiles, groups = views
        batch = StepBatch(
            num_tokens=R, num_requests=R, num_prefill_requests=0, num_prefill_tokens=0,
            max_q_len=1, max_kv_len=max_kv, token_ids=fixed[0], positions=fixed[1],
            token_request=fixed[2], cu_q=fixed[3], ctx_len=fixed[4], state_slot=fixed[5],
            logit_rows=fixed[6], tiles=tiles, groups=groups,
            host=HostBatch(cu_q=np.arange(R + 1, dtype=np.int64), ctx_len=pos_np,
                           state_slot=slots_np, requests=reqs),
            layout_key=tuple(sizes) + (0, 0))
        return batch, list(range(R))

    def _current_stream(self):
        """The current stream as an object, looked up by its raw handle: the plain lookup goes
        through several Python layers and costs tens of microseconds a step."""
        raw = torch._C._cuda_getCurrentRawStream(self._device_index)
        if raw != self._stream_raw:
            self._stream_raw = raw
            self._stream_obj = torch.cuda.current_stream(self.device)
        return self._stream_obj

    def _upload(self, sizes, arrays) -> tuple[list[int], int]:
        """Lay the arrays out (each section aligned to 16 bytes), fill the next pinned buffer
        and copy it to the device in one transfer."""
        offsets = []
        off = 0
        for n in sizes:
            offsets.append(off)
            off += _align(max(n, 1))
        total = off
        if total > self._capacity:
            torch.cuda.synchronize() if self.device.type == "cuda" else None
            self._alloc(max(total, 2 * self._capacity))
        self._turn ^= 1
        ev = self._events[self._turn]
        if ev is not None:
            ev.synchronize()
        host = self._host[self._turn].numpy()
        for a, o, n in zip(arrays, offsets, sizes):
            if n:
                host[o:o + n] = a
        self._dev[:total].copy_(self._host[self._turn][:total], non_blocking=True)
        if self.device.type == "cuda":
            ev = self._event_pool[self._turn]
            ev.record(self._current_stream())
            self._events[self._turn] = ev
        self._last_bytes = total * 4
        self.uploads += 1                # the device descriptor now belongs to this build
        return offsets, total
