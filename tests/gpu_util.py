"""Helpers of the GPU tests: attention cases built on the real cache manager and batch builder."""

from __future__ import annotations

import copy

import torch

from somi_inference_b200.cache import CacheManager
from somi_inference_b200.engine.batch import BatchBuilder, StepEntry
from somi_inference_b200.parts.base import CacheNeeds, PagedKVNeeds


def attention_case(ops, *, nq, nkv, hd, page_size, window, requests, dtype, seed=0,
                   num_pages=None, shuffle_pages=True):
    """`requests`: list of (tokens already cached, tokens in this step).

    Returns (manager, batch, qkv, view): the cache storage is filled with random
    numbers, so every slot that attention may read holds something.
    """
    g = torch.Generator().manual_seed(seed)
    total = sum(-(-(c + q) // page_size) for c, q in requests)
    num_pages = num_pages or total + 3
    mgr = CacheManager([CacheNeeds(paged=PagedKVNeeds(nkv, hd, window))], [None],
                       num_pages=num_pages, page_size=page_size, max_requests=len(requests) + 1,
                       max_positions=max(c + q for c, q in requests) + page_size,
                       dtype=dtype, device="cuda")
    if shuffle_pages:   # take and give back pages so that tables are not 0,1,2,...
        pool = mgr.groups[0].pool
        taken = pool.take(pool.num_free)
        perm = torch.randperm(len(taken), generator=g).tolist()
        pool.give_back([taken[i] for i in perm])
    store = mgr.groups[0].storage
    store.copy_(torch.randn(store.shape, generator=g).to(dtype))
    entries = []
    for i, (c, q) in enumerate(requests):
        mgr.register(i)
        if c:
            mgr.reserve(i, c)
            mgr.commit(i)
        mgr.reserve(i, q)
        entries.append(StepEntry(i, [0] * q, []))
    builder = BatchBuilder(mgr, device="cuda", q_tile_sizes=ops.q_tile_sizes)
    batch, order = builder.build(entries)
    qkv = torch.randn((batch.num_tokens, (nq + 2 * nkv) * hd), generator=g).to(dtype).cuda()
    return mgr, batch, qkv, mgr.view(0).paged, order


def batch_to_cpu(batch):
    """A copy of the batch whose device arrays live on the CPU (for the host reference)."""
    b = copy.copy(batch)
    for name in ("token_ids", "positions", "token_request", "cu_q", "ctx_len", "state_slot",
                 "logit_rows"):
        setattr(b, name, getattr(batch, name).cpu())
    b.tiles = {k: v.cpu() for k, v in batch.tiles.items()}
    b.groups = [copy.copy(g) for g in batch.groups]
    for g in b.groups:
        g.block_table = g.block_table.cpu()
        g.slot_map = g.slot_map.cpu()
    return b
