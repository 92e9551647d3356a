"""Position encodings that act on queries and keys before they reach the cache.

Rotary encoding as the reference computes it (somi_inference/models/qwen2.py:65-113):
inv_freq[i] = 1 / theta^(2i/d) for i in [0, d/2), angle = position * inv_freq[i]
in float32, and the rotation pairs element i with element i + d/2 ("rotate half"):
    out[i]       = x[i] * cos - x[i + d/2] * sin
    out[i + d/2] = x[i + d/2] * cos + x[i] * sin
Values are left untouched.  inv_freq is computed here once, on the host, in
float32 with the reference's expression; angles, sines and cosines are computed
in float32 inside the kernel, which also writes the rotated keys and the values
to their cache slots.

A position encoding answers
    encode_and_store(qkv, num_heads, num_kv_heads, head_dim, batch, paged, write)
where `qkv` is [T, (num_heads + 2 num_kv_heads) * head_dim], rotated in place.  One that sets
`takes_partial_sums = True` also accepts `partials=` (float32 [splits, T, width] partial sums of
the projection) and `bias=`, adds them up itself and leaves the queries in `qkv`.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl
from .registry import POSITION_ENCODINGS


@POSITION_ENCODINGS.register("rope")
class RotaryEncoding:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return []

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        self.theta = float(params["theta"])
        self.max_positions = int(params["max_positions"])
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.ctx = ctx
        exponent = torch.arange(0, self.rotary_dim, 2) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta ** exponent)).to(torch.float32).to(ctx.device)

    takes_partial_sums = True     # encode_and_store accepts `partials=` and `bias=`

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, batch, paged, write,
                         partials=None, bias=None):
        group = batch.groups[paged.group] if paged is not None else None
        self.ctx.ops.rope_store(
            qkv, batch.positions, self.inv_freq, num_heads, num_kv_heads, head_dim,
            self.rotary_dim,
            group.slot_map if (write and group is not None) else None,
            paged.keys if paged is not None else None,
            paged.values if paged is not None else None, partials=partials, bias=bias)


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding:
    """Stores keys and values as they are (rotary_dim 0)."""

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return []

    takes_partial_sums = True

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.inv_freq = torch.zeros(1, dtype=torch.float32, device=ctx.device)

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, batch, paged, write,
                         partials=None, bias=None):
        group = batch.groups[paged.group] if paged is not None else None
        self.ctx.ops.rope_store(
            qkv, batch.positions, self.inv_freq, num_heads, num_kv_heads, head_dim, 0,
            group.slot_map if (write and group is not None) else None,
            paged.keys if paged is not None else None,
            paged.values if paged is not None else None, partials=partials, bias=bias)
