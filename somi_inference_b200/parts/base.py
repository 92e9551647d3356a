"""What every part of a layer has in common: declared tensors and a build context.

A part is built from (a) its parameters, taken verbatim from a `PartSpec`,
(b) the tensors it declared, already on the device, and (c) a `BuildContext`
that carries the compute dtype, the device and the table of kernels.  A part
never sees a model config and never names an architecture.

Interfaces (duck-typed; the classes below only document them):

* Norm:          `forward(residual, delta=None, rows=None) -> Tensor`
                 adds `delta` into the fp32 `residual` (in place) and returns the
                 normalised rows in the compute dtype; with `rows`, only those
                 rows are produced and `residual` is left untouched.  `delta` is
                 what a mixer or feed-forward returned: [T, H], or float32
                 [splits, T, H] partial sums that the norm adds up in order.
* FeedForward:   `forward(x, batch) -> Tensor` of the same shape as `x`.
* Mixer:         `cache_needs() -> CacheNeeds`, and
                 `forward(x, batch, cache, owns_cache) -> Tensor`.
                 `cache` is the view the cache manager made for this run from
                 `cache_needs()`; `owns_cache` is False when the run reads
                 another run's cache and must not write it.
* PositionEncoding: `encode_and_store(qkv, geometry, batch, paged, write)`.
* Embedding:     `forward(batch) -> Tensor` float32 [T, H]: the residual stream's start, from
                 `batch.token_ids` (and whatever else of the batch it needs: positions, ...).
* Block arrangement: built as `cls(mixer, feed_forward, norms)` (`norms`: name -> norm; a
                 part the layer does not have is None); `forward(residual, pending, batch,
                 cache, owns_cache)` returns the delta that the next norm has to add.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import torch


@dataclass(frozen=True)
class TensorDecl:
    """A tensor that a part expects in the weight file."""

    name: str
    shape: tuple[int, ...]
    init: str = "normal"          # "normal" | "ones" | "zeros": used by the random-weights mode
    matrix: bool = True           # matrices feed GEMMs and are held in the compute dtype
    optional: bool = False        # the file may lack it; the part then finds no such name
    ignored: bool = False         # tolerated in the file (shape-checked) but never read: a
                                  # redundant copy, such as the head's matrix of a tied model


@dataclass
class BuildContext:
    dtype: torch.dtype            # compute dtype: torch.bfloat16 or torch.float32
    device: torch.device
    ops: Any                      # kernel table (ops.CudaOps on the product path)

    def place(self, t: torch.Tensor, *, matrix: bool) -> torch.Tensor:
        """Move a loaded tensor to the device in the precision it is held in.

        float32 compute: every floating tensor becomes float32.  bfloat16
        compute: matrices become bfloat16; other tensors keep the precision they
        were stored in (a tensor stored in 32-bit stays so); integer tensors
        become int32.
        """
        if not t.is_floating_point():
            return t.to(device=self.device, dtype=torch.int32).contiguous()
        if self.dtype == torch.float32:
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        if matrix or t.dtype != torch.float32:
            return t.to(device=self.device, dtype=self.dtype).contiguous()
        return t.to(device=self.device).contiguous()


@dataclass(frozen=True)
class PagedKVNeeds:
    """Keys and values that grow with the sequence, kept in pages."""

    num_kv_heads: int
    head_dim: int                 # width of a key
    window: int | None = None     # None: all keys; n: only the last n positions are ever read
    value_dim: int | None = None  # width of a value; None: the same as a key's

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim


@dataclass(frozen=True)
class StateNeeds:
    """Per-request state of fixed size: name -> (shape, dtype)."""

    tensors: Mapping[str, tuple[tuple[int, ...], torch.dtype]] = field(default_factory=dict)


@dataclass(frozen=True)
class CacheNeeds:
    paged: PagedKVNeeds | None = None
    state: StateNeeds | None = None


def names_of(params: Mapping[str, Any]) -> Mapping[str, str]:
    names = params.get("names")
    if not isinstance(names, Mapping):
        raise ValueError("part parameters carry no 'names' mapping (logical -> tensor name)")
    return names
