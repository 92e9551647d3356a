"""The engine: a model, its cache and the one step function.

The reference runs a step as separate forward passes: one whole prompt per new
sequence, then one batch of single tokens (somi_inference/core/continuous_batching.py:200-203,
somi_inference/core/model_runner.py:24-60).  Here `Engine.step` takes any mixture
of (request, its next tokens) and runs exactly those tokens as one batch against
the cache that earlier steps left, returning float32 logits at the wanted places.
"""

from __future__ import annotations

from collections import OrderedDict
from typing import Sequence

import torch

from ..cache import CacheManager, OutOfPages
from ..config import load_config
from ..parts import BuildContext, Decoder, declared_tensors
from ..weights import load_tensors
from .batch import BatchBuilder, StepBatch, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be 'bfloat16' or 'float32', got {dtype!r}") from None


class LayoutCache:
    """Which step layouts have a captured graph.  A layout is captured at its second sighting;
    when `capacity` graphs are held, the one replayed longest ago makes room (a serving run
    passes through many layouts as requests come, grow and go, and only the recent ones return).
    """

    def __init__(self, capacity: int, max_sightings: int = 4096) -> None:
        if capacity < 1:
            raise ValueError("a layout cache needs room for at least one graph")
        self.capacity = capacity
        self.max_sightings = max_sightings
        self._entries: OrderedDict = OrderedDict()
        self._seen: dict = {}
        self.hits = self.captures = self.evictions = 0

    def __len__(self) -> int:
        return len(self._entries)

    def __contains__(self, key) -> bool:
        return key in self._entries

    def get(self, key):
        """The entry captured for `key`, marked as just used; None if there is none."""
        entry = self._entries.get(key)
        if entry is not None:
            self._entries.move_to_end(key)
            self.hits += 1
        return entry

    def sighted(self, key) -> bool:
        """Count an eager run of `key`; True when the layout should be captured now."""
        if len(self._seen) > self.max_sightings:      # many layouts that never came back
            self._seen.clear()
        n = self._seen.get(key, 0) + 1
        self._seen[key] = n
        return n >= 2

    def put(self, key, entry) -> None:
        while len(self._entries) >= self.capacity:
            old, _ = self._entries.popitem(last=False)     # dropping the graph frees its memory
            self._seen.pop(old, None)      # it has to be seen twice again before it is captured anew
            self.evictions += 1
        self._entries[key] = entry
        self.captures += 1

    def clear(self) -> None:
        self._entries.clear()
        self._seen.clear()


class Engine:
    def __init__(self, model_dir: str, *, dtype="bfloat16", page_size: int = 16,
                 num_pages: int | None = None, max_tokens: int | None = None,
                 max_requests: int = 16, device: str | torch.device = "cuda:0",
                 ops=None, use_graphs: bool = True) -> None:
        """Load `model_dir` (config.json + safetensors) and lay out its cache.

        The page pool holds `num_pages` pages per group, or enough for
        `max_tokens` tokens (rounded up to whole pages) when that is given.
        """
        config = load_config(model_dir)
        spec = config.to_model_spec()
        tensors = load_tensors(model_dir, declared_tensors(spec))
        self._setup(config, tensors, dtype=dtype, page_size=page_size, num_pages=num_pages,
                    max_tokens=max_tokens, max_requests=max_requests, device=device, ops=ops,
                    use_graphs=use_graphs)

    @classmethod
    def from_tensors(cls, config, tensors: dict, **kwargs) -> "Engine":
        """An engine over tensors that are already in memory (name -> tensor, any device),
        e.g. random weights made on the device; `config` is a typed architecture config."""
        self = cls.__new__(cls)
        self._setup(config, tensors, **kwargs)
        return self

    def _setup(self, config, tensors, *, dtype="bfloat16", page_size: int = 16,
               num_pages: int | None = None, max_tokens: int | None = None,
               max_requests: int = 16, device="cuda:0", ops=None,
               use_graphs: bool = True) -> None:
        self.device = torch.device(device)
        self.dtype = resolve_dtype(dtype)
        if ops is None:
            from ..ops import cuda_ops
            ops = cuda_ops()
        self.ops = ops
        self.config = config
        self.spec = config.to_model_spec()
        ctx = BuildContext(dtype=self.dtype, device=self.device, ops=ops)
        with torch.no_grad():
            self.model = Decoder(self.spec, tensors, ctx)
            needs, owners = self.model.cache_needs()
            if num_pages is None:
                if max_tokens is None:
                    raise ValueError("give num_pages or max_tokens")
                num_pages = -(-int(max_tokens) // page_size)
            self.page_size = page_size
            self.num_pages = int(num_pages)
            self.cache = CacheManager(needs, owners, num_pages=self.num_pages,
                                      page_size=page_size, max_requests=max_requests,
                                      max_positions=self.spec.max_positions, dtype=self.dtype,
                                      device=self.device)
        self.builder = BatchBuilder(self.cache, device=self.device,
                                    q_tile_sizes=ops.q_tile_sizes,
                                    vocab_size=self.spec.vocab_size,
                                    max_positions=self.spec.max_positions)
        self.last_batch: StepBatch | None = None
        self.use_graphs = use_graphs
        self._token_stage = None
        self._prebuilt = None
        self.token_patch_bytes = 0
        self.graph_max_tokens = 8192     # larger steps are bound by the GPU, not by the host
        self._graphs = LayoutCache(capacity=128)
        self._graph_pool = None
        self._graph_generation = self.builder.generation

    # ------------------------------------------------------------------ step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; return float32 logits [wanted, vocab] in the entries' order.

        New requests are registered on first sight.  If the pages for this step
        cannot all be had, `OutOfPages` is raised and the cache is as before.
        """
        registered: list[object] = []
        reserved: list[object] = []
        ids = [e.request for e in entries]
        if len(set(ids)) != len(ids):
            raise ValueError("a request appears twice in one step")
        if any(len(e.tokens) < 1 for e in entries):
            raise ValueError("every entry of a step needs at least one token")
        try:
            for e in entries:
                if not self.cache.is_registered(e.request):
                    self.cache.register(e.request)
                    registered.append(e.request)
                self.cache.reserve(e.request, len(e.tokens))
                reserved.append(e.request)
            batch, _ = self.builder.build(entries)
            logits = self._run(batch)
        except Exception:
            # also when a launch failed: nothing stays reserved, the lengths are as before
            for r in reserved:
                self.cache.cancel(r)
            for r in registered:
                self.cache.release(r)
            raise
        for e in entries:
            self.cache.commit(e.request)
        return logits

    def run_reserved(self, entries: Sequence[StepEntry], keep: bool = True) -> torch.Tensor:
        """As `step`, for a caller (the scheduler) that registered the requests and reserved
        their pages itself and will commit afterwards.  With `keep=False` the returned logits
        may be a buffer that the next step overwrites (the caller samples from it at once)."""
        batch, _ = self.builder.build(entries)
        return self._run(batch, keep)

    def _run(self, batch: StepBatch, keep: bool = True) -> torch.Tensor:
        """Forward pass of one batch.  A step is a sequence of a few hundred kernels; for
        single-token steps and for portions of a small model the host cannot issue them as fast
        as the GPU runs them.  So the kernel sequence is captured in a CUDA graph the second time
        a layout (tokens and rows of every request class, tiles, table width, wanted rows) is
        seen and replayed from then on; the batch descriptor lives at fixed device addresses, so
        a replay reads the new step's data."""
        self.last_batch = batch
        graphable = (self.use_graphs and self.device.type == "cuda" and self.model.graph_safe
                     and batch.num_tokens <= self.graph_max_tokens)
        if not graphable:
            with torch.no_grad():
                return self.model.forward(batch, self.cache)
        if self._graph_generation != self.builder.generation:
            # the descriptor buffer moved: graphs captured over the old addresses are void
            self._graphs.clear()
            self._graph_generation = self.builder.generation
        key = batch.layout_key
        entry = self._graphs.get(key)
        if entry is not None:
            graph, logits, launches = entry
            graph.replay()
            self.ops.launches += launches
            # the graph's own output buffer is overwritten by the next replay
            return logits.clone() if keep else logits
        with torch.no_grad():
            logits = self.model.forward(batch, self.cache)      # also warms up the libraries
        if self._graphs.sighted(key):
            # Capturing runs nothing; recording the same step again is harmless because a step
            # only writes the cache slots of its own tokens, with the same values.
            before = self.ops.launches
            graph = torch.cuda.CUDAGraph()
            if len(self._graphs) == 0:
                # the shared memory pool lives only as long as a graph uses it: after every
                # graph has gone (the descriptor moved) this capture starts a new one
                self._graph_pool = None
            with torch.no_grad(), torch.cuda.graph(graph, pool=self._graph_pool):
                static_logits = self.model.forward(batch, self.cache)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            self._graphs.put(key, (graph, static_logits, self.ops.launches - before))
            self.ops.launches = before
        return logits

    def prebuild(self, entries: Sequence[StepEntry]) -> StepBatch:
        """The batch descriptor of a step whose token ids are not known yet (`entries` carry
        placeholders): built and uploaded now, run later by `run_prebuilt`.  No other step may
        be built in between; the requests' pages are reserved by the caller."""
        batch, _ = self.builder.build(entries)
        self._prebuilt = (batch, self.builder.uploads)
        return batch

    def prebuilt_is_current(self, batch: StepBatch) -> bool:
        """Whether the device still holds this batch's descriptor (no other step was built since)."""
        return (self._prebuilt is not None and self._prebuilt[0] is batch
                and self._prebuilt[1] == self.builder.uploads)

    def run_prebuilt(self, batch: StepBatch, token_ids: Sequence[int], keep: bool = True) -> torch.Tensor:
        """Run a batch from `prebuild` with its token ids, one per token of the batch in the
        entries' order (single-token requests only, so that order is the batch's order)."""
        n = len(token_ids)
        if n != batch.num_tokens or batch.num_prefill_requests:
            raise ValueError("run_prebuilt takes one token id for every single-token request")
        if not self.prebuilt_is_current(batch):
            raise RuntimeError("another step was built after this one was prepared")
        if self._token_stage is None or self._token_stage.numel() < n:
            self._token_stage = torch.empty(max(n, 256), dtype=torch.int32,
                                            pin_memory=self.device.type == "cuda")
        self._token_stage[:n] = torch.as_tensor(token_ids, dtype=torch.int32)
        batch.token_ids.copy_(self._token_stage[:n], non_blocking=True)
        self.token_patch_bytes = 4 * n
        return self._run(batch, keep)

    def run_prebuilt_fed(self, batch: StepBatch, token_ids: torch.Tensor, keep: bool = True) -> torch.Tensor:
        """As `run_prebuilt`, with the token ids taken from an int32 device tensor (the sampler's
        output of the step before): nothing waits for the host to have seen them."""
        if token_ids.numel() != batch.num_tokens or batch.num_prefill_requests:
            raise ValueError("run_prebuilt_fed takes one token id for every single-token request")
        if token_ids.dtype != torch.int32 or token_ids.device != batch.token_ids.device:
            raise ValueError("token ids must be int32 on the engine's device")
        if not self.prebuilt_is_current(batch):
            raise RuntimeError("another step was built after this one was prepared")
        batch.token_ids.copy_(token_ids, non_blocking=True)
        self.token_patch_bytes = 0
        return self._run(batch, keep)

    def end(self, request: object) -> None:
        """The request is finished: everything it holds goes back to the pools."""
        self.cache.release(request)

    def has(self, request: object) -> bool:
        return self.cache.is_registered(request)

    def length(self, request: object) -> int:
        return self.cache.length(request)
