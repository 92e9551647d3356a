"""The generic decoder: embedding, the scheduled runs of layers, final norm, head.

The reference's `QwenModel` hard-wires one layer class N times
(somi_inference/models/qwen2.py:342-386) and its adapter adds the head
(somi_inference/models/qwen2_adapter.py:60-62,95,146).  This decoder is built
from a `ModelSpec`: every layer names its own parts, and the order of execution
is the spec's schedule, which may run a layer twice or let a run read another
run's cache.  It knows no architecture.
"""

from __future__ import annotations

import torch

from ..config.spec import LayerSpec, ModelSpec
from .base import BuildContext, CacheNeeds, TensorDecl
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS)


def declared_tensors(spec: ModelSpec) -> dict[str, TensorDecl]:
    """Every tensor the weight file must hold, by name."""
    out: dict[str, TensorDecl] = {}

    def add(decls) -> None:
        for d in decls:
            if d.name in out and out[d.name].shape != d.shape:
                raise ValueError(f"tensor {d.name!r} is declared twice with different shapes")
            out.setdefault(d.name, d)

    add(EMBEDDINGS.declare(spec.embedding))
    for layer in spec.layers:
        if layer.mixer is not None:
            add(MIXERS.declare(layer.mixer))
        if layer.feed_forward is not None:
            add(FEED_FORWARDS.declare(layer.feed_forward))
        for norm in layer.norms.values():
            add(NORMS.declare(norm))
    add(NORMS.declare(spec.final_norm))
    add(HEADS.declare(spec.head))
    return out


class Decoder:
    def __init__(self, spec: ModelSpec, tensors: dict[str, torch.Tensor], ctx: BuildContext) -> None:
        spec.validate()
        self.spec = spec
        self.ctx = ctx
        decls = declared_tensors(spec)
        lacking = [n for n, d in decls.items() if n not in tensors and not (d.optional or d.ignored)]
        if lacking:
            raise KeyError(f"tensors missing for the model: {', '.join(sorted(lacking))}")
        placed = {name: ctx.place(tensors[name], matrix=d.matrix) for name, d in decls.items()
                  if name in tensors and not d.ignored}
        self.embedding = EMBEDDINGS.build(spec.embedding, placed, ctx)
        self.layers = [self._build_layer(layer, placed) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, placed, ctx)
        self.head = HEADS.build(spec.head, placed, ctx)
        self.schedule = spec.schedule
        # a step can be captured in a CUDA graph only if no part plans on the host per step
        self.graph_safe = all(getattr(p, "graph_safe", False)
                              for b in self.layers for p in (b.mixer, b.feed_forward)
                              if p is not None)

    def _build_layer(self, layer: LayerSpec, placed):
        mixer = None if layer.mixer is None else MIXERS.build(layer.mixer, placed, self.ctx)
        ff = (None if layer.feed_forward is None
              else FEED_FORWARDS.build(layer.feed_forward, placed, self.ctx))
        norms = {name: NORMS.build(spec, placed, self.ctx) for name, spec in layer.norms.items()}
        return ARRANGEMENTS.get(layer.arrangement)(mixer, ff, norms)

    def cache_needs(self) -> tuple[list[CacheNeeds | None], list[int | None]]:
        """Per run of the schedule: what its mixer needs (None: no mixer, or nothing), and
        whose cache it reads."""
        mixers = [self.layers[run.layer].mixer for run in self.schedule]
        needs = [None if m is None else m.cache_needs() for m in mixers]
        owners = [run.cache_of for run in self.schedule]
        return needs, owners

    def forward(self, batch, cache) -> torch.Tensor:
        """Run the step's tokens; return float32 logits [len(batch.logit_rows), vocab]."""
        residual = self.embedding.forward(batch)
        pending = None
        for i, run in enumerate(self.schedule):
            pending = self.layers[run.layer].forward(residual, pending, batch, cache.view(i),
                                                     run.cache_of is None)
        if batch.logit_rows.shape[0] == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32,
                               device=residual.device)
        h = self.final_norm.forward(residual, pending, rows=batch.logit_rows)
        return self.head.forward(h)
