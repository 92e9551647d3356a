"""Architecture-neutral description of a decoder: parts, layers and their order.

A model is data: a list of `LayerSpec` (which mixer, which feed-forward, which
norm, which arrangement, each with its own numbers) and a `schedule`, the list
of runs that one forward pass makes.  A run names a layer and, optionally, an
earlier run whose cache it reads instead of keeping one of its own.  Nothing in
this file knows an architecture; an architecture's config class produces a
`ModelSpec` (see `config/qwen2.py`).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and its parameters.

    `kind` is looked up in the matching registry of `parts/registry.py`;
    `params` are passed to the part's constructor unchanged, so every size and
    constant a part uses is stated here and nowhere else.
    """

    kind: str
    params: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One decoder layer: weight-name prefix, its parts and their arrangement.

    A layer has at most one mixer and at most one feed-forward (either may be None) and any
    number of norms, each under the name by which the layer's arrangement asks for it: the
    pre-norm arrangement wants "mixer" and "feed_forward"; an arrangement that also normalises
    what its parts return can name four.  The arrangement's constructor is called with
    `(mixer, feed_forward, norms)`, `norms` being a dict from those names to built norms.
    """

    prefix: str  # e.g. "model.layers.3"
    mixer: PartSpec | None
    feed_forward: PartSpec | None
    norms: Mapping[str, PartSpec] = field(default_factory=dict)
    arrangement: str = "pre_norm"


@dataclass(frozen=True)
class RunSpec:
    """One entry of the schedule: run `layer`; read the cache of run `cache_of`.

    `cache_of is None` means the run owns a cache (and writes it).  Otherwise it
    is the index, in the schedule, of an earlier run whose cache this run reads
    without writing.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything the generic decoder needs to be built."""

    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("a model needs a non-empty schedule")
        for i, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {run.layer}, "
                                 f"but there are {len(self.layers)} layers")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"schedule[{i}].cache_of={run.cache_of} must "
                                     "name an earlier run")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}].cache_of={run.cache_of} names "
                                     "a run that owns no cache")
