"""Registries of part kinds.  A `PartSpec.kind` is looked up here.

Each registry maps a kind to a class with
    `declare(params) -> list[TensorDecl]`          (static: what the weight file must hold)
    `__init__(params, tensors, ctx)`                (tensors: name -> placed tensor)
Registering a new kind is all that a new mixer, feed-forward, norm, position
encoding, embedding, head or block arrangement needs; see `parts/base.py` for
the call each kind must answer.
"""

from __future__ import annotations

from typing import Any, Callable

from ..config.spec import PartSpec


class PartRegistry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, type] = {}

    def register(self, kind: str, cls: type | None = None) -> Callable[[type], type] | type:
        def put(c: type) -> type:
            if kind in self._kinds and self._kinds[kind] is not c:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._kinds[kind] = c
            return c
        return put(cls) if cls is not None else put

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> type:
        try:
            return self._kinds[kind]
        except KeyError:
            raise ValueError(f"unknown {self.what} kind {kind!r}; registered: "
                             f"{sorted(self._kinds)}") from None

    def declare(self, spec: PartSpec) -> list:
        return list(self.get(spec.kind).declare(spec.params))

    def build(self, spec: PartSpec, tensors: dict[str, Any], ctx: Any) -> Any:
        return self.get(spec.kind)(spec.params, tensors, ctx)

    def kinds(self) -> list[str]:
        return sorted(self._kinds)


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
EMBEDDINGS = PartRegistry("embedding")
HEADS = PartRegistry("head")
ARRANGEMENTS = PartRegistry("block arrangement")
