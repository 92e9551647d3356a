"""Weights by tensor name, checked against what the model's parts declared.

The reference loads through the library's model class and `load_state_dict(strict=True)`
(somi_inference/models/qwen2_adapter.py:228-251), which raises on the first kind
of mismatch.  This loader reads the safetensors file(s) directly and raises one
`WeightError` that lists every missing tensor, every unexpected tensor and every
wrong shape at once.
"""

from __future__ import annotations

import json
import os
from typing import Mapping

import torch

from ..parts.base import TensorDecl
from .safetensors_io import SafetensorsFile

# Buffers that exporters write but that are computed, not learned
# (somi_inference/models/qwen2_adapter.py:165-167 skips them too).
_IGNORED_SUFFIXES = ("rotary_emb.inv_freq",)


class WeightError(ValueError):
    """The weight file does not match the model: lists what is missing, extra or misshapen."""

    def __init__(self, missing, unexpected, wrong_shape, where: str) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {where} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {tuple(got)}, model needs {tuple(want)}"
                for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def _open_files(model_dir: str) -> dict[str, SafetensorsFile]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            weight_map = json.load(f)["weight_map"]
        files = {fn: SafetensorsFile(os.path.join(model_dir, fn)) for fn in set(weight_map.values())}
        return {name: files[fn] for name, fn in weight_map.items()}
    if os.path.isfile(single):
        f = SafetensorsFile(single)
        return {name: f for name in f.names()}
    raise FileNotFoundError(f"{model_dir!r} holds neither model.safetensors nor "
                            "model.safetensors.index.json")


def load_tensors(model_dir: str, declared: Mapping[str, TensorDecl],
                 optional: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    """Return {name: CPU tensor in its stored dtype} for every declared tensor that is read.

    A declaration marked `optional` may be absent from the file (it is then absent from the
    result); one marked `ignored` is checked for its shape when present but never read.  Names
    in `optional` may be present in the file without being declared at all.
    """
    files = _open_files(model_dir)
    present = {n for n in files if not n.endswith(_IGNORED_SUFFIXES)}
    missing = sorted(n for n, d in declared.items()
                     if n not in present and not (d.optional or d.ignored))
    unexpected = sorted(n for n in present if n not in declared and n not in optional)
    wrong = []
    for name in sorted(present & set(declared)):
        _, shape = files[name].info(name)
        if tuple(shape) != tuple(declared[name].shape):
            wrong.append((name, shape, declared[name].shape))
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, model_dir)
    return {name: files[name].tensor(name) for name, d in declared.items()
            if name in present and not d.ignored}
