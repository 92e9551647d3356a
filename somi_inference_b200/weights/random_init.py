"""Random-weights mode: write a model folder from a configuration and a seed.

The reference has no such mode (its tests use default module initialisation,
tests/integration/test_paged_attention_integration.py:12-24).  Tensors are drawn
in the order the model declares them, each from N(0, std) in float32 on the CPU
generator seeded once with `seed` ("ones" and "zeros" tensors are constant), and
then stored in `dtype`.  The folder holds config.json and model.safetensors and
is read back through the ordinary loader.
"""

from __future__ import annotations

import json
import os

import torch

from ..parts.model import declared_tensors
from .safetensors_io import save_safetensors


def random_tensors(config, seed: int, *, std: float = 0.02,
                   dtype: torch.dtype = torch.bfloat16) -> dict[str, torch.Tensor]:
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    out: dict[str, torch.Tensor] = {}
    for name, decl in declared_tensors(config.to_model_spec()).items():
        if decl.ignored:
            continue
        if decl.init == "ones":
            t = torch.ones(decl.shape, dtype=torch.float32)
        elif decl.init == "zeros":
            t = torch.zeros(decl.shape, dtype=torch.float32)
        elif decl.init == "normal":
            t = torch.empty(decl.shape, dtype=torch.float32).normal_(0.0, std, generator=gen)
        else:
            raise ValueError(f"tensor {name!r}: unknown init {decl.init!r}")
        out[name] = t.to(dtype)
    return out


def write_random_model(config, seed: int, out_dir: str, *, std: float = 0.02,
                       dtype: torch.dtype = torch.bfloat16) -> str:
    """Write `out_dir/config.json` and `out_dir/model.safetensors`; return `out_dir`."""
    os.makedirs(out_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = {torch.bfloat16: "bfloat16", torch.float32: "float32",
                          torch.float16: "float16"}[dtype]
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f, indent=1)
    save_safetensors(random_tensors(config, seed, std=std, dtype=dtype),
                     os.path.join(out_dir, "model.safetensors"))
    return out_dir
