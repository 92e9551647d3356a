"""Dense projection y = x W^T (+ b) through the library matrix product.

The reference's engine uses `nn.Linear` for every projection
(somi_inference/models/qwen2.py:221-222,268-271), i.e. the library GEMM; so does
this class.  In float32 the product is a true 32-bit one: the reduced-precision
matrix mode (TF32) is switched off process-wide when the package is imported.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None) -> None:
        self.weight = weight                      # [out, in], compute dtype
        self.bias = None if bias is None else bias.to(weight.dtype)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.weight, self.bias)


def project_to_float32(h: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """h W^T with a float32 result (the library product accumulates in float32)."""
    if h.dtype == torch.float32:
        return F.linear(h, weight)
    try:
        return torch.mm(h, weight.t(), out_dtype=torch.float32)
    except (TypeError, RuntimeError):
        return F.linear(h, weight).float()
