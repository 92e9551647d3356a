"""RMS normalisation over the last dimension, fused with the residual sum.

Formula (somi_inference/models/qwen2.py:46-62): x32 = float(x);
y = x32 * rsqrt(mean(x32^2) + eps); out = weight * y.  The reference casts y to
the input dtype before the weight multiply; here the residual stream stays in
float32 and the product is rounded once, at the end.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .registry import NORMS


@NORMS.register("rmsnorm")
class RMSNorm:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"], (int(params["size"]),), init="ones",
                           matrix=False)]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]

    def forward(self, residual: torch.Tensor, delta: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """`delta` is [T, size], or float32 [splits, T, size] partial sums that are added up."""
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=residual.device)
        self.ctx.ops.add_rmsnorm(residual, delta, self.weight, self.eps, out, rows)
        return out
