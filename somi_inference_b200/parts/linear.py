"""Dense projection y = x W^T (+ b).

The reference's engine uses `nn.Linear` for every projection
(somi_inference/models/qwen2.py:221-222,268-271), i.e. the library GEMM.  Here a step with few
tokens (bfloat16, at most `ops.skinny_max_tokens` rows) runs the engine's own tcgen05 kernel,
which streams the weight once through TMA and tensor memory and can leave split-K partial sums
or apply SiLU(gate)*up in its epilogue; larger bfloat16 steps (prompt portions) go to the library
product.  float32 goes to the engine's own float32 kernel (`csrc/gemm_f32.cu`: plain FMAs, every
output summed over K in ascending order whatever the step's size), not to the library.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import trace


class Linear:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None = None, ops=None) -> None:
        self.weight = weight                      # [out, in], compute dtype
        self.bias = None if bias is None else bias.to(weight.dtype)
        self.ops = ops
        self.out_features, self.in_features = weight.shape

    def skinny(self, x: torch.Tensor) -> bool:
        ops = self.ops
        return (ops is not None and x.is_cuda and getattr(ops, "skinny_supported", None) is not None
                and ops.skinny_supported(x.shape[0], self.out_features, self.in_features, x.dtype))

    def own_f32(self, x: torch.Tensor) -> bool:
        return (x.dtype == torch.float32 and x.is_cuda and self.weight.dtype == torch.float32
                and getattr(self.ops, "gemm_f32", None) is not None)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.skinny(x):
            return self.ops.skinny_gemm(x, self.weight, self.bias, self.ops.GEMM_BF16)
        if self.own_f32(x):
            return self.ops.gemm_f32(x, self.weight, self.bias)
        y = F.linear(x, self.weight, self.bias)
        self._note(x, y)
        return y

    def _note(self, x: torch.Tensor, y: torch.Tensor) -> None:
        if trace.active():
            M, N, K = x.shape[0], self.out_features, self.in_features
            trace.note("library_gemm", (N * K + M * K) * x.element_size() + y.numel() * y.element_size(),
                       2.0 * M * N * K, detail=f"M={M} N={N} K={K}")

    def partial_sums(self, x: torch.Tensor) -> torch.Tensor | None:
        """float32 [splits, M, out] partial sums over ranges of K (bias in the first), for a
        consumer that adds them up (the next norm, the rotary kernel); None when the step is not
        one for the tcgen05 kernel."""
        if not self.skinny(x):
            return None
        ops = self.ops
        return ops.skinny_gemm(x, self.weight, self.bias, ops.GEMM_PARTIAL_F32,
                               splits=ops.skinny_splits(x.shape[0], self.out_features, self.in_features))

    def swiglu(self, x: torch.Tensor) -> torch.Tensor | None:
        """silu(gate) * up for a weight whose rows alternate gate, up; None when not available."""
        if not self.skinny(x):
            return None
        return self.ops.skinny_gemm(x, self.weight, None, self.ops.GEMM_SWIGLU)

    def to_float32(self, x: torch.Tensor) -> torch.Tensor:
        """x W^T with a float32 result (accumulation is float32 in every path)."""
        if self.skinny(x):
            return self.ops.skinny_gemm(x, self.weight, None, self.ops.GEMM_F32)
        if self.own_f32(x):
            return self.ops.gemm_f32(x, self.weight, None)
        if x.dtype == torch.float32:
            y = F.linear(x, self.weight)
        elif _MM_TAKES_OUT_DTYPE:
            y = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
        else:
            y = F.linear(x, self.weight).float()      # rounds the logits to bfloat16 first
        self._note(x, y)
        return y


def _mm_takes_out_dtype() -> bool:
    """Whether this torch has `torch.mm(..., out_dtype=)` (asked once, without a device)."""
    try:
        torch.mm(torch.zeros(1, 1, device="meta", dtype=torch.bfloat16),
                 torch.zeros(1, 1, device="meta", dtype=torch.bfloat16), out_dtype=torch.float32)
        return True
    except (TypeError, RuntimeError, NotImplementedError):
        return False


_MM_TAKES_OUT_DTYPE = _mm_takes_out_dtype()
