"""Dense gated feed-forward (SwiGLU).

Formula (somi_inference/models/qwen2.py:209-229): gu = h W_gu^T with
W_gu = cat(gate_proj, up_proj) on the output dimension
(somi_inference/models/qwen2_adapter.py:182-189,244-248); gate, up = the two
halves; y = (silu(gate) * up) W_down^T; silu(z) = z * sigmoid(z), in float32.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .linear import Linear
from .registry import FEED_FORWARDS


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    graph_safe = True     # launches kernels only; nothing is decided on the host per step

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, inter = int(params["hidden_size"]), int(params["intermediate_size"])
        return [TensorDecl(n["gate_weight"], (inter, hidden)),
                TensorDecl(n["up_weight"], (inter, hidden)),
                TensorDecl(n["down_weight"], (hidden, inter))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.inter = int(params["intermediate_size"])
        # rows alternate gate_i, up_i, so that one thread pair of the product's epilogue (or one
        # vector load of the activation kernel) holds a matching gate and up
        gate, up = tensors[n["gate_weight"]], tensors[n["up_weight"]]
        self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, -1).contiguous(),
                              None, ctx.ops)
        self.down = Linear(tensors[n["down_weight"]], None, ctx.ops)

    def forward(self, x: torch.Tensor, batch) -> torch.Tensor:
        act = self.gate_up.swiglu(x)
        if act is None:
            gu = self.gate_up(x)
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            self.ctx.ops.silu_mul(gu, act, interleaved=True)
        partial = self.down.partial_sums(act)
        return partial if partial is not None else self.down(act)
