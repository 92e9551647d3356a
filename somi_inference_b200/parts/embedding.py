"""Token embedding and the output head.

Embedding: x = E[ids] (somi_inference/models/qwen2.py:360,382), written straight
into the float32 residual stream.  Head: logits = h E^T when tied
(somi_inference/models/qwen2_adapter.py:60-62), else h W_lm^T with the file's
`lm_head.weight`; logits are produced in float32 for the wanted rows only.
"""

from __future__ import annotations

import torch

from .base import BuildContext, TensorDecl, names_of
from .linear import Linear
from .registry import EMBEDDINGS, HEADS


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        return [TensorDecl(names_of(params)["weight"],
                           (int(params["vocab_size"]), int(params["hidden_size"])))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.weight = tensors[names_of(params)["weight"]]
        self.hidden = int(params["hidden_size"])

    def forward(self, batch) -> torch.Tensor:
        token_ids = batch.token_ids
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32,
                          device=token_ids.device)
        self.ctx.ops.embed(token_ids, self.weight, out)
        return out


@HEADS.register("lm_head")
class LMHead:
    @staticmethod
    def declare(params) -> list[TensorDecl]:
        shape = (int(params["vocab_size"]), int(params["hidden_size"]))
        # a tied model's file may still carry the head's matrix (the reference drops it as well:
        # somi_inference/models/qwen2_adapter.py:161-162): tolerated, never read
        return [TensorDecl(names_of(params)["weight"], shape, optional=bool(params["tied"]),
                           ignored=bool(params["tied"]))]

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.proj = Linear(tensors[n["tied_to"] if params["tied"] else n["weight"]], None, ctx.ops)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.proj.to_float32(h)
