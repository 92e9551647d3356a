"""Attention mixer: grouped-query causal attention over the paged cache.

Formulas (somi_inference/models/qwen2.py:252-300 for the projections,
:158-186 for the scores; somi_inference/core/paged_attention.py:352-413 for the
cached form): q = h Wq^T + bq, k = h Wk^T + bk, v = h Wv^T + bv; rotary encoding
of q and k; query head h reads kv head h // (heads / kv_heads); scores
q.k * head_dim^-0.5, causal, softmax in float32; output through Wo.

The three projections are one matrix product over the concatenated weight
[(heads + 2 kv_heads) * head_dim, hidden].  Keys and values of the step's tokens
go to their cache slots first; attention then reads everything, old and new,
from the cache, whether the request brought one token or a portion of a prompt.
"""

from __future__ import annotations

import torch

from .base import BuildContext, CacheNeeds, PagedKVNeeds, TensorDecl, names_of
from .linear import Linear
from .registry import MIXERS, POSITION_ENCODINGS


@MIXERS.register("attention")
class AttentionMixer:
    graph_safe = True     # launches kernels only; nothing is decided on the host per step

    @staticmethod
    def declare(params) -> list[TensorDecl]:
        n = names_of(params)
        hidden, heads = int(params["hidden_size"]), int(params["num_heads"])
        kv_heads, hd = int(params["num_kv_heads"]), int(params["head_dim"])
        decl = [TensorDecl(n["q_weight"], (heads * hd, hidden)),
                TensorDecl(n["k_weight"], (kv_heads * hd, hidden)),
                TensorDecl(n["v_weight"], (kv_heads * hd, hidden)),
                TensorDecl(n["o_weight"], (hidden, heads * hd))]
        if params.get("qkv_bias"):
            decl += [TensorDecl(n["q_bias"], (heads * hd,), matrix=False),
                     TensorDecl(n["k_bias"], (kv_heads * hd,), matrix=False),
                     TensorDecl(n["v_bias"], (kv_heads * hd,), matrix=False)]
        if params.get("out_bias"):
            decl.append(TensorDecl(n["o_bias"], (hidden,), matrix=False))
        decl += POSITION_ENCODINGS.declare(params["position"])
        return decl

    def __init__(self, params, tensors, ctx: BuildContext) -> None:
        n = names_of(params)
        self.ctx = ctx
        self.hidden = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads ({self.num_heads}) must be divisible by "
                             f"num_kv_heads ({self.num_kv_heads})")
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        w = torch.cat([tensors[n["q_weight"]], tensors[n["k_weight"]], tensors[n["v_weight"]]], 0)
        b = None
        if params.get("qkv_bias"):
            b = torch.cat([tensors[n["q_bias"]].float(), tensors[n["k_bias"]].float(),
                           tensors[n["v_bias"]].float()], 0)
        self.qkv = Linear(w.contiguous(), b, ctx.ops)
        self.out = Linear(tensors[n["o_weight"]],
                          tensors[n["o_bias"]] if params.get("out_bias") else None, ctx.ops)
        self.position = POSITION_ENCODINGS.build(params["position"], tensors, ctx)
        ctx.ops.check_attention_geometry(self.num_heads, self.num_kv_heads, self.head_dim)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(paged=PagedKVNeeds(self.num_kv_heads, self.head_dim, self.window))

    def forward(self, x: torch.Tensor, batch, cache, owns_cache: bool) -> torch.Tensor:
        paged = cache.paged
        partial = self.qkv.partial_sums(x) if self.position.takes_partial_sums else None
        if partial is not None:
            # the split-K product's partial sums (the bias is in the first) are added up by the
            # rotary kernel itself
            qkv = torch.empty((x.shape[0], self.qkv.out_features), dtype=x.dtype, device=x.device)
            self.position.encode_and_store(qkv, self.num_heads, self.num_kv_heads, self.head_dim,
                                           batch, paged, owns_cache, partials=partial)
        else:
            qkv = self.qkv(x)
            self.position.encode_and_store(qkv, self.num_heads, self.num_kv_heads, self.head_dim,
                                           batch, paged, owns_cache)
        out = torch.empty((x.shape[0], self.num_heads * self.head_dim), dtype=x.dtype,
                          device=x.device)
        self.ctx.ops.paged_attention(qkv, paged.keys, paged.values, batch,
                                     batch.groups[paged.group], self.num_heads,
                                     self.num_kv_heads, self.head_dim, self.scale,
                                     self.window, out, storage=paged.storage)
        partial = self.out.partial_sums(out)
        return partial if partial is not None else self.out(out)
