"""Toy parts defined by the tests, to show that the framework takes a new mixer, feed-forward
or position encoding without a change to its files.  None of them is anybody's model.

* `ToyDecayMixer`: a mixer with per-request state of fixed size and no paged cache:
  s_t = decay * s_{t-1} + x_t W_in,  y_t = s_t W_out.  The state lives in the cache manager's
  state slots, so a request can be continued in portions.
* `ToyRoutedFF`: a feed-forward with routing: top-1 of `n_experts` tiny SwiGLU-free experts,
  router logits in float32.
* `ToyShiftEncoding`: a position encoding that adds position * step to one key/query dim.
Each has its plain whole-sequence formula beside it.
"""

from __future__ import annotations

import torch

from somi_inference_b200.parts import FEED_FORWARDS, MIXERS, POSITION_ENCODINGS
from somi_inference_b200.parts.base import CacheNeeds, StateNeeds, TensorDecl, names_of


class ToyDecayMixer:
    @staticmethod
    def declare(params):
        n = names_of(params)
        h, s = int(params["hidden_size"]), int(params["state_size"])
        return [TensorDecl(n["w_in"], (s, h)), TensorDecl(n["w_out"], (h, s))]

    def __init__(self, params, tensors, ctx):
        n = names_of(params)
        self.decay = float(params["decay"])
        self.state_size = int(params["state_size"])
        self.w_in, self.w_out = tensors[n["w_in"]].float(), tensors[n["w_out"]].float()

    def cache_needs(self):
        return CacheNeeds(state=StateNeeds({"s": ((self.state_size,), torch.float32)}))

    def forward(self, x, batch, cache, owns_cache):
        state = cache.state["s"]
        u = x.float() @ self.w_in.T
        out = torch.empty_like(u)
        cu = batch.host.cu_q
        for r, slot in enumerate(batch.host.state_slot.tolist()):
            s = state[slot].clone()
            for t in range(int(cu[r]), int(cu[r + 1])):
                s = self.decay * s + u[t]
                out[t] = s
            if owns_cache:
                state[slot] = s
        return (out @ self.w_out.T).to(x.dtype)

    @staticmethod
    def plain(x, w_in, w_out, decay):
        s = torch.zeros(w_in.shape[0])
        ys = []
        for t in range(x.shape[0]):
            s = decay * s + x[t] @ w_in.T
            ys.append(s @ w_out.T)
        return torch.stack(ys)


class ToyRoutedFF:
    @staticmethod
    def declare(params):
        n = names_of(params)
        h, e, i = int(params["hidden_size"]), int(params["n_experts"]), int(params["inner"])
        return [TensorDecl(n["router"], (e, h)), TensorDecl(n["w1"], (e * i, h)),
                TensorDecl(n["w2"], (e * h, i))]

    def __init__(self, params, tensors, ctx):
        n = names_of(params)
        self.h, self.e, self.i = int(params["hidden_size"]), int(params["n_experts"]), int(params["inner"])
        self.router = tensors[n["router"]].float()
        self.w1 = tensors[n["w1"]].float().view(self.e, self.i, self.h)
        self.w2 = tensors[n["w2"]].float().view(self.e, self.h, self.i)

    def forward(self, x, batch):
        return self.plain(x.float(), self.router, self.w1, self.w2).to(x.dtype)

    @staticmethod
    def plain(x, router, w1, w2):
        choice = torch.argmax(x @ router.T, dim=-1)
        out = torch.empty_like(x)
        for t in range(x.shape[0]):
            e = int(choice[t])
            out[t] = torch.relu(x[t] @ w1[e].T) @ w2[e].T
        return out


class ToyShiftEncoding:
    """q[..., 0] and k[..., 0] get position * step added; keys and values are then stored."""

    takes_partial_sums = False

    @staticmethod
    def declare(params):
        return []

    def __init__(self, params, tensors, ctx):
        self.step = float(params["step"])
        self.ctx = ctx
        self.zero = torch.zeros(1, dtype=torch.float32, device=ctx.device)

    def encode_and_store(self, qkv, num_heads, num_kv_heads, head_dim, batch, paged, write):
        x = qkv.view(qkv.shape[0], num_heads + 2 * num_kv_heads, head_dim)
        x[:, :num_heads + num_kv_heads, 0] += (batch.positions.float() * self.step).unsqueeze(1).to(x.dtype)
        group = batch.groups[paged.group]
        self.ctx.ops.rope_store(qkv, batch.positions, self.zero, num_heads, num_kv_heads, head_dim,
                                0, group.slot_map if write else None, paged.keys, paged.values)


def register_toys():
    MIXERS.register("toy_decay", ToyDecayMixer)
    FEED_FORWARDS.register("toy_routed", ToyRoutedFF)
    POSITION_ENCODINGS.register("toy_shift", ToyShiftEncoding)


def unregister_toys():
    MIXERS.unregister("toy_decay")
    FEED_FORWARDS.unregister("toy_routed")
    POSITION_ENCODINGS.unregister("toy_shift")
