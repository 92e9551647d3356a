"""Toy parts defined by the tests, to show that the framework takes a new mixer, feed-forward
or position encoding without a change to its files.  None of them is anybody's model.

* `ToyDecayMixer`: a mixer with per-request state of fixed size and no paged cache:
  s_t = decay * s_{t-1} + x_t W_in,  y_t = s_t W_out.  The state lives in the cache manager's
  state slots, so a request can be continued in portions.
* `ToyRoutedFF`: a feed-forward with routing: top-1 of `n_experts` tiny SwiGLU-free experts,
  router logits in float32.
* `ToyShiftEncoding`: a position encoding that adds position * step to one key/query dim.
* `ToyWideValueMixer`: attention whose values are wider than its keys (the cache keeps keys and
  values of different widths), with its own gather over the block table and an optional bias.
* `ToyPositionEmbedding`: an embedding that adds a learned row per position (needs the batch's
  positions, not only its token ids).
* `ToySandwichBlock`: an arrangement with four norms (before and after each part);
  `ToyMixerOnlyBlock`: a layer without a feed-forward.
Each has its plain whole-sequence formula beside it.
"""

from __future__ import annotations

import torch


def mm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a[..., K] times b[N, K] transposed, written as a product and a sum: the toy parts' sizes
    are tiny, and on the GPU this keeps them off the library's float32 matrix product (whose
    results the engine's own float32 path deliberately does not rely on)."""
    if not a.is_cuda:
        return a @ b.T
    return (a.unsqueeze(-2) * b).sum(-1)

from somi_inference_b200.parts import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, MIXERS,
                                       POSITION_ENCODINGS)
from somi_inference_b200.parts.base import (CacheNeeds, PagedKVNeeds, StateNeeds, TensorDecl,
                                            names_of)


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
        u = mm(x.float(), self.w_in)
        out = torch.empty_like(u)
        cu = batch.host.cu_q
        for r, slot in enumerate(batch.host.state_slot.tolist()):
            s = state[slot].clone()
            for t in range(int(cu[r]), int(cu[r + 1])):
                s = self.decay * s + u[t]
                out[t] = s
            if owns_cache:
                state[slot] = s
        return mm(out, self.w_out).to(x.dtype)

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
        choice = torch.argmax(mm(x, router), dim=-1)
        out = torch.empty_like(x)
        for t in range(x.shape[0]):
            e = int(choice[t])
            out[t] = mm(torch.relu(mm(x[t], w1[e])), w2[e])
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


class ToyWideValueMixer:
    """Causal attention with `heads` heads over one key/value head: keys of width `key_dim`,
    values of width `value_dim` (not the same), no position encoding, an output bias that the
    weight file may lack.  It writes and gathers its pages itself, with tensor indexing, and
    plans on the host (so its steps are not captured in graphs)."""

    graph_safe = False

    @staticmethod
    def declare(params):
        n = names_of(params)
        h, nh = int(params["hidden_size"]), int(params["heads"])
        kd, vd = int(params["key_dim"]), int(params["value_dim"])
        return [TensorDecl(n["wq"], (nh * kd, h)), TensorDecl(n["wk"], (kd, h)),
                TensorDecl(n["wv"], (vd, h)), TensorDecl(n["wo"], (h, nh * vd)),
                TensorDecl(n["bo"], (h,), matrix=False, optional=True)]

    def __init__(self, params, tensors, ctx):
        n = names_of(params)
        self.nh, self.kd, self.vd = int(params["heads"]), int(params["key_dim"]), int(params["value_dim"])
        self.wq, self.wk = tensors[n["wq"]].float(), tensors[n["wk"]].float()
        self.wv, self.wo = tensors[n["wv"]].float(), tensors[n["wo"]].float()
        self.bo = tensors[n["bo"]].float() if n["bo"] in tensors else None

    def cache_needs(self):
        return CacheNeeds(paged=PagedKVNeeds(1, self.kd, None, value_dim=self.vd))

    def forward(self, x, batch, cache, owns_cache):
        paged = cache.paged
        group = batch.groups[paged.group]
        ps = paged.page_size
        xf = x.float()
        T = xf.shape[0]
        q = mm(xf, self.wq).view(T, self.nh, self.kd)
        if owns_cache:
            slot = group.slot_map.long()
            paged.keys[slot // ps, 0, slot % ps] = mm(xf, self.wk).to(paged.keys.dtype)
            paged.values[slot // ps, 0, slot % ps] = mm(xf, self.wv).to(paged.values.dtype)
        out = torch.empty((T, self.nh * self.vd), dtype=torch.float32, device=x.device)
        cu, ctx = batch.host.cu_q, batch.host.ctx_len
        for r in range(batch.num_requests):
            t0, t1, c = int(cu[r]), int(cu[r + 1]), int(ctx[r])
            n = c + (t1 - t0)
            pos = torch.arange(n, device=x.device)
            pages = group.block_table[r, pos // ps].long()
            k = paged.keys[pages, 0, pos % ps].float()              # [n, kd]
            v = paged.values[pages, 0, pos % ps].float()            # [n, vd]
            scores = (q[t0:t1].unsqueeze(2) * k).sum(-1) * self.kd ** -0.5          # [t, h, n]
            seen = pos.unsqueeze(0) <= (c + torch.arange(t1 - t0, device=x.device)).unsqueeze(1)
            scores = scores.masked_fill(~seen.unsqueeze(1), float("-inf"))
            probs = torch.softmax(scores, -1)
            out[t0:t1] = (probs.unsqueeze(-1) * v).sum(2).reshape(t1 - t0, -1)         # [t, h, v]
        y = mm(out, self.wo)
        if self.bo is not None:
            y = y + self.bo
        return y.to(x.dtype)

    @staticmethod
    def plain(x, wq, wk, wv, wo, bo, nh):
        T = x.shape[0]
        kd, vd = wk.shape[0], wv.shape[0]
        q, k, v = (x @ wq.T).view(T, nh, kd), x @ wk.T, x @ wv.T
        scores = torch.einsum("thd,nd->thn", q, k) * kd ** -0.5
        mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
        p = torch.softmax(scores.masked_fill(~mask.unsqueeze(1), float("-inf")), -1)
        y = torch.einsum("thn,nv->thv", p, v).reshape(T, nh * vd) @ wo.T
        return y if bo is None else y + bo


class ToyPositionEmbedding:
    """x_t = E[token_t] + P[position_t]: needs the batch's positions as well as its token ids."""

    @staticmethod
    def declare(params):
        n = names_of(params)
        v, h, m = int(params["vocab_size"]), int(params["hidden_size"]), int(params["max_positions"])
        return [TensorDecl(n["weight"], (v, h)), TensorDecl(n["positions"], (m, h))]

    def __init__(self, params, tensors, ctx):
        n = names_of(params)
        self.table, self.rows = tensors[n["weight"]].float(), tensors[n["positions"]].float()

    def forward(self, batch):
        return (self.table[batch.token_ids.long()] + self.rows[batch.positions.long()]).contiguous()


class ToySandwichBlock:
    """x = x + norm_b(mixer(norm_a(x)));  x = x + norm_d(feed_forward(norm_c(x))): four norms.
    A part's output is normalised through the norm interface itself, over a zero stream."""

    def __init__(self, mixer, feed_forward, norms):
        assert set(norms) == {"pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward"}
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, residual, pending, batch, cache, owns_cache):
        h = self.norms["pre_mixer"].forward(residual, pending)
        a = self.mixer.forward(h, batch, cache, owns_cache)
        a = self.norms["post_mixer"].forward(torch.zeros_like(residual), a)
        h = self.norms["pre_feed_forward"].forward(residual, a)
        f = self.feed_forward.forward(h, batch)
        return self.norms["post_feed_forward"].forward(torch.zeros_like(residual), f)


class ToyMixerOnlyBlock:
    """x = x + mixer(norm(x)): a layer without a feed-forward."""

    def __init__(self, mixer, feed_forward, norms):
        assert feed_forward is None and set(norms) == {"mixer"}
        self.mixer, self.feed_forward, self.norm = mixer, None, norms["mixer"]

    def forward(self, residual, pending, batch, cache, owns_cache):
        return self.mixer.forward(self.norm.forward(residual, pending), batch, cache, owns_cache)


def register_toys():
    MIXERS.register("toy_decay", ToyDecayMixer)
    MIXERS.register("toy_wide_value", ToyWideValueMixer)
    FEED_FORWARDS.register("toy_routed", ToyRoutedFF)
    POSITION_ENCODINGS.register("toy_shift", ToyShiftEncoding)
    EMBEDDINGS.register("toy_position_embedding", ToyPositionEmbedding)
    ARRANGEMENTS.register("toy_sandwich", ToySandwichBlock)
    ARRANGEMENTS.register("toy_mixer_only", ToyMixerOnlyBlock)


def unregister_toys():
    MIXERS.unregister("toy_decay")
    MIXERS.unregister("toy_wide_value")
    FEED_FORWARDS.unregister("toy_routed")
    POSITION_ENCODINGS.unregister("toy_shift")
    EMBEDDINGS.unregister("toy_position_embedding")
    ARRANGEMENTS.unregister("toy_sandwich")
    ARRANGEMENTS.unregister("toy_mixer_only")
