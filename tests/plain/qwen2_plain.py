"""Plain, slow implementation of the Qwen2.5 dense decoder: whole sequences, no cache.

One function per part, written from the reference's formulas (file:line cited
per function, paths inside luke396/somi-inference).  It shares no code with the
engine: it reads config.json with `json` and the safetensors file with its own
few lines, and computes in float32 (or float64) on the CPU with elementary
tensor operations only.

Its agreement with the reference's own model code on a tiny random model is
recorded under tests/golden/ (made by tests/golden/make_golden.py) and checked
by tests/test_plain.py.
"""

from __future__ import annotations

import json
import math
import os
import struct

import torch


# --------------------------------------------------------------------- loading
def read_safetensors(path: str) -> dict[str, torch.Tensor]:
    """Own reader: 8-byte header length, JSON header, raw little-endian data."""
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
             "F64": torch.float64, "I32": torch.int32, "I64": torch.int64}
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, t = e["data_offsets"]
        if t == b:
            out[name] = torch.empty(e["shape"], dtype=kinds[e["dtype"]])
            continue
        out[name] = torch.frombuffer(bytearray(data[b:t]), dtype=kinds[e["dtype"]]).reshape(e["shape"]).clone()
    return out


def load_folder(model_dir: str, dtype=torch.float32):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {k: v.to(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
    return cfg, w


# ----------------------------------------------------------------------- parts
def embed(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x = E[ids]  (somi_inference/models/qwen2.py:360,382)."""
    return table[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2, -1) + eps); out = weight * y  (somi_inference/models/qwen2.py:46-62)."""
    var = x.pow(2).mean(dim=-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def rope_tables(head_dim: int, theta: float, n_pos: int, dtype=torch.float32):
    """inv_freq = 1/theta^(arange(0,d,2)/d); freq = outer(t, inv_freq); emb = cat(freq, freq);
    cos/sin of emb  (somi_inference/models/qwen2.py:71-81)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2) / head_dim))
    t = torch.arange(n_pos, dtype=inv_freq.dtype)
    freq = torch.outer(t, inv_freq)
    emb = torch.cat((freq, freq), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    """[x1, x2] -> [-x2, x1], halves split at d/2  (somi_inference/models/qwen2.py:92-96)."""
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x*cos + rotate_half(x)*sin, cos/sin [T, d] broadcast over heads; x is [heads, T, d]
    (somi_inference/models/qwen2.py:99-113)."""
    return x * cos.unsqueeze(0) + rotate_half(x) * sin.unsqueeze(0)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: int | None = None) -> torch.Tensor:
    """q [nq,T,d], k,v [nkv,T,d] -> [nq,T,d].  scale = d^-0.5; kv heads repeated
    nq/nkv times each (repeat_interleave); scores + triu(-inf, 1); softmax; P V
    (somi_inference/models/qwen2.py:158-186).  `window` n additionally hides keys
    j <= i - n (the reference never sets one: qwen2.py:262,272)."""
    nq, T, d = q.shape
    nkv = k.shape[0]
    if nq % nkv:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    rep = nq // nkv
    k = k.repeat_interleave(rep, dim=0)
    v = v.repeat_interleave(rep, dim=0)
    scores = torch.einsum("hid,hjd->hij", q, k) * (d ** -0.5)
    i = torch.arange(T).unsqueeze(1)
    j = torch.arange(T).unsqueeze(0)
    hidden = j > i
    if window is not None:
        hidden = hidden | (j <= i - window)
    scores = scores.masked_fill(hidden.unsqueeze(0), float("-inf"))
    return torch.einsum("hij,hjd->hid", torch.softmax(scores, dim=-1), v)


def attention_block(h: torch.Tensor, w: dict, p: str, cfg: dict, cos, sin,
                    window: int | None) -> torch.Tensor:
    """q/k/v projections with bias, view to heads, rope on q and k, attention, o_proj without
    bias  (somi_inference/models/qwen2.py:268-271,279-299)."""
    T = h.shape[0]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // nq
    q = (h @ w[f"{p}.self_attn.q_proj.weight"].T + w[f"{p}.self_attn.q_proj.bias"]).view(T, nq, d).transpose(0, 1)
    k = (h @ w[f"{p}.self_attn.k_proj.weight"].T + w[f"{p}.self_attn.k_proj.bias"]).view(T, nkv, d).transpose(0, 1)
    v = (h @ w[f"{p}.self_attn.v_proj.weight"].T + w[f"{p}.self_attn.v_proj.bias"]).view(T, nkv, d).transpose(0, 1)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window)
    return o.transpose(0, 1).reshape(T, nq * d) @ w[f"{p}.self_attn.o_proj.weight"].T


def swiglu(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    """down(silu(gate(h)) * up(h)), silu(z) = z*sigmoid(z); gate = first half of the merged
    projection, up = second  (somi_inference/models/qwen2.py:226-229;
    somi_inference/models/qwen2_adapter.py:182-189)."""
    g = h @ w[f"{p}.mlp.gate_proj.weight"].T
    u = h @ w[f"{p}.mlp.up_proj.weight"].T
    return (g * torch.sigmoid(g) * u) @ w[f"{p}.mlp.down_proj.weight"].T


def layer_window(cfg: dict, layer: int) -> int | None:
    if cfg.get("use_sliding_window") and layer >= cfg["max_window_layers"]:
        return cfg["sliding_window"]
    return None


def rope_theta(cfg: dict) -> float:
    """rope_parameters.rope_theta (somi_inference/models/qwen2_adapter.py:208-210) or the
    top-level key that raw config.json files carry."""
    if "rope_theta" in cfg:
        return float(cfg["rope_theta"])
    return float(cfg["rope_parameters"]["rope_theta"])


def hidden_states(cfg: dict, w: dict, ids: torch.Tensor) -> torch.Tensor:
    """Embedding, the layers (pre-norm attention + residual, pre-norm MLP + residual), final norm
    (somi_inference/models/qwen2.py:325-339,380-386).  ids [T] -> [T, H], positions 0..T-1
    (somi_inference/models/qwen2_adapter.py:91)."""
    T = ids.shape[0]
    eps = cfg["rms_norm_eps"]
    d = cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]
    x = embed(ids, w["model.embed_tokens.weight"])
    cos, sin = rope_tables(d, rope_theta(cfg), T, x.dtype)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        h = rms_norm(x, w[f"{p}.input_layernorm.weight"], eps)
        x = x + attention_block(h, w, p, cfg, cos, sin, layer_window(cfg, i))
        h = rms_norm(x, w[f"{p}.post_attention_layernorm.weight"], eps)
        x = x + swiglu(h, w, p)
    return rms_norm(x, w["model.norm.weight"], eps)


def lm_head(cfg: dict, w: dict, h: torch.Tensor) -> torch.Tensor:
    """logits = h E^T with the embedding matrix when tied (somi_inference/models/qwen2_adapter.py:60-62);
    with lm_head.weight when tie_word_embeddings is false (the architecture's rule; the reference
    always ties)."""
    table = w["model.embed_tokens.weight"] if cfg["tie_word_embeddings"] else w["lm_head.weight"]
    return h @ table.T


def logits(cfg: dict, w: dict, ids) -> torch.Tensor:
    """Logits at every position of one whole sequence: [T, vocab]."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    return lm_head(cfg, w, hidden_states(cfg, w, ids))


def greedy(cfg: dict, w: dict, prompt: list[int], n_new: int) -> list[int]:
    """Greedy continuation by re-running the whole sequence for every new token."""
    ids = list(prompt)
    out = []
    for _ in range(n_new):
        nxt = int(torch.argmax(logits(cfg, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out
