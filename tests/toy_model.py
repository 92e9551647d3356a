"""A toy architecture defined entirely by the tests: different mixers and feed-forwards in
different layers, a layer that runs twice, a run that reads another run's cache, an embedding
that reads positions, a layer with four norms, a layer without a feed-forward, and a mixer whose
values are wider than its keys (with a bias that the file may lack).  It is
registered, built and stepped through the framework's public registries only; its plain
whole-sequence forward is written out below for comparison.  It is nobody's model."""

from __future__ import annotations

import json
import os
from dataclasses import dataclass

import torch

from somi_inference_b200.config import LayerSpec, ModelSpec, PartSpec, RunSpec
from somi_inference_b200.parts import declared_tensors
from somi_inference_b200.weights import save_safetensors
from tests.plain import qwen2_plain as plain
from tests.toy_parts import ToyDecayMixer, ToyRoutedFF, ToyWideValueMixer

ARCH = "ToyMixedForCausalLM"
H, V, EPS = 48, 211, 1e-5


@dataclass(frozen=True)
class ToyConfig:
    raw: tuple
    architecture = ARCH

    @classmethod
    def from_dict(cls, d):
        return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

    def to_dict(self):
        return {k: json.loads(v) for k, v in self.raw}

    def to_model_spec(self) -> ModelSpec:
        d = self.to_dict()

        def norm(name):
            return PartSpec("rmsnorm", {"size": H, "eps": EPS, "names": {"weight": name}})

        def attn(p, nq, nkv, hd, window, position):
            return PartSpec("attention", {
                "hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                "qkv_bias": True, "out_bias": False, "window": window, "position": position,
                "names": {f"{x}_{y}": f"{p}.{x}.{y}" for x in "qkvo" for y in ("weight", "bias")}})

        def swiglu(p, inter):
            return PartSpec("swiglu", {"hidden_size": H, "intermediate_size": inter,
                                       "names": {"gate_weight": f"{p}.gate", "up_weight": f"{p}.up",
                                                 "down_weight": f"{p}.down"}})

        def two(p):
            return {"mixer": norm(f"{p}.n1"), "feed_forward": norm(f"{p}.n2")}
        layers = (
            LayerSpec("l0", attn("l0", 4, 2, 16, None, PartSpec("rope", {
                "head_dim": 16, "theta": d["theta"], "max_positions": d["max_positions"]})),
                swiglu("l0", 72), two("l0")),
            LayerSpec("l1", PartSpec("toy_decay", {"hidden_size": H, "state_size": 24, "decay": 0.8,
                                                   "names": {"w_in": "l1.w_in", "w_out": "l1.w_out"}}),
                      PartSpec("toy_routed", {"hidden_size": H, "n_experts": d["n_experts"], "inner": 20,
                                              "names": {"router": "l1.router", "w1": "l1.w1",
                                                        "w2": "l1.w2"}}),
                      two("l1")),
            LayerSpec("l2", attn("l2", 2, 1, 32, 6, PartSpec("toy_shift", {"step": 0.05})),
                      swiglu("l2", 40), two("l2")),
            # four norms around the two parts
            LayerSpec("l3", attn("l3", 2, 2, 16, None, PartSpec("none", {})), swiglu("l3", 56),
                      {k: norm(f"l3.{k}") for k in ("pre_mixer", "post_mixer", "pre_feed_forward",
                                                    "post_feed_forward")},
                      arrangement="toy_sandwich"),
            # no feed-forward; values wider than keys; a bias the file may lack
            LayerSpec("l4", PartSpec("toy_wide_value", {
                "hidden_size": H, "heads": 3, "key_dim": 8, "value_dim": 24,
                "names": {"wq": "l4.wq", "wk": "l4.wk", "wv": "l4.wv", "wo": "l4.wo", "bo": "l4.bo"}}),
                None, {"mixer": norm("l4.n1")}, arrangement="toy_mixer_only"),
        )
        return ModelSpec(ARCH, H, V, d["max_positions"],
                         PartSpec("toy_position_embedding", {
                             "vocab_size": V, "hidden_size": H, "max_positions": d["max_positions"],
                             "names": {"weight": "emb", "positions": "pos"}}),
                         layers,
                         (RunSpec(0), RunSpec(1), RunSpec(3), RunSpec(2), RunSpec(4), RunSpec(1),
                          RunSpec(0, cache_of=0)),
                         norm("final"),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False,
                                              "names": {"weight": "head", "tied_to": "emb"}}))


def write_toy_model(out_dir: str, seed: int = 5, dtype=torch.float32, n_experts: int = 3,
                    with_optional: bool = False) -> str:
    """Tensors declared optional are left out unless `with_optional`.  `n_experts` = 1 switches the hard top-1 routing off: under bfloat16 rounding a token
    whose two best router logits nearly tie may legitimately go to the other expert, which no
    tolerance on logits can express; the bfloat16 test therefore routes trivially."""
    os.makedirs(out_dir, exist_ok=True)
    raw = {"architectures": [ARCH], "theta": 5000.0, "max_positions": 256, "n_experts": n_experts}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for name, decl in declared_tensors(ToyConfig.from_dict(raw).to_model_spec()).items():
        if decl.ignored or (decl.optional and not with_optional):
            continue
        if decl.init == "ones":
            t = 1 + 0.1 * torch.randn(decl.shape, generator=g)
        else:
            t = 0.12 * torch.randn(decl.shape, generator=g)
        tensors[name] = t.to(dtype)
    save_safetensors(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def _attention(h, w, p, nq, nkv, hd, window, encode, kv=None):
    T = h.shape[0]
    q = (h @ w[f"{p}.q.weight"].T + w[f"{p}.q.bias"]).view(T, nq, hd).transpose(0, 1)
    k = (h @ w[f"{p}.k.weight"].T + w[f"{p}.k.bias"]).view(T, nkv, hd).transpose(0, 1)
    v = (h @ w[f"{p}.v.weight"].T + w[f"{p}.v.bias"]).view(T, nkv, hd).transpose(0, 1)
    q, k = encode(q), encode(k)
    if kv is not None:
        k, v = kv
    o = plain.causal_attention(q, k, v, window)
    return o.transpose(0, 1).reshape(T, nq * hd) @ w[f"{p}.o.weight"].T, (k, v)


def _swiglu(h, w, p):
    g, u = h @ w[f"{p}.gate"].T, h @ w[f"{p}.up"].T
    return (g * torch.sigmoid(g) * u) @ w[f"{p}.down"].T


def plain_logits(model_dir: str, ids: list[int]) -> torch.Tensor:
    """Whole-sequence forward of the toy model with elementary operations."""
    cfg, w = plain.load_folder(model_dir)
    T = len(ids)
    x = w["emb"][torch.tensor(ids)] + w["pos"][:T]
    cos, sin = plain.rope_tables(16, cfg["theta"], T)

    def rope(t):
        return plain.apply_rope(t, cos, sin)

    def shift(t):
        t = t.clone()
        t[:, :, 0] += torch.arange(T).float() * 0.05
        return t

    def l0(x, kv=None):
        a, kv_out = _attention(plain.rms_norm(x, w["l0.n1"], EPS), w, "l0", 4, 2, 16, None, rope, kv)
        x = x + a
        return x + _swiglu(plain.rms_norm(x, w["l0.n2"], EPS), w, "l0"), kv_out

    def l1(x):
        x = x + ToyDecayMixer.plain(plain.rms_norm(x, w["l1.n1"], EPS), w["l1.w_in"], w["l1.w_out"], 0.8)
        return x + ToyRoutedFF.plain(plain.rms_norm(x, w["l1.n2"], EPS), w["l1.router"],
                                     w["l1.w1"].view(-1, 20, H), w["l1.w2"].view(-1, H, 20))

    def l2(x):
        a, _ = _attention(plain.rms_norm(x, w["l2.n1"], EPS), w, "l2", 2, 1, 32, 6, shift)
        x = x + a
        return x + _swiglu(plain.rms_norm(x, w["l2.n2"], EPS), w, "l2")

    def l3(x):
        a, _ = _attention(plain.rms_norm(x, w["l3.pre_mixer"], EPS), w, "l3", 2, 2, 16, None,
                          lambda t: t)
        x = x + plain.rms_norm(a, w["l3.post_mixer"], EPS)
        f = _swiglu(plain.rms_norm(x, w["l3.pre_feed_forward"], EPS), w, "l3")
        return x + plain.rms_norm(f, w["l3.post_feed_forward"], EPS)

    def l4(x):
        return x + ToyWideValueMixer.plain(plain.rms_norm(x, w["l4.n1"], EPS), w["l4.wq"], w["l4.wk"],
                                           w["l4.wv"], w["l4.wo"], w.get("l4.bo"), 3)

    x, kv0 = l0(x)
    x = l1(x)
    x = l3(x)
    x = l2(x)
    x = l4(x)
    x = l1(x)
    x, _ = l0(x, kv0)
    return plain.rms_norm(x, w["final"], EPS) @ w["head"].T
