"""A part that brings a CUDA kernel of its own.

The feed-forward below is defined here, not in the framework: its kernel lies in
`tests/toy_kernels/`, is compiled by the engine's builder (`ops.build_library`) and is launched
by the part itself on the current stream.  It is registered, put into a two-layer architecture
beside the engine's attention, stepped (whole prompts, portions, single tokens, CUDA-graph
replay of repeated layouts) and compared with a plain whole-sequence forward.  No file of the
framework changes for it.  It is nobody's model.
"""

from __future__ import annotations

import ctypes
import json
import os
from dataclasses import dataclass

import pytest
import torch

from somi_inference_b200.config import (LayerSpec, ModelSpec, PartSpec, RunSpec, register_architecture,
                                         unregister_architecture)
from somi_inference_b200.parts import FEED_FORWARDS, TensorDecl, declared_tensors
from somi_inference_b200.weights import save_safetensors
from tests import replay
from tests.plain import qwen2_plain as plain
from tests.tiny import random_tokens
from tests.toy_model import _attention

pytestmark = pytest.mark.gpu

ARCH = "ToyOwnKernelForCausalLM"
H, V, EPS, THETA, POSITIONS = 40, 173, 1e-5, 20000.0, 256
KERNELS = os.path.join(os.path.dirname(os.path.abspath(__file__)), "toy_kernels")


class ToyGatedShiftFF:
    """y[t, i] = x[t, i] * sigmoid(g[i] * x[t, i]) + b[i] * x[t, (i + 1) mod H], by its own kernel."""

    graph_safe = True          # it launches one kernel and decides nothing on the host

    @staticmethod
    def declare(params):
        n, h = params["names"], int(params["hidden_size"])
        return [TensorDecl(n["g"], (h,)), TensorDecl(n["b"], (h,))]

    def __init__(self, params, tensors, ctx):
        from somi_inference_b200.ops import build_library
        self.h = int(params["hidden_size"])
        self.g = tensors[params["names"]["g"]].float().contiguous()
        self.b = tensors[params["names"]["b"]].float().contiguous()
        self.lib = ctypes.CDLL(build_library(KERNELS, "libtoy_part_kernels.so"))
        self.lib.toy_gated_shift.restype = ctypes.c_int

    def forward(self, x, batch):
        x = x.contiguous()
        y = torch.empty_like(x)
        code = {torch.float32: 0, torch.bfloat16: 1}[x.dtype]
        rc = self.lib.toy_gated_shift(
            ctypes.c_void_p(x.data_ptr()), ctypes.c_int(code), ctypes.c_void_p(self.g.data_ptr()),
            ctypes.c_void_p(self.b.data_ptr()), ctypes.c_void_p(y.data_ptr()),
            ctypes.c_int(x.shape[0]), ctypes.c_int(self.h),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError(f"toy_gated_shift failed with code {rc}")
        return y

    @staticmethod
    def plain(x, g, b):
        return x * torch.sigmoid(g * x) + b * torch.roll(x, -1, dims=-1)


@dataclass(frozen=True)
class OwnKernelConfig:
    raw: tuple
    architecture = ARCH

    @classmethod
    def from_dict(cls, d):
        return cls(tuple(sorted((k, json.dumps(v)) for k, v in d.items())))

    def to_dict(self):
        return {k: json.loads(v) for k, v in self.raw}

    def to_model_spec(self) -> ModelSpec:
        def norm(name):
            return PartSpec("rmsnorm", {"size": H, "eps": EPS, "names": {"weight": name}})

        def layer(p, nq, nkv, hd):
            rope = PartSpec("rope", {"head_dim": hd, "theta": THETA, "max_positions": POSITIONS})
            attn = PartSpec("attention", {
                "hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                "qkv_bias": True, "out_bias": False, "window": None, "position": rope,
                "names": {f"{x}_{y}": f"{p}.{x}.{y}" for x in "qkvo" for y in ("weight", "bias")}})
            ff = PartSpec("toy_gated_shift", {"hidden_size": H, "names": {"g": f"{p}.g", "b": f"{p}.b"}})
            return LayerSpec(p, attn, ff, {"mixer": norm(f"{p}.n1"), "feed_forward": norm(f"{p}.n2")})
        return ModelSpec(ARCH, H, V, POSITIONS,
                         PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H,
                                                "names": {"weight": "emb"}}),
                         (layer("a", 5, 1, 16), layer("b", 2, 2, 32)),
                         (RunSpec(0), RunSpec(1)),
                         norm("final"),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True,
                                              "names": {"weight": "head", "tied_to": "emb"}}))


def write_model(out_dir: str, dtype) -> str:
    os.makedirs(out_dir, exist_ok=True)
    raw = {"architectures": [ARCH]}
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(raw, f)
    g = torch.Generator().manual_seed(11)
    tensors = {}
    for name, decl in declared_tensors(OwnKernelConfig.from_dict(raw).to_model_spec()).items():
        if decl.ignored or decl.optional:
            continue
        t = (1 + 0.1 * torch.randn(decl.shape, generator=g)) if decl.init == "ones" else \
            0.15 * torch.randn(decl.shape, generator=g)
        tensors[name] = t.to(dtype)
    save_safetensors(tensors, os.path.join(out_dir, "model.safetensors"))
    return out_dir


def plain_logits(model_dir: str, ids: list[int]) -> torch.Tensor:
    _, w = plain.load_folder(model_dir)
    T = len(ids)
    x = w["emb"][torch.tensor(ids)]
    for p, nq, nkv, hd in (("a", 5, 1, 16), ("b", 2, 2, 32)):
        cos, sin = plain.rope_tables(hd, THETA, T)
        a, _ = _attention(plain.rms_norm(x, w[f"{p}.n1"], EPS), w, p, nq, nkv, hd, None,
                          lambda t: plain.apply_rope(t, cos, sin))
        x = x + a
        x = x + ToyGatedShiftFF.plain(plain.rms_norm(x, w[f"{p}.n2"], EPS), w[f"{p}.g"], w[f"{p}.b"])
    return plain.rms_norm(x, w["final"], EPS) @ w["emb"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_part_with_a_kernel_of_its_own(tmp_path, dtype):
    from somi_inference_b200.engine import Engine, StepEntry
    FEED_FORWARDS.register("toy_gated_shift", ToyGatedShiftFF)
    register_architecture(ARCH, OwnKernelConfig)
    try:
        d = write_model(str(tmp_path / dtype), getattr(torch, dtype))
        reqs = {f"k{i}": random_tokens(n, V, 40 + i) for i, n in enumerate([37, 64, 9, 80])}
        ref = {k: plain_logits(d, v) for k, v in reqs.items()}
        scale = max(v.abs().max().item() for v in ref.values())
        atol, rms = (5e-5, 2e-5) if dtype == "float32" else (4e-2 * scale, 4e-3 * scale)
        for mode in (replay.whole, replay.last_one_by_one, replay.portions, replay.mixed):
            steps, max_tokens = mode(reqs)
            eng = Engine(d, dtype=dtype, page_size=16, max_tokens=max_tokens)
            assert eng.model.graph_safe
            got = replay.run_steps(eng, steps)
            replay.compare(got, ref, atol, f"own kernel/{dtype}/{mode.__name__}", rms)
            eng.ops.check_errors()
        # one decode layout many times: the part's kernel is captured in the step's graph
        eng = Engine(d, dtype=dtype, page_size=16, max_tokens=256)
        toks = reqs["k1"]
        got = {}
        logits = eng.step([StepEntry("g", toks[:8], [7])]).float().cpu()
        got[("k1", 7)] = logits[0]
        for i in range(8, len(toks)):
            got[("k1", i)] = eng.step([StepEntry("g", [toks[i]], [0])]).float().cpu()[0]
        assert eng._graphs.hits >= 40, f"only {eng._graphs.hits} steps were replayed from a graph"
        replay.compare(got, ref, atol, f"own kernel/{dtype}/graph", rms)
    finally:
        unregister_architecture(ARCH)
        FEED_FORWARDS.unregister("toy_gated_shift")
