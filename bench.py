"""Benchmark of the flagship serving step: decode tokens per second, Qwen2.5-0.5B-shaped.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 0.5b|7b|14b] [--layers L]
    python bench.py --impl reference      (prints that the reference arm is unavailable)

A step is one decode step of the whole engine: batch of 8 requests with 2,048 cached tokens
each, random bfloat16 weights, one new token per request (batch layout upload, all layers,
head, sampling kernel).  `value` times K such steps on the device with CUDA events;
`e2e` runs the same through `LLM.step()` with host token ids in and sampled ids out.
Also reported: a 2,048-token prefill, the HBM roofline of the decode step, and decode at
batch 1 and 64.  One JSON line on stdout.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {
    # the three benchmark shapes: Qwen2.5-0.5B, 7B and 14B sizes
    "0.5b": dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14,
                 num_key_value_heads=2, head_dim=64, intermediate_size=4864, vocab_size=151936,
                 rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "7b": dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28,
               num_key_value_heads=4, head_dim=128, intermediate_size=18944, vocab_size=152064,
               rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40,
                num_key_value_heads=8, head_dim=128, intermediate_size=13824, vocab_size=152064,
                rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
FULL_LAYERS = {k: v["num_hidden_layers"] for k, v in SHAPES.items()}
CONTEXT = 2048          # cached tokens per request when decode is timed
MAX_CONTEXT = 4096      # "benchmark at context 4096": positions the model is laid out for
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}
            if "bf16_tflops_sustained" in raw:
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out, "measured"
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nv = None

    def _loop(self) -> None:
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def build_engine(shape: str, layers: int, batches: list[int], extra_tokens: int,
                 context: int = CONTEXT, prefill_tokens: int = PREFILL_TOKENS):
    import torch

    from somi_inference_b200.config import Qwen2Config
    from somi_inference_b200.engine import Engine
    from somi_inference_b200.parts import declared_tensors
    raw = dict(SHAPES[shape], num_hidden_layers=layers, max_position_embeddings=max(MAX_CONTEXT, context + extra_tokens, prefill_tokens),
               architectures=["Qwen2ForCausalLM"], hidden_act="silu", use_sliding_window=False)
    cfg = Qwen2Config.from_dict(raw)
    gen = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, d in declared_tensors(cfg.to_model_spec()).items():
        if d.init == "ones":
            tensors[name] = torch.ones(d.shape, dtype=torch.bfloat16, device="cuda")
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=gen)
            tensors[name] = t.to(torch.bfloat16)
            del t
    page = 16
    most = max(batches) * (context + extra_tokens) + prefill_tokens + 4 * page
    eng = Engine.from_tensors(cfg, tensors, dtype="bfloat16", page_size=page, max_tokens=most,
                              max_requests=max(batches) + 1)
    return cfg, eng


def model_bytes_and_flops(cfg, layers: int) -> dict:
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer = (nq + 2 * nkv) * hd * H + (nq + 2 * nkv) * hd + nq * hd * H + 3 * H * I + 2 * H
    head = V * H
    weight_params = layers * per_layer + head + H        # every weight a decode step reads once
    kv_bytes_per_token = layers * 2 * nkv * hd * 2
    matmul_params = layers * ((nq + 2 * nkv) * hd * H + nq * hd * H + 3 * H * I)
    return {"weight_bytes": 2 * weight_params, "kv_bytes_per_token": kv_bytes_per_token,
            "matmul_params": matmul_params, "head_params": head,
            "attn_flops_per_layer": lambda T: 4 * nq * hd * (T * (T + 1) // 2)}


def fill_context(eng, batch: int, vocab: int, tag: str, context: int = CONTEXT):
    """Prefill `batch` requests to `context` tokens through the step function."""
    import torch

    from somi_inference_b200.engine import StepEntry
    g = torch.Generator().manual_seed(1)
    ids = []
    for b in range(batch):
        toks = torch.randint(0, vocab, (context,), generator=g).tolist()
        eng.step([StepEntry((tag, b), toks, [])])
        ids.append((tag, b))
    torch.cuda.synchronize()
    return ids


def time_decode(eng, sampler, reqs, vocab: int, steps: int, warmup: int):
    """K decode steps, enqueued back to back, timed with CUDA events."""
    import torch

    from somi_inference_b200.engine import StepEntry
    from somi_inference_b200.sampling import SamplingParams
    B = len(reqs)
    g = torch.Generator().manual_seed(2)
    feed = torch.randint(0, vocab, (steps + warmup, B), generator=g).tolist()
    params = [SamplingParams(temperature=0.0)] * B

    def one(i: int):
        logits = eng.step([StepEntry(r, [feed[i][b]], [0]) for b, r in enumerate(reqs)])
        return sampler.sample(logits, params, [i] * B, [0] * B)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    launches0 = eng.ops.launches
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(warmup, warmup + steps):
        out = one(i)
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end) / steps
    return ms, (eng.ops.launches - launches0), out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--shape", choices=list(SHAPES), default="0.5b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run only this phase and print its figures (for profiling runs)")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="cached tokens per request (with --only decode)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (with --only prefill)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "luke396/somi-inference does not install offline (its build backend "
                          "uv_build is not in the wheelhouse) and its public API loads models and "
                          "tokenizers from the Hugging Face hub, which needs a network"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    from somi_inference_b200.engine import LLM, StepEntry
    from somi_inference_b200.sampling import Sampler, SamplingParams

    layers = args.layers or FULL_LAYERS[args.shape]
    batches = [args.batch] if args.no_points else sorted({1, args.batch, 64})
    extra = 2 * (args.steps + args.warmup) + 8
    if args.only is None and (args.context != CONTEXT or args.prefill_tokens != PREFILL_TOKENS):
        print("bench.py: --context and --prefill-tokens go with --only decode / --only prefill")
        return 2
    if args.only is not None:
        batches = [args.batch]
    n_prefill = args.prefill_tokens
    cfg, eng = build_engine(args.shape, layers, batches, extra, args.context, n_prefill)
    sampler = Sampler(eng.ops, eng.device)
    sizes = model_bytes_and_flops(cfg, layers)
    pk, pk_kind = peaks()
    V = cfg.vocab_size

    if args.only == "decode":
        reqs = fill_context(eng, args.batch, V, "main", args.context)
        ms, launches, _ = time_decode(eng, sampler, reqs, V, args.steps, args.warmup)
        print(json.dumps({"only": "decode", "batch": args.batch, "context": args.context,
                          "ms_per_step": round(ms, 4), "tokens_per_s": round(args.batch / ms * 1e3, 1),
                          "gpu_launches": int(launches)}))
        return 0

    # ---- prefill of 2,048 tokens (one request, one step), timed over a few repetitions
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, V, (n_prefill,), generator=g).tolist()
    pre_ms = []
    # the same layout every time: from its third run on the step is replayed from the CUDA graph
    # that the engine captured at the second
    for rep in range(7):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        eng.step([StepEntry(("prefill", rep), prompt, [n_prefill - 1])])
        e.record()
        torch.cuda.synchronize()
        eng.end(("prefill", rep))
        pre_ms.append(s.elapsed_time(e))
    prefill_ms = sorted(pre_ms[2:])[len(pre_ms[2:]) // 2]
    prefill_flops = (2 * sizes["matmul_params"] * n_prefill + 2 * sizes["head_params"]
                     + layers * sizes["attn_flops_per_layer"](n_prefill))
    prefill = {"value": round(n_prefill / prefill_ms * 1e3, 1), "tokens": n_prefill,
               "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", **prefill}))
        return 0

    # ---- decode at the headline batch, device-timed
    reqs = fill_context(eng, args.batch, V, "main")
    with ClockSampler() as clocks:
        ms, launches, _ = time_decode(eng, sampler, reqs, V, args.steps, args.warmup)
    value = args.batch / ms * 1e3
    ctx_mid = CONTEXT + args.warmup + args.steps / 2
    step_bytes = sizes["weight_bytes"] + args.batch * ctx_mid * sizes["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_kind}
    for r in reqs:
        eng.end(r)

    # ---- the same through the Python entry point: host token ids in, sampled ids out
    llm = LLM(eng, max_concurrent=max(batches) + 1, max_num_batched_tokens=8192, chunk_size=2048)
    gq = torch.Generator().manual_seed(4)
    e2e_reqs = [llm.make_request(torch.randint(0, V, (CONTEXT,), generator=gq).tolist(),
                                 max_new_tokens=args.steps + args.warmup + 4,
                                 sampling_params=SamplingParams(temperature=0.0), ignore_eos=True)
                for _ in range(args.batch)]
    for r in e2e_reqs:
        llm.scheduler.add_request(r)
    while any(r.num_computed < CONTEXT for r in e2e_reqs):
        llm.step()
    for _ in range(args.warmup):
        llm.step()
    torch.cuda.synchronize()
    n0 = sum(len(r.output_tokens) for r in e2e_reqs)
    with ClockSampler() as e2e_clocks:
        t0 = time.perf_counter()
        for _ in range(args.steps):
            llm.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    n1 = sum(len(r.output_tokens) for r in e2e_reqs)
    e2e = {"value": round((n1 - n0) / dt, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(llm.engine.builder.h2d_bytes_last + llm.sampler_h2d_bytes()
                                     + llm.engine.token_patch_bytes),
           "d2h_bytes_per_step": int(llm.d2h_bytes_last), "ms_per_step": round(dt / args.steps * 1e3, 3),
           # this region runs later than the device-timed one, under the power cap often at a lower clock
           "sm_mhz": e2e_clocks.summary().get("sm_mhz")}
    for r in e2e_reqs:
        if llm.engine.has(r.request_id):
            llm.engine.end(r.request_id)
    llm.scheduler.running.clear()

    # ---- decode at batch 1 and 64
    points = {}
    if not args.no_points:
        for b in (1, 64):
            rq = fill_context(eng, b, V, f"b{b}")
            pms, _, _ = time_decode(eng, sampler, rq, V, max(10, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b / pms * 1e3, 1)
            for r in rq:
                eng.end(r)

    line = {
        "metric": "decode tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "config": {"model": f"Qwen2.5-{args.shape.upper()}-shaped", "layers": layers,
                   "layers_full": FULL_LAYERS[args.shape], "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size,
                   "vocab": cfg.vocab_size, "tied": cfg.tie_word_embeddings,
                   "global_batch": args.batch, "seq_len": CONTEXT, "max_context": MAX_CONTEXT,
                   "kv_block": 16, "parallelism": "single GPU",
                   "l2": "no flush: a step reads more than the 126 MB L2"},
        "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches),
        "prefill": prefill, "roofline": roofline, "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
