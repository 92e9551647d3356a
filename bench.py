"""Benchmark of the serving step: decode tokens per second of a Qwen2.5-7B-shaped model.

    python bench.py [--gpus 1] [--steps K] [--warmup W]          the whole line (default)
    python bench.py --impl reference [--steps K] [--warmup W]    luke396/somi-inference, same step
    python bench.py --only decode|prefill|mixed [--shape 0.5b|7b|14b] [--layers L] [--batch B]
                    [--context C] [--prefill-tokens T] [--profile]      one phase (profiling runs)

A step is one decode step of the whole engine: 8 requests with 2,048 cached tokens each,
random bfloat16 weights, one new token per request (batch layout upload, all layers, head,
sampling kernel).  `value` times K such steps on the device with CUDA events; `e2e` runs the
same through `LLM.step()` with host token ids in and sampled ids out.  The same line carries
a 2,048-token prefill, the HBM roofline of the decode step, latency statistics, decode at
batch 1 and 64 and at longer contexts, prefill at longer prompts (`points`), the 0.5B-shaped
model's figures (`shape_0_5b`), and a mixed step of the 14B-shaped model (64 decoding requests
beside a 512-token portion of a prompt, `mixed_14b`).  `--profile` adds one row per kernel of an
eager step: time, bytes, flops and the fraction of the measured peak.  One JSON line on stdout;
`--output-file` appends it, with an environment block, to a JSONL file.
"""

from __future__ import annotations

import argparse
import json
import os
import platform
import subprocess
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
LONG_CONTEXT = 40960    # ... when the points at 8 k and 32 k cached tokens are measured too
PREFILL_TOKENS = 2048
PAGE = 16
MIXED_PORTION = 512
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
REFERENCE_DIR = os.path.join(ROOT, "baseline", "_ref")


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
            self._stop.wait(0.02)

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


def environment() -> dict:
    """Where and with what the numbers were taken (as benchmarks/common.py:231-251 records)."""
    import torch

    def git(*args: str):
        try:
            r = subprocess.run(["git", *args], cwd=ROOT, capture_output=True, text=True, check=True)
            return r.stdout.strip()
        except (OSError, subprocess.CalledProcessError):
            return None

    env = {"git_sha": git("rev-parse", "HEAD"),
           "git_dirty": (lambda s: None if s is None else bool(s))(
               git("status", "--porcelain", "--untracked-files=no")),
           "python_version": platform.python_version(), "platform": platform.platform(),
           "torch_version": torch.__version__, "cuda_version": torch.version.cuda,
           "device_name": None, "device_capability": None, "driver": None}
    if torch.cuda.is_available():
        env["device_name"] = torch.cuda.get_device_name(0)
        env["device_capability"] = "%d.%d" % torch.cuda.get_device_capability(0)
        try:
            import pynvml
            pynvml.nvmlInit()
            v = pynvml.nvmlSystemGetDriverVersion()
            env["driver"] = v.decode() if isinstance(v, bytes) else str(v)
        except Exception:
            pass
    return env


def latency_stats(ms: list[float]) -> dict:
    """Mean, median and 95th percentile of the per-step times (benchmarks/common.py:159-170)."""
    s = sorted(ms)
    n = len(s)

    def pct(p: float) -> float:
        k = (n - 1) * p
        lo, hi = int(k), min(int(k) + 1, n - 1)
        return s[lo] + (s[hi] - s[lo]) * (k - lo)

    return {"mean_ms": round(sum(s) / n, 4), "median_ms": round(pct(0.5), 4),
            "p95_ms": round(pct(0.95), 4), "min_ms": round(s[0], 4), "max_ms": round(s[-1], 4)}


def shape_config(shape: str, layers: int, positions: int) -> dict:
    return dict(SHAPES[shape], num_hidden_layers=layers, max_position_embeddings=positions,
                architectures=["Qwen2ForCausalLM"], hidden_act="silu", use_sliding_window=False)


def config_record(shape: str, layers: int, batch: int, positions: int) -> dict:
    """The `config` entry of the line: every size, flat (both arms print the same)."""
    s = SHAPES[shape]
    return {"model": f"Qwen2.5-{shape.upper()}-shaped", "layers": layers,
            "layers_full": FULL_LAYERS[shape], "hidden": s["hidden_size"],
            "heads": s["num_attention_heads"], "kv_heads": s["num_key_value_heads"],
            "head_dim": s["head_dim"], "intermediate": s["intermediate_size"],
            "vocab": s["vocab_size"], "tied": s["tie_word_embeddings"],
            "rms_norm_eps": s["rms_norm_eps"], "rope_theta": s["rope_theta"],
            "global_batch": batch, "seq_len": CONTEXT, "max_context": positions,
            "kv_block": PAGE, "prefill_tokens": PREFILL_TOKENS, "parallelism": "single GPU",
            "l2": "no flush: a step reads more than the 126 MB L2"}


def build_engine(shape: str, layers: int, max_tokens: int, max_requests: int, positions: int):
    import torch

    from somi_inference_b200.config import Qwen2Config
    from somi_inference_b200.engine import Engine
    from somi_inference_b200.parts import declared_tensors
    cfg = Qwen2Config.from_dict(shape_config(shape, layers, positions))
    gen = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, d in declared_tensors(cfg.to_model_spec()).items():
        if d.ignored:
            continue
        if d.init == "ones":
            tensors[name] = torch.ones(d.shape, dtype=torch.bfloat16, device="cuda")
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device="cuda").normal_(0.0, 0.02, generator=gen)
            tensors[name] = t.to(torch.bfloat16)
            del t
    eng = Engine.from_tensors(cfg, tensors, dtype="bfloat16", page_size=PAGE,
                              max_tokens=max_tokens + 4 * PAGE, max_requests=max_requests)
    return cfg, eng


def model_sizes(cfg, layers: int) -> dict:
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    nq, nkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    per_layer = (nq + 2 * nkv) * hd * H + (nq + 2 * nkv) * hd + nq * hd * H + 3 * H * I + 2 * H
    head = V * H
    return {"weight_bytes": 2 * (layers * per_layer + head + H),   # every weight a decode step reads once
            "kv_bytes_per_token": layers * 2 * nkv * hd * 2,
            "matmul_params": layers * ((nq + 2 * nkv) * hd * H + nq * hd * H + 3 * H * I),
            "head_params": head, "attn_flops_per_pair": 4 * nq * hd * layers}


def step_flops(sizes: dict, tokens: int, wanted: int, pairs: int) -> float:
    """Products of all layers for `tokens` rows, the head for `wanted` rows, attention over
    `pairs` (query, key) pairs per head."""
    return (2.0 * sizes["matmul_params"] * tokens + 2.0 * sizes["head_params"] * wanted
            + float(sizes["attn_flops_per_pair"]) * pairs)


def fill_context(eng, batch: int, vocab: int, tag: str, context: int):
    """Prefill `batch` requests to `context` tokens through the step function."""
    import torch

    from somi_inference_b200.engine import StepEntry
    g = torch.Generator().manual_seed(1)
    ids = []
    for b in range(batch):
        toks = torch.randint(0, vocab, (context,), generator=g).tolist()
        for lo in range(0, context, 8192):
            eng.step([StepEntry((tag, b), toks[lo:lo + 8192], [])])
        ids.append((tag, b))
    torch.cuda.synchronize()
    return ids


def time_decode(eng, sampler, reqs, vocab: int, steps: int, warmup: int):
    """K decode steps, enqueued back to back, timed with CUDA events (one after every step)."""
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
    events = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    events[0].record()
    for i in range(steps):
        one(warmup + i)
        events[i + 1].record()
    torch.cuda.synchronize()
    ms = events[0].elapsed_time(events[-1]) / steps
    per_step = [events[i].elapsed_time(events[i + 1]) for i in range(steps)]
    return ms, (eng.ops.launches - launches0), per_step


def decode_roofline(sizes: dict, batch: int, context_mid: float, ms: float, pk: dict, kind: str) -> dict:
    step_bytes = sizes["weight_bytes"] + batch * context_mid * sizes["kv_bytes_per_token"]
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": kind}


def time_prefill(eng, vocab: int, n_tokens: int, sizes: dict, pk: dict, reps: int = 7) -> dict:
    """One request, one step of `n_tokens` (prompts beyond 8,192 tokens in portions of 8,192,
    as the engine's entry point would cut them), timed over a few repetitions."""
    import torch

    from somi_inference_b200.engine import StepEntry
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, vocab, (n_tokens,), generator=g).tolist()
    portion = 8192
    times = []
    # the same layout every time: from its third run on a step is replayed from the CUDA graph
    # that the engine captured at the second
    for rep in range(reps):
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for lo in range(0, n_tokens, portion):
            last = lo + portion >= n_tokens
            eng.step([StepEntry(("prefill", rep), prompt[lo:lo + portion],
                                [min(portion, n_tokens - lo) - 1] if last else [])])
        e.record()
        torch.cuda.synchronize()
        eng.end(("prefill", rep))
        times.append(s.elapsed_time(e))
    tail = sorted(times[2:])
    ms = tail[len(tail) // 2]
    flops = step_flops(sizes, n_tokens, 1, n_tokens * (n_tokens + 1) // 2)
    return {"value": round(n_tokens / ms * 1e3, 1), "tokens": n_tokens, "ms": round(ms, 3),
            "frac": round(flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}


def time_e2e(eng, vocab: int, batch: int, steps: int, warmup: int, max_concurrent: int) -> dict:
    """The decode step through the Python entry point: host token ids in, sampled ids out."""
    import torch

    from somi_inference_b200.engine import LLM
    from somi_inference_b200.sampling import SamplingParams
    llm = LLM(eng, max_concurrent=max_concurrent, max_num_batched_tokens=8192, chunk_size=2048)
    gq = torch.Generator().manual_seed(4)
    reqs = [llm.make_request(torch.randint(0, vocab, (CONTEXT,), generator=gq).tolist(),
                             max_new_tokens=steps + warmup + 4,
                             sampling_params=SamplingParams(temperature=0.0), ignore_eos=True)
            for _ in range(batch)]
    for r in reqs:
        llm.scheduler.add_request(r)
    while any(r.num_computed < CONTEXT for r in reqs):
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    n0 = sum(len(r.output_tokens) for r in reqs)
    with ClockSampler() as clocks:
        t0 = time.perf_counter()
        for _ in range(steps):
            llm.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
    n1 = sum(len(r.output_tokens) for r in reqs)
    out = {"value": round((n1 - n0) / dt, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(llm.engine.builder.h2d_bytes_last + llm.sampler_h2d_bytes()
                                     + llm.engine.token_patch_bytes),
           "d2h_bytes_per_step": int(llm.d2h_bytes_last),
           "ms_per_step": round(dt / steps * 1e3, 3),
           # this region runs later than the device-timed one, under the power cap often at a lower clock
           "sm_mhz": clocks.summary().get("sm_mhz")}
    for r in reqs:
        if llm.engine.has(r.request_id):
            llm.engine.end(r.request_id)
    llm.scheduler.running.clear()
    return out


def time_mixed(eng, vocab: int, sizes: dict, pk: dict, n_decode: int, reps: int, warm: int) -> dict:
    """`n_decode` requests at 2,048 cached tokens take one token each while one prompt of 2,048
    tokens goes through in portions of 512: four steps of 512 + n_decode tokens per prompt."""
    import torch

    from somi_inference_b200.engine import StepEntry
    g = torch.Generator().manual_seed(5)
    reqs = fill_context(eng, n_decode, vocab, "mixed", CONTEXT)
    portions = PREFILL_TOKENS // MIXED_PORTION
    times: list[float] = []
    flops = moved = 0.0
    ctx_now = CONTEXT
    for rep in range(warm + reps):
        prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        feed = torch.randint(0, vocab, (portions, n_decode), generator=g).tolist()
        for p in range(portions):
            lo = p * MIXED_PORTION
            entries = [StepEntry(("mixed-prompt", rep), prompt[lo:lo + MIXED_PORTION],
                                 [MIXED_PORTION - 1] if p == portions - 1 else [])]
            entries += [StepEntry(r, [feed[p][b]], [0]) for b, r in enumerate(reqs)]
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            eng.step(entries)
            e.record()
            torch.cuda.synchronize()
            if rep >= warm:
                times.append(s.elapsed_time(e))
                pairs = MIXED_PORTION * lo + MIXED_PORTION * (MIXED_PORTION + 1) // 2 + n_decode * (ctx_now + 1)
                flops += step_flops(sizes, MIXED_PORTION + n_decode,
                                    n_decode + (1 if p == portions - 1 else 0), pairs)
                moved += sizes["weight_bytes"] + sizes["kv_bytes_per_token"] * (
                    n_decode * (ctx_now + 1) + lo + MIXED_PORTION)
            ctx_now += 1
        eng.end(("mixed-prompt", rep))
    for r in reqs:
        eng.end(r)
    total_s = sum(times) * 1e-3
    tokens = (MIXED_PORTION + n_decode) * len(times)
    return {"decode_requests": n_decode, "context": CONTEXT, "portion": MIXED_PORTION,
            "prompt_tokens": PREFILL_TOKENS, "tokens_per_step": MIXED_PORTION + n_decode,
            "steps": len(times), "value": round(tokens / total_s, 1), "unit": "tokens/s",
            **latency_stats(times),
            "flops_frac": round(flops / total_s / (pk["bf16_tflops"] * 1e12), 4),
            "hbm_frac": round(moved / total_s / 1e9 / pk["hbm_gbs"], 4)}


def profile_step(eng, run, pk: dict) -> list[dict]:
    """Rows of `--profile`: `run()` makes one step; it is run eagerly (no CUDA graph) under a
    launch trace, after one untimed eager run."""
    import torch

    from somi_inference_b200.ops import trace
    was = eng.use_graphs
    eng.use_graphs = False
    try:
        run()
        torch.cuda.synchronize()
        with trace.LaunchTrace() as t:
            run()
        return trace.summarise(t.rows(), pk["hbm_gbs"], pk["bf16_tflops"])
    finally:
        eng.use_graphs = was


def free_device_memory() -> None:
    import gc

    import torch
    gc.collect()
    torch.cuda.empty_cache()


# ----------------------------------------------------------------------------- the phases
def run_shape(shape: str, layers: int, batch: int, steps: int, warmup: int, pk: dict, kind: str,
              points: bool, long_points: bool, profile: bool) -> dict:
    """Everything that is measured on one model shape: prefill at 2,048 tokens, decode at
    `batch` (device-timed and end to end), decode at batch 1 and 64, and the long points."""
    import torch

    from somi_inference_b200.engine import StepEntry
    from somi_inference_b200.sampling import Sampler, SamplingParams
    batches = sorted({1, batch, 64}) if points else [batch]
    extra = 2 * (steps + warmup) + 8
    most = max(batches) * (CONTEXT + extra) + PREFILL_TOKENS
    positions = MAX_CONTEXT
    if long_points:
        most = max(most, 64 * (8192 + extra), 8 * (32768 + extra))
        positions = LONG_CONTEXT
    cfg, eng = build_engine(shape, layers, most, max(batches) + 1, positions)
    sampler = Sampler(eng.ops, eng.device)
    sizes = model_sizes(cfg, layers)
    V = cfg.vocab_size
    out: dict = {}

    # the headline first, on a GPU that the long products of the other measurements have not
    # yet driven to its power cap
    reqs = fill_context(eng, batch, V, "main", CONTEXT)
    with ClockSampler() as clocks:
        ms, launches, per_step = time_decode(eng, sampler, reqs, V, steps, warmup)
    out.update(ms=ms, launches=launches, clocks=clocks.summary(), latency=latency_stats(per_step),
               roofline=decode_roofline(sizes, batch, CONTEXT + warmup + steps / 2, ms, pk, kind))
    if profile:
        g = torch.Generator().manual_seed(6)
        tok = torch.randint(0, V, (batch,), generator=g).tolist()
        params = [SamplingParams(temperature=0.0)] * batch

        def one():
            logits = eng.step([StepEntry(r, [tok[b]], [0]) for b, r in enumerate(reqs)])
            sampler.sample(logits, params, [0] * batch, [0] * batch)
        out["profile_decode"] = profile_step(eng, one, pk)
    for r in reqs:
        eng.end(r)

    out["e2e"] = time_e2e(eng, V, batch, steps, warmup, max(batches) + 1)
    out["prefill"] = time_prefill(eng, V, PREFILL_TOKENS, sizes, pk)

    pts: dict = {}
    if points:
        for b in (1, 64):
            rq = fill_context(eng, b, V, f"b{b}", CONTEXT)
            n = max(10, steps // 2)
            pms, _, _ = time_decode(eng, sampler, rq, V, n, warmup)
            pts[f"decode_b{b}"] = round(b / pms * 1e3, 1)
            pts[f"decode_b{b}_frac"] = decode_roofline(sizes, b, CONTEXT + warmup + n / 2, pms, pk, kind)["frac"]
            for r in rq:
                eng.end(r)
    if long_points:
        for b, ctx in ((8, 8192), (64, 8192), (8, 32768)):
            rq = fill_context(eng, b, V, f"b{b}c{ctx}", ctx)
            n = max(10, steps // 2)
            pms, _, _ = time_decode(eng, sampler, rq, V, n, warmup)
            pts[f"decode_b{b}_ctx{ctx // 1024}k"] = round(b / pms * 1e3, 1)
            pts[f"decode_b{b}_ctx{ctx // 1024}k_frac"] = decode_roofline(
                sizes, b, ctx + warmup + n / 2, pms, pk, kind)["frac"]
            for r in rq:
                eng.end(r)
        for n_tok in (8192, 32768):
            p = time_prefill(eng, V, n_tok, sizes, pk, reps=5)
            pts[f"prefill_{n_tok // 1024}k"] = p["value"]
            pts[f"prefill_{n_tok // 1024}k_frac"] = p["frac"]
    out["points"] = pts
    eng._graphs.clear()
    del eng, sampler
    free_device_memory()
    return out


def run_only(args, pk: dict, kind: str) -> int:
    """One phase on one shape, for profiling runs and sweeps; prints its own small line."""
    import torch

    from somi_inference_b200.engine import StepEntry
    from somi_inference_b200.sampling import Sampler, SamplingParams
    shape = args.shape
    layers = args.layers or FULL_LAYERS[shape]
    extra = 2 * (args.steps + args.warmup) + 8
    if args.only == "decode":
        cfg, eng = build_engine(shape, layers, args.batch * (args.context + extra), args.batch + 1,
                                max(MAX_CONTEXT, args.context + extra))
        sizes = model_sizes(cfg, layers)
        sampler = Sampler(eng.ops, eng.device)
        reqs = fill_context(eng, args.batch, cfg.vocab_size, "main", args.context)
        ms, launches, per_step = time_decode(eng, sampler, reqs, cfg.vocab_size, args.steps, args.warmup)
        line = {"only": "decode", "shape": shape, "layers": layers, "batch": args.batch,
                "context": args.context, "ms_per_step": round(ms, 4),
                "tokens_per_s": round(args.batch / ms * 1e3, 1), "gpu_launches": int(launches),
                "latency": latency_stats(per_step),
                "roofline": decode_roofline(sizes, args.batch, args.context + args.warmup + args.steps / 2,
                                            ms, pk, kind)}
        if args.profile:
            tok = [1] * args.batch
            params = [SamplingParams(temperature=0.0)] * args.batch

            def one():
                logits = eng.step([StepEntry(r, [tok[b]], [0]) for b, r in enumerate(reqs)])
                sampler.sample(logits, params, [0] * args.batch, [0] * args.batch)
            line["profile"] = profile_step(eng, one, pk)
    elif args.only == "prefill":
        n = args.prefill_tokens
        cfg, eng = build_engine(shape, layers, n + 64, 2, max(MAX_CONTEXT, n))
        sizes = model_sizes(cfg, layers)
        line = {"only": "prefill", "shape": shape, "layers": layers,
                **time_prefill(eng, cfg.vocab_size, n, sizes, pk)}
        if args.profile:
            g = torch.Generator().manual_seed(6)
            prompt = torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
            count = [0]

            def one():
                count[0] += 1
                rid = ("profile", count[0])
                for lo in range(0, n, 8192):
                    eng.step([StepEntry(rid, prompt[lo:lo + 8192], [])])
                eng.end(rid)
            line["profile"] = profile_step(eng, one, pk)
    else:
        cfg, eng = build_engine(shape, layers, args.batch * (CONTEXT + 64) + PREFILL_TOKENS,
                                args.batch + 2, MAX_CONTEXT)
        sizes = model_sizes(cfg, layers)
        line = {"only": "mixed", "shape": shape, "layers": layers,
                **time_mixed(eng, cfg.vocab_size, sizes, pk, args.batch, reps=3, warm=2)}
        if args.profile:
            reqs = fill_context(eng, args.batch, cfg.vocab_size, "p", CONTEXT)
            count = [0]

            def one():
                count[0] += 1
                entries = [StepEntry(("pp", count[0]), [1] * MIXED_PORTION, [])]
                entries += [StepEntry(r, [1], [0]) for r in reqs]
                eng.step(entries)
                eng.end(("pp", count[0]))
            line["profile"] = profile_step(eng, one, pk)
    print(json.dumps(line))
    if args.output_file:
        with open(args.output_file, "a") as f:
            f.write(json.dumps({**line, "environment": environment()}) + "\n")
    return 0


# ------------------------------------------------------------------------ the reference arm
def reference_arm(args) -> int:
    """The same decode step on the unmodified reference (a plain copy of its package under
    baseline/_ref): its `QwenModel` with random bfloat16 weights of the same shape behind its own
    `QwenAdapter`, `KVCacheManager`, `ModelRunner`, `Sampler` and `ContinuousBatchingEngine`.
    Nothing of this repository's engine is imported here."""
    shape, batch = args.shape, args.batch
    layers = args.layers or FULL_LAYERS[shape]
    base = {"impl": "reference"}
    if not os.path.isfile(os.path.join(REFERENCE_DIR, "somi_inference", "__init__.py")):
        print(json.dumps({**base, "unavailable": "baseline/_ref holds no copy of the reference's "
                          "somi_inference package (pip cannot build it offline: its build backend "
                          "uv_build is not in the wheelhouse; a plain copy of the package is used "
                          "instead and was not found)"}))
        return 0
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({**base, "unavailable": "no CUDA device"}))
        return 0
    # Triton's cache of the reference's kernels: where a copy from an earlier run of this arm lies
    # beside the reference (baseline/_triton_cache, not under version control), a temporary folder
    # is seeded with it, which saves the minutes its unrolled decode kernel takes to compile.  It
    # holds nothing but what Triton made of the reference's own sources on this image.
    if "TRITON_CACHE_DIR" not in os.environ:
        import shutil
        import tempfile
        seed = os.path.join(os.path.dirname(REFERENCE_DIR), "_triton_cache")
        cache = os.path.join(tempfile.gettempdir(), f"somi_reference_triton_cache_{os.getuid()}")
        if os.path.isdir(seed) and not os.path.isdir(cache):
            shutil.copytree(seed, cache)
            # an entry's group file names its files by absolute path: point them to the copy
            for entry in os.listdir(cache):
                for f in os.listdir(os.path.join(cache, entry)):
                    if f.startswith("__grp__") and f.endswith(".json"):
                        path = os.path.join(cache, entry, f)
                        with open(path) as fh:
                            grp = json.load(fh)
                        grp["child_paths"] = {k: os.path.join(cache, entry, os.path.basename(v))
                                              for k, v in grp.get("child_paths", {}).items()}
                        with open(path, "w") as fh:
                            json.dump(grp, fh)
        os.makedirs(cache, exist_ok=True)
        os.environ["TRITON_CACHE_DIR"] = cache
    sys.path.insert(0, REFERENCE_DIR)
    from somi_inference.core.continuous_batching import (ContinuousBatchingEngine, Scheduler,
                                                         Sequence, SequenceStatus)
    from somi_inference.core.model_runner import ModelRunner
    from somi_inference.core.paged_attention import KVCacheManager
    from somi_inference.core.sampler import Sampler, SamplingParams
    from somi_inference.models.qwen2 import QwenModel
    from somi_inference.models.qwen2_adapter import QwenAdapter

    s = SHAPES[shape]
    dev = torch.device("cuda:0")
    steps, warmup = args.steps, max(args.warmup, 3)
    positions = MAX_CONTEXT if args.no_points else LONG_CONTEXT
    torch.manual_seed(0)
    with torch.device(dev):
        model = QwenModel(vocab_size=s["vocab_size"], hidden_size=s["hidden_size"],
                          intermediate_size=s["intermediate_size"], num_hidden_layers=layers,
                          num_attention_heads=s["num_attention_heads"],
                          num_key_value_heads=s["num_key_value_heads"], head_dim=s["head_dim"],
                          max_seq_size=positions, rms_norm_eps=s["rms_norm_eps"],
                          rope_theta=s["rope_theta"])
    gen = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("layernorm.weight"):
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02, generator=gen)
    # as the reference's LLM does after loading (somi_inference/entrypoints/llm.py:89-93)
    model.to(device=dev, dtype=torch.bfloat16)
    model.eval()
    model.requires_grad_(requires_grad=False)
    V = s["vocab_size"]
    greedy = SamplingParams(temperature=0.0)

    def make(batch_n: int, backends: dict):
        adapter = QwenAdapter(model, **backends)
        blocks = batch_n * (-(-(CONTEXT + steps + warmup + 8) // PAGE)) + PREFILL_TOKENS // PAGE + 4
        kv = KVCacheManager(num_blocks=blocks, block_size=PAGE, num_kv_heads=s["num_key_value_heads"],
                            head_dim=s["head_dim"], n_layers=layers, device=dev, dtype=torch.bfloat16)
        runner = ModelRunner(adapter, Sampler(), kv)
        sched = Scheduler(max_concurrent=batch_n + 1, block_size=PAGE, total_blocks=blocks)
        return adapter, kv, runner, ContinuousBatchingEngine(runner, sched, eos_token_id=-1)

    def decode_run(batch_n: int, backends: dict, n_steps: int, n_warm: int):
        """Prefill `batch_n` prompts of 2,048 tokens through the reference's engine, then time
        `n_steps` of its decode steps: on the device around `ModelRunner.decode`, and end to end
        around `ContinuousBatchingEngine._decode_batch` (host ids in, sampled ids out)."""
        adapter, kv, runner, engine = make(batch_n, backends)
        g = torch.Generator().manual_seed(1)
        seqs = [Sequence(seq_id=i, status=SequenceStatus.RUNNING,
                         prompt_tokens=torch.randint(0, V, (CONTEXT,), generator=g).tolist(),
                         output_tokens=[], max_new_tokens=10 ** 6, sampling_params=greedy)
                for i in range(batch_n)]
        with torch.inference_mode():
            for sq in seqs:
                engine._prefill(sq)
            for _ in range(n_warm):
                engine._decode_batch(seqs)
            torch.cuda.synchronize()
            ids = torch.tensor([sq.output_tokens[-1] for sq in seqs], device=dev).unsqueeze(1)
            seq_ids = [sq.seq_id for sq in seqs]
            hist = [[] for _ in seqs]
            s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_ev.record()
            for _ in range(n_steps):
                out = runner.decode(ids, seq_ids, [greedy] * batch_n, hist)
                ids = out.unsqueeze(1)
            e_ev.record()
            torch.cuda.synchronize()
            dev_ms = s_ev.elapsed_time(e_ev) / n_steps
            for sq, t in zip(seqs, ids[:, 0].tolist()):
                sq.output_tokens.append(int(t))
            t0 = time.perf_counter()
            for _ in range(n_steps):
                engine._decode_batch(seqs)
            torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t0) / n_steps * 1e3
        del kv, runner, engine
        torch.cuda.empty_cache()
        return dev_ms, e2e_ms

    def prefill_run(backends: dict):
        adapter, kv, runner, engine = make(1, backends)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, V, (1, PREFILL_TOKENS), generator=g).to(dev)
        times = []
        with torch.inference_mode():
            for rep in range(5):
                kv.register_sequence(rep)
                torch.cuda.synchronize()
                s_ev, e_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s_ev.record()
                adapter.prefill(prompt, kv, rep)
                e_ev.record()
                torch.cuda.synchronize()
                kv.free_sequence(rep)
                times.append(s_ev.elapsed_time(e_ev))
        del kv, runner, engine
        torch.cuda.empty_cache()
        tail = sorted(times[2:])
        return tail[len(tail) // 2]

    arms = {"torch_ref": dict(prefill_attention_backend="torch_ref", decode_attention_backend="torch_ref",
                              mlp_backend="torch_ref"),
            # its Triton attention kernels take bfloat16; its Triton MLP takes float16 only
            # (somi_inference/core/mlp_triton.py:24), so the MLP stays on the library product
            "triton_attention": dict(prefill_attention_backend="triton",
                                     decode_attention_backend="triton", mlp_backend="torch_ref")}
    # The reference's Triton decode kernel is unrolled over the block table's width
    # (`MAX_BLOCKS_PER_SEQ` is a compile-time constant, somi_inference/core/
    # paged_attention_triton.py:53,93,228): at 2,048 cached tokens it is compiled anew each time
    # the longest request enters another block of 16, which takes minutes where Triton's cache
    # does not hold that width yet.  Its steps are therefore timed inside one block (one warm-up
    # step, then at most 7 on the device and 7 end to end: tokens 2,049 to 2,063), whatever the
    # cache holds; the compilation itself is outside the timed steps.
    within_one_block = (PAGE - 2) // 2
    results: dict = {}
    for name, backends in arms.items():
        jit = name != "torch_ref"
        k_steps, k_warm = (min(steps, within_one_block), 1) if jit else (steps, warmup)
        try:
            t0 = time.perf_counter()
            print(f"[bench] reference arm: backend {name} ...", file=sys.stderr, flush=True)
            with ClockSampler() as clocks:
                dev_ms, e2e_ms = decode_run(batch, backends, k_steps, k_warm)
            pre_ms = prefill_run(backends)
            results[name] = {"ms_per_step": round(dev_ms, 3), "value": round(batch / dev_ms * 1e3, 1),
                             "e2e_ms_per_step": round(e2e_ms, 3),
                             "e2e_value": round(batch / e2e_ms * 1e3, 1),
                             "prefill_ms": round(pre_ms, 3),
                             "prefill_value": round(PREFILL_TOKENS / pre_ms * 1e3, 1),
                             "steps": k_steps, "warmup": k_warm,
                             "wall_s": round(time.perf_counter() - t0, 1),
                             "clocks": clocks.summary()}
            if jit:
                results[name]["note"] = ("timed inside one block of 16 positions: its decode kernel "
                                         "is compiled anew for every block-table width")
        except Exception as exc:        # a backend its own predicates refuse, or that fails to compile
            results[name] = {"failed": f"{type(exc).__name__}: {str(exc)[:200]}"}
            torch.cuda.empty_cache()
    ok = {k: v for k, v in results.items() if "value" in v}
    if not ok:
        print(json.dumps({**base, "unavailable": "the reference's decode step failed in every "
                          f"backend: {results}"}))
        return 0
    best = max(ok, key=lambda k: ok[k]["value"])
    b = ok[best]
    points = {}
    if not args.no_points:
        for pb in (1, 64):
            try:
                pms, _ = decode_run(pb, arms[best], *((min(5, within_one_block), 1) if best != "torch_ref"
                                                      else (max(5, steps // 4), 3)))
                points[f"decode_b{pb}"] = round(pb / pms * 1e3, 1)
            except Exception as exc:
                points[f"decode_b{pb}"] = None
                points[f"decode_b{pb}_failed"] = f"{type(exc).__name__}: {str(exc)[:120]}"
                torch.cuda.empty_cache()
    tokens_in = batch * 8     # int64 ids of one step: torch.tensor([...]) of the last tokens
    line = {"impl": "reference", "metric": "decode tokens/s", "value": b["value"], "unit": "tokens/s",
            "n_gpus": 1, "steps": b["steps"], "warmup": b["warmup"], "ms_per_step": b["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
            "config": config_record(shape, layers, batch, positions), "clocks": b["clocks"],
            "e2e": {"value": b["e2e_value"], "unit": "tokens/s", "h2d_bytes_per_step": tokens_in,
                    "d2h_bytes_per_step": tokens_in, "ms_per_step": b["e2e_ms_per_step"]},
            "prefill": {"value": b["prefill_value"], "tokens": PREFILL_TOKENS, "ms": b["prefill_ms"]},
            "points": points, "backend": best, "backends": results,
            "path": "QwenModel + QwenAdapter + KVCacheManager + ModelRunner + Sampler + "
                    "ContinuousBatchingEngine._decode_batch, unmodified, from baseline/_ref"}
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--shape", choices=list(SHAPES), default="7b")
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-points", action="store_true",
                    help="skip decode at batch 1 and 64 and the longer contexts")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the 0.5B-shaped figures and the 14B-shaped mixed step")
    ap.add_argument("--only", choices=["decode", "prefill", "mixed"], default=None,
                    help="run only this phase and print its figures (for profiling runs)")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="cached tokens per request (with --only decode)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (with --only prefill)")
    ap.add_argument("--profile", action="store_true",
                    help="add one row per kernel of an eager step: time, bytes, flops, fraction of peak")
    ap.add_argument("--output-file", type=str, default=None,
                    help="append the line, with an environment block, to this JSONL file")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)
    if args.only is None and (args.context != CONTEXT or args.prefill_tokens != PREFILL_TOKENS):
        print("bench.py: --context and --prefill-tokens go with --only decode / --only prefill")
        return 2
    pk, kind = peaks()
    if args.only is not None:
        return run_only(args, pk, kind)

    layers = args.layers or FULL_LAYERS[args.shape]
    main_run = run_shape(args.shape, layers, args.batch, args.steps, args.warmup, pk, kind,
                         points=not args.no_points, long_points=not args.no_points,
                         profile=args.profile)
    line = {
        "metric": "decode tokens/s", "value": round(args.batch / main_run["ms"] * 1e3, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random N(0,0.02) weights, uniform random token ids",
        "config": config_record(args.shape, layers, args.batch,
                                MAX_CONTEXT if args.no_points else LONG_CONTEXT),
        "clocks": main_run["clocks"], "e2e": main_run["e2e"],
        "gpu_launches": int(main_run["launches"]), "prefill": main_run["prefill"],
        "roofline": main_run["roofline"], "latency": main_run["latency"],
        "points": main_run["points"],
    }
    if args.profile:
        line["profile_decode"] = main_run["profile_decode"]
    if not args.no_extras:
        # the 0.5B-shaped model (the benchmark description's small shape): the same measurements
        small = run_shape("0.5b", FULL_LAYERS["0.5b"], args.batch, args.steps, args.warmup, pk, kind,
                          points=not args.no_points, long_points=False, profile=False)
        line["shape_0_5b"] = {
            "model": "Qwen2.5-0.5B-shaped", "layers": FULL_LAYERS["0.5b"],
            "value": round(args.batch / small["ms"] * 1e3, 1), "ms_per_step": round(small["ms"], 4),
            "e2e": small["e2e"]["value"], "prefill": small["prefill"], "roofline": small["roofline"],
            "latency": small["latency"], "points": small["points"], "gpu_launches": int(small["launches"])}
        # the 14B-shaped mixed step
        l14 = FULL_LAYERS["14b"]
        cfg14, eng14 = build_engine("14b", l14, 64 * (CONTEXT + 64) + PREFILL_TOKENS, 66, MAX_CONTEXT)
        line["mixed_14b"] = {"model": "Qwen2.5-14B-shaped", "layers": l14,
                             **time_mixed(eng14, cfg14.vocab_size, model_sizes(cfg14, l14), pk, 64,
                                          reps=3, warm=2)}
        eng14._graphs.clear()
        del eng14
        free_device_memory()
    line["environment"] = environment()
    print(json.dumps(line))
    if args.output_file:
        with open(args.output_file, "a") as f:
            f.write(json.dumps(line) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
