"""The engine at the layer sizes of the large models (0.5B, 7B and 14B shapes, two layers).

The tiny configurations cannot reach the kernels' large-size variants (rings that are not deep,
more output tiles than SMs, the vocabulary-sized head, token widths of 32 and 64 with long K).
Random weights whose values are bfloat16 in every engine.

* Against the plain implementation on the CPU (tests/plain/qwen2_plain.py), in float32 and in
  bfloat16: a few requests of up to 290 tokens, each whole and then mixed (portions beside
  single tokens, pages handed on), and one step of a 512-token portion beside 64 single tokens.
* bfloat16 against the engine's float32 path where the plain implementation would take minutes:
  batches on both sides of the kernels' token widths (16, 32, 64), a decode step with thousands
  of 128-key chunks, and the 512 + 64 step at contexts of 2,048 tokens.
Bounds.  float32: rounding grows with the length of the sums (widths of 896 to 5,120, inner sizes
up to 18,944), so the yardstick is measured, not assumed: the plain implementation is run in
float64 and in float32, and the engine's largest difference from the float64 logits may be at
most four times that of the plain float32 logits (measured: 2.1 to 3.4 times, the library's
float32 product on the GPU adding up a row of up to 18,944 terms in longer runs than the CPU's
does; in absolute terms 3e-6 to 1.2e-5 of the largest logit, against 1e-5 for the tiny models).  bfloat16: root mean square 4e-3 and largest difference
4e-2 of the largest logit, as in the replay tests.  Weights are N(0, 0.03) for the 0.5B and 7B
shapes and N(0, 0.02), the benchmark description's spread, for the 14B shape: at width 5,120 a
spread of 0.03 makes the pre-activations (variance width * spread^2 = 4.6) large enough for
softmax and SiLU to amplify bfloat16 rounding to the bound itself (measured 3.2e-3 to 4.5e-3).
"""

import pytest
import torch

from tests import replay
from tests.plain import qwen2_plain as plain

pytestmark = pytest.mark.gpu

SHAPES = {
    "7b": dict(hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, intermediate_size=18944,
               vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False),
    "0.5b": dict(hidden_size=896, num_attention_heads=14, num_key_value_heads=2, intermediate_size=4864,
                 vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=True),
    "14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, intermediate_size=13824,
                vocab_size=152064, rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False),
}
SPREAD = {"7b": 0.03, "0.5b": 0.03, "14b": 0.02}


@pytest.fixture(scope="module", params=list(SHAPES))
def weights(request):
    from somi_inference_b200.config import Qwen2Config
    from somi_inference_b200.parts import declared_tensors
    raw = dict(SHAPES[request.param], num_hidden_layers=2, max_position_embeddings=4608,
               architectures=["Qwen2ForCausalLM"], hidden_act="silu", use_sliding_window=False)
    cfg = Qwen2Config.from_dict(raw)
    gen = torch.Generator(device="cuda").manual_seed(0)
    tensors = {}
    for name, d in declared_tensors(cfg.to_model_spec()).items():
        if d.ignored:
            continue
        if d.init == "ones":
            tensors[name] = torch.ones(d.shape, dtype=torch.bfloat16, device="cuda")
        else:
            t = torch.empty(d.shape, dtype=torch.float32, device="cuda").normal_(
                0.0, SPREAD[request.param], generator=gen)
            tensors[name] = t.to(torch.bfloat16)
    _RAW[request.param] = raw
    yield request.param, cfg, tensors
    tensors.clear()
    _PLAIN.clear()
    torch.cuda.empty_cache()


_PLAIN: dict = {}
_RAW: dict = {}     # shape name -> the config as the plain implementation reads it


def plain_rows(name, cfg, tensors, requests: dict, rows: set) -> tuple[dict, dict]:
    """Plain logits, computed on the CPU, at the (request, position) pairs in `rows`: whole-sequence
    hidden states of every request, the head only where a row is wanted.  Returns the float64
    logits and the float32 logits."""
    if name not in _PLAIN:
        _PLAIN.clear()
        w64 = {k: v.double().cpu() for k, v in tensors.items()}
        _PLAIN[name] = (w64, {k: v.float() for k, v in w64.items()})
    out64, out32 = {}, {}
    for w, out, dt in ((_PLAIN[name][0], out64, torch.float64), (_PLAIN[name][1], out32, torch.float32)):
        for rid, toks in requests.items():
            pos = sorted(p for r, p in rows if r == rid)
            if not pos:
                continue
            h = plain.hidden_states(_RAW[name], w, torch.tensor(toks, dtype=torch.long))
            assert h.dtype == dt
            lg = plain.lm_head(_RAW[name], w, h[pos])
            for i, p in enumerate(pos):
                out[(rid, p)] = lg[i]
    return out64, out32


def check_against_plain(got: dict, ref: tuple[dict, dict], dtype: str, what: str) -> None:
    ref64, ref32 = ref
    scale = max(float(v.abs().max()) for v in ref64.values())
    worst, sq, n, noise = 0.0, 0.0, 0, 0.0
    for key, row in got.items():
        diff = row.double() - ref64[key]
        worst = max(worst, float(diff.abs().max()))
        sq += float(diff.pow(2).sum())
        n += diff.numel()
        noise = max(noise, float((ref32[key].double() - ref64[key]).abs().max()))
    rms = (sq / n) ** 0.5
    print(f"{what}: worst {worst / scale:.2e}, rms {rms / scale:.2e} of the largest logit ({scale:.2f}); "
          f"plain float32 against float64: {noise / scale:.2e}")
    if dtype == "float32":
        assert worst <= 4 * noise, (f"{what}: worst {worst:.3e}, four times the plain float32 "
                                    f"implementation's own {noise:.3e} is allowed")
    else:
        assert rms <= 4e-3 * scale, f"{what}: rms {rms / scale:.2e} of the largest logit"
        assert worst <= 4e-2 * scale, f"{what}: worst {worst / scale:.2e} of the largest logit"


def few_wanted(steps: list[dict], keep_last: int = 1) -> list[dict]:
    """The same trace with fewer logits asked for (the head's plain product is what costs)."""
    for rec in steps:
        for e in rec["entries"]:
            e["want"] = sorted(e["want"])[-keep_last:]
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_against_plain_whole_and_mixed(weights, dtype):
    """Each request alone and whole, then all of them mixed with so few pages that they are handed
    on, against the plain implementation's logits."""
    from somi_inference_b200.engine import Engine
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(11)
    requests = {f"r{i}": torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()
                for i, n in enumerate([37, 150, 290, 75, 129])}
    tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
    for mode in (replay.whole, replay.mixed):
        steps, max_tokens = mode(requests)
        steps = few_wanted(steps, keep_last=4 if mode is replay.whole else 1)
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=max_tokens,
                                  max_requests=8)
        got = replay.run_steps(eng, steps)
        eng.ops.check_errors()
        assert all(f == eng.num_pages for f in eng.cache.free_pages())
        del eng
        ref = plain_rows(name, cfg, tensors, requests, set(got))
        check_against_plain(got, ref, dtype, f"{name}/{dtype}/{mode.__name__}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portion_of_512_beside_64_single_tokens_against_plain(weights, dtype):
    """One step with a 512-token portion of a prompt (88 tokens already cached) beside 64 requests
    that bring one token each: library products at 576 rows, prompt attention and decode attention
    in one step.  Run three times with different tokens (the third is replayed from a CUDA graph)."""
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(12)
    tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
    eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=3 * 640 + 64 * 128,
                              max_requests=70)
    ctxs = [20 + (7 * i) % 41 for i in range(64)]
    singles = {f"d{i}": torch.randint(0, cfg.vocab_size, (c + 3,), generator=g).tolist()
               for i, c in enumerate(ctxs)}
    for rid, toks in singles.items():
        eng.step([StepEntry(rid, toks[:-3], [])])
    got, requests = {}, dict(singles)
    for rep in range(3):
        prompt = torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist()
        requests[f"p{rep}"] = prompt
        eng.step([StepEntry(f"p{rep}", prompt[:88], [])])
        entries = [StepEntry(f"p{rep}", prompt[88:], [511])]
        entries += [StepEntry(rid, [toks[len(toks) - 3 + rep]], [0]) for rid, toks in singles.items()]
        logits = eng.step(entries).float().cpu()
        got[(f"p{rep}", 599)] = logits[0]
        if rep != 1:                              # the plain head costs: two of the three steps
            for k, (rid, toks) in enumerate(singles.items()):
                got[(rid, len(toks) - 3 + rep)] = logits[1 + k]
        eng.end(f"p{rep}")
    eng.ops.check_errors()
    assert len(eng._graphs) > 0 and eng._graphs.hits >= 1
    del eng
    ref = plain_rows(name, cfg, tensors, requests, set(got))
    check_against_plain(got, ref, dtype, f"{name}/{dtype}/512+64")


def test_long_prompt_in_two_portions_against_plain(weights):
    """A prompt of 700 tokens in portions of 400 and 300 through the prompt-attention kernel with
    two query tiles per CTA (made to take the step whatever its size), bfloat16, against the plain
    implementation at rows on both sides of the 128- and 256-row tile edges."""
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(14)
    prompt = torch.randint(0, cfg.vocab_size, (700,), generator=g).tolist()
    eng = Engine.from_tensors(cfg, tensors, dtype="bfloat16", page_size=16, max_tokens=768, max_requests=2)
    was = eng.ops.pp_prefill_min_ctas
    eng.ops.pp_prefill_min_ctas = 0
    try:
        want_a = [0, 127, 128, 255, 256, 399]
        want_b = [0, 111, 112, 113, 299]           # positions 400, 511, 512, 513, 699
        la = eng.step([StepEntry("p", prompt[:400], want_a)]).float().cpu()
        lb = eng.step([StepEntry("p", prompt[400:], want_b)]).float().cpu()
        eng.ops.check_errors()
    finally:
        eng.ops.pp_prefill_min_ctas = was
    got = {("p", w): la[i] for i, w in enumerate(want_a)}
    got.update({("p", 400 + w): lb[i] for i, w in enumerate(want_b)})
    del eng
    ref = plain_rows(name, cfg, tensors, {"p": prompt}, set(got))
    check_against_plain(got, ref, "bfloat16", f"{name}/bfloat16/700 tokens in two portions")


def test_portion_of_512_beside_64_single_tokens_at_2048_context(weights):
    """The same step at the benchmark's sizes: 64 requests with 2,048 cached tokens and a prompt
    with 1,024 cached tokens; bfloat16 against the engine's float32 path."""
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(13)
    lens = [2048 + 3 * (i % 5) for i in range(64)]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    long = torch.randint(0, cfg.vocab_size, (1536,), generator=g).tolist()
    feed = torch.randint(0, cfg.vocab_size, (2, 64), generator=g).tolist()
    outs = []
    for dtype in ("bfloat16", "float32"):
        tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16,
                                  max_tokens=sum(lens) + 64 * 32 + 2048, max_requests=66)
        for i, p in enumerate(prompts):
            eng.step([StepEntry(i, p, [])])
        res = []
        for s in range(2):
            eng.step([StepEntry("long", long[:1024], [])])
            entries = [StepEntry("long", long[1024:], [511])]
            entries += [StepEntry(i, [feed[s][i]], [0]) for i in range(64)]
            res.append(eng.step(entries).float())
            eng.end("long")
        eng.ops.check_errors()
        outs.append(torch.cat(res))
        del eng, tt
    got, ref = outs
    scale = ref.abs().max().item()
    rms = ((got - ref) ** 2).mean().sqrt().item()
    assert rms <= 4e-3 * scale, f"{name}: rms {rms / scale:.2e} of the largest logit"
    assert (got - ref).abs().max().item() <= 4e-2 * scale


@pytest.mark.parametrize("batch", [5, 17, 32, 33, 64])
def test_bfloat16_against_float32_at_large_layer_sizes(weights, batch):
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    g = torch.Generator().manual_seed(batch)
    lens = [int(x) for x in torch.randint(20, 300, (batch,), generator=g)]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    feed = torch.randint(0, cfg.vocab_size, (3, batch), generator=g).tolist()
    outs = []
    for dtype in ("bfloat16", "float32"):
        tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=batch * 320 + 64,
                                  max_requests=batch + 1)
        res = [eng.step([StepEntry(i, p, [len(p) - 1]) for i, p in enumerate(prompts)])]
        for s in range(3):
            res.append(eng.step([StepEntry(i, [feed[s][i]], [0]) for i in range(batch)]))
        eng.ops.check_errors()
        outs.append(torch.cat([r.float() for r in res]))
        del eng, tt
    got, ref = outs
    scale = ref.abs().max().item()
    rms = ((got - ref) ** 2).mean().sqrt().item()
    assert rms <= 4e-3 * scale, f"{name} batch {batch}: rms {rms / scale:.2e} of the largest logit"
    assert (got - ref).abs().max().item() <= 4e-2 * scale


def test_bfloat16_against_float32_with_thousands_of_chunks(weights):
    """A decode step with more than 16 chunks of 128 keys per SM takes the attention kernel whose
    CTAs walk through several chunks, and a merge over fewer, larger partial results: many
    requests with contexts of a few thousand tokens, of different lengths."""
    from somi_inference_b200.engine import Engine, StepEntry
    name, cfg, tensors = weights
    batch, ctx = {"7b": (40, 2100), "0.5b": (48, 4200), "14b": (20, 2100)}[name]
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    assert -(-ctx // 128) * cfg.num_key_value_heads * batch >= 16 * sms, "the step is meant to be large"
    g = torch.Generator().manual_seed(7)
    lens = [ctx - 37 * (i % 7) for i in range(batch)]
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    feed = torch.randint(0, cfg.vocab_size, (4, batch), generator=g).tolist()
    outs = []
    for dtype in ("bfloat16", "float32"):
        tt = tensors if dtype == "bfloat16" else {k: v.float() for k, v in tensors.items()}
        eng = Engine.from_tensors(cfg, tt, dtype=dtype, page_size=16, max_tokens=sum(lens) + 64 * batch,
                                  max_requests=batch)
        for i, p in enumerate(prompts):
            eng.step([StepEntry(i, p, [])])
        res = [eng.step([StepEntry(i, [feed[s][i]], [0]) for i in range(batch)]) for s in range(4)]
        eng.ops.check_errors()
        outs.append(torch.cat([r.float() for r in res]))
        del eng, tt
    got, ref = outs
    scale = ref.abs().max().item()
    rms = ((got - ref) ** 2).mean().sqrt().item()
    assert rms <= 4e-3 * scale, f"{name}: rms {rms / scale:.2e} of the largest logit"
    assert (got - ref).abs().max().item() <= 4e-2 * scale
