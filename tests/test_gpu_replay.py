"""The engine against the plain implementation under every way of cutting the work.

Same requests: whole; most in one step and the last 32 tokens one by one; in portions of
changing size down to two tokens; and mixed, up to four live requests with so few pages that
they are used again.  In float32 and bfloat16, for three tiny configurations, in-process and
through the bin/trace_run program.
"""

import os

import pytest
import torch

from tests import replay
from tests.plain import qwen2_plain as plain
from tests.tiny import PAGE_SIZES, TINY, make_model, random_tokens

pytestmark = pytest.mark.gpu

# Weights are drawn with a larger spread than 0.02 so that attention scores differ by several
# units and a wrong key or a wrong mask moves the logits by far more than the tolerance.
STD = 0.08
LENGTHS = [5, 97, 40, 70, 33, 100, 64, 81]
# D: several 128-key tiles and 128-row query tiles, and lengths on both sides of their edges
LENGTHS_BY_MODEL = {"D": [300, 150, 260, 33, 129, 200]}
# float32: logits are of size 3-5; differences between orders of summation stay below 3e-5.
# bfloat16: every activation that passes between kernels is rounded to 8 bits of mantissa
# (2^-9 relative each).  Measured on whole prompts (no cache or batching involved) and under
# every cut and every kernel variant (TMA or cp.async attention, tcgen05 or library products):
# the root mean square of the logit differences is 1.0e-3 to 2.4e-3 of the largest logit and
# hardly moves, while the largest single difference among a million logits moves between
# 0.5e-2 and 2.0e-2 with the order of summation.  Bounds: RMS 4e-3 and largest 4e-2 of the
# largest logit, the same for every way of cutting; a fault of the cache or the batch moves a
# position's logits by the logits' own size, twenty-five times the bound.
ATOL = {"float32": lambda scale: 3e-5, "bfloat16": lambda scale: 4e-2 * scale}
RMS = {"float32": lambda scale: 1e-5, "bfloat16": lambda scale: 4e-3 * scale}
MODES = {"whole": replay.whole, "last32": replay.last_one_by_one, "portions": replay.portions,
         "mixed": replay.mixed}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = str(tmp_path_factory.mktemp("models"))
    out = {}
    for name in TINY:
        for dt in (torch.float32, torch.bfloat16):
            d = make_model(name, root, dt, std=STD)
            cfg, w = plain.load_folder(d)       # float32 arithmetic on the stored values
            reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 10 + i)
                    for i, n in enumerate(LENGTHS_BY_MODEL.get(name, LENGTHS))}
            ref = {k: plain.logits(cfg, w, v) for k, v in reqs.items()}
            scale = max(v.abs().max().item() for v in ref.values())
            out[(name, dt)] = (d, cfg, reqs, ref, scale)
    return out


@pytest.mark.parametrize("mode", list(MODES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_in_process(models, name, dtype, mode):
    from somi_inference_b200.engine import Engine
    d, cfg, reqs, ref, scale = models[(name, getattr(torch, dtype))]
    steps, max_tokens = MODES[mode](reqs)
    eng = Engine(d, dtype=dtype, page_size=PAGE_SIZES[name], max_tokens=max_tokens)
    got = replay.run_steps(eng, steps)
    assert len(got) >= sum(1 for _ in reqs)
    replay.compare(got, ref, ATOL[dtype](scale), f"{name}/{dtype}/{mode}", RMS[dtype](scale))
    assert all(f == eng.num_pages for f in eng.cache.free_pages()), "pages were lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_replay_program(models, tmp_path, name, dtype):
    d, cfg, reqs, ref, scale = models[(name, getattr(torch, dtype))]
    for mode in ("mixed", "last32"):
        sub = {k: reqs[k] for k in list(reqs)[:5]} if mode == "last32" else reqs
        steps, max_tokens = MODES[mode](sub)
        out_dir = str(tmp_path / mode)
        got = replay.run_trace_program(d, dtype, steps, max_tokens, out_dir, cfg["vocab_size"])
        replay.compare(got, ref, ATOL[dtype](scale), f"trace_run {name}/{dtype}/{mode}", RMS[dtype](scale))


def test_cut_independence_float32(models):
    """The same position computed whole and token by token differs by rounding only."""
    from somi_inference_b200.engine import Engine
    d, cfg, reqs, ref, scale = models[("C", torch.float32)]
    sub = {"r1": reqs["r1"]}
    outs = []
    for mode in ("whole", "last32", "portions"):
        steps, mt = MODES[mode](sub)
        eng = Engine(d, dtype="float32", page_size=16, max_tokens=mt)
        outs.append(replay.run_steps(eng, steps))
    for key in outs[0]:
        for o in outs[1:]:
            assert (outs[0][key] - o[key]).abs().max().item() < 1e-5


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_replay_with_the_two_tile_prompt_attention(models, name, mode):
    """The prompt-attention kernel with two query tiles per CTA is chosen by itself only for steps
    with at least a CTA per SM, which no tiny model reaches: here it is made to take every prompt
    portion (head sizes 64 and 128; whole prompts of several tiles, portions down to two tokens,
    portions beside single tokens with pages handed on)."""
    from somi_inference_b200.engine import Engine
    d, cfg, reqs, ref, scale = models[(name, torch.bfloat16)]
    steps, max_tokens = MODES[mode](reqs)
    eng = Engine(d, dtype="bfloat16", page_size=PAGE_SIZES[name], max_tokens=max_tokens)
    was = eng.ops.pp_prefill_min_ctas
    eng.ops.pp_prefill_min_ctas = 0
    try:
        got = replay.run_steps(eng, steps)
        eng.ops.check_errors()
    finally:
        eng.ops.pp_prefill_min_ctas = was
    replay.compare(got, ref, ATOL["bfloat16"](scale), f"two-tile {name}/{mode}", RMS["bfloat16"](scale))
    assert all(f == eng.num_pages for f in eng.cache.free_pages())


def test_cut_independence_bfloat16(models):
    """In bfloat16 the bits of a cached key depend on the product that made it: a step of few
    tokens sums the projection in float32 and rounds once, after the rotation; a larger step takes
    the library's product, which rounds to bfloat16 before the rotation rounds again.  So the same
    position computed whole, token by token (as after a preemption that recomputes) or in portions
    differs, but by rounding only: directly compared, within the bounds that each cut keeps against
    the plain implementation."""
    from somi_inference_b200.engine import Engine
    d, cfg, reqs, ref, scale = models[("D", torch.bfloat16)]
    sub = {"r2": reqs["r2"]}
    outs = []
    for mode in ("whole", "last32", "portions"):
        steps, mt = MODES[mode](sub)
        eng = Engine(d, dtype="bfloat16", page_size=16, max_tokens=mt)
        outs.append(replay.run_steps(eng, steps))
    for o in outs[1:]:
        diff = torch.stack([outs[0][k] - o[k] for k in outs[0]])
        assert diff.abs().max().item() <= 4e-2 * scale
        assert diff.pow(2).mean().sqrt().item() <= 4e-3 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_steps_replayed_from_graphs_match_plain(models, name, dtype):
    """A step whose layout has been seen twice is captured in a CUDA graph and replayed from then
    on.  One prompt-portion layout (16 tokens of one request) and one decode layout (two requests,
    one token each) are fed many times, with different tokens, cached lengths and pages; the
    replayed steps must give the plain logits like any other."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, cfg, reqs, ref, scale = models[(name, getattr(torch, dtype))]
    ids = list(reqs)[:4]
    portion = 16
    eng = Engine(d, dtype=dtype, page_size=PAGE_SIZES[name],
                 max_tokens=2 * max(replay.round_up(len(reqs[r]), 64) for r in ids))
    got = {}
    for pair in (ids[:2], ids[2:]):
        fed = {r: 0 for r in pair}
        # the prompts, in portions of 16 (the tail, shorter than that, in one step of its own)
        for r in pair:
            head = (len(reqs[r]) - 8) // portion * portion
            while fed[r] < head:
                toks = reqs[r][fed[r]:fed[r] + portion]
                logits = eng.step([StepEntry(r, toks, [0, portion - 1])]).float().cpu()
                got[(r, fed[r])], got[(r, fed[r] + portion - 1)] = logits[0], logits[1]
                fed[r] += portion
        # both requests decode together while both have tokens left: one layout, many steps
        while all(fed[r] < len(reqs[r]) for r in pair):
            logits = eng.step([StepEntry(r, [reqs[r][fed[r]]], [0]) for r in pair]).float().cpu()
            for k, r in enumerate(pair):
                got[(r, fed[r])] = logits[k]
                fed[r] += 1
        for r in pair:
            eng.end(r)                      # the next pair gets these pages
        eng.cache.check_consistency()
    graphs = eng._graphs
    assert len(graphs) >= 2, "the portion layout and the decode layout should both be captured"
    assert graphs.hits >= 12, f"only {graphs.hits} steps were replayed"
    eng.ops.check_errors()
    replay.compare(got, ref, ATOL[dtype](scale), f"graphs {name}/{dtype}", RMS[dtype](scale))


def test_graphs_are_captured_anew_after_the_descriptor_buffer_moved(models):
    """When a step needs a larger descriptor buffer than the engine holds, the buffer is
    allocated anew and every captured graph is void.  The next layouts are captured again
    (in a memory pool of their own: the old one went with its last graph) and their steps give
    the plain logits like any other."""
    from somi_inference_b200.engine import Engine, StepEntry
    d, cfg, reqs, ref, scale = models[("A", torch.bfloat16)]
    rid = list(reqs)[1]
    toks = reqs[rid]
    eng = Engine(d, dtype="bfloat16", page_size=PAGE_SIZES["A"], max_tokens=256)
    got = {}
    logits = eng.step([StepEntry("x", toks[:8], [7])]).float().cpu()
    got[(rid, 7)] = logits[0]
    for i in range(8, 40):
        got[(rid, i)] = eng.step([StepEntry("x", [toks[i]], [0])]).float().cpu()[0]
    assert len(eng._graphs) >= 1 and eng._graphs.hits >= 20
    captures = eng._graphs.captures
    eng.builder._alloc(2 * eng.builder._capacity)          # what a step beyond the capacity does
    for i in range(40, len(toks)):
        got[(rid, i)] = eng.step([StepEntry("x", [toks[i]], [0])]).float().cpu()[0]
    assert eng._graphs.captures > captures, "no layout was captured after the buffer moved"
    eng.ops.check_errors()
    replay.compare(got, ref, ATOL["bfloat16"](scale), "graphs after a moved descriptor", RMS["bfloat16"](scale))
