"""The sampling kernel against the plain sampler (tests/plain/sampler_plain.py), row by row."""

import pytest
import torch

from somi_inference_b200.sampling import Sampler, SamplingParams
from tests.plain import sampler_plain

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sampler():
    from somi_inference_b200.ops import cuda_ops
    return Sampler(cuda_ops(), "cuda")


def test_uniform_matches_python(sampler):
    for seed, c in [(0, 0), (5, 17), (2 ** 63 + 12345, 4000000000), (2 ** 64 - 1, 1)]:
        assert sampler.ops.uniform(seed, c) == pytest.approx(sampler_plain.uniform(seed, c), abs=0)


@pytest.mark.parametrize("V", [5, 517, 1000, 151936])
def test_greedy_lowest_index_wins_ties(sampler, V):
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(6, V, generator=g)
    logits[1, V // 2] = logits[1, V - 1] = 50.0
    logits[2, 0] = logits[2, 3] = 50.0
    logits[3] = -1e30
    out = sampler.sample(logits.cuda(), [SamplingParams(temperature=0.0)] * 6, [0] * 6, [0] * 6)
    assert out.tolist() == torch.argmax(logits, -1).tolist()
    assert out[1] == V // 2 and out[2] == 0 and out[3] == 0


def check_rows(sampler, logits, params, histories, n_counters=12):
    rows = logits.shape[0]
    dev = logits.cuda()
    for counter in range(n_counters):
        seeds = [1000 + 7 * r for r in range(rows)]
        got = sampler.sample(dev, params, [counter] * rows, seeds, histories).tolist()
        for r in range(rows):
            p = params[r]
            tok, cdf, target = sampler_plain.sample_row(
                logits[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                histories[r] if histories else [], seeds[r], counter)
            if cdf is None or got[r] == tok:
                assert got[r] == tok
                continue
            # A different token is only acceptable where float32 summation order decides:
            # the target lies within rounding of the boundary between the two tokens.
            kept = torch.isfinite(sampler_plain.filtered_logits(
                logits[r], p.temperature, p.top_k, p.top_p, p.repetition_penalty,
                histories[r] if histories else []))
            assert kept[got[r]], f"row {r}: token {got[r]} was filtered out"
            lo = float(cdf[got[r] - 1]) if got[r] > 0 else 0.0
            assert lo - 1e-5 <= target <= float(cdf[got[r]]) + 1e-5, (r, counter, got[r], tok)


@pytest.mark.parametrize("V", [64, 1000, 32003])
def test_temperature_top_k_top_p_penalty(sampler, V):
    g = torch.Generator().manual_seed(V + 1)
    logits = torch.randn(8, V, generator=g) * 3
    params = [SamplingParams(temperature=1.0), SamplingParams(temperature=0.7),
              SamplingParams(temperature=1.3, top_k=5), SamplingParams(temperature=1.0, top_k=1),
              SamplingParams(temperature=0.9, top_p=0.8),
              SamplingParams(temperature=1.0, top_k=40, top_p=0.5),
              SamplingParams(temperature=0.8, repetition_penalty=1.7),
              SamplingParams(temperature=0.0, repetition_penalty=3.0, top_k=3, top_p=0.2)]
    hist = [torch.randint(0, V, (50,), generator=g).tolist() for _ in range(8)]
    hist[7] = [int(torch.argmax(logits[7]))]
    check_rows(sampler, logits, params, hist)


def test_kept_sets_are_exact(sampler):
    """With a spread-out distribution, sampling many times never leaves the plain kept set and
    reaches all of it."""
    V = 50
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(1, V, generator=g) * 2
    for p in (SamplingParams(temperature=1.0, top_k=4), SamplingParams(temperature=1.5, top_p=0.6)):
        kept = torch.isfinite(sampler_plain.filtered_logits(logits[0], p.temperature, p.top_k,
                                                            p.top_p, 1.0, []))
        dev = logits.cuda().expand(64, V).contiguous()
        seen = set()
        for rep in range(8):
            out = sampler.sample(dev, [p] * 64, list(range(rep * 64, rep * 64 + 64)), [9] * 64)
            seen |= set(out.tolist())
        assert seen == set(torch.nonzero(kept).flatten().tolist())


def test_distribution_and_batch_independence(sampler):
    V = 11
    logits = torch.linspace(-2, 2, V).unsqueeze(0)
    probs = torch.softmax(logits[0] / 0.9, 0)
    n = 4096
    dev = logits.cuda().expand(n, V).contiguous()
    p = SamplingParams(temperature=0.9)
    out = sampler.sample(dev, [p] * n, list(range(n)), [77] * n)
    freq = torch.bincount(out.cpu().long(), minlength=V).float() / n
    assert (freq - probs).abs().max().item() < 0.03
    # the same (seed, counter) gives the same token whatever else is in the batch
    alone = sampler.sample(dev[:1], [p], [123], [77]).item()
    other = torch.randn(5, V).cuda()
    mixed = sampler.sample(torch.cat([other[:3], dev[:1], other[3:]]), [p] * 6,
                           [1, 2, 3, 123, 5, 6], [1, 2, 3, 77, 5, 6])
    assert mixed[3].item() == alone
