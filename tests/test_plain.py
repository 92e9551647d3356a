"""The plain implementation against hand formulas and against the recorded outputs of the
reference's own model code (tests/golden/golden_tiny.json, made by tests/golden/make_golden.py)."""

import json
import math
import os

import pytest
import torch

from somi_inference_b200.config import Qwen2Config
from somi_inference_b200.weights import random_tensors
from tests.plain import qwen2_plain as plain
from tests.plain import sampler_plain
from tests.tiny import SEEDS, TINY

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "golden_tiny.json")


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]])
    out = plain.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0)     # rms = sqrt(12.5)
    r = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 / r, 8 / r]]), atol=1e-6)


def test_rope_tables_and_rotation():
    cos, sin = plain.rope_tables(8, 1e6, 16)
    assert cos.shape == (16, 8) and torch.all(cos[0] == 1) and torch.all(sin[0] == 0)
    inv = 1.0 / (1e6 ** (torch.arange(0, 8, 2) / 8))
    assert torch.allclose(cos[5, :4], torch.cos(5 * inv)) and torch.allclose(cos[5, 4:], cos[5, :4])
    x = torch.randn(2, 16, 8)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    assert torch.equal(plain.rotate_half(torch.tensor([1.0, 2.0, 3.0, 4.0])),
                       torch.tensor([-3.0, -4.0, 1.0, 2.0]))


def test_attention_is_causal_windowed_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(4, 6, 8), torch.randn(2, 6, 8), torch.randn(2, 6, 8)
    o = plain.causal_attention(q, k, v)
    assert torch.allclose(o[:, 0], v.repeat_interleave(2, 0)[:, 0], atol=1e-6)   # first sees itself only
    k2, v2 = k.clone(), v.clone()
    k2[:, 4:], v2[:, 4:] = 9.0, 9.0
    assert torch.allclose(plain.causal_attention(q, k2, v2)[:, :4], o[:, :4], atol=1e-6)
    ow = plain.causal_attention(q, k, v, window=2)
    s = torch.einsum("d,jd->j", q[3, 5], k[1, 4:6]) * 8 ** -0.5
    assert torch.allclose(ow[3, 5], torch.softmax(s, 0) @ v[1, 4:6], atol=1e-6)
    assert torch.allclose(plain.causal_attention(q, k, v, window=6), o, atol=1e-6)
    with pytest.raises(ValueError):
        plain.causal_attention(torch.randn(3, 2, 8), k[:, :2], v[:, :2])


def test_swiglu_by_hand():
    w = {"p.mlp.gate_proj.weight": torch.tensor([[1.0, 0.0]]),
         "p.mlp.up_proj.weight": torch.tensor([[0.0, 2.0]]),
         "p.mlp.down_proj.weight": torch.tensor([[1.0], [-1.0]])}
    h = torch.tensor([[0.5, 3.0]])
    g = 0.5 / (1 + math.exp(-0.5))
    assert torch.allclose(plain.swiglu(h, w, "p"), torch.tensor([[g * 6, -g * 6]]), atol=1e-6)


@pytest.mark.parametrize("name", ["A", "B"])
def test_against_the_reference_models_recorded_outputs(name):
    with open(GOLDEN) as f:
        gold = json.load(f)
    cfg = dict(TINY[name])
    w = {k: v.float() for k, v in random_tensors(Qwen2Config.from_dict(cfg), SEEDS[name],
                                                 std=gold["std"], dtype=torch.float32).items()}
    e = gold[name]
    assert e["hidden_max_abs_diff"] < 1e-5
    ids = e["ids"]
    if name == "A":
        assert e["logits_max_abs_diff"] < 1e-5
        logits = plain.logits(cfg, w, ids)
        for pos, row in e["reference_logits_rows"].items():
            assert torch.allclose(logits[int(pos), :16], torch.tensor(row), atol=2e-5)
        for n, g in e["greedy"].items():
            assert plain.greedy(cfg, w, g["prompt"], len(g["tokens"])) == g["tokens"]
    else:
        h = plain.hidden_states(cfg, w, torch.tensor(ids))
        for pos, row in e["reference_hidden_rows"].items():
            assert torch.allclose(h[int(pos), :16], torch.tensor(row), atol=2e-5)


def test_plain_sampler_pipeline():
    x = torch.tensor([1.0, 3.0, 2.0, -1.0, 0.5])
    assert sampler_plain.sample_row(x, 0.0, -1, 1.0, 1.0, [], 0, 0)[0] == 1
    # repetition penalty flips the greedy choice (positive logit divided)
    assert sampler_plain.sample_row(x, 0.0, -1, 1.0, 2.0, [1], 0, 0)[0] == 2
    f = sampler_plain.filtered_logits(x, 1.0, 2, 1.0, 1.0, [])
    assert torch.isfinite(f).tolist() == [False, True, True, False, False]
    p = torch.softmax(x, 0)
    f = sampler_plain.filtered_logits(x, 1.0, -1, float(p[1]) + 0.01, 1.0, [])
    assert torch.isfinite(f).tolist() == [False, True, True, False, False]   # the crossing token stays
    f = sampler_plain.filtered_logits(x, 1.0, -1, 0.1, 1.0, [])
    assert torch.isfinite(f).tolist() == [False, True, False, False, False]
    us = [sampler_plain.uniform(5, c) for c in range(2000)]
    assert 0.0 <= min(us) and max(us) < 1.0 and abs(sum(us) / 2000 - 0.5) < 0.03
    counts = [0] * 5
    for c in range(4000):
        counts[sampler_plain.sample_row(x, 1.0, -1, 1.0, 1.0, [], 11, c)[0]] += 1
    assert all(abs(counts[i] / 4000 - float(p[i])) < 0.03 for i in range(5))
