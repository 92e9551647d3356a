"""Plain generation with sampling: whole-sequence logits from tests/plain/qwen2_plain.py, one
token at a time, through the plain sampler.  The loop is the reference's: prefill samples the
first token from the last prompt position with the prompt as history, every decode step samples
from the newest position with prompt + output as history
(somi_inference/core/model_runner.py:24-60, somi_inference/core/continuous_batching.py:141-177).
The random number of a request's i-th sampled token is uniform(seed, i).
"""

from __future__ import annotations

import torch

from . import qwen2_plain as plain
from . import sampler_plain


def _row(cfg, w, tokens):
    return plain.logits(cfg, w, tokens)[-1]


def generate(cfg, w, prompt, n_new, *, temperature=1.0, top_k=-1, top_p=1.0,
             repetition_penalty=1.0, seed=0) -> list[int]:
    out: list[int] = []
    for i in range(n_new):
        tok, _, _ = sampler_plain.sample_row(_row(cfg, w, list(prompt) + out), temperature, top_k,
                                             top_p, repetition_penalty, list(prompt) + out, seed, i)
        out.append(tok)
    return out


def check_sampled(cfg, w, prompt, got, *, temperature=1.0, top_k=-1, top_p=1.0,
                  repetition_penalty=1.0, seed=0, slack=2e-4) -> int:
    """Check `got` (an engine's output for `prompt`) token by token against the plain pipeline,
    each token given the engine's own earlier tokens.  A token that differs from the plain one is
    accepted only where rounding decides: it survived the filters, and the draw's target lies
    within `slack` of the boundary between the two tokens in the cumulative distribution.
    Returns how many tokens were such boundary cases."""
    boundary = 0
    for i, tok in enumerate(got):
        history = list(prompt) + list(got[:i])
        row = _row(cfg, w, history)
        want, cdf, target = sampler_plain.sample_row(row, temperature, top_k, top_p,
                                                     repetition_penalty, history, seed, i)
        if tok == want:
            continue
        assert cdf is not None, f"token {i}: greedy gives {want}, got {tok}"
        kept = torch.isfinite(sampler_plain.filtered_logits(row, temperature, top_k, top_p,
                                                            repetition_penalty, history))
        assert kept[tok], f"token {i}: {tok} was filtered out by the plain pipeline"
        lo = float(cdf[tok - 1]) if tok > 0 else 0.0
        assert lo - slack <= target <= float(cdf[tok]) + slack, \
            f"token {i}: got {tok}, plain gives {want}; target {target} not at their boundary"
        boundary += 1
    return boundary
