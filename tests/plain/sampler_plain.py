"""Plain sampler: the reference's pipeline, row by row, with sorting (no kernels' tricks).

Formulas from somi_inference/core/sampler.py: repetition penalty over set(history)
(:81-104), division by temperature (:106-115), top-k by `topk` indices (:117-134), top-p on
the sorted softmax with the shift that keeps the first token crossing p (:136-159), then
argmax for temperature 0 or a draw from the softmax (:161-176).  The reference draws with
torch.multinomial from the global generator; the engine's draw is an inverse-CDF walk in
index order with a uniform number from splitmix64(seed, counter), restated here in Python.
"""

from __future__ import annotations

import torch

MASK64 = (1 << 64) - 1


def uniform(seed: int, counter: int) -> float:
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def filtered_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                    repetition_penalty: float, history) -> torch.Tensor:
    """One row after penalty, temperature, top-k and top-p (-inf where removed)."""
    x = logits.clone().float()
    if repetition_penalty != 1.0 and len(history):
        ids = torch.tensor(sorted(set(history)), dtype=torch.long)
        v = x[ids]
        x[ids] = torch.where(v > 0, v / repetition_penalty, v * repetition_penalty)
    if temperature > 0.0:
        x = x / temperature
    if temperature == 0.0:
        return x
    if top_k != -1:
        k = min(top_k, x.numel())
        keep = torch.zeros_like(x, dtype=torch.bool)
        keep[torch.topk(x, k=k).indices] = True
        x = x.masked_fill(~keep, float("-inf"))
    if top_p != 1.0:
        sorted_x, order = torch.sort(x, descending=True)
        cum = torch.cumsum(torch.softmax(sorted_x, dim=-1, dtype=torch.float32), dim=-1)
        remove = cum > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        x[order[remove]] = float("-inf")
    return x


def sample_row(logits, temperature, top_k, top_p, repetition_penalty, history, seed, counter):
    """Returns (token, cdf, target): cdf is the index-order cumulative softmax of what is left."""
    x = filtered_logits(logits, temperature, top_k, top_p, repetition_penalty, history)
    if temperature == 0.0:
        return int(torch.argmax(x)), None, None
    probs = torch.softmax(x.double(), dim=-1)
    cdf = torch.cumsum(probs, dim=-1)
    target = uniform(seed, counter) * float(cdf[-1])
    token = int(torch.searchsorted(cdf, torch.tensor(target, dtype=cdf.dtype), right=True))
    token = min(token, x.numel() - 1)
    return token, cdf, target
