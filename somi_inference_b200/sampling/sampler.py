"""Turns logits rows into token ids on the device.

Same interface idea as the reference's `Sampler.sample(logits, params, token_histories)`
(somi_inference/core/sampler.py:31-55), but the whole pipeline (repetition
penalty, temperature, top-k, top-p, argmax or draw) is one kernel launch for
all rows, and each row carries (seed, counter) for its random number.
"""

from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .params import SamplingParams


class Sampler:
    def __init__(self, ops, device: torch.device | str) -> None:
        self.ops = ops
        self.device = torch.device(device)
        self.h2d_bytes_last = 0
        self._greedy: dict = {}

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams],
               counters: Sequence[int], seeds: Sequence[int],
               histories: Sequence[Sequence[int]] | None = None) -> torch.Tensor:
        """logits [rows, vocab] float32 on the device -> int32 [rows] on the device.

        `counters[i]` is how many tokens row i's request has sampled so far;
        `seeds[i]` its seed; `histories[i]` its prompt and output tokens (only
        read where the row's repetition penalty is not 1).
        """
        rows = logits.shape[0]
        if logits.dim() != 2:
            raise ValueError(f"logits must be 2D, got shape {tuple(logits.shape)}")
        if not (len(params) == len(counters) == len(seeds) == rows):
            raise ValueError("one SamplingParams, counter and seed per logits row is needed")
        if all(p.temperature == 0.0 and p.repetition_penalty == 1.0 for p in params):
            # argmax rows need neither seeds, counters nor histories: one cached parameter block
            cached = self._greedy.get(rows)
            if cached is None:
                cached = self._pack(params, [0] * rows, [0] * rows, None)
                self._greedy[rows] = cached
            self.h2d_bytes_last = 0
            return self._launch(logits, rows, *cached)
        return self._launch(logits, rows, *self._pack(params, counters, seeds, histories))

    def _pack(self, params, counters, seeds, histories):
        rows = len(params)
        # one packed upload: 4 float/int arrays of `rows`, seeds as two int32 each, offsets, tokens
        hist_off = np.zeros(rows + 1, dtype=np.int64)
        toks: list[np.ndarray] = []
        for i, p in enumerate(params):
            n = 0
            if p.repetition_penalty != 1.0 and histories is not None and len(histories[i]):
                h = np.unique(np.asarray(histories[i], dtype=np.int64))
                toks.append(h)
                n = len(h)
            hist_off[i + 1] = hist_off[i] + n
        n_hist = int(hist_off[-1])
        r8 = -(-rows // 2) * 2
        buf = np.zeros(7 * r8 + 2 + rows + 1 + max(n_hist, 1), dtype=np.int32)
        buf[0:rows].view(np.float32)[:] = [p.temperature for p in params]
        buf[r8:r8 + rows] = [p.top_k for p in params]
        buf[2 * r8:2 * r8 + rows].view(np.float32)[:] = [p.top_p for p in params]
        buf[3 * r8:3 * r8 + rows].view(np.float32)[:] = [p.repetition_penalty for p in params]
        buf[4 * r8:4 * r8 + 2 * rows].view(np.uint64)[:] = np.asarray(
            [int(s) % (1 << 64) for s in seeds], dtype=np.uint64)
        buf[6 * r8:6 * r8 + rows].view(np.uint32)[:] = np.asarray(counters, dtype=np.uint32)
        o = 7 * r8
        buf[o:o + rows + 1] = hist_off
        h = o + rows + 1
        h += h % 2
        if n_hist:
            buf[h:h + n_hist] = np.concatenate(toks)
        self.h2d_bytes_last = buf.nbytes
        dev = torch.from_numpy(buf).to(self.device, non_blocking=True)
        # the kernel's arguments as views of the one uploaded buffer (made once per upload: the
        # block of an all-greedy step is cached with them)
        return (dev[0:rows].view(torch.float32), dev[r8:r8 + rows],
                dev[2 * r8:2 * r8 + rows].view(torch.float32),
                dev[3 * r8:3 * r8 + rows].view(torch.float32),
                dev[4 * r8:4 * r8 + 2 * rows], dev[6 * r8:6 * r8 + rows],
                dev[o:o + rows + 1], dev[h:h + max(n_hist, 1)])

    def _launch(self, logits, rows, *views):
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        self.ops.sample(logits, *views, out)
        return out
