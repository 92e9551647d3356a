"""Traces for the replay tests: the same requests cut into steps in four ways.

A trace is a list of step records as `bin/trace_run` reads them.  `run_steps`
feeds a trace to an `Engine` in-process; `run_trace_program` feeds it to the
`bin/trace_run` program.  Both return {(request, position): logits row}.
"""

from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import torch

from somi_inference_b200.engine import StepEntry

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def whole(requests: dict[str, list[int]]) -> tuple[list[dict], int]:
    """Each request alone and whole, all positions wanted."""
    steps = []
    for s, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks,
                                              "want": list(range(len(toks)))}], "end": [rid]})
    return steps, max(round_up(len(t), 64) for t in requests.values())


def last_one_by_one(requests: dict[str, list[int]], tail: int = 32) -> tuple[list[dict], int]:
    """Most of a request in one step, then its last `tail` tokens one by one."""
    steps = []
    s = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[:head],
                                              "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, len(toks)):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[i:i + 1], "want": [0]}],
                          "end": [rid] if i == len(toks) - 1 else []})
            s += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps, max(round_up(len(t), 64) for t in requests.values())


def portions(requests: dict[str, list[int]], sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 9)) -> tuple[list[dict], int]:
    """Portions of changing size, down to two tokens."""
    steps = []
    s = 0
    for rid, toks in requests.items():
        i = 0
        k = 0
        while i < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            i += c
            steps.append({"step": s, "entries": [{"id": rid, "tokens": toks[i - c:i],
                                                  "want": list(range(c))}],
                          "end": [rid] if i == len(toks) else []})
            s += 1
    return steps, max(round_up(len(t), 64) for t in requests.values())


def mixed(requests: dict[str, list[int]], seed: int = 0, live: int = 4,
          tail: int = 32) -> tuple[list[dict], int]:
    """Up to `live` requests at a time: portions of some beside single tokens of others.

    A request's prompt part is fed in random portions (2..24 tokens), its last
    `tail` tokens one by one; now and then a request sits a step out.  As soon
    as one ends the next one starts, so its pages are handed on.  The second
    value is the most tokens (each request rounded up to 64) held at any time.
    """
    rng = random.Random(seed)
    waiting = list(requests.items())
    active: list[list] = []      # [rid, toks, fed]
    steps = []
    s = 0
    peak = 0
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active.append([rid, toks, 0])
        entries, ended = [], []
        for a in active:
            rid, toks, fed = a
            if rng.random() < 0.15 and len(active) > 1:
                continue
            left = len(toks) - fed
            if left > tail:
                c = min(rng.choice([2, 2, 3, 5, 8, 13, 16, 17, 24]), left - tail)
                if c == 1 and left - tail == 1:
                    c = 1
            else:
                c = 1
            want = sorted(set(rng.sample(range(c), k=min(c, rng.choice([1, 2, c])))) | {c - 1})
            entries.append({"id": rid, "tokens": toks[fed:fed + c], "want": want})
            a[2] = fed + c
            if a[2] == len(toks):
                ended.append(rid)
        if not entries:
            continue
        peak = max(peak, sum(round_up(a[2], 64) for a in active if a[2] > 0))
        steps.append({"step": s, "entries": entries, "end": ended})
        s += 1
        active = [a for a in active if a[0] not in ended]
    return steps, peak


LAST_RUN: dict = {}      # (request, position) -> (step, tokens in the step, replayed from a graph?)


def run_steps(engine, steps: list[dict]) -> dict[tuple[str, int], torch.Tensor]:
    out: dict[tuple[str, int], torch.Tensor] = {}
    fed: dict[str, int] = {}
    LAST_RUN.clear()
    for rec in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in rec["entries"]]
        graphs = getattr(engine, "_graphs", None)
        hits = graphs.hits if graphs is not None else 0
        logits = engine.step(entries).float().cpu()
        replayed = graphs is not None and graphs.hits > hits
        k = 0
        for e in rec["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = logits[k]
                LAST_RUN[(e["id"], base + w)] = (rec["step"], [len(x["tokens"]) for x in rec["entries"]],
                                                 replayed)
                k += 1
            fed[e["id"]] = base + len(e["tokens"])
        assert k == logits.shape[0]
        for rid in rec["end"]:
            engine.end(rid)
            fed.pop(rid, None)
        engine.cache.check_consistency()
    return out


def run_trace_program(model_dir: str, dtype: str, steps: list[dict], max_tokens: int,
                      out_dir: str, vocab: int, env: dict | None = None,
                      prefix: list[str] | None = None) -> dict[tuple[str, int], torch.Tensor]:
    """Feed the trace to bin/trace_run, one step at a time, waiting for `done <step>`."""
    cmd = (prefix or []) + [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                            model_dir, "--dtype", dtype, "--out", out_dir, "--max-tokens",
                            str(max_tokens)]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for rec in steps:
            proc.stdin.write(json.dumps(rec) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline()
            assert line.strip() == f"done {rec['step']}", f"trace_run answered {line!r}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out: dict[tuple[str, int], torch.Tensor] = {}
    fed: dict[str, int] = {}
    for rec in steps:
        n_want = sum(len(e["want"]) for e in rec["entries"])
        path = os.path.join(out_dir, f"{rec['step']}.f32")
        if n_want == 0:
            assert not os.path.exists(path)
        else:
            logits = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, vocab).copy())
        k = 0
        for e in rec["entries"]:
            base = fed.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], base + w)] = logits[k]
                k += 1
            fed[e["id"]] = base + len(e["tokens"])
        for rid in rec["end"]:
            fed.pop(rid, None)
    return out


def compare(got: dict, reference: dict[str, torch.Tensor], atol: float, what: str,
            rms_tol: float | None = None) -> float:
    """Every produced row against the plain logits of its request; returns the worst error.

    `atol` bounds the largest single difference; `rms_tol`, when given, bounds the root mean
    square of all differences (rounding noise has a stable RMS, while the largest of a million
    differences moves with every change of summation order)."""
    worst = 0.0
    where = None
    sq, n = 0.0, 0
    off = []
    for (rid, pos), row in got.items():
        diff = row.double() - reference[rid][pos].double()
        err = diff.abs().max().item()
        sq += float(diff.pow(2).sum())
        n += diff.numel()
        if not err <= atol:
            off.append((rid, pos, float(f"{err:.3g}")))
        if not err <= worst:      # also catches NaN
            worst, where = err, (rid, pos)
    assert worst <= atol, (f"{what}: worst error {worst:.3e} at request/position {where} (allowed "
                           f"{atol:.1e}); {len(off)} rows off, the first: {off[:12]}; their steps "
                           f"(step, tokens of its entries, replayed from a graph): "
                           f"{[LAST_RUN.get((r, p)) for r, p, _ in off[:12]]}")
    if rms_tol is not None:
        rms = (sq / max(n, 1)) ** 0.5
        assert rms <= rms_tol, f"{what}: rms error {rms:.3e} (allowed {rms_tol:.1e})"
    return worst
