"""Trace replay: feed given token ids through the engine step by step, write logits.

Usage:  trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Reads one JSON object per line from standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries` are one batch for `Engine.step` (the step function that generation
uses: same model, cache and kernels).  For a step in which logits are wanted,
`OUT/<step>.f32` receives them as little-endian float32 [wanted, vocab], in the
order of the entries and of `want`.  Requests named in `end` give back what they
hold after the step.  After every step `done <step>` is printed and flushed.
It samples nothing.  The reference has no counterpart; its closest relative is
the hand-driven prefill/decode loop of tests/models/test_qwen2_e2e.py:63-77.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

TRACE_PAGE_SIZE = 16       # divides 64, so a request's pages never exceed its count rounded up to 64
MAX_LIVE_REQUESTS = 16


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=TRACE_PAGE_SIZE)
    args = ap.parse_args(argv)

    os.makedirs(args.out, exist_ok=True)
    from ..engine import Engine, StepEntry

    page = args.page_size
    unit = max(64, page)
    unit = -(-unit // page) * page
    pool_tokens = -(-args.max_tokens // unit) * unit
    engine = Engine(args.model, dtype=args.dtype, page_size=page, max_tokens=pool_tokens,
                    max_requests=MAX_LIVE_REQUESTS)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                logits.detach().to("cpu").contiguous().numpy().astype("<f4").tofile(
                    os.path.join(args.out, f"{step}.f32"))
            engine.ops.check_errors()       # a kernel that gave up on a bounded wait says so here
        for rid in rec.get("end", []):
            if engine.has(rid):
                engine.end(rid)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
