"""Per-launch timing of one step: a CUDA event after every kernel launch.

The reference profiles a prompt step stage by stage with events around each stage
(benchmarks/profile_prefill.py:183-285).  Here every wrapper of the kernel table, and the
library matrix product, reports each launch with the bytes it has to move and the
floating-point operations it has to do; while a `LaunchTrace` is active an event is recorded
after each of them, and the time of a launch is the distance to the event before it.  Without
an active trace `note` costs one comparison.

Times taken this way are those of an eager step (no CUDA graph, no overlap of a kernel's start
with its predecessor's end).  The host needs longer to issue a short kernel than the GPU to run
it, so the trace first puts a spinning kernel of a few milliseconds on the stream: the host
issues the step's launches behind it, and when it ends they run back to back with nothing but
the events between them.
"""

from __future__ import annotations

import torch

_active: "LaunchTrace | None" = None


def active() -> bool:
    return _active is not None


def note(label: str, nbytes: float = 0.0, flops: float = 0.0, detail: str = "") -> None:
    """Report the launch that was just made (call after the launch, on its stream)."""
    if _active is not None:
        _active.note(label, nbytes, flops, detail)


class LaunchTrace:
    def __init__(self, head_start_ms: float = 8.0) -> None:
        self._events: list[torch.cuda.Event] = []
        self._rows: list[tuple[str, float, float, str]] = []
        self._head_start_cycles = int(head_start_ms * 1e-3 * 1.9e9)

    def __enter__(self) -> "LaunchTrace":
        global _active
        if _active is not None:
            raise RuntimeError("a launch trace is already active")
        if self._head_start_cycles > 0:
            torch.cuda._sleep(self._head_start_cycles)       # a bounded spin, then the step
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append(ev)
        _active = self
        return self

    def __exit__(self, *exc) -> None:
        global _active
        _active = None

    def note(self, label: str, nbytes: float, flops: float, detail: str) -> None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append(ev)
        self._rows.append((label, float(nbytes), float(flops), detail))

    def rows(self) -> list[dict]:
        """One record per launch, in launch order: label, detail, microseconds, bytes, flops."""
        torch.cuda.synchronize()
        out = []
        for i, (label, nbytes, flops, detail) in enumerate(self._rows):
            us = self._events[i].elapsed_time(self._events[i + 1]) * 1e3
            out.append({"label": label, "detail": detail, "us": us, "bytes": nbytes, "flops": flops})
        return out


def summarise(rows: list[dict], hbm_gbs: float, tflops: float) -> list[dict]:
    """Rows with equal (label, detail) added up; achieved rates and their fractions of the peaks.

    `frac` is the larger of bytes / time / copy peak and flops / time / tensor peak: the
    fraction of the roofline that bounds the launch.
    """
    merged: dict[tuple[str, str], dict] = {}
    for r in rows:
        m = merged.setdefault((r["label"], r["detail"]),
                              {"label": r["label"], "detail": r["detail"], "launches": 0,
                               "us": 0.0, "bytes": 0.0, "flops": 0.0})
        m["launches"] += 1
        for k in ("us", "bytes", "flops"):
            m[k] += r[k]
    total = sum(m["us"] for m in merged.values()) or 1.0
    out = []
    for m in merged.values():
        s = m["us"] * 1e-6
        gbs = m["bytes"] / s / 1e9 if s > 0 else 0.0
        tf = m["flops"] / s / 1e12 if s > 0 else 0.0
        out.append({**m, "us": round(m["us"], 1), "share": round(m["us"] / total, 4),
                    "gb_s": round(gbs, 1), "tflop_s": round(tf, 1),
                    "frac": round(max(gbs / hbm_gbs, tf / tflops), 4)})
    out.sort(key=lambda m: -m["us"])
    return out
