"""Timing helpers shared by the op-level benchmarks.

CUDA events on the launching stream, warm-up first, an L2 flush (a 256 MiB write, twice the 126 MB
L2) before every timed iteration, median over repeats.  Multi-GPU numbers take the maximum over
ranks.  Roofline fractions are against the measured peaks in ``MEASURED_PEAKS.json`` when present,
else the fallback 6.65 TB/s and 1.59 PFLOP/s.
"""

from __future__ import annotations

import json
import os
import statistics

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_flush = None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as stream:
            data = json.load(stream)
        return dict(hbm_gbs=data["hbm_gbs"], bf16_tflops=data["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, device="cuda", dtype=torch.uint8)
    _flush.zero_()


def measure(fn, *, warmup=5, repeats=15):
    """Median milliseconds of ``fn()`` with a cold L2."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(repeats):
        flush_l2()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    return statistics.median(times)


def report(rows, path=None):
    for row in rows:
        print(json.dumps(row), flush=True)
    if path:
        with open(path, "w") as stream:
            json.dump(rows, stream, indent=1)
