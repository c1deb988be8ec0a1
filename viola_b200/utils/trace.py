"""Phase ranges for profilers and per-phase timings of the engine step.

The reference has no tracing hooks (its trainer logs wall time per step, experiments/train_dit.py:196-200).
Here every phase of a step (``backward``, ``reduce``, ``optimizer``, ``writeback``, ``ema``) is wrapped in
:func:`phase`:

* ``VIOLA_TRACE=1`` pushes an NVTX range per phase (visible in Nsight Systems / Compute timelines);
* ``VIOLA_PHASE_TIMES=1`` (or :func:`enable_timing`) also records a CUDA-event pair per phase on the current
  stream; :func:`phase_times` synchronises and returns the accumulated milliseconds per phase, which is how the
  per-step optimizer and communication times of the benchmarks are obtained without a profiler.

Both are off by default and then cost one dictionary lookup per phase.
"""

from __future__ import annotations

import os
import time
from contextlib import contextmanager

import torch

_nvtx = os.environ.get("VIOLA_TRACE", "0") not in ("", "0")
_timing = os.environ.get("VIOLA_PHASE_TIMES", "0") not in ("", "0")
_pending = []          # (name, start event | start seconds, end event | end seconds)
_totals = {}


def enable_timing(enabled=True):
    """Turn per-phase timing on or off at run time; clears what was collected."""
    global _timing
    _timing = bool(enabled)
    _pending.clear()
    _totals.clear()


def enable_nvtx(enabled=True):
    global _nvtx
    _nvtx = bool(enabled)


@contextmanager
def phase(name):
    """Mark one phase of the step.  A no-op unless tracing or timing is enabled."""
    if not (_nvtx or _timing):
        yield
        return
    cuda = torch.cuda.is_available() and torch.cuda.is_initialized()
    if cuda and torch.cuda.is_current_stream_capturing():
        yield                      # timing events cannot be recorded into a CUDA graph
        return
    if _nvtx and cuda:
        torch.cuda.nvtx.range_push(f"viola.{name}")
    start = None
    if _timing:
        if cuda:
            start = torch.cuda.Event(enable_timing=True)
            start.record()
        else:
            start = time.perf_counter()
    try:
        yield
    finally:
        if _timing:
            if cuda:
                end = torch.cuda.Event(enable_timing=True)
                end.record()
            else:
                end = time.perf_counter()
            _pending.append((name, start, end))
        if _nvtx and cuda:
            torch.cuda.nvtx.range_pop()


def phase_times(reset=True):
    """Milliseconds per phase accumulated since the last reset (synchronises the device once)."""
    if _pending and not isinstance(_pending[0][1], float):
        torch.cuda.synchronize()
    for name, start, end in _pending:
        elapsed = (end - start) * 1e3 if isinstance(start, float) else start.elapsed_time(end)
        _totals[name] = _totals.get(name, 0.0) + elapsed
    _pending.clear()
    result = dict(_totals)
    if reset:
        _totals.clear()
    return result
