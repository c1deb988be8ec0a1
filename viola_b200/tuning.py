"""Per-shape tile selection for the tcgen05 GEMMs, measured once and remembered on disk.

The GEMM kernel picks its output-tile width (128 or 256 columns) from a wave-count heuristic.  With tuning
switched on (``Linear(autotune=True)``, ``MLP(autotune=True)``, ``FP8Muon(ns_autotune=True)`` or
``viola_b200.tuning.enable()``), the first call with a new *signature* (epilogue, shapes, operand layouts and
dtypes, batch count) times every candidate width on the call's own operands and keeps the fastest; later calls
and later processes take the recorded choice.  This is the role of the reference's five autotuners and their
JSON caches (viola/nn/_linear_tuning.py:101-208, _grouped_tuning.py:40-77, _mlp_tuning.py:72-91,
_gated_kernels.py, viola/optim/_orthogonalize_kernels.py:115-197), collapsed into one mechanism because all of
those products run on one kernel template here.

Method (as in the reference's tuners): untimed warm-up, CUDA events around a burst of launches, median of
several repeats, candidates visited in rotating order so that none always runs first, and a determinism check
(two runs of a candidate must give bit-identical output, otherwise it is rejected).  A candidate must beat the
heuristic's choice by more than ``margin`` to replace it.

Cache: ``$VIOLA_B200_CACHE`` or ``~/.cache/viola_b200/<family>/<sha256>.json``; the key covers the GPU name,
compute capability, SM count, shared memory per block, the torch and CUDA versions and a hash of the kernel
library, so a rebuilt library or another GPU never reuses stale choices.  Nothing is timed while a CUDA graph
is being captured (the recorded or heuristic choice is used).
"""

from __future__ import annotations

import hashlib
import json
import os
import statistics
import threading
from pathlib import Path

import torch

FAMILIES = {0: "linear", 1: "orthogonalize", 2: "mlp", 3: "mlp", 4: "activation"}     # by epilogue code
CANDIDATES = (128, 256)

_enabled = False
_lock = threading.Lock()
_choices = {}                # signature -> tile width (0 = heuristic)
_not_on_disk = set()         # signatures whose cache file was looked for and not found
_fingerprint = None
margin = 0.03
repeats, burst, warmup = 5, 8, 3
log = []                     # (signature, {candidate: milliseconds}, chosen) of every search in this process


def enable(enabled=True):
    """Switch first-use tuning on or off for the whole process (layers with ``autotune=True`` switch it on)."""
    global _enabled
    _enabled = bool(enabled)


def enabled():
    return _enabled


def cache_root():
    return Path(os.environ.get("VIOLA_B200_CACHE", "~/.cache/viola_b200")).expanduser()


def fingerprint():
    """What a recorded choice depends on besides the call's signature."""
    global _fingerprint
    if _fingerprint is None:
        from . import ops
        entry = {"torch": torch.__version__, "cuda": torch.version.cuda}
        try:
            entry["library"] = hashlib.sha256(Path(ops._LIB_PATH).read_bytes()).hexdigest()[:16]
        except OSError:
            entry["library"] = "missing"
        if torch.cuda.is_available():
            props = torch.cuda.get_device_properties(torch.cuda.current_device())
            entry.update(gpu=props.name, capability=[props.major, props.minor], sms=props.multi_processor_count,
                         shared_memory=getattr(props, "shared_memory_per_block_optin", 0))
        _fingerprint = entry
    return _fingerprint


def _cache_path(signature):
    family = FAMILIES.get(signature[0], "gemm")
    digest = hashlib.sha256(json.dumps([fingerprint(), list(signature)], sort_keys=True, default=str).encode()).hexdigest()
    return cache_root() / family / f"{digest}.json"


def recall(signature):
    """Choice recorded in memory or on disk for ``signature`` (None when there is none)."""
    if signature in _choices:
        return _choices[signature]
    if signature in _not_on_disk:
        return None
    path = _cache_path(signature)
    try:
        record = json.loads(path.read_text())
        if record.get("signature") == [str(v) for v in signature]:
            _choices[signature] = int(record["tile"])
            return _choices[signature]
    except (OSError, ValueError, KeyError):
        pass
    _not_on_disk.add(signature)
    return None


def remember(signature, tile, timings=None):
    _choices[signature] = int(tile)
    path = _cache_path(signature)
    try:
        path.parent.mkdir(parents=True, exist_ok=True)
        scratch = path.with_suffix(".tmp")
        scratch.write_text(json.dumps({"signature": [str(v) for v in signature], "tile": int(tile),
                                       "milliseconds": timings or {}, "fingerprint": fingerprint()}, indent=1))
        scratch.replace(path)
    except OSError:
        pass                      # a read-only home directory only costs the persistence


def forget():
    """Drop the in-memory choices (the files stay)."""
    _choices.clear()
    _not_on_disk.clear()
    log.clear()


def measure_cuda(run):
    """Median milliseconds of one ``run()`` from CUDA events around bursts of back-to-back launches."""
    for _ in range(warmup):
        run()
    samples = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(burst):
            run()
        stop.record()
        stop.synchronize()
        samples.append(start.elapsed_time(stop) / burst)
    return statistics.median(samples)


def search(signature, run, output, *, candidates=CANDIDATES, measure=measure_cuda, baseline=0):
    """Time ``run(tile)`` for the heuristic (``baseline``) and every candidate; record and return the winner.

    ``output``: callable returning the tensor a run wrote (for the determinism check)."""
    order = [baseline, *candidates]
    timings, rejected = {}, set()
    for tile in order:
        run(tile)
        first = output().clone()
        run(tile)
        if not torch.equal(first, output()):
            rejected.add(tile)            # two runs disagree: never pick a non-deterministic configuration
    for rotation in range(len(order)):
        for tile in order[rotation:] + order[:rotation]:
            if tile in rejected:
                continue
            timings.setdefault(tile, []).append(measure(lambda: run(tile)))
    medians = {tile: statistics.median(values) for tile, values in timings.items()}
    chosen = baseline
    if medians:
        best = min(medians, key=medians.get)
        reference_time = medians.get(baseline, float("inf"))
        if best != baseline and medians[best] < reference_time * (1.0 - margin):
            chosen = best
    log.append((signature, medians, chosen))
    remember(signature, chosen, {str(k): v for k, v in medians.items()})
    return chosen


def choose(signature, run, output, *, tunable=True, candidates=CANDIDATES):
    """Tile width for a GEMM call: the recorded choice, or a search when tuning is on and timing is possible.
    ``candidates``: 128 and 256 (columns of a single-CTA tile) and, where the kernel has it, 512 = a 256 x 256 tile
    computed by a CTA pair."""
    found = recall(signature)
    if found is not None:
        return found
    if not (_enabled and tunable) or not torch.cuda.is_available() or torch.cuda.is_current_stream_capturing():
        return 0
    with _lock:
        return search(signature, run, output, candidates=candidates)
