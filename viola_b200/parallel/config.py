"""Engine configuration: a YAML file, a dict, or ``$VIOLA_CONFIG`` merged one level deep over defaults.

Keys and defaults are the reference's (viola/distributed/config.py:18-42): ``num_processes``,
``mixed_precision``, ``gradient_accumulation_steps``, ``sharding{parameters, gradients, optimizer, ema,
blocks}``, ``precision{master_weight_dtype, gradient_dtype, master_rounding, master_rounding_seed}``,
``communication{dtype, bucket_mb, fp8_format, fp8_tile_size}``, ``ema{decay, dtype}`` and the optional
``device``.  One addition: ``communication.backend`` selects the transport of the hot paths —
``"auto"`` (peer-memory kernels on CUDA when every rank can map its peers, else collectives),
``"p2p"`` or ``"nccl"`` — and ``communication.overlap``: true runs the gradient reduction on a side stream bucket by
bucket while backward is still producing gradients; false (default) runs it once backward is done, with kernels
that take the whole GPU (measured faster at 2-8 GPUs: the narrow overlapped kernels cost more than they hide).
``communication.reduce_once`` (default true): with sharded gradients every microbatch adds its gradients into a
rank-local fp32 sum and the owners receive that sum once per optimizer step; false sends every microbatch's
gradients to the owners as the reference does (viola/distributed/gradients.py:86-125), which saves one
gradient-sized buffer per rank and costs one reduction per accumulation step.
``sharding.resident`` (``"auto"`` / true / false) keeps the gathered copy of sharded parameters allocated between
uses when it is small next to the device memory.
"""

from __future__ import annotations

import copy
import os
from pathlib import Path

import torch

from ..precision import settings

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def dtype(value):
    if value is None or isinstance(value, torch.dtype):
        return value
    return _DTYPES[value]


def read_config(config=None):
    if config is None:
        config = os.environ.get("VIOLA_CONFIG")
    if isinstance(config, (str, Path)):
        import yaml
        with open(config) as stream:
            config = yaml.safe_load(stream)
    supplied = copy.deepcopy(config or {})
    policy = settings()
    result = {
        "num_processes": 1,
        "mixed_precision": "bf16",
        "gradient_accumulation_steps": 1,
        "sharding": {"parameters": False, "gradients": False, "optimizer": True, "ema": True, "blocks": None,
                     "resident": "auto"},
        "precision": {"master_weight_dtype": policy["master_weight_dtype"],
                      "gradient_dtype": policy["gradient_dtype"] or torch.float32,
                      "master_rounding": policy["master_rounding"],
                      "master_rounding_seed": policy["master_rounding_seed"]},
        "communication": {"dtype": None, "bucket_mb": 25, "fp8_format": "e4m3", "fp8_tile_size": 256,
                          "backend": "auto", "overlap": False, "reduce_once": True},
        "ema": {"decay": 0, "dtype": "fp32"},
    }
    for key, value in supplied.items():
        if isinstance(value, dict) and isinstance(result.get(key), dict):
            result[key].update(value)
        else:
            result[key] = value
    return result
