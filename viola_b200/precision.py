"""Process-wide training precision policy.

Two independent knobs, read when optimizers are constructed / bound and when the engine starts:
the storage dtype of master weights (``None`` = update the model parameters in place, no second
copy) together with the rounding used when a master is stored in 16 bits, and the dtype in which
parameter gradients are received and accumulated.  Same surface as the reference policy module
(viola/precision.py:16-35).
"""

from __future__ import annotations

import torch

_NAMES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}
_policy = {
    "master_weight_dtype": torch.float32,
    "gradient_dtype": None,
    "master_rounding": "nearest",
    "master_rounding_seed": 0,
}


def _dtype(value):
    """Accept 'fp32' / 'bf16' / 'fp16' or the torch dtype itself."""
    if isinstance(value, str):
        value = _NAMES[value]
    if value not in _NAMES.values():
        raise ValueError(f"unsupported precision {value!r}")
    return value


def set_master_weight_dtype(dtype, *, rounding="nearest", seed=0):
    """Select master-weight storage; ``None`` keeps no separate master copy."""
    if rounding not in ("nearest", "stochastic"):
        raise ValueError("rounding must be 'nearest' or 'stochastic'")
    if not 0 <= seed < (1 << 63):
        raise ValueError("seed must fit in 63 bits")
    _policy["master_weight_dtype"] = None if dtype is None else _dtype(dtype)
    _policy["master_rounding"] = rounding
    _policy["master_rounding_seed"] = seed


def set_gradient_dtype(dtype):
    """Select the dtype in which parameter gradients are produced and accumulated.

    Applies to optimizers bound (or FP8Muon instances built) afterwards; activation gradients and
    the operators' own arithmetic are unaffected.
    """
    _policy["gradient_dtype"] = _dtype(dtype)


def settings():
    """A copy of the current policy."""
    return dict(_policy)
