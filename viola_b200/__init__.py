"""viola_b200: a Blackwell-datacenter (B200, sm_100a) native FP8 training framework.

``import viola_b200 as viola`` gives the reference's public surface (viola/__init__.py:5-9):
``viola.nn``, ``viola.optim``, ``viola.distributed``, ``viola.precision``, ``viola.violaEngine``,
``viola.set_master_weight_dtype`` and ``viola.set_gradient_dtype``.
"""

__version__ = "0.1.0"

import sys as _sys

from . import nn, ops, optim, parallel, precision
from .parallel import violaEngine
from .precision import set_gradient_dtype, set_master_weight_dtype

distributed = parallel
_sys.modules[__name__ + ".distributed"] = parallel

__all__ = ["distributed", "parallel", "nn", "optim", "ops", "precision", "violaEngine", "set_master_weight_dtype",
           "set_gradient_dtype"]
