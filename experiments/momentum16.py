"""Muon with one BF16 (or FP16) momentum buffer: the baseline that FP8 momentum is compared against.

Same update rule, Newton-Schulz and weight update as :class:`viola_b200.optim.FP8Muon`; only the momentum
storage differs (2 bytes per element, no scales).  Used by ``train_dit.py --momentum-dtype bf16`` for matched
independent runs (counterpart of experiments/momentum16.py:25-40 of the reference).
"""
from __future__ import annotations

import torch

from viola_b200 import ops
from viola_b200.optim import FP8Muon


class Momentum16(FP8Muon):
    def __init__(self, params, *, momentum_dtype=torch.bfloat16, **options):
        if momentum_dtype not in (torch.bfloat16, torch.float16):
            raise ValueError("momentum_dtype must be bfloat16 or float16")
        self.momentum_dtype = momentum_dtype
        super().__init__(params, **options)

    def _begin_local(self):
        super()._begin_local()
        self._deferred = None               # the batched path is written for the FP8 state; go one matrix at a time

    def _momentum(self, param, grad, state, group, key, out=None):
        buffer = state.get("momentum_buffer")
        if buffer is None:
            buffer = state["momentum_buffer"] = torch.zeros_like(param, dtype=self.momentum_dtype)
        shape = tuple(param.shape) if group["batched"] else (param.shape[0], param.numel() // param.shape[0])
        if out is None:
            work = self._workspace.get(param.device)
            if work is None or work.numel() < param.numel():
                work = self._workspace[param.device] = torch.empty(param.numel(), device=param.device,
                                                                   dtype=torch.bfloat16)
            out = work[:param.numel()].view(shape)
        ops.momentum16(grad, buffer, out.view(-1), group["momentum"], group["nesterov"])
        return out
