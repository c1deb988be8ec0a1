"""Master-weight binding between a model and any ``torch.optim.Optimizer``.

``bind_optimizer(model, optimizer)`` swaps every optimizer parameter for a master parameter in the
policy's master dtype (or keeps the model parameter itself when masters are disabled), aliases the
model-side gradient onto the master before each step, and after each step re-derives the compute
weight: FP8 layers re-quantise from the master (``Linear.refresh_weight``), other parameters receive
a cast copy.  The optimizer's ``state_dict`` gains a ``viola_masters`` entry so that model + optimizer
checkpoints resume exactly.  Semantics follow viola/optim/master_weights.py:13-179.
"""

from __future__ import annotations

import weakref

import torch
from torch import nn

from .. import ops
from ..nn import Linear
from ..precision import settings
from .matrix import MatrixOptimizer


@torch.no_grad()
def step_mixed_adamw(optimizer, precision):
    """Run stock ``torch.optim.AdamW`` entries whose gradient dtype differs from the weight dtype (or
    that use stochastic master rounding) through the fused Adam kernel; returns the (parameter,
    gradient) pairs whose ``.grad`` was detached so the native step skips them."""
    handled = []
    rounding = precision["master_rounding"]
    for group in optimizer.param_groups:
        for parameter in group["params"]:
            gradient = parameter.grad
            if gradient is None:
                continue
            mixed = gradient.dtype != parameter.dtype or rounding != "nearest"
            if mixed and type(optimizer) is torch.optim.AdamW:
                if any(group.get(flag, False) for flag in ("amsgrad", "capturable", "differentiable", "fused")):
                    raise RuntimeError("mixed-precision AdamW supports the plain (non-amsgrad, non-fused) variant")
                state = optimizer.state[parameter]
                if not state:
                    state.update(step=torch.tensor(0.0), exp_avg=torch.zeros_like(parameter),
                                 exp_avg_sq=torch.zeros_like(parameter))
                state["step"] += 1
                ops.adam_update(parameter, gradient, state["exp_avg"], state["exp_avg_sq"], lr=group["lr"],
                                weight_decay=group["weight_decay"], betas=group["betas"], eps=group["eps"],
                                step=int(state["step"]), rounding=rounding, key=precision["master_rounding_seed"],
                                maximize=group.get("maximize", False))
                handled.append((parameter, gradient))
                parameter.grad = None
            elif mixed and type(optimizer) is torch.optim.SGD:
                if rounding != "nearest":
                    raise RuntimeError("stochastic master rounding is not available for SGD")
                group["foreach"] = False
    return handled


class _MasterWeights:
    def __init__(self, model, optimizer):
        if optimizer.state:
            raise RuntimeError("bind the optimizer before its first step or load_state_dict")
        policy = settings()
        self.master_dtype = policy["master_weight_dtype"]
        self.gradient_dtype = policy["gradient_dtype"] or torch.float32
        self.rounding, self.seed = policy["master_rounding"], policy["master_rounding_seed"]
        self.optimizer = optimizer
        self.pairs, self.active = [], []
        layers = {id(m.weight): m for m in model.modules() if isinstance(m, Linear)}
        masters = {}
        for group in optimizer.param_groups:
            if isinstance(optimizer, MatrixOptimizer):
                group["master_rounding"], group["master_rounding_seed"] = self.rounding, self.seed
            replaced = []
            for param in group["params"]:
                param.grad_dtype = self.gradient_dtype
                if id(param) not in masters:
                    masters[id(param)] = self._make_master(param, layers.get(id(param)))
                replaced.append(masters[id(param)])
            group["params"] = replaced
        if isinstance(optimizer, MatrixOptimizer):
            optimizer._partition = None
        optimizer.register_step_pre_hook(self._before_step)
        optimizer.register_step_post_hook(self._after_step)
        optimizer.register_state_dict_post_hook(self._save)
        optimizer.register_load_state_dict_pre_hook(self._load)
        optimizer.register_load_state_dict_post_hook(self._after_load)
        self._wrap_zero_grad(optimizer)

    def _make_master(self, param, layer):
        if layer is not None and layer.weight_dtype == "fp8":
            if self.master_dtype is None:
                raise RuntimeError("disabling the master needs BF16 / FP16 / FP32 weight storage")
            initial = layer._initial_weight
            if initial is None:      # model-only checkpoint: a full resume overwrites this from the optimizer state
                initial = layer.dequantize_weight()
            master = nn.Parameter(initial.detach().to(self.master_dtype), requires_grad=param.requires_grad)
        elif self.master_dtype is not None and param.dtype != self.master_dtype:
            master = nn.Parameter(param.detach().to(self.master_dtype), requires_grad=param.requires_grad)
        else:
            master = param
        if layer is not None:
            layer._initial_weight = None
            layer._master_ref = weakref.ref(master)
        master.grad_dtype = self.gradient_dtype
        self.pairs.append((param, master, layer))
        return master

    def _wrap_zero_grad(self, optimizer):
        inner = optimizer.zero_grad

        def zero_grad(set_to_none=True):
            inner(set_to_none=set_to_none)
            for param, master, _ in self.pairs:
                if param is master or param.grad is None:
                    continue
                if set_to_none:
                    param.grad = None
                else:
                    param.grad.detach_()
                    param.grad.zero_()

        optimizer.zero_grad = zero_grad

    @torch.no_grad()
    def _before_step(self, optimizer, args, kwargs):
        # torch passes (optimizer, *step_args) here
        if any(value is not None for value in args[1:]) or kwargs.get("closure") is not None:
            raise RuntimeError("master binding needs explicit forward/backward; optimizer closures are not supported")
        self.active = []
        for param, master, layer in self.pairs:
            if param.grad is not None:
                master.grad = param.grad        # alias: no second gradient buffer
                self.active.append((param, master, layer, param.grad))
        step_mixed_adamw(optimizer, dict(master_rounding=self.rounding, master_rounding_seed=self.seed))

    @torch.no_grad()
    def _after_step(self, optimizer, args, kwargs):
        skipped = isinstance(optimizer, MatrixOptimizer) and optimizer.step_was_skipped
        for param, master, layer, gradient in self.active:
            if not skipped and layer is not None:
                layer.refresh_weight(master)
            elif not skipped and param is not master:
                param.copy_(master)
            if param is not master:
                master.grad = None
            else:
                param.grad = gradient
        self.active.clear()

    def _save(self, optimizer, state):
        state["viola_masters"] = {
            "weights": [master.detach() if master is not param else None for param, master, _ in self.pairs],
            "gradient_dtype": self.gradient_dtype,
            "master_dtype": self.master_dtype,
            "rounding": self.rounding,
            "seed": self.seed,
        }

    @torch.no_grad()
    def _load(self, optimizer, state):
        state = dict(state)
        saved = state.pop("viola_masters")
        if saved["master_dtype"] != self.master_dtype or saved["gradient_dtype"] != self.gradient_dtype:
            raise RuntimeError("checkpoint master / gradient precision differs from the current policy")
        if len(saved["weights"]) != len(self.pairs):
            raise RuntimeError("checkpoint holds a different number of bound parameters")
        self.rounding, self.seed = saved["rounding"], saved["seed"]
        for (_, master, _), value in zip(self.pairs, saved["weights"]):
            if value is not None:
                master.copy_(value)
        return state

    @torch.no_grad()
    def _after_load(self, optimizer):
        # FP8 compute weights come from the model checkpoint (exact codes, scales and histories);
        # re-quantising here would advance delayed-scaling state.  Only plain copies are refreshed.
        for param, master, layer in self.pairs:
            if (layer is None or layer.weight_dtype != "fp8") and param is not master:
                param.copy_(master)
        optimizer.zero_grad()


def bind_optimizer(model, optimizer):
    """Install the master-weight hooks on ``optimizer`` (returned unchanged).

    Move the model to its device first and set the precision policy before binding.  Save and load both
    the model's and the optimizer's ``state_dict`` for an exact resume.
    """
    if hasattr(optimizer, "_viola_linear_masters"):
        raise RuntimeError("this optimizer is already bound")
    optimizer._viola_linear_masters = _MasterWeights(model, optimizer)
    return optimizer
