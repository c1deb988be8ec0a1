"""Master weights behind any ``torch.optim.Optimizer``: ``bind_optimizer(model, optimizer)``.

What binding does (contract of viola/optim/master_weights.py:13-179):

* every optimizer parameter is replaced by a *master* in the policy's master dtype (``viola_b200.precision``);
  FP8 layers seed theirs from the layer's real-valued initial weight (or from the decoded codes when a
  model-only checkpoint was loaded), parameters that already have the master dtype are used as they are;
* before a step the model-side gradient becomes the master's gradient (same tensor, no copy); closures are
  refused because forward / backward must have run on the compute weights;
* after a step FP8 layers re-quantise from their master and other parameters receive a cast copy; a step
  the optimizer skipped (``step_was_skipped``) refreshes nothing;
* ``optimizer.state_dict()`` gains ``viola_masters`` and loading it restores the masters without touching
  FP8 codes (they come from the model's own state dict, bit for bit);
* ``optimizer.zero_grad`` also clears the model-side gradients.

Stock ``torch.optim.AdamW`` cannot step a parameter whose gradient has another dtype, nor round
stochastically; :class:`MixedAdamW` runs exactly those entries through this library's Adam kernel, all
entries of a group that share a step count in one multi-tensor launch.
"""

from __future__ import annotations

import weakref
from dataclasses import dataclass

import torch
from torch import nn

from .. import ops
from ..nn import Linear
from ..precision import settings
from .matrix import MatrixOptimizer

_UNSUPPORTED_ADAMW_FLAGS = ("amsgrad", "capturable", "differentiable", "fused")


class MixedAdamW:
    """Adapter for one ``optimizer.step()``: takes over the AdamW entries torch's own loop cannot handle.

    ``run()`` updates them and hides their gradients so that the native step passes them by;
    ``restore_gradients()`` puts the gradients back afterwards.  For ``torch.optim.SGD`` with mixed dtypes the
    adapter only switches the group to the single-tensor loop, which accepts them.  Other optimizers are left alone.
    """

    def __init__(self, optimizer, *, rounding="nearest", seed=0):
        self.optimizer, self.rounding, self.seed = optimizer, rounding, seed
        self.hidden = []

    def _needs_kernel(self, parameter):
        return parameter.grad is not None and (parameter.grad.dtype != parameter.dtype or self.rounding != "nearest")

    def _state(self, parameter):
        state = self.optimizer.state[parameter]
        if not state:
            state["step"] = torch.tensor(0.0)
            state["exp_avg"] = torch.zeros_like(parameter)
            state["exp_avg_sq"] = torch.zeros_like(parameter)
        return state

    def _launch(self, group, entries, step):
        """One update for ``entries`` (all at optimizer step ``step``): a single table-driven launch on a GPU."""
        options = dict(lr=group["lr"], weight_decay=group["weight_decay"], betas=group["betas"], eps=group["eps"],
                       step=step, rounding=self.rounding, maximize=group.get("maximize", False))
        batched = all(p.is_cuda and p.is_contiguous() and p.dtype in ops._DT and p.grad.dtype in ops._DT
                      for p, _ in entries)
        if not batched:
            for parameter, state in entries:
                ops.adam_update(parameter, parameter.grad, state["exp_avg"], state["exp_avg_sq"], key=self.seed,
                                **options)
            return
        codes = ops._DT
        rows = []
        for parameter, state in entries:
            gradient = parameter.grad if parameter.grad.is_contiguous() else parameter.grad.contiguous()
            rows.append((parameter, gradient, state["exp_avg"], state["exp_avg_sq"], parameter.numel(), self.seed, 0.0,
                         0.0, codes[parameter.dtype], codes[gradient.dtype] | (codes[state["exp_avg"].dtype] << 8)))
        cache = self.optimizer.__dict__.setdefault("_viola_adam_tables", {})
        key = (id(group), len(rows))
        table = cache.get(key)
        if table is None or not table.matches(rows):
            table = cache[key] = ops.TensorTable(rows, entries[0][0].device)
        ops.multi_adam(table, **options)

    @torch.no_grad()
    def run(self):
        kind = type(self.optimizer)
        for group in self.optimizer.param_groups:
            selected = [p for p in group["params"] if self._needs_kernel(p)]
            if not selected:
                continue
            if kind is torch.optim.SGD:
                if self.rounding != "nearest":
                    raise RuntimeError("stochastic master rounding is not available for SGD")
                group["foreach"] = False
                continue
            if kind is not torch.optim.AdamW:
                continue
            if any(group.get(flag, False) for flag in _UNSUPPORTED_ADAMW_FLAGS):
                raise RuntimeError("mixed-precision AdamW supports the plain (non-amsgrad, non-fused) variant")
            by_step = {}
            for parameter in selected:
                state = self._state(parameter)
                state["step"] += 1
                by_step.setdefault(int(state["step"]), []).append((parameter, state))
            for step, entries in by_step.items():
                self._launch(group, entries, step)
            for parameter in selected:
                self.hidden.append((parameter, parameter.grad))
                parameter.grad = None
        return self.hidden

    def restore_gradients(self):
        for parameter, gradient in self.hidden:
            parameter.grad = gradient
        self.hidden = []


@dataclass
class Binding:
    parameter: nn.Parameter      # what the model computes with
    master: nn.Parameter         # what the optimizer updates (may be the same object)
    layer: Linear | None

    @property
    def separate(self):
        return self.master is not self.parameter


class _MasterWeights:
    """The hook set installed by :func:`bind_optimizer`; one instance per optimizer."""

    def __init__(self, model, optimizer):
        if optimizer.state:
            raise RuntimeError("bind the optimizer before its first step or load_state_dict")
        policy = settings()
        self.optimizer = optimizer
        self.master_dtype = policy["master_weight_dtype"]
        self.gradient_dtype = policy["gradient_dtype"] or torch.float32
        self.rounding, self.seed = policy["master_rounding"], policy["master_rounding_seed"]
        self.bindings = []
        self._stepping = []                     # (binding, gradient) of the step in flight
        owner_layer = {id(module.weight): module for module in model.modules() if isinstance(module, Linear)}
        known = {}
        matrix_optimizer = isinstance(optimizer, MatrixOptimizer)
        for group in optimizer.param_groups:
            if matrix_optimizer:
                group["master_rounding"], group["master_rounding_seed"] = self.rounding, self.seed
            masters = []
            for parameter in group["params"]:
                parameter.grad_dtype = self.gradient_dtype
                binding = known.get(id(parameter))
                if binding is None:
                    binding = known[id(parameter)] = self._bind(parameter, owner_layer.get(id(parameter)))
                masters.append(binding.master)
            group["params"] = masters
        if matrix_optimizer:
            optimizer._partition = None
        self._install(optimizer)

    # ------------------------------------------------------------------ construction
    def _bind(self, parameter, layer):
        fp8_layer = layer is not None and layer.weight_dtype == "fp8"
        if fp8_layer and self.master_dtype is None:
            raise RuntimeError("disabling the master needs BF16 / FP16 / FP32 weight storage")
        if fp8_layer:
            # without an initial weight (model-only checkpoint) start from the decoded codes; a full resume
            # overwrites this from the optimizer state
            seed = layer._initial_weight if layer._initial_weight is not None else layer.dequantize_weight()
            master = nn.Parameter(seed.detach().to(self.master_dtype), requires_grad=parameter.requires_grad)
        elif self.master_dtype is None or parameter.dtype == self.master_dtype:
            master = parameter
        else:
            master = nn.Parameter(parameter.detach().to(self.master_dtype), requires_grad=parameter.requires_grad)
        master.grad_dtype = self.gradient_dtype
        if layer is not None:
            layer._initial_weight = None
            layer._master_ref = weakref.ref(master)
        binding = Binding(parameter, master, layer)
        self.bindings.append(binding)
        return binding

    def _install(self, optimizer):
        optimizer.register_step_pre_hook(self._before_step)
        optimizer.register_step_post_hook(self._after_step)
        optimizer.register_state_dict_post_hook(self._add_masters)
        optimizer.register_load_state_dict_pre_hook(self._take_masters)
        optimizer.register_load_state_dict_post_hook(self._after_load)
        clear_masters = optimizer.zero_grad

        def zero_grad(set_to_none=True):
            clear_masters(set_to_none=set_to_none)
            for binding in self.bindings:
                gradient = binding.parameter.grad
                if not binding.separate or gradient is None:
                    continue
                if set_to_none:
                    binding.parameter.grad = None
                else:
                    gradient.detach_()
                    gradient.zero_()

        optimizer.zero_grad = zero_grad

    # ------------------------------------------------------------------ step hooks
    @torch.no_grad()
    def _before_step(self, optimizer, args, kwargs):
        closure = kwargs.get("closure")
        if closure is None:
            closure = next((value for value in args[1:] if value is not None), None)     # args[0] is the optimizer
        if closure is not None:
            raise RuntimeError("master binding needs explicit forward/backward; optimizer closures are not supported")
        self._stepping = [(b, b.parameter.grad) for b in self.bindings if b.parameter.grad is not None]
        for binding, gradient in self._stepping:
            binding.master.grad = gradient                     # the same tensor: no second gradient buffer
        self._adapter = MixedAdamW(optimizer, rounding=self.rounding, seed=self.seed)
        self._adapter.run()

    @torch.no_grad()
    def _after_step(self, optimizer, args, kwargs):
        skipped = isinstance(optimizer, MatrixOptimizer) and optimizer.step_was_skipped
        for binding, gradient in self._stepping:
            if not skipped:
                if binding.layer is not None:
                    binding.layer.refresh_weight(binding.master)
                elif binding.separate:
                    binding.parameter.copy_(binding.master)
            if binding.separate:
                binding.master.grad = None
            else:
                binding.parameter.grad = gradient              # the adapter may have hidden it
        self._stepping = []
        self._adapter.hidden = []

    # ------------------------------------------------------------------ state-dict hooks
    def _add_masters(self, optimizer, state):
        state["viola_masters"] = dict(
            weights=[b.master.detach() if b.separate else None for b in self.bindings],
            gradient_dtype=self.gradient_dtype, master_dtype=self.master_dtype, rounding=self.rounding, seed=self.seed)

    @torch.no_grad()
    def _take_masters(self, optimizer, state):
        remaining = {key: value for key, value in state.items() if key != "viola_masters"}
        saved = state["viola_masters"]
        if (saved["master_dtype"], saved["gradient_dtype"]) != (self.master_dtype, self.gradient_dtype):
            raise RuntimeError("checkpoint master / gradient precision differs from the current policy")
        if len(saved["weights"]) != len(self.bindings):
            raise RuntimeError("checkpoint holds a different number of bound parameters")
        self.rounding, self.seed = saved["rounding"], saved["seed"]
        for binding, value in zip(self.bindings, saved["weights"]):
            if value is not None:
                binding.master.copy_(value)
        return remaining

    @torch.no_grad()
    def _after_load(self, optimizer):
        # FP8 compute weights are restored by the model's state dict (exact codes, scales, histories);
        # quantising again here would advance delayed-scaling state, so only plain copies are refreshed.
        for binding in self.bindings:
            fp8_layer = binding.layer is not None and binding.layer.weight_dtype == "fp8"
            if binding.separate and not fp8_layer:
                binding.parameter.copy_(binding.master)
        optimizer.zero_grad()


def bind_optimizer(model, optimizer):
    """Install the master-weight hooks on ``optimizer`` and return it.

    Order of operations for the caller: move the model to its device, set the precision policy, construct
    the optimizer, bind, train.  For an exact resume save and load both ``model.state_dict()`` and
    ``optimizer.state_dict()``.
    """
    if hasattr(optimizer, "_viola_linear_masters"):
        raise RuntimeError("this optimizer is already bound")
    optimizer._viola_linear_masters = _MasterWeights(model, optimizer)
    return optimizer
