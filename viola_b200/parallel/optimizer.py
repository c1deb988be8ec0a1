"""Optimizer placement: owner-local (or replicated) full master parameters behind a stock optimizer.

Follows the reference's ``OptimizerState`` (viola/distributed/optimizer.py:12-136): the optimizer
handed to the engine must be unused and unbound; its parameter groups are rewritten to hold, for
every record this rank is responsible for, a *full-matrix* master parameter (FP8 layers start from
their real-valued initial weight), plus ``viola_parameter_indices`` so that per-parameter Philox
keys do not depend on the sharding layout.  ``attach_gradients`` points each master's ``.grad`` at
its slice of the gradient accumulator, ``writeback`` sends updated masters through the parameter
store, ``full_value`` broadcasts a master for a replicated EMA.
"""

from __future__ import annotations

import torch

from .config import dtype as to_dtype
from .parameters import broadcast_tensor


class OptimizerState:
    def __init__(self, store, optimizer, config):
        if optimizer.state or hasattr(optimizer, "_viola_linear_masters"):
            raise RuntimeError("prepare an unused, unbound optimizer: the engine owns master-weight binding")
        self.store, self.optimizer = store, optimizer
        self.shard = config["sharding"]["optimizer"]
        self.master_dtype = to_dtype(config["precision"]["master_weight_dtype"])
        self.gradient_dtype = to_dtype(config["precision"]["gradient_dtype"])
        self.precision = config["precision"]
        self.saved_precision = dict(self.precision, master_weight_dtype=self.master_dtype,
                                    gradient_dtype=self.gradient_dtype)
        self.parameters, self.transient = {}, set()
        self.records = [r for r in store.records if not self.shard or r.owner == store.rank]
        for record in store.records:
            param, layer = record.parameter, record.layer
            mine = not self.shard or record.owner == store.rank
            sharded_storage = record.unit is not None
            full = None
            if layer is not None and layer.weight_dtype == "fp8":
                if self.master_dtype is None:
                    raise RuntimeError("FP8 weight storage needs floating-point master weights")
                full = layer._initial_weight
                if full is None:
                    codes = store.full(record)                      # collective: every rank takes part
                    scale = layer._scale_float() if layer._grouped_scaling else layer.weight_scale
                    full = _decode(layer, codes, scale)
            elif sharded_storage:
                full = store.full(record)                            # collective
            if not mine:
                continue
            target = self.master_dtype or record.dtype
            if not sharded_storage and target == record.dtype and full is None:
                master = param                                       # update the model parameter in place
            else:
                source = full if full is not None else param.detach()
                master = torch.nn.Parameter(source.to(dtype=target, copy=True).view(record.shape))
            master.grad_dtype = self.gradient_dtype
            self.parameters[record.index] = master
            if self.master_dtype is None and sharded_storage:
                self.transient.add(record.index)
        for group in optimizer.param_groups:
            records = [store.by_parameter[p] for p in group["params"] if p in store.by_parameter]
            records = [r for r in records if r.index in self.parameters]
            group["params"] = [self.parameters[r.index] for r in records]
            group["viola_parameter_indices"] = [r.index for r in records]
            group["master_rounding"] = self.precision["master_rounding"]
            group["master_rounding_seed"] = self.precision["master_rounding_seed"]
        if hasattr(optimizer, "_partition"):
            optimizer._partition = None
        self.release()
        store.release_initializers()

    @torch.no_grad()
    def materialize(self):
        """Without masters and with sharded storage, gather the live weights just for this update."""
        if self.master_dtype is not None:
            return
        for record in self.store.records:
            if record.unit is None:
                continue
            full = self.store.full(record)
            if record.index in self.parameters:
                param = self.parameters[record.index]
                param.untyped_storage().resize_(param.numel() * param.element_size())
                param.copy_(full.view(record.shape))

    @torch.no_grad()
    def attach_gradients(self, gradients, active):
        for position, record in enumerate(self.store.records):
            if not active[position]:
                continue
            value = gradients.local.get(position)
            if gradients.shard and not self.shard:
                if value is None:
                    value = torch.empty(record.numel, device=record.parameter.device, dtype=self.gradient_dtype)
                broadcast_tensor(value, self.store.global_ranks[record.owner], self.store.group)
            if record.index in self.parameters:
                self.parameters[record.index].grad = value.view(record.shape)

    @torch.no_grad()
    def step(self):
        from ..optim.master_weights import step_mixed_adamw
        handled = step_mixed_adamw(self.optimizer, self.precision)
        self.optimizer.step()
        for parameter, gradient in handled:
            parameter.grad = gradient

    @torch.no_grad()
    def writeback(self, active):
        self.store.begin_writes()
        for record, used in zip(self.store.records, active):
            if used:
                # always one source, even with replicated state: stochastic / FP8 results stay identical
                self.store.write(record, self.parameters.get(record.index), record.owner)
        self.store.end_writes()

    @torch.no_grad()
    def full_value(self, record):
        value = self.parameters.get(record.index)
        if not self.shard:
            return value.detach()
        if value is None:
            value = torch.empty(record.shape, device=record.parameter.device,
                                dtype=self.master_dtype or record.dtype)
        broadcast_tensor(value.detach(), self.store.global_ranks[record.owner], self.store.group)
        return value.detach()

    @torch.no_grad()
    def release(self):
        self.optimizer.zero_grad(set_to_none=True)
        for index in self.transient:
            self.parameters[index].untyped_storage().resize_(0)

    def state_dict(self):
        return dict(optimizer=self.optimizer.state_dict(), precision=self.saved_precision,
                    masters={r.name: self.parameters[r.index].detach() for r in self.records
                             if r.index not in self.transient and self.parameters[r.index] is not r.parameter})

    @torch.no_grad()
    def load_state_dict(self, saved):
        if saved["precision"] != self.saved_precision:
            raise RuntimeError("checkpoint master / gradient precision differs from this run")
        self.optimizer.load_state_dict(saved["optimizer"])
        for record in self.records:
            if record.name in saved["masters"]:
                self.parameters[record.index].copy_(saved["masters"][record.name])
        self.release()


def _decode(layer, codes, scale):
    """Real-valued weight from gathered FP8 codes (used when no initial master is available)."""
    from .. import ops
    if layer._grouped_scaling:
        return ops.group_dequantize(codes, scale, layer.weight_group_shape)
    weight = codes.float() * scale
    return ops.hadamard64(weight) if layer.rotation_size else weight
