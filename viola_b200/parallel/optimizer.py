"""Where the optimizer's master weights live and how an update travels back to the compute weights.

The engine hands a stock ``torch.optim.Optimizer`` full-matrix masters: for every parameter record this
rank is responsible for (its owned records when ``sharding.optimizer`` is on, all of them otherwise)
a :class:`MasterSlot` holds one ``nn.Parameter`` in the master dtype.  FP8 layers seed it from their
real-valued initial weight (or from the decoded codes when that was dropped), everything else from
the gathered parameter.  The optimizer's groups are rewritten to those masters and annotated with the
records' stable indices, so Philox keys of stochastic rounding do not depend on the sharding layout.

Per step: gradients of the active records are views of the gradient accumulator; after the optimizer
ran, the updated masters of *all* active records go back to compute storage in one
:meth:`ParameterStore.write_many` call, which on a GPU is two kernel launches per owner (EMA included).

Behavioural contract (viola/distributed/optimizer.py:12-136): the optimizer must be unused and unbound;
write-back always has a single source rank per record, also with replicated state; records no rank
used keep weight, state and step count; checkpoints refuse another precision.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .config import dtype as to_dtype
from .parameters import broadcast_tensor


@dataclass
class MasterSlot:
    record: object
    master: torch.nn.Parameter
    aliased: bool            # the master *is* the model parameter (no separate copy to save or write back)
    transient: bool          # storage exists only during an update (no masters + sharded storage)


def _real_weight(store, record):
    """Real-valued full weight of ``record`` for seeding a master; collective when storage is sharded."""
    layer = record.layer
    if layer is not None and layer.weight_dtype == "fp8":
        if layer._initial_weight is not None:
            return layer._initial_weight
        from .. import ops
        codes = store.full(record)
        if layer._grouped_scaling:
            return ops.group_dequantize(codes, layer._scale_float(), layer.weight_group_shape)
        weight = codes.float() * layer.weight_scale
        return ops.hadamard64(weight) if layer.rotation_size else weight
    return store.full(record) if record.unit is not None else None


class OptimizerState:
    def __init__(self, store, optimizer, config):
        if optimizer.state or hasattr(optimizer, "_viola_linear_masters"):
            raise RuntimeError("prepare an unused, unbound optimizer: the engine owns master-weight binding")
        precision = config["precision"]
        self.store, self.optimizer = store, optimizer
        self.shard = bool(config["sharding"]["optimizer"])
        self.master_dtype = to_dtype(precision["master_weight_dtype"])
        self.gradient_dtype = to_dtype(precision["gradient_dtype"])
        self.precision = precision
        self._fingerprint = {**precision, "master_weight_dtype": self.master_dtype,
                             "gradient_dtype": self.gradient_dtype}
        self.slots = {}
        for record in store.records:
            needs_master = record.layer is not None and record.layer.weight_dtype == "fp8"
            if needs_master and self.master_dtype is None:
                raise RuntimeError("FP8 weight storage needs floating-point master weights")
            seed = _real_weight(store, record)           # every rank takes part in the gathers
            if self.shard and record.owner != store.rank:
                continue
            self.slots[record.index] = self._make_slot(record, seed)
        self.records = [slot.record for slot in self.slots.values()]
        self.parameters = {index: slot.master for index, slot in self.slots.items()}
        self._rewrite_groups()
        self.release()
        store.release_initializers()

    def _make_slot(self, record, seed):
        wanted = self.master_dtype or record.dtype
        in_place = seed is None and record.unit is None and wanted == record.dtype
        if in_place:
            master = record.parameter
        else:
            source = seed if seed is not None else record.parameter.detach()
            master = torch.nn.Parameter(source.to(dtype=wanted, copy=True).view(record.shape))
        master.grad_dtype = self.gradient_dtype
        return MasterSlot(record, master, aliased=in_place,
                          transient=self.master_dtype is None and record.unit is not None)

    def _rewrite_groups(self):
        by_parameter = self.store.by_parameter
        for group in self.optimizer.param_groups:
            kept = [by_parameter[p].index for p in group["params"]
                    if p in by_parameter and by_parameter[p].index in self.slots]
            group["params"] = [self.slots[index].master for index in kept]
            group["viola_parameter_indices"] = kept
            group["master_rounding"] = self.precision["master_rounding"]
            group["master_rounding_seed"] = self.precision["master_rounding_seed"]
        if hasattr(self.optimizer, "_partition"):
            self.optimizer._partition = None

    # ------------------------------------------------------------------ one update
    @torch.no_grad()
    def materialize(self):
        """Masters disabled + sharded storage: gather the live weights for the duration of this update."""
        if self.master_dtype is not None:
            return
        for record in self.store.records:
            if record.unit is None:
                continue
            value = self.store.full(record)
            slot = self.slots.get(record.index)
            if slot is not None:
                master = slot.master
                master.untyped_storage().resize_(master.numel() * master.element_size())
                master.copy_(value.view(record.shape))

    @torch.no_grad()
    def attach_gradients(self, gradients, active):
        """Point every active master's ``.grad`` at its slice of the accumulator (owner -> all ranks first when
        gradients are sharded but optimizer state is not)."""
        spread = gradients.shard and not self.shard
        for position, record in enumerate(self.store.records):
            if not active[position]:
                continue
            value = gradients.local.get(position)
            if spread:
                if value is None:
                    value = torch.empty(record.numel, device=record.parameter.device, dtype=self.gradient_dtype)
                broadcast_tensor(value, self.store.global_ranks[record.owner], self.store.group)
            slot = self.slots.get(record.index)
            if slot is not None:
                slot.master.grad = value.view(record.shape)

    @torch.no_grad()
    def step(self):
        from ..optim.master_weights import MixedAdamW
        adapter = MixedAdamW(self.optimizer, rounding=self.precision["master_rounding"],
                             seed=self.precision["master_rounding_seed"])
        adapter.run()
        self.optimizer.step()
        adapter.restore_gradients()

    @torch.no_grad()
    def writeback(self, active, *, averages=None, decay=0.0):
        """Send the updated masters of the active records to compute storage; returns True when the EMA lerp of
        ``averages`` was folded into the same kernels (the caller then skips its own EMA update)."""
        records = [record for record, used in zip(self.store.records, active) if used]
        values = {index: slot.master.detach() for index, slot in self.slots.items()}
        return self.store.write_many(records, values, averages=averages, decay=decay, purpose="step")

    @torch.no_grad()
    def full_value(self, record):
        """The master of ``record`` on every rank (owner -> all when optimizer state is sharded)."""
        slot = self.slots.get(record.index)
        if not self.shard:
            return slot.master.detach()
        value = slot.master.detach() if slot is not None else torch.empty(
            record.shape, device=record.parameter.device, dtype=self.master_dtype or record.dtype)
        broadcast_tensor(value, self.store.global_ranks[record.owner], self.store.group)
        return value

    @torch.no_grad()
    def release(self):
        self.optimizer.zero_grad(set_to_none=True)
        for slot in self.slots.values():
            if slot.transient:
                slot.master.untyped_storage().resize_(0)

    # ------------------------------------------------------------------ checkpoints
    def state_dict(self):
        masters = {slot.record.name: slot.master.detach() for slot in self.slots.values()
                   if not slot.transient and not slot.aliased}
        return {"optimizer": self.optimizer.state_dict(), "precision": self._fingerprint, "masters": masters}

    @torch.no_grad()
    def load_state_dict(self, saved):
        if saved["precision"] != self._fingerprint:
            raise RuntimeError("checkpoint master / gradient precision differs from this run")
        self.optimizer.load_state_dict(saved["optimizer"])
        stored = saved["masters"]
        for slot in self.slots.values():
            if slot.record.name in stored:
                slot.master.copy_(stored[slot.record.name])
        self.release()
