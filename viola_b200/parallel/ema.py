"""Exponential moving averages of the master weights.

``EMAState`` is the engine's EMA (owner-local when ``sharding.ema`` is on, a full replica per rank
otherwise; viola/distributed/ema.py:78-132).  ``ShardedEMA`` is the standalone variant for DTensor
parameters that hooks itself onto ``optimizer.step`` (viola/distributed/ema.py:7-75).  The update is
the fused ``ema <- decay * ema + (1 - decay) * master`` kernel on CUDA.
"""

from __future__ import annotations

import torch

from .. import ops


class EMAState:
    """The engine's running average of the master weights.

    Placement: with ``shard`` each rank averages the records it owns (no communication at all); without it
    every rank averages every record and receives the owners' masters each step.  ``update`` is one
    multi-tensor launch; when the step's write-back already folded the lerp into its kernels the engine calls
    :meth:`mark_updated` instead.  ``apply`` pushes the averages into the compute weights through the same
    owner write-back an optimizer step uses, so FP8 codes and scales are identical on all ranks.
    """

    def __init__(self, store, optimizer, *, decay=0, dtype=torch.float32, shard=True):
        if not 0 <= decay < 1:
            raise ValueError("ema decay must be in [0, 1)")
        self.store, self.optimizer = store, optimizer
        self.decay, self.dtype, self.shard = decay, dtype, shard
        self.updates = 0
        self.weights = {}
        self._table = None
        if decay:
            optimizer.materialize()
            for record, master in self._tracked():
                self.weights[record.name] = master.to(dtype=dtype, copy=True)
            optimizer.release()

    def _tracked(self):
        """(record, current master) for every record this rank averages; communicates when replicated."""
        for record in self.store.records:
            if not self.shard:
                yield record, self.optimizer.full_value(record)
            elif record.owner == self.store.rank:
                yield record, self.optimizer.parameters[record.index].detach()

    @property
    def fusable(self):
        """The averages sit beside the owners' masters, so the write-back kernels can update them in passing."""
        return bool(self.decay) and self.shard

    def mark_updated(self):
        self.updates += 1

    @torch.no_grad()
    def update(self):
        if not self.decay:
            return
        pairs = [(self.weights[record.name], master) for record, master in self._tracked()]
        on_gpu = bool(pairs) and pairs[0][0].is_cuda and all(a.is_contiguous() and m.is_contiguous() for a, m in pairs)
        if on_gpu:
            rows = [(average, master, None, None, average.numel(), 0, 0.0, 0.0, ops._DT[average.dtype], ops._DT[master.dtype])
                    for average, master in pairs]
            if self._table is None or not self._table.matches(rows):
                self._table = ops.TensorTable(rows, pairs[0][0].device)
            ops.multi_ema(self._table, self.decay)
        else:
            for average, master in pairs:
                ops.ema_lerp(average, master, self.decay)
        self.updates += 1

    @torch.no_grad()
    def apply(self):
        """Overwrite the compute weights with the averages (used inside ``ema_scope``)."""
        values = {record.index: self.weights[record.name] for record in self.store.records
                  if record.name in self.weights}
        self.store.write_many(list(self.store.records), values, purpose="ema")

    def state_dict(self):
        if not self.decay:
            return {}
        return {"decay": self.decay, "dtype": self.dtype, "shard": self.shard, "updates": self.updates,
                "weights": self.weights}

    @torch.no_grad()
    def load_state_dict(self, state):
        if not self.decay:
            return
        if (state["dtype"], state["shard"]) != (self.dtype, self.shard):
            raise RuntimeError("checkpoint EMA dtype / placement differs from this run")
        if set(state["weights"]) != set(self.weights):
            raise RuntimeError("checkpoint EMA covers different parameters")
        self.decay, self.updates = state["decay"], state["updates"]
        for name, saved in state["weights"].items():
            self.weights[name].copy_(saved)


def _average_placement(source):
    """Where the average of a DTensor lives: row-sharded for replicated tensors with rows, else as the source."""
    from torch.distributed.tensor import Replicate, Shard
    (placement,) = source.placements
    if isinstance(placement, Replicate):
        return Shard(0) if source.ndim else placement
    if isinstance(placement, Shard):
        return placement
    raise ValueError("parameters must be Replicate or Shard")


class ShardedEMA:
    """Stand-alone EMA for DTensor parameters on a 1-D mesh, updated from an ``optimizer.step`` post-hook.

    ``parameters``: a module or ``(name, DTensor)`` pairs.  A replicated parameter's average is kept as its
    local row slice (``Shard(0)``), so the state is one copy across the mesh and the update needs no
    communication; sharded parameters keep their placement.  After ``bind_optimizer`` the average follows the
    master weights.  ``decay=0`` allocates nothing and installs no hook.  Steps the optimizer skipped
    (``step_was_skipped``) do not advance the average.  (viola/distributed/ema.py:7-75)
    """

    def __init__(self, parameters, optimizer, *, decay=0, dtype=torch.float32):
        from torch.distributed.tensor import DTensor
        if not 0 <= decay < 1:
            raise ValueError("ema decay must be in [0, 1)")
        self.decay, self.dtype, self.updates = decay, dtype, 0
        self.weights, self._sources, self._hook = {}, {}, None
        if not decay:
            return
        named = parameters.named_parameters() if isinstance(parameters, torch.nn.Module) else parameters
        binding = getattr(optimizer, "_viola_linear_masters", None)
        master_of = {id(b.parameter): b.master for b in binding.bindings} if binding is not None else {}
        for name, parameter in named:
            if not parameter.requires_grad:
                continue
            source = master_of.get(id(parameter), parameter)
            if not isinstance(source, DTensor) or source.device_mesh.ndim != 1:
                raise ValueError("ShardedEMA expects DTensor parameters on a 1-D mesh")
            placement = _average_placement(source)
            self._sources[name] = source
            self.weights[name] = source.detach().redistribute(placements=[placement]).to(dtype=dtype, copy=True)
        self._hook = optimizer.register_step_post_hook(
            lambda opt, args, kwargs: None if getattr(opt, "step_was_skipped", False) else self.update())

    @torch.no_grad()
    def update(self):
        if not self.decay:
            return
        for name, average in self.weights.items():
            local = average.to_local()
            if local.numel():
                fresh = self._sources[name].detach().redistribute(placements=average.placements).to_local()
                ops.ema_lerp(local, fresh.to(self.dtype), self.decay)
        self.updates += 1

    def state_dict(self):
        if not self.decay:
            return {}
        return {"decay": self.decay, "updates": self.updates, "dtype": self.dtype, "weights": self.weights}

    @torch.no_grad()
    def load_state_dict(self, state):
        if not self.decay:
            return
        if state["dtype"] != self.dtype or set(state["weights"]) != set(self.weights):
            raise RuntimeError("checkpoint EMA differs from this instance")
        self.decay, self.updates = state["decay"], state["updates"]
        for name, average in self.weights.items():
            incoming = state["weights"][name].redistribute(placements=average.placements)
            average.to_local().copy_(incoming.to_local())

    def close(self):
        if self._hook is not None:
            self._hook.remove()
            self._hook = None
