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
    def __init__(self, store, optimizer, *, decay=0, dtype=torch.float32, shard=True):
        if not 0 <= decay < 1:
            raise ValueError("ema decay must be in [0, 1)")
        self.store, self.optimizer = store, optimizer
        self.decay, self.dtype, self.shard = decay, dtype, shard
        self.updates = 0
        self.weights = {}
        if not decay:
            return
        self.optimizer.materialize()
        for record in store.records:
            source = self._source(record)
            if source is not None:
                self.weights[record.name] = source.to(dtype=dtype, copy=True)
        self.optimizer.release()

    def _source(self, record):
        if not self.shard:
            return self.optimizer.full_value(record)
        if record.owner == self.store.rank:
            return self.optimizer.parameters[record.index].detach()
        return None

    @torch.no_grad()
    def update(self):
        if not self.decay:
            return
        pairs = []
        for record in self.store.records:
            source = self._source(record)
            if source is not None:
                pairs.append((self.weights[record.name], source))
        if pairs and pairs[0][0].is_cuda and all(a.is_contiguous() and b.is_contiguous() for a, b in pairs):
            # one launch for every average (the sources are the optimizer's master parameters)
            rows = [(ema, source, None, None, ema.numel(), 0, 0.0, 0.0, ops._DT[ema.dtype], ops._DT[source.dtype])
                    for ema, source in pairs]
            if getattr(self, "_table", None) is None or not self._table.matches(rows):
                self._table = ops.TensorTable(rows, pairs[0][0].device)
            ops.multi_ema(self._table, self.decay)
        else:
            for ema, source in pairs:
                ops.ema_lerp(ema, source, self.decay)
        self.updates += 1

    def state_dict(self):
        if not self.decay:
            return {}
        return dict(decay=self.decay, dtype=self.dtype, shard=self.shard, updates=self.updates, weights=self.weights)

    @torch.no_grad()
    def load_state_dict(self, state):
        if not self.decay:
            return
        if state["dtype"] != self.dtype or state["shard"] != self.shard:
            raise RuntimeError("checkpoint EMA dtype / placement differs from this run")
        if state["weights"].keys() != self.weights.keys():
            raise RuntimeError("checkpoint EMA covers different parameters")
        self.decay, self.updates = state["decay"], state["updates"]
        for name, average in self.weights.items():
            average.copy_(state["weights"][name])

    @torch.no_grad()
    def apply(self):
        """Write the averages into the compute weights (through the owners, like an optimizer step)."""
        self.store.begin_writes()
        for record in self.store.records:
            self.store.write(record, self.weights.get(record.name), record.owner)
        self.store.end_writes()


class ShardedEMA:
    """EMA bound to ``optimizer.step`` for DTensor parameters on a 1-D mesh; ``decay=0`` allocates nothing.

    ``parameters`` is a module or an iterable of ``(name, DTensor)``.  Replicated parameters keep a
    ``Shard(0)`` average (local row slice, no communication); sharded parameters keep their placement.
    With ``bind_optimizer`` in use the average tracks the master weights.
    """

    def __init__(self, parameters, optimizer, *, decay=0, dtype=torch.float32):
        from torch.distributed.tensor import DTensor, Replicate, Shard
        if not 0 <= decay < 1:
            raise ValueError("ema decay must be in [0, 1)")
        self.decay, self.dtype, self.updates = decay, dtype, 0
        self.weights, self._sources, self._hook = {}, {}, None
        if decay == 0:
            return
        pairs = parameters.named_parameters() if isinstance(parameters, torch.nn.Module) else parameters
        binding = getattr(optimizer, "_viola_linear_masters", None)
        masters = {id(p): master for p, master, _ in binding.pairs} if binding is not None else {}
        for name, param in pairs:
            if not param.requires_grad:
                continue
            source = masters.get(id(param), param)
            if not isinstance(source, DTensor) or source.device_mesh.ndim != 1:
                raise ValueError("ShardedEMA expects DTensor parameters on a 1-D mesh")
            placement, = source.placements
            if not isinstance(placement, (Replicate, Shard)):
                raise ValueError("parameters must be Replicate or Shard")
            if isinstance(placement, Replicate) and source.ndim:
                placement = Shard(0)
            self._sources[name] = source
            self.weights[name] = source.detach().redistribute(placements=[placement]).to(dtype=dtype, copy=True)
        self._hook = optimizer.register_step_post_hook(self._after_step)

    def _after_step(self, optimizer, args, kwargs):
        if not getattr(optimizer, "step_was_skipped", False):
            self.update()

    @torch.no_grad()
    def update(self):
        if self.decay == 0:
            return
        for name, average in self.weights.items():
            source = self._sources[name].detach().redistribute(placements=average.placements)
            local = average.to_local()
            if local.numel():
                ops.ema_lerp(local, source.to_local().to(self.dtype), self.decay)
        self.updates += 1

    def state_dict(self):
        if self.decay == 0:
            return {}
        return dict(decay=self.decay, updates=self.updates, dtype=self.dtype, weights=self.weights)

    @torch.no_grad()
    def load_state_dict(self, state):
        if self.decay == 0:
            return
        if state["dtype"] != self.dtype or state["weights"].keys() != self.weights.keys():
            raise RuntimeError("checkpoint EMA differs from this instance")
        self.decay, self.updates = state["decay"], state["updates"]
        for name, saved in state["weights"].items():
            current = self.weights[name]
            current.to_local().copy_(saved.redistribute(placements=current.placements).to_local())

    def close(self):
        if self._hook is not None:
            self._hook.remove()
            self._hook = None
