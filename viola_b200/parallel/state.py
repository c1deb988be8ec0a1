"""Composition of the four independent placements: parameters, gradients, optimizer state, EMA.

Counterpart of viola/distributed/state.py:14-75.  ``step`` = reduce gradients (and agree on which
parameters were used anywhere) -> optional all-rank non-finite skip -> attach gradients to the
owners' masters -> optimizer step -> write updated weights back to compute storage -> EMA update
-> clear.  ``state_dict`` / ``load_state_dict`` carry rank, mesh, sharding flags and parameter
metadata and refuse to load into a different layout.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..utils.trace import phase
from .config import dtype as to_dtype
from .ema import EMAState
from .gradients import GradientState
from .optimizer import OptimizerState
from .parameters import ParameterStore


class DistributedState:
    def __init__(self, model, optimizer, engine, sharder=None, transport=None):
        config = engine.config
        self.group, self.rank, self.world = engine.group, engine.rank, engine.world_size
        self.mesh_ranks = list(engine.global_ranks)
        self.sharding = {key: config["sharding"][key] for key in ("parameters", "gradients", "optimizer", "ema")}
        gradient_dtype = to_dtype(config["precision"]["gradient_dtype"])
        self.parameters = ParameterStore(model, optimizer, self.group, self.rank, self.world, self.mesh_ranks,
                                         gradient_dtype, sharder, transport)
        self.optimizer = OptimizerState(self.parameters, optimizer, config)
        communication = config["communication"]
        self.gradients = GradientState(self.parameters, gradient_dtype=gradient_dtype,
                                       communication_dtype=communication["dtype"], bucket_mb=communication["bucket_mb"],
                                       fp8_format=communication["fp8_format"],
                                       fp8_tile_size=communication["fp8_tile_size"], shard=self.sharding["gradients"],
                                       defer_reduction=(sharder is not None and transport is None) or (transport is not None and not transport.overlap),
                                       transport=transport)
        for position, record in enumerate(self.parameters.records):
            self.gradients.bind(position, record.parameter)
        if transport is not None:
            transport.finalize()
            if self.gradients.transport is not None:
                if self.gradients.shard:
                    transport.finalize_gradients()
                else:
                    transport.finalize_all_reduce()
            if self.parameters.transport is not None:
                transport.finalize_parameters()
        self.ema = EMAState(self.parameters, self.optimizer, decay=config["ema"]["decay"],
                            dtype=to_dtype(config["ema"]["dtype"]), shard=self.sharding["ema"])

    def backward(self, loss):
        self.gradients.begin_backward()
        try:
            with phase("backward"):
                loss.backward()
        finally:
            with phase("reduce"):
                self.gradients.finish_backward()

    @torch.no_grad()
    def step(self, divisor):
        with phase("reduce"):
            active = self.gradients.reduce(divisor)
        if not any(active):
            self.zero_grad()
            return False
        optimizer = self.optimizer.optimizer
        if getattr(optimizer, "skip_nonfinite", False):
            bad = (~torch.isfinite(self.gradients.accumulator).all()).to(torch.int32)
            if self.world > 1:
                dist.all_reduce(bad, op=dist.ReduceOp.MAX, group=self.group)
            if bad.item():
                optimizer.step_was_skipped = True
                self.zero_grad()
                return False
        with phase("optimizer"):
            self.optimizer.materialize()
            self.optimizer.attach_gradients(self.gradients, active)
            self.optimizer.step()
        with phase("writeback"):
            self.optimizer.writeback(active)
        with phase("ema"):
            self.ema.update()
        self.zero_grad()
        return True

    def zero_grad(self):
        self.optimizer.release()
        self.gradients.zero_grad()

    def state_dict(self):
        return dict(rank=dist.get_rank(), mesh=self.mesh_ranks, sharding=self.sharding,
                    parameters=self.parameters.metadata(), optimizer=self.optimizer.state_dict(),
                    ema=self.ema.state_dict())

    def load_state_dict(self, state):
        if (state["rank"] != dist.get_rank() or state["mesh"] != self.mesh_ranks
                or state["sharding"] != self.sharding or state["parameters"] != self.parameters.metadata()):
            raise RuntimeError("checkpoint parameter ownership / layout differs from this run")
        self.optimizer.load_state_dict(state["optimizer"])
        self.ema.load_state_dict(state["ema"])

    def close(self):
        for handle in [*self.parameters.hooks, *self.gradients.hooks]:
            handle.remove()
        if self.parameters.sharder is not None:
            self.parameters.sharder.close()
