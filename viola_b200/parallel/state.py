"""The engine's distributed state: four independently placed stores and the step that ties them together.

``ParameterStore`` (compute weights, replicated or row-sharded), ``GradientState`` (accumulator,
replicated or reduced to per-tensor owners), ``OptimizerState`` (full-matrix masters, owner-local or
replicated) and ``EMAState`` are built from the four ``sharding.*`` switches, which do not constrain each
other (viola/distributed/state.py:14-75 composes the same four).

One optimizer step runs these stages; on a GPU with the peer-memory transport none of them waits on the
host, so the host enqueues the whole tail while the GPU is still in backward:

1. *agree*: finish gradient reduction and learn which records produced a gradient on any rank; the same
   exchange carries every rank's kernel status word, and a recorded failure raises on all ranks together;
2. *guard* (``skip_nonfinite`` optimizers only): all ranks agree to skip a step with Inf / NaN gradients;
3. *update*: gradients become the masters' ``.grad`` and the optimizer steps;
4. *publish*: owners write the new weights into compute storage everywhere and, in the same kernels,
   advance the EMA; otherwise the EMA is advanced by its own launch;
5. gradients and transient storage are cleared.

``state_dict`` / ``load_state_dict`` carry rank, mesh, sharding flags and per-record metadata and refuse to
load into another layout.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..utils.trace import phase
from .config import dtype as to_dtype
from .ema import EMAState
from .gradients import GradientState
from .optimizer import OptimizerState
from .parameters import ParameterStore

_SHARDING_KEYS = ("parameters", "gradients", "optimizer", "ema")


class DistributedState:
    def __init__(self, model, optimizer, engine, sharder=None, transport=None):
        config = engine.config
        self.group, self.rank, self.world = engine.group, engine.rank, engine.world_size
        self.mesh_ranks = list(engine.global_ranks)
        self.sharding = {key: config["sharding"][key] for key in _SHARDING_KEYS}
        self.transport = transport
        self.monitor = ops.StatusMonitor(engine.device)
        gradient_dtype = to_dtype(config["precision"]["gradient_dtype"])
        wire = config["communication"]
        self.parameters = ParameterStore(model, optimizer, self.group, self.rank, self.world, self.mesh_ranks,
                                         gradient_dtype, sharder, transport)
        self.optimizer = OptimizerState(self.parameters, optimizer, config)
        # With a sharder that gathers through collectives, reducing inside backward would interleave two
        # collective sequences that ranks may enter in different orders, so reduction waits for the end of
        # backward; one-sided peer kernels have no such order and may run as gradients arrive.
        after_backward = (sharder is not None and transport is None) or (transport is not None and not transport.overlap)
        self.gradients = GradientState(self.parameters, gradient_dtype=gradient_dtype, communication_dtype=wire["dtype"],
                                       bucket_mb=wire["bucket_mb"], fp8_format=wire["fp8_format"],
                                       fp8_tile_size=wire["fp8_tile_size"], shard=self.sharding["gradients"],
                                       defer_reduction=after_backward, transport=transport, monitor=self.monitor,
                                       landing=wire.get("gradient_slots", True),
                                       reduce_once=wire.get("reduce_once", True)
                                       and not (transport is not None and transport.overlap))
        for position, record in enumerate(self.parameters.records):
            self.gradients.bind(position, record.parameter)
        if transport is not None:
            self._lay_out_heap(transport)
        self.ema = EMAState(self.parameters, self.optimizer, decay=config["ema"]["decay"],
                            dtype=to_dtype(config["ema"]["dtype"]), shard=self.sharding["ema"])

    def _lay_out_heap(self, transport):
        """All users have filed their requests: allocate the symmetric heap and hand out offsets and flags."""
        transport.attach_usage(len(self.parameters.records))
        transport.finalize()
        transport.finalize_usage()
        if self.gradients.transport is not None:
            if self.gradients.shard:
                transport.finalize_gradients()
            else:
                transport.finalize_all_reduce()
        if self.parameters.transport is not None:
            transport.finalize_parameters()

    # ------------------------------------------------------------------ microbatch
    def backward(self, loss):
        self.gradients.begin_backward()
        try:
            with phase("backward"):
                loss.backward()
        finally:
            with phase("reduce"):
                self.gradients.finish_backward()

    # ------------------------------------------------------------------ optimizer step
    def _nonfinite_everywhere(self):
        flag = torch.isfinite(self.gradients.accumulator).all().logical_not().to(torch.int32)
        if self.world > 1:
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.group)
        return bool(flag.item())

    @torch.no_grad()
    def step(self, divisor):
        # A status code recorded since the last step travels with the usage agreement inside reduce(), so
        # that with several ranks all of them raise in the same step instead of one leaving the others
        # inside a collective.
        with phase("reduce"):
            active = self.gradients.reduce(divisor)
        updated = any(active)
        inner = self.optimizer.optimizer
        if updated and getattr(inner, "skip_nonfinite", False) and self._nonfinite_everywhere():
            inner.step_was_skipped = True
            updated = False
        if updated:
            with phase("optimizer"):
                self.optimizer.materialize()
                self.optimizer.attach_gradients(self.gradients, active)
                self.optimizer.step()
            fuse_ema = self.ema.fusable and all(active)
            with phase("writeback"):
                folded = self.optimizer.writeback(active, averages=self.ema.weights if fuse_ema else None,
                                                  decay=self.ema.decay if fuse_ema else 0.0)
            with phase("ema"):
                if folded:
                    self.ema.mark_updated()
                else:
                    self.ema.update()
        self.zero_grad()
        self.monitor.snapshot()
        return updated

    def zero_grad(self):
        self.optimizer.release()
        self.gradients.zero_grad()

    def check_status(self):
        """Synchronising check of this rank's kernel status word (before anything durable is written)."""
        self.monitor.check()

    # ------------------------------------------------------------------ checkpoints
    def _identity(self):
        return {"rank": dist.get_rank(), "mesh": self.mesh_ranks, "sharding": self.sharding,
                "parameters": self.parameters.metadata()}

    def state_dict(self):
        return {**self._identity(), "optimizer": self.optimizer.state_dict(), "ema": self.ema.state_dict()}

    def load_state_dict(self, state):
        mine = self._identity()
        if any(state[key] != value for key, value in mine.items()):
            raise RuntimeError("checkpoint parameter ownership / layout differs from this run")
        self.optimizer.load_state_dict(state["optimizer"])
        self.ema.load_state_dict(state["ema"])

    def close(self):
        for handle in (*self.parameters.hooks, *self.gradients.hooks):
            handle.remove()
        if self.parameters.sharder is not None:
            self.parameters.sharder.close()
        self.monitor.check()
