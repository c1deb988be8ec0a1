"""``MatrixOptimizer``: base class for update rules that need a whole logical matrix (Muon and relatives).

A subclass writes one method, ``_step_local(parameter, gradient, state, group, index)``, which updates a
full ordinary tensor in place.  This class does the rest:

* plain tensors are handed to ``_step_local`` directly (``_begin_local`` / ``_finish_local`` bracket that
  pass so a subclass can collect same-shape matrices and run them as one batched launch);
* DTensor parameters (``Replicate`` or ``Shard`` on a 1-D mesh) have per-tensor owners
  (:class:`~viola_b200.parallel.partition.MatrixPartition`).  They are worked through in rounds of one
  tensor per owner: the gradient and the weight are assembled on the owner, updated there, and the result
  is written back into the existing layout, so every rank is busy in every round.  With
  ``shard_state=False`` every rank assembles and updates every tensor (replicated state), but the value
  that is written back still comes from the owner alone, which keeps stochastic and FP8 results bit-identical;
* ``skip_nonfinite=True`` makes all ranks agree (one flag, one reduction per mesh) to skip a step whose
  gradients contain Inf / NaN; ``step_was_skipped`` tells hooks about it;
* ``group["viola_parameter_indices"]`` (set by the engine) replaces positional indices, so Philox keys stay
  the same under any sharding layout;
* ``state_dict`` carries the ownership layout as ``viola_dtensor`` and ``load_state_dict`` refuses another
  layout and keeps every state tensor's own dtype (raw uint8 momentum, bf16 Adam moments), which the stock
  loader would cast to the parameter dtype.

Behaviour and checkpoint keys follow the reference base class (viola/optim/matrix.py:13-135).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel.partition import MatrixPartition

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = ()


def _local(tensor):
    return tensor.to_local() if isinstance(tensor, DTensor) else tensor


class MatrixOptimizer(torch.optim.Optimizer):
    def __init__(self, params, defaults, *, shard_state=True, skip_nonfinite=False):
        self.shard_state, self.skip_nonfinite = shard_state, skip_nonfinite
        self.step_was_skipped = False
        self._partition = None
        super().__init__(params, defaults)

    # ------------------------------------------------------------------ ownership
    @property
    def partition(self):
        if self._partition is None:
            self._partition = MatrixPartition(p for group in self.param_groups for p in group["params"])
        return self._partition

    def add_param_group(self, group):
        if self._partition is not None and self._partition.owners:
            raise RuntimeError("add DTensor parameter groups before the first step or checkpoint")
        super().add_param_group(group)
        self._partition = None

    # ------------------------------------------------------------------ subclass interface
    def _step_local(self, parameter, gradient, state, group, index):
        """Update one full parameter in place; ``index`` is stable across sharding layouts."""
        raise NotImplementedError

    def _begin_local(self):
        """Called before the plain-tensor parameters are visited (subclasses may start batching)."""

    def _finish_local(self):
        """Called after the plain-tensor parameters were visited, before DTensor owner rounds."""

    # ------------------------------------------------------------------ the step
    def _work_items(self):
        """(parameter, group, stable index) for every parameter that has a gradient."""
        position = 0
        for group in self.param_groups:
            stable = group.get("viola_parameter_indices")
            for slot, parameter in enumerate(group["params"]):
                index = position if stable is None else stable[slot]
                position += 1
                if parameter.grad is not None:
                    yield parameter, group, index

    def _gradients_nonfinite(self):
        """One device-side flag over all local gradients, then one MAX reduction per mesh so ranks agree."""
        flags = [torch.isfinite(_local(p.grad)).all().logical_not() for p, _, _ in self._work_items()]
        bad = torch.stack(flags).any() if flags else None
        for mesh in self.partition.meshes:
            vote = torch.zeros((), device=mesh.device_type, dtype=torch.int32)
            if bad is not None:
                vote += bad.to(device=vote.device, dtype=torch.int32)
            dist.all_reduce(vote, op=dist.ReduceOp.MAX, group=mesh.get_group())
            bad = vote.bool()
        return bool(bad) if bad is not None else False

    @torch.no_grad()
    def step(self, closure=None):
        self.step_was_skipped = False
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.skip_nonfinite and self._gradients_nonfinite():
            self.step_was_skipped = True
            return loss
        owned_elsewhere = {}
        self._begin_local()
        for parameter, group, index in self._work_items():
            if isinstance(parameter, DTensor):
                owned_elsewhere[parameter] = (group, index)
            else:
                self._step_local(parameter, parameter.grad, self.state[parameter], group, index)
        self._finish_local()
        if owned_elsewhere:
            for round_ in self.partition.batches:
                self._owner_round([p for p in round_ if p in owned_elsewhere], owned_elsewhere)
        return loss

    def _owner_round(self, parameters, contexts):
        """One tensor per owner: assemble, update on the owner(s), write back from the owner."""
        from ..parallel.communication import gather_to_owner, replicate_tensor, write_from_owner
        assembled = []
        for parameter in parameters:
            owner = self.partition.owner(parameter)
            if self.shard_state:
                weight, gradient = gather_to_owner(parameter, owner), gather_to_owner(parameter.grad, owner)
            else:
                weight, gradient = replicate_tensor(parameter), replicate_tensor(parameter.grad)
            assembled.append((parameter, owner, None if weight is None else weight.contiguous(), gradient))
        for parameter, _, weight, gradient in assembled:
            if weight is not None:
                group, index = contexts[parameter]
                self._step_local(weight, gradient.contiguous(), self.state[parameter], group, index)
        for parameter, owner, weight, _ in assembled:
            write_from_owner(parameter, weight, owner)

    # ------------------------------------------------------------------ checkpoints
    def _layout(self):
        if not self.partition.owners:
            return {}
        return {"shard_state": self.shard_state, "partition": self.partition.state_dict()}

    def state_dict(self):
        state = super().state_dict()
        layout = self._layout()
        if layout:
            state["viola_dtensor"] = layout
        return state

    def load_state_dict(self, state_dict):
        if state_dict.get("viola_dtensor", {}) != self._layout():
            raise RuntimeError("matrix-optimizer checkpoint ownership / layout differs from this run")
        incoming = {key: value for key, value in state_dict.items() if key != "viola_dtensor"}
        # split the per-parameter state: scalars go through the stock loader, tensors are re-attached
        # afterwards exactly as saved (torch would cast floating tensors to the parameter dtype)
        tensors, scalars = {}, {}
        for saved_id, entries in incoming["state"].items():
            tensors[saved_id] = {k: v for k, v in entries.items() if isinstance(v, torch.Tensor)}
            scalars[saved_id] = {k: v for k, v in entries.items() if not isinstance(v, torch.Tensor)}
        super().load_state_dict({**incoming, "state": scalars})
        saved_groups = incoming["param_groups"]
        for saved_group, group in zip(saved_groups, self.param_groups):
            for saved_id, parameter in zip(saved_group["params"], group["params"]):
                for name, value in tensors.get(saved_id, {}).items():
                    self.state[parameter][name] = value.to(device=parameter.device, copy=True)
