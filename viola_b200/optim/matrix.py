"""Base class for optimizers whose update rule needs a whole logical matrix.

Subclasses implement ``_step_local(parameter, gradient, state, group, index)`` on ordinary full
tensors.  Plain parameters are updated in place; DTensor parameters (Replicate or Shard on a 1-D
mesh) are processed in owner rounds: gather gradient and weight to the owner, update there, write
the result back into the existing layout.  ``shard_state=False`` keeps replicated state but still
writes back from one source so stochastic / FP8 results agree bit for bit.  Behaviour and
checkpoint keys follow the reference base class (viola/optim/matrix.py:13-135).
"""

from __future__ import annotations

from abc import abstractmethod

import torch
import torch.distributed as dist

from ..parallel.partition import MatrixPartition

try:
    from torch.distributed.tensor import DTensor
except Exception:  # pragma: no cover
    DTensor = ()


class MatrixOptimizer(torch.optim.Optimizer):
    def __init__(self, params, defaults, *, shard_state=True, skip_nonfinite=False):
        self.shard_state = shard_state
        self.skip_nonfinite = skip_nonfinite
        self.step_was_skipped = False
        self._partition = None
        super().__init__(params, defaults)
        self.register_state_dict_post_hook(self._save_partition)
        self.register_load_state_dict_pre_hook(self._before_load)
        self.register_load_state_dict_post_hook(self._after_load)

    def add_param_group(self, group):
        if self._partition is not None and self._partition.owners:
            raise RuntimeError("add DTensor parameter groups before the first step or checkpoint")
        super().add_param_group(group)
        self._partition = None

    @property
    def partition(self):
        if self._partition is None:
            self._partition = MatrixPartition(p for g in self.param_groups for p in g["params"])
        return self._partition

    @abstractmethod
    def _step_local(self, parameter, gradient, state, group, index):
        """Update one full parameter in place; ``index`` is stable across sharding layouts."""
        raise NotImplementedError

    def _has_nonfinite(self):
        bad = False
        for group in self.param_groups:
            for param in group["params"]:
                if param.grad is None:
                    continue
                grad = param.grad.to_local() if isinstance(param.grad, DTensor) else param.grad
                if not torch.isfinite(grad).all():
                    bad = True
        for mesh in self.partition.meshes:          # all ranks must agree before anyone skips
            flag = torch.tensor(int(bad), device=mesh.device_type, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=mesh.get_group())
            bad = bool(flag.item())
        return bad

    @torch.no_grad()
    def step(self, closure=None):
        self.step_was_skipped = False
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.skip_nonfinite and self._has_nonfinite():
            self.step_was_skipped = True
            return loss
        distributed, running = {}, 0
        self._begin_local()
        for group in self.param_groups:
            indices = group.get("viola_parameter_indices")
            for position, param in enumerate(group["params"]):
                index = indices[position] if indices is not None else running
                running += 1
                if param.grad is None:
                    continue
                if isinstance(param, DTensor):
                    distributed[param] = (group, index)
                else:
                    self._step_local(param, param.grad, self.state[param], group, index)
        self._finish_local()
        if distributed:
            for batch in self.partition.batches:
                self._step_batch(batch, distributed)
        return loss

    def _begin_local(self):
        """Called before the plain-tensor parameters are visited (subclasses may start batching)."""

    def _finish_local(self):
        """Called after the plain-tensor parameters were visited, before DTensor owner rounds."""

    def _step_batch(self, batch, contexts):
        from ..parallel.communication import gather_to_owner, replicate_tensor, write_from_owner
        work = []
        for param in batch:
            if param not in contexts:
                continue
            owner = self.partition.owner(param)
            if self.shard_state:
                gradient, value = gather_to_owner(param.grad, owner), gather_to_owner(param, owner)
            else:
                gradient, value = replicate_tensor(param.grad), replicate_tensor(param)
            if value is not None:
                value = value.contiguous()
            work.append((param, value, gradient, owner))
        for param, value, gradient, _ in work:
            if value is not None:
                group, index = contexts[param]
                self._step_local(value, gradient.contiguous(), self.state[param], group, index)
        for param, value, _, owner in work:
            write_from_owner(param, value, owner)

    # ------------------------------------------------------------------ checkpoint hooks
    def _save_partition(self, optimizer, state):
        if self.partition.owners:
            state["viola_dtensor"] = dict(shard_state=self.shard_state, partition=self.partition.state_dict())
        return state

    def _before_load(self, optimizer, saved):
        saved = dict(saved)
        layout = saved.pop("viola_dtensor", {})
        expected = (dict(shard_state=self.shard_state, partition=self.partition.state_dict())
                    if self.partition.owners else {})
        if layout != expected:
            raise RuntimeError("matrix-optimizer checkpoint ownership / layout differs from this run")
        # torch would cast every floating state tensor to the parameter dtype; keep raw FP8 momentum
        # bytes and independently chosen Adam state dtypes by loading tensors ourselves.
        self._loading = {pid: {k: v for k, v in state.items() if isinstance(v, torch.Tensor)}
                         for pid, state in saved["state"].items()}
        self._loading_groups = saved["param_groups"]
        stripped = {pid: {k: v for k, v in state.items() if not isinstance(v, torch.Tensor)}
                    for pid, state in saved["state"].items()}
        return dict(saved, state=stripped)

    def _after_load(self, optimizer):
        for old, group in zip(self._loading_groups, self.param_groups):
            for pid, param in zip(old["params"], group["params"]):
                for name, value in self._loading.get(pid, {}).items():
                    self.state[param][name] = value.to(device=param.device, copy=True)
        del self._loading, self._loading_groups
