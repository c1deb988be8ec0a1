"""FP8Muon: Muon with one E4M3 momentum buffer + fp32 tile scales, and an auxiliary AdamW.

Constructor, per-group options, state layout (``momentum_q`` uint8, ``momentum_scale`` fp32, ``step`` /
``exp_avg``, ``exp_avg_sq``), Philox key derivation and the update rule follow the reference
(viola/optim/muon.py:14-141).  The kernels are this library's: a register-resident momentum kernel
(optional stochastic rounding), Newton-Schulz on the tcgen05 GEMM (every ``ns_backend`` value runs that
kernel; naming the kernel backend explicitly, ``"tilelang"`` or ``"tcgen05"``, together with ``ns_autotune``
switches on the per-shape tile search of :mod:`viola_b200.tuning`) and fused master-weight / AdamW updates.
"""

from __future__ import annotations

import os
import warnings

import torch

from .. import ops
from ..precision import _dtype, settings
from .matrix import MatrixOptimizer
from .orthogonalize import METHODS, OUTPUT_DTYPE

_MODES = {"fast": (256, 3), "balanced": (256, 5), "stable": (128, 5)}
_MASK63 = (1 << 63) - 1


def _matrix_shape(param, group):
    return tuple(param.shape) if group["batched"] else (param.shape[0], param.numel() // param.shape[0])


def _use_muon(param, group):
    return param.ndim >= 2 if group["use_muon"] is None else group["use_muon"]


class FP8Muon(MatrixOptimizer):
    """Matrices (``ndim >= 2``) take the Muon update, everything else AdamW.

    Per-group ``use_muon=False`` forces AdamW (embeddings, output heads); convolution filters are
    flattened to ``[out_channels, -1]``; ``batched=True`` treats the last two dimensions as independent
    (expert) matrices.  DTensor parameters on a 1-D mesh are updated by whole-tensor owners.
    """

    def __init__(self, params, lr=1e-3, *, weight_decay=0.0, momentum=0.95, nesterov=True, mode="balanced",
                 granularity="tile", tile_size=None, block_shape=None, rounding="nearest", rounding_seed=0,
                 ns_steps=None, ns_method="standard", ns_backend="torch", ns_autotune=True,
                 adjust_lr_fn="match_rms_adamw", betas=(0.9, 0.95), eps=1e-8, adam_state_dtype="fp32",
                 skip_nonfinite=False, shard_state=True):
        default_tile, default_steps = _MODES[mode]
        policy = settings()
        defaults = dict(lr=lr, weight_decay=weight_decay, momentum=momentum, nesterov=nesterov, use_muon=None,
                        batched=False, granularity=granularity,
                        tile_size=default_tile if tile_size is None else tile_size,
                        block_shape=(16, 16) if block_shape is None else tuple(block_shape), rounding=rounding,
                        rounding_seed=rounding_seed, ns_steps=default_steps if ns_steps is None else ns_steps,
                        ns_method=ns_method, ns_backend=ns_backend, ns_autotune=ns_autotune,
                        adjust_lr_fn=adjust_lr_fn, betas=betas, eps=eps, adam_state_dtype=_dtype(adam_state_dtype),
                        master_rounding=policy["master_rounding"],
                        master_rounding_seed=policy["master_rounding_seed"])
        if ns_autotune and ns_backend in ("tilelang", "tcgen05"):
            from .. import tuning
            tuning.enable()          # per-shape tile search for the Newton-Schulz GEMMs (cached on disk)
        self.observer = None
        self._workspace = {}
        self._deferred = None
        self.ns_batch = 32          # matrices of one shape orthogonalised per batched launch
        super().__init__(params, defaults, shard_state=shard_state, skip_nonfinite=skip_nonfinite)

    def add_param_group(self, group):
        super().add_param_group(group)
        group = self.param_groups[-1]
        if group["lr"] < 0 or group["weight_decay"] < 0:
            raise ValueError("lr and weight_decay must be non-negative")
        if not 0 <= group["momentum"] < 1 or group["ns_steps"] <= 0:
            raise ValueError("momentum must be in [0, 1) and ns_steps positive")
        if group["ns_method"] not in METHODS or group["ns_backend"] not in ("torch", "tilelang", "tcgen05"):
            raise ValueError("unknown Newton-Schulz method / backend")
        if group["adjust_lr_fn"] not in ("original", "match_rms_adamw"):
            raise ValueError("adjust_lr_fn must be 'original' or 'match_rms_adamw'")
        if group["granularity"] not in ("tile", "block") or group["rounding"] not in ("nearest", "stochastic"):
            raise ValueError("unknown granularity / rounding")
        if not 0 <= group["rounding_seed"] < (1 << 63):
            raise ValueError("rounding_seed must fit in 63 bits")
        if group["tile_size"] not in (64, 128, 256, 512, 1024):
            raise ValueError("tile_size must be one of 64, 128, 256, 512, 1024")
        if len(group["block_shape"]) != 2 or any(v not in (8, 16, 32, 64) for v in group["block_shape"]):
            raise ValueError("block_shape entries must be 8, 16, 32 or 64")
        group["adam_state_dtype"] = _dtype(group["adam_state_dtype"])
        grad_dtype = settings()["gradient_dtype"]
        unaligned = []
        for param in group["params"]:
            if grad_dtype is not None:
                param.grad_dtype = grad_dtype
            if not _use_muon(param, group):
                continue
            if param.ndim < 2:
                raise ValueError("Muon parameters must have at least two dimensions")
            shape = _matrix_shape(param, group)
            if group["granularity"] == "tile":
                partial = shape[-1] % group["tile_size"]
            else:
                partial = shape[-2] % group["block_shape"][0] or shape[-1] % group["block_shape"][1]
            if partial:
                unaligned.append(shape)
        if unaligned and int(os.environ.get("RANK", "0")) == 0:
            warnings.warn(f"FP8Muon: {len(unaligned)} matrices have partial {group['granularity']} groups "
                          f"(e.g. {unaligned[:3]}); shapes are kept and edge groups cover the valid elements only.",
                          stacklevel=3)

    def _momentum(self, param, grad, state, group, key, out=None):
        shape = _matrix_shape(param, group)
        quant = {name: group[name] for name in ("granularity", "tile_size", "block_shape")}
        if "momentum_q" not in state:
            codes, scales = ops.state_sizes(shape, **quant)
            state["momentum_q"] = torch.zeros(codes, device=param.device, dtype=torch.uint8)
            state["momentum_scale"] = torch.ones(scales, device=param.device, dtype=torch.float32)
        if out is not None:
            matrix = out
        else:
            work = self._workspace.get(param.device)
            if work is None or work.numel() < param.numel():
                work = self._workspace[param.device] = torch.empty(param.numel(), device=param.device,
                                                                   dtype=torch.bfloat16)
            matrix = work[:param.numel()].view(shape)
        q, scale = state["momentum_q"], state["momentum_scale"]
        before = (q.clone(), scale.clone()) if self.observer is not None else (None, None)
        ops.momentum_update(grad, q, scale, q, scale, matrix.view(-1), beta=group["momentum"],
                            nesterov=group["nesterov"], matrix_shape=shape, rounding=group["rounding"],
                            rounding_step=state["step"], rounding_key=key, **quant)
        if self.observer is not None:
            self.observer.momentum(param, grad, before[0], before[1], q, scale, matrix, group, 1.0, quant)
        return matrix

    def _step_local(self, param, grad, state, group, index):
        key = (group["rounding_seed"] + index * 0x9E3779B97F4A7C15) & _MASK63
        master_key = (group["master_rounding_seed"] + index * 0x517CC1B727220A95) & _MASK63
        if grad.is_sparse:
            raise RuntimeError("FP8Muon does not support sparse gradients")
        if param.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise RuntimeError("bind FP8 modules with viola_b200.optim.bind_optimizer before stepping")
        state.setdefault("step", 0)
        if (_use_muon(param, group) and self._deferred is not None and param.is_cuda
                and len(_matrix_shape(param, group)) == 2):
            # same-shape matrices are orthogonalised together after the parameter loop
            shape = _matrix_shape(param, group)
            self._deferred.setdefault((shape, id(group), state["step"], param.device), []).append(
                (param, grad, state, group, key, master_key))
            return
        if not _use_muon(param, group) and self._deferred is not None and param.is_cuda and param.is_contiguous():
            # vectors of one group that are at the same step share one multi-tensor AdamW launch
            self._deferred_adam.setdefault((id(group), state["step"], param.device), []).append(
                (param, grad, state, group, master_key))
            return
        if _use_muon(param, group):
            matrix = self._momentum(param, grad, state, group, key)
            method = METHODS[group["ns_method"]]
            update = method(matrix, steps=group["ns_steps"])
            if self.observer is not None:
                self.observer.update(param, update, group, method)
            rows, cols = matrix.shape[-2:]
            if group["adjust_lr_fn"] == "match_rms_adamw":
                scale = 0.2 * max(rows, cols) ** 0.5
            else:
                scale = max(1.0, rows / cols) ** 0.5
            ops.weight_update(param, update, group["lr"], group["weight_decay"], update_scale=scale,
                              rounding=group["master_rounding"], step=state["step"], key=master_key)
        else:
            if "exp_avg" not in state:
                state["exp_avg"] = torch.zeros_like(param, dtype=group["adam_state_dtype"])
                state["exp_avg_sq"] = torch.zeros_like(param, dtype=group["adam_state_dtype"])
            ops.adam_update(param, grad, state["exp_avg"], state["exp_avg_sq"], lr=group["lr"],
                            weight_decay=group["weight_decay"], betas=group["betas"], eps=group["eps"],
                            step=state["step"] + 1, rounding=group["master_rounding"], key=master_key)
        state["step"] += 1

    # ------------------------------------------------------------------ batched / multi-tensor tail of the step
    def _begin_local(self):
        self._deferred = {} if self.observer is None else None
        self._deferred_adam = {}

    def _table(self, name, rows, device):
        """Cached descriptor table; rebuilt only when a tensor of the set moved."""
        cached = self._workspace.get(name)
        if cached is None or not cached.matches(rows):
            cached = self._workspace[name] = ops.TensorTable(rows, device)
        return cached

    def _finish_local(self):
        deferred, self._deferred = self._deferred, None
        adam, self._deferred_adam = getattr(self, "_deferred_adam", {}), {}
        codes = ops._DT
        for (group_id, step, device), items in adam.items():
            group = items[0][3]
            rows = []
            for param, grad, state, _, master_key in items:
                if "exp_avg" not in state:
                    state["exp_avg"] = torch.zeros_like(param, dtype=group["adam_state_dtype"])
                    state["exp_avg_sq"] = torch.zeros_like(param, dtype=group["adam_state_dtype"])
                flat = grad if grad.is_contiguous() else grad.contiguous()
                rows.append((param, flat, state["exp_avg"], state["exp_avg_sq"], param.numel(), master_key, 0.0, 0.0,
                             codes[param.dtype], codes[flat.dtype] | (codes[state["exp_avg"].dtype] << 8)))
            table = self._table(("adam", group_id, device), rows, device)
            ops.multi_adam(table, lr=group["lr"], weight_decay=group["weight_decay"], betas=group["betas"],
                           eps=group["eps"], step=step + 1, rounding=group["master_rounding"])
            for _, _, state, _, _ in items:
                state["step"] += 1
        if not deferred:
            return
        for (shape, group_id, step, device), items in deferred.items():
            group = items[0][3]
            rows_, cols_ = shape
            if group["adjust_lr_fn"] == "match_rms_adamw":
                update_scale = 0.2 * max(rows_, cols_) ** 0.5
            else:
                update_scale = max(1.0, rows_ / cols_) ** 0.5
            tiled = group["granularity"] == "tile"
            for start in range(0, len(items), self.ns_batch):
                chunk = items[start:start + self.ns_batch]
                key = ("stack", shape, device)
                stack = self._workspace.get(key)
                if stack is None or stack.shape[0] < len(chunk):
                    stack = self._workspace[key] = torch.empty((min(self.ns_batch, len(items)), *shape), device=device,
                                                               dtype=torch.bfloat16)
                stack = stack[:len(chunk)]
                if tiled:
                    rows = []
                    for slot, (param, grad, state, _, rounding_key, _) in enumerate(chunk):
                        if "momentum_q" not in state:
                            count, scales = ops.state_sizes(shape, granularity="tile", tile_size=group["tile_size"])
                            state["momentum_q"] = torch.zeros(count, device=device, dtype=torch.uint8)
                            state["momentum_scale"] = torch.ones(scales, device=device, dtype=torch.float32)
                        flat = grad if grad.is_contiguous() else grad.contiguous()
                        rows.append((flat, state["momentum_q"], state["momentum_scale"], stack[slot], param.numel(),
                                     rounding_key, 0.0, 0.0, codes[flat.dtype], 0))
                    table = self._table(("momentum", shape, group_id, start, device), rows, device)
                    ops.multi_momentum(table, tile_size=group["tile_size"], beta=group["momentum"],
                                       nesterov=group["nesterov"], rounding=group["rounding"], step=step)
                else:
                    for slot, (param, grad, state, _, rounding_key, _) in enumerate(chunk):
                        self._momentum(param, grad, state, group, rounding_key, out=stack[slot])
                # a persistent result buffer keeps the addresses in the update table stable across steps
                out_key = ("ns_out", shape, group["ns_method"], device)
                result = self._workspace.get(out_key)
                if result is None or result.shape[0] < len(chunk):
                    result = self._workspace[out_key] = torch.empty((min(self.ns_batch, len(items)), *shape),
                                                                    device=device,
                                                                    dtype=OUTPUT_DTYPE[group["ns_method"]])
                updates = METHODS[group["ns_method"]](stack, steps=group["ns_steps"], out=result[:len(chunk)])
                rows = [(param, updates[slot], None, None, param.numel(), master_key, update_scale, 0.0,
                         codes[param.dtype], codes[updates.dtype])
                        for slot, (param, _, _, _, _, master_key) in enumerate(chunk)]
                table = self._table(("update", shape, group_id, start, device), rows, device)
                ops.multi_weight_update(table, group["lr"], group["weight_decay"], rounding=group["master_rounding"],
                                        step=step)
                for _, _, state, _, _, _ in chunk:
                    state["step"] += 1
