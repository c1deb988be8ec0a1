"""``MomentumAudit``: per-step, per-matrix diagnostics of FP8 momentum against a BF16 shadow momentum.

Attach an instance to ``FP8Muon.observer``.  The optimizer then reports, for every matrix it updates, the
gradient, the FP8 state before and after, and the Newton-Schulz input it used; the audit advances a BF16
shadow momentum on the *same* gradients and records how far the two drift apart, plus, every ``ns_interval``
steps, how much the orthogonalised update differs when the shadow momentum is fed to the same Newton-Schulz.
The shadow buffers are diagnostic state (2 bytes per element) and not part of the optimizer's footprint.

Output: ``momentum-rank{r}-{n:06d}.parquet`` (or ``.jsonl`` when pyarrow is not importable) with one row per
(step, matrix) and the columns of :data:`FIELDS`; ``ns-rank{r}.jsonl`` with the update comparisons.
``finish()`` returns a per-step summary for the trainer's log.  Same role and metric definitions as the
reference's audit (experiments/audit.py:12-139).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from viola_b200 import ops

COMPARISON = ("error_squared_sum", "reference_squared_sum", "relative_l2", "cosine", "max_abs", "bias")
FIELDS = ("grad_rms", "fp8_rms", "fp8_absmax", "zero_fraction", "nonfinite_fraction", "code_unchanged_fraction",
          "endpoint_fraction", "scale_min", "scale_max", "local_quant_relative_l2", "local_quant_bias",
          "bf16_rms", "bf16_zero_fraction", "bf16_nonfinite_fraction",
          *(f"fp8_bf16_{name}" for name in COMPARISON),
          "input_fp8_bf16_relative_l2", "input_fp8_bf16_cosine", "fp8_bf16_norm_ratio",
          "fp8_bf16_scale_aligned_relative_l2")


def compare(actual, reference):
    """(sum of squared error, sum of squared reference, relative L2, cosine, max |error|, mean error)."""
    actual, reference = actual.float().flatten(), reference.float().flatten()
    delta = actual - reference
    error, energy, own = delta.square().sum(), reference.square().sum(), actual.square().sum()
    cosine = (actual * reference).sum() / (energy * own).sqrt().clamp_min(1e-30)
    cosine = torch.where((energy == 0) & (own == 0), torch.ones_like(cosine), cosine).clamp(-1, 1)
    return torch.stack((error, energy, (error / energy.clamp_min(1e-30)).sqrt(), cosine, delta.abs().max(), delta.mean()))


class MomentumAudit:
    def __init__(self, model, output, rank=0, ns_interval=100, rows_per_file=20000):
        self.names = {id(p): name for name, p in model.named_parameters()}
        self.output = Path(output)
        self.output.mkdir(parents=True, exist_ok=True)
        self.rank, self.ns_interval, self.rows_per_file = rank, ns_interval, rows_per_file
        self.shadow, self.staged, self.ns_inputs = {}, {}, {}
        self.pending, self.records = [], []
        self.step = 0
        self.files = 0

    def alias(self, master, parameter):
        """Make ``master`` (what the optimizer sees after binding) report under ``parameter``'s name."""
        self.names[id(master)] = self.names[id(parameter)]

    # ------------------------------------------------------------------ FP8Muon.observer interface
    @torch.no_grad()
    def momentum(self, param, grad, q, scale, new_q, new_scale, matrix, group, loss_scale, quant):
        name = self.names.get(id(param), f"param{id(param)}")
        beta = group["momentum"]
        count = param.numel()
        g = grad.float().flatten() / loss_scale
        shadow = self.shadow.get(name)
        if shadow is None:
            shadow = torch.zeros(count, device=param.device, dtype=torch.bfloat16)
        fresh16 = beta * shadow.float() + (1 - beta) * g
        # like the optimizer: this step's Newton-Schulz input uses the fresh momentum before storage rounding
        reference_input = ((1 - beta) * g + beta * fresh16 if group.get("nesterov", True) else fresh16).bfloat16()
        stored16 = fresh16.bfloat16()
        shape = tuple(matrix.shape)
        old = ops.momentum_dequantize(q, scale, shape, **quant).flatten()[:count]
        current = ops.momentum_dequantize(new_q, new_scale, shape, **quant).flatten()[:count]
        fresh8 = beta * old + (1 - beta) * g
        local = compare(current, fresh8)
        codes = new_q[:count].view(torch.float8_e4m3fn).float()
        reference = stored16.float()
        pair = compare(matrix.flatten(), reference_input)
        energy, own = reference.square().sum(), current.square().sum()
        fitted = (current * reference).sum() / energy.clamp_min(1e-30)
        metrics = torch.stack((
            g.square().mean().sqrt(), current.square().mean().sqrt(), current.abs().max(),
            (current == 0).float().mean(), (~current.isfinite()).float().mean(),
            (q[:count] == new_q[:count]).float().mean(), (codes.abs() == 448).float().mean(),
            new_scale.min(), new_scale.max(), local[2], local[5],
            reference.square().mean().sqrt(), (stored16 == 0).float().mean(), (~stored16.isfinite()).float().mean(),
            *compare(current, reference), pair[2], pair[3],
            (own / energy.clamp_min(1e-30)).sqrt(),
            ((current - fitted * reference).square().sum() / own.clamp_min(1e-30)).sqrt()))
        self.staged[name] = stored16
        self.pending.append((name, list(param.shape), metrics))
        if self.ns_interval and self.step % self.ns_interval == 0:
            self.ns_inputs[name] = reference_input.view(shape)

    @torch.no_grad()
    def update(self, param, actual, group, method):
        name = self.names.get(id(param), f"param{id(param)}")
        reference_input = self.ns_inputs.pop(name, None)
        if reference_input is not None:
            reference = method(reference_input, steps=group.get("ns_steps", 5))
            self.pending.append((name + ":NS", list(param.shape), compare(actual, reference)))

    # ------------------------------------------------------------------ per-step bookkeeping
    def finish(self, overflow=False):
        """Commit the shadow state of this step and return a summary; ``overflow=True`` discards the step."""
        if overflow:
            self.staged.clear(); self.pending.clear(); self.ns_inputs.clear()
            return {"overflow_skipped": True}
        self.shadow.update(self.staged)
        self.staged.clear()
        matrices = [row for row in self.pending if not row[0].endswith(":NS")]
        updates = [row for row in self.pending if row[0].endswith(":NS")]
        self.pending = []
        shadow_bytes = sum(t.numel() * t.element_size() for t in self.shadow.values())
        summary = {"reference_precision": "bf16", "local_matrices": len(matrices), "diagnostic_shadow_bytes": shadow_bytes}
        if matrices:
            values = torch.stack([row[2] for row in matrices]).float().cpu()
            for (name, shape, _), row in zip(matrices, values.tolist()):
                self.records.append({"step": self.step, "rank": self.rank, "name": name, "shape": shape,
                                     **dict(zip(FIELDS, row))})
            first = FIELDS.index("fp8_bf16_error_squared_sum")
            summary["fp8_bf16_local_relative_l2"] = math.sqrt(float(values[:, first].sum())
                                                             / max(float(values[:, first + 1].sum()), 1e-30))
            summary["fp8_bf16_max_matrix_relative_l2"] = float(values[:, first + 2].max())
            summary["fp8_bf16_min_matrix_cosine"] = float(values[:, first + 3].min())
        if updates:
            rows = torch.stack([row[2] for row in updates]).float().cpu().tolist()
            with (self.output / f"ns-rank{self.rank}.jsonl").open("a") as handle:
                for (name, shape, _), row in zip(updates, rows):
                    handle.write(json.dumps({"step": self.step, "name": name, "shape": shape,
                                             "reference_precision": "bf16", **dict(zip(COMPARISON, row))}) + "\n")
        if len(self.records) >= self.rows_per_file:
            self.flush()
        return summary

    def flush(self):
        if not self.records:
            return None
        stem = self.output / f"momentum-rank{self.rank}-{self.files:06d}"
        try:
            import pyarrow as pa
            import pyarrow.parquet as pq
            path = stem.with_suffix(".parquet")
            pq.write_table(pa.Table.from_pylist(self.records), path, compression="zstd")
        except ImportError:
            path = stem.with_suffix(".jsonl")
            path.write_text("".join(json.dumps(record) + "\n" for record in self.records))
        self.records = []
        self.files += 1
        return path
