"""Compare two finished ``train_dit.py`` runs (e.g. FP8 momentum against BF16 momentum): loss curves and final masters.

    python experiments/compare_runs.py --run runs/fp8 --baseline runs/bf16 --output runs/fp8-vs-bf16

Refuses runs whose settings differ in anything that changes the data or the model (seed, batch sizes, world
size, epochs, learning rate, model, dataset, source of the model file).  Writes ``loss_curves.csv``,
``weight_errors.json`` (per parameter: relative L2, cosine, max / mean absolute difference, RMSE of the fp32
masters held by rank 0 .. n of the engine checkpoints) and ``summary.json``.  The two runs are independent
trajectories, so the weight difference includes accumulated divergence, not only quantisation error.
Same purpose as the reference's experiments/compare_runs.py:19-82.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
from pathlib import Path

import torch

MATCHED = ("seed", "batch", "micro_batch", "world_size", "epochs", "lr", "model", "dataset")


def read_json(path):
    return json.loads(Path(path).read_text())


def step_records(run):
    records = {}
    with (run / "steps-rank0.jsonl").open() as handle:
        for line in handle:
            record = json.loads(line)
            records[record["step"]] = record
    return records


def masters(run):
    """name -> fp32 master, merged over the per-rank files of the run's engine checkpoint."""
    merged, names = {}, set()
    for path in sorted((run / "checkpoint").glob("rank-*.pt")):
        state = torch.load(path, map_location="cpu", weights_only=False)["state"]
        merged.update(state["optimizer"]["masters"])
        names.update(entry["name"] for entry in state["parameters"])
    # parameters that are their own master (same dtype, unsharded) are only in the full model file
    model = torch.load(run / "checkpoint" / "model.pt", map_location="cpu", weights_only=False)["model"]
    for name in names - set(merged):
        if name in model and model[name].is_floating_point() and model[name].dtype not in (torch.float8_e4m3fn, torch.float8_e5m2):
            merged[name] = model[name]
    return merged


class Accumulator:
    def __init__(self):
        self.error = self.reference = self.actual = self.dot = self.absolute = 0.0
        self.maximum, self.elements = 0.0, 0

    def add(self, x, y):
        delta = x - y
        error, reference, actual = delta.square().sum().item(), y.square().sum().item(), x.square().sum().item()
        dot, absolute, maximum = (x * y).sum().item(), delta.abs().sum().item(), delta.abs().max().item()
        self.error += error; self.reference += reference; self.actual += actual
        self.dot += dot; self.absolute += absolute
        self.maximum = max(self.maximum, maximum)
        self.elements += x.numel()
        return {"relative_l2": math.sqrt(error / reference) if reference else None,
                "cosine": dot / math.sqrt(actual * reference) if actual and reference else None,
                "max_abs": maximum, "mean_abs": absolute / x.numel(), "rmse": math.sqrt(error / x.numel())}

    def summary(self):
        return {"parameters": self.elements, "relative_l2": math.sqrt(self.error / max(self.reference, 1e-300)),
                "cosine": self.dot / math.sqrt(max(self.actual * self.reference, 1e-300)), "max_abs": self.maximum,
                "mean_abs": self.absolute / max(self.elements, 1), "rmse": math.sqrt(self.error / max(self.elements, 1))}


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--run", type=Path, required=True)
    parser.add_argument("--baseline", type=Path, required=True)
    parser.add_argument("--output", type=Path, required=True)
    args = parser.parse_args()
    ours, theirs = read_json(args.run / "settings.json"), read_json(args.baseline / "settings.json")
    for key in MATCHED:
        if ours.get(key) != theirs.get(key):
            raise SystemExit(f"training settings differ: {key}: {ours.get(key)!r} vs {theirs.get(key)!r}")
    model_file = "viola_b200/models/dit.py"
    if ours["source_sha256"].get(model_file) != theirs["source_sha256"].get(model_file):
        raise SystemExit("the two runs used different model sources")
    steps = read_json(args.run / "complete.json")["steps"]
    if steps != read_json(args.baseline / "complete.json")["steps"]:
        raise SystemExit("the two runs finished after different numbers of updates")
    args.output.mkdir(parents=True, exist_ok=True)
    a, b = step_records(args.run), step_records(args.baseline)
    shared = sorted(set(a) & set(b))
    with (args.output / "loss_curves.csv").open("w", newline="") as handle:
        writer = csv.writer(handle)
        writer.writerow(("step", "run_loss", "baseline_loss", "loss_difference", "run_probe", "baseline_probe"))
        for step in shared:
            writer.writerow((step, a[step]["loss"], b[step]["loss"], a[step]["loss"] - b[step]["loss"],
                             a[step].get("fixed_probe_loss", ""), b[step].get("fixed_probe_loss", "")))
    left, right = masters(args.run), masters(args.baseline)
    if left.keys() != right.keys():
        raise SystemExit("the checkpoints hold different parameters")
    totals, rows = Accumulator(), []
    for name in sorted(left):
        x, y = left[name].double().flatten(), right[name].double().flatten()
        rows.append({"name": name, "shape": list(left[name].shape), **totals.add(x, y)})
    tail = shared[-100:]
    summary = {"steps": steps, "note": "independent trajectories: weight differences include accumulated divergence",
               **totals.summary(),
               "final_100_loss": {"run": sum(a[s]["loss"] for s in tail) / max(len(tail), 1),
                                  "baseline": sum(b[s]["loss"] for s in tail) / max(len(tail), 1)}}
    (args.output / "weight_errors.json").write_text(json.dumps(rows, indent=2))
    (args.output / "summary.json").write_text(json.dumps(summary, indent=2))
    print(json.dumps(summary), flush=True)


if __name__ == "__main__":
    main()
