"""The user-facing scripts run end to end on a CPU: examples, the DiT trainer with the momentum audit, the run
comparison and the job queue's helpers (small sizes; the kernels' PyTorch restatements do the arithmetic)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def run(*command, timeout=600):
    environment = {key: value for key, value in os.environ.items()
                   if key not in ("MASTER_ADDR", "MASTER_PORT", "RANK", "WORLD_SIZE", "LOCAL_RANK", "VIOLA_CONFIG")}
    environment.update(PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, *map(str, command)], cwd=ROOT, env=environment, capture_output=True, text=True,
                          timeout=timeout)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    return done.stdout


def test_examples_run_on_cpu(tmp_path):
    assert "step=1" in run("examples/linear.py", "--steps", "2", "--device", "cpu", "--width", "64")
    assert "step=1" in run("examples/train.py", "--steps", "2")
    first = run("examples/train_distributed.py", "--steps", "2", "--batch-size", "8", "--checkpoint", tmp_path / "ck")
    assert "step=1" in first and (tmp_path / "ck" / "metadata.json").exists()
    resumed = run("examples/train_distributed.py", "--steps", "5", "--batch-size", "8", "--resume", tmp_path / "ck")
    assert "step=5" in resumed and "step=1 " not in resumed
    assert "step=1" in run("-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1", "--nproc-per-node", "2",
                           "examples/train_dtensor.py", "--steps", "2", "--ema-decay", "0.9")


def test_launcher_runs_the_engine_example_on_two_ranks(tmp_path):
    config = tmp_path / "two.yaml"
    config.write_text("num_processes: 2\ndevice: cpu\nmixed_precision: 'no'\ngradient_accumulation_steps: 2\n"
                      "sharding: {parameters: true, gradients: true, optimizer: true, ema: true}\n"
                      "communication: {dtype: fp32}\nema: {decay: 0.99}\n")
    output = run("-m", "viola_b200", "launch", "--config", config, "examples/train_distributed.py", "--steps", "2",
                 "--batch-size", "4")
    assert "step=1" in output and "ema_updates=1" in output


def test_dit_trainer_audit_and_comparison(tmp_path):
    common = ["experiments/train_dit.py", "--synthetic", "64", "--model", "tiny", "--linear", "torch", "--batch", "16",
              "--micro-batch", "8", "--max-steps", "3"]
    run(*common, "--output", tmp_path / "fp8", "--audit", "--ns-interval", "1", "--probe-interval", "2")
    run(*common, "--output", tmp_path / "bf16", "--momentum-dtype", "bf16", "--probe-interval", "2")
    records = [json.loads(line) for line in (tmp_path / "fp8" / "steps-rank0.jsonl").read_text().splitlines()]
    assert [r["step"] for r in records] == [1, 2, 3] and "fixed_probe_loss" in records[1]
    assert records[2]["fp8_bf16_max_matrix_relative_l2"] < 0.06          # FP8 momentum stays within a few percent
    assert (tmp_path / "fp8" / "settings.json").exists() and (tmp_path / "fp8" / "complete.json").exists()
    assert list((tmp_path / "fp8" / "metrics").glob("momentum-rank0-*")) and (tmp_path / "fp8" / "metrics" / "ns-rank0.jsonl").exists()
    summary = json.loads(run("experiments/compare_runs.py", "--run", tmp_path / "fp8", "--baseline", tmp_path / "bf16",
                             "--output", tmp_path / "cmp").strip().splitlines()[-1])
    assert summary["steps"] == 3 and summary["parameters"] > 0 and summary["relative_l2"] < 0.05
    assert (tmp_path / "cmp" / "loss_curves.csv").exists()


def test_queue_helpers():
    sys.path.insert(0, str(ROOT / "experiments"))
    try:
        import run_queue
    finally:
        sys.path.pop(0)
    assert run_queue.idle_gpus("0, 12, 0\n1, 70000, 99\n2, 100, 3\n") == [0, 2]
    names = [job["name"] for job in run_queue.default_jobs()]
    assert names[:2] == ["gpus1-batch256-fp8", "gpus1-batch256-bf16"] and len(names) == len(set(names)) == 7
    command, environment = run_queue.launch_command({"name": "x", "gpus": 2, "args": ["--batch", "64"]}, "/d", "/o", None)
    assert "--nproc-per-node=2" in command and command[-2:] == ["--batch", "64"]
