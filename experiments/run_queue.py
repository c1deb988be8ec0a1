"""Run a list of ``train_dit.py`` jobs one after another on whichever GPUs are idle, resumably.

    python experiments/run_queue.py --data /data/latents/mmap --root runs --jobs jobs.json

``jobs.json``: a list of ``{"name", "gpus", "args": [...extra train_dit.py arguments...]}``.  Without it a default
sweep runs: FP8 and BF16 momentum on one GPU, then FP8 momentum at global batch 256 / 128 / 64 on 1 and 2 GPUs,
and finally the FP8-vs-BF16 comparison.  A job whose ``complete.json`` exists is skipped, so the queue can be
restarted.  GPUs count as idle below 500 MiB used and 5 % utilisation (read with ``nvidia-smi``; nothing on the
GPU is changed).  Progress goes to ``<root>/status.json`` (written atomically) and one log per job.
(Role of the reference's experiments/run_queue.py:17-99.)
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

HERE = Path(__file__).resolve().parent


def idle_gpus(query=None):
    """Indices of GPUs with < 500 MiB in use and < 5 % utilisation."""
    if query is None:
        query = subprocess.run(["nvidia-smi", "--query-gpu=index,memory.used,utilization.gpu",
                                "--format=csv,noheader,nounits"], check=True, capture_output=True, text=True).stdout
    idle = []
    for line in query.splitlines():
        fields = [field.strip() for field in line.split(",")]
        if len(fields) == 3 and int(fields[1]) < 500 and int(fields[2]) < 5:
            idle.append(int(fields[0]))
    return idle


def default_jobs():
    jobs = [{"name": "gpus1-batch256-fp8", "gpus": 1, "args": ["--batch", "256", "--audit"]},
            {"name": "gpus1-batch256-bf16", "gpus": 1, "args": ["--batch", "256", "--momentum-dtype", "bf16"]}]
    for gpus in (1, 2):
        for batch in (256, 128, 64):
            if (gpus, batch) != (1, 256):
                jobs.append({"name": f"gpus{gpus}-batch{batch}-fp8", "gpus": gpus, "args": ["--batch", str(batch)]})
    return jobs


class Status:
    def __init__(self, root):
        self.path = root / "status.json"

    def write(self, stage, **fields):
        record = {"stage": stage, "updated_at": time.time(), **fields}
        scratch = self.path.with_suffix(".tmp")
        scratch.write_text(json.dumps(record, indent=2))
        scratch.replace(self.path)
        print(json.dumps(record), flush=True)


def launch_command(job, data, output, config):
    command = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
               f"--nproc-per-node={job['gpus']}", str(HERE / "train_dit.py"), "--data", str(data), "--output", str(output),
               *job.get("args", [])]
    environment = dict(os.environ, OMP_NUM_THREADS="4")
    if config:
        environment["VIOLA_CONFIG"] = str(Path(config).resolve())
    return command, environment


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--data", required=True)
    parser.add_argument("--root", required=True)
    parser.add_argument("--jobs")
    parser.add_argument("--config", help="engine YAML exported to every job as $VIOLA_CONFIG")
    parser.add_argument("--poll-seconds", type=float, default=30)
    args = parser.parse_args()
    root = Path(args.root)
    root.mkdir(parents=True, exist_ok=True)
    status = Status(root)
    jobs = json.loads(Path(args.jobs).read_text()) if args.jobs else default_jobs()
    try:
        for job in jobs:
            output = root / job["name"]
            if (output / "complete.json").exists():
                continue
            while True:
                idle = idle_gpus()
                if len(idle) >= job["gpus"]:
                    chosen = idle[:job["gpus"]]
                    break
                status.write("waiting_for_idle_gpus", next_run=job["name"], required=job["gpus"], idle=idle)
                time.sleep(args.poll_seconds)
            status.write("training", run=job["name"], gpus=chosen, started_at=time.time())
            command, environment = launch_command(job, args.data, output, args.config)
            environment["CUDA_VISIBLE_DEVICES"] = ",".join(map(str, chosen))
            with (root / f"{job['name']}.log").open("a") as log:
                subprocess.run(command, env=environment, stdout=log, stderr=subprocess.STDOUT, check=True)
        fp8, bf16 = root / "gpus1-batch256-fp8", root / "gpus1-batch256-bf16"
        if (fp8 / "complete.json").exists() and (bf16 / "complete.json").exists():
            status.write("comparing")
            with (root / "comparison.log").open("w") as log:
                subprocess.run([sys.executable, str(HERE / "compare_runs.py"), "--run", str(fp8), "--baseline", str(bf16),
                                "--output", str(root / "fp8-vs-bf16")], stdout=log, stderr=subprocess.STDOUT, check=True)
        status.write("complete")
    except Exception as error:
        status.write("failed", error=repr(error))
        raise


if __name__ == "__main__":
    main()
