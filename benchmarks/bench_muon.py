"""FP8Muon optimizer step on a Llama-7B-shaped parameter set (or the DiT-XL/2 set).

32 layers x (4 x 4096x4096 + 3 x 11008x4096) matrices ~N(0, 0.02) with gradients ~N(0, 1e-3), plus
65 RMSNorm vectors on the auxiliary AdamW; balanced mode (tile 256, 5 NS steps), weight decay 0.01,
match_rms_adamw; standard (bf16) and gram (fp16) orthogonalisation, nearest and stochastic rounding.
With N ranks the set is owner-sharded by the engine's greedy partition and every rank times its own
share (max over ranks reported); ``--layers`` shrinks the set for quick runs.

    python benchmarks/bench_muon.py --layers 32
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_muon.py
"""

from __future__ import annotations

import argparse
import gc
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks.common import measure, report  # noqa: E402
from viola_b200 import ops  # noqa: E402
from viola_b200.optim import FP8Muon  # noqa: E402
from viola_b200.parallel.partition import assign_owners  # noqa: E402


def ns_flops(rows, cols, steps=5):
    small, large = min(rows, cols), max(rows, cols)
    return steps * (2 * small * small * large * 2 + 2 * small ** 3)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--layers", type=int, default=32)
    parser.add_argument("--out", default=None)
    args = parser.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    rank = int(os.environ.get("RANK", 0))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if world > 1:
        dist.init_process_group("nccl")
    device = torch.device("cuda")
    shapes = ([(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)]) * args.layers
    owners = assign_owners([r * c for r, c in shapes], world)
    mine = [shape for shape, owner in zip(shapes, owners) if owner == rank]
    torch.manual_seed(rank)
    rows = []
    for method in ("standard", "gram"):
        for rounding in ("nearest", "stochastic"):
            matrices = [torch.nn.Parameter(torch.randn(shape, device=device) * 0.02) for shape in mine]
            vectors = [torch.nn.Parameter(torch.ones(4096, device=device)) for _ in range(65 if rank == 0 else 0)]
            optimizer = FP8Muon(matrices + vectors, lr=1e-3, weight_decay=0.01, mode="balanced", ns_method=method,
                                rounding=rounding)
            optimizer.ns_batch = 8
            for p in matrices + vectors:
                p.grad = torch.randn_like(p) * 1e-3
            ms = measure(optimizer.step, warmup=2, repeats=4)
            flops = sum(ns_flops(*shape) for shape in mine)
            timing = torch.tensor([ms], device=device)
            if world > 1:
                dist.all_reduce(timing, op=dist.ReduceOp.MAX)
            if rank == 0:
                rows.append(dict(op="fp8muon_step", layers=args.layers, ns_method=method, rounding=rounding, world=world,
                                 step_ms_max_over_ranks=timing.item(), ns_tflop_this_rank=flops / 1e12,
                                 ns_tflops_rate=flops / ms / 1e9,
                                 state_bytes_per_element=1 + 4 / 256))
            del optimizer, matrices, vectors, p
            gc.collect()
            torch.cuda.empty_cache()
    ops.check_status()
    if rank == 0:
        report(rows, args.out)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
