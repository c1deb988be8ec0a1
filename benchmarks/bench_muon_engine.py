"""FP8Muon step on a Llama-7B-shaped parameter set through the engine, owner-sharded over 1 / 2 / 4 / 8 GPUs.

What is timed, per step and as the maximum over ranks (CUDA events, no host wait inside):

* ``gather``: every rank's full gradient of every matrix goes to the matrix's owner: FP8 (e4m3, tile 256)
  quantise + peer push, owner-side dequantise + ordered fp32 sum into its accumulator (the engine's
  per-microbatch gradient path; one pass = one microbatch);
* ``step``: the optimizer step on the owners (FP8 momentum, Newton-Schulz, weight update; AdamW on the 65 norm
  vectors), the write-back of the new FP8 weights into every rank's row shard by peer stores, the re-gather of
  the resident copies, and the cross-rank barriers around them.

The reference does the same work as gather-to-owner / step / scatter + broadcasts per parameter over NCCL
(viola/optim/matrix.py:86-108, viola/distributed/parameters.py:121-147).  ``--layers`` shrinks the set;
32 layers are 6.5 B parameters.

    python benchmarks/bench_muon_engine.py --layers 32
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_muon_engine.py
"""

from __future__ import annotations

import argparse
import os
import statistics
import sys

import torch
import torch.distributed as dist
from torch import nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks.common import report  # noqa: E402
import viola_b200 as viola  # noqa: E402
from viola_b200 import ops, utils  # noqa: E402
from viola_b200.nn import Linear  # noqa: E402


class Layer(nn.Module):
    """The seven matrices and two norm vectors of one Llama-7B layer (never run forward here)."""

    def __init__(self, width=4096, hidden=11008):
        super().__init__()
        self.q, self.k, self.v, self.o = (Linear(width, width, bias=False) for _ in range(4))
        self.gate, self.up = Linear(width, hidden, bias=False), Linear(width, hidden, bias=False)
        self.down = Linear(hidden, width, bias=False)
        self.norm1, self.norm2 = nn.Parameter(torch.ones(width)), nn.Parameter(torch.ones(width))


class Stack(nn.Module):
    def __init__(self, layers):
        super().__init__()
        self.layers = nn.ModuleList([Layer() for _ in range(layers)])
        self.norm = nn.Parameter(torch.ones(4096))


def ns_flops(rows, cols, steps=5):
    small, large = min(rows, cols), max(rows, cols)
    return steps * (2 * small * small * large * 2 + 2 * small ** 3)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--layers", type=int, default=32)
    parser.add_argument("--steps", type=int, default=4)
    parser.add_argument("--ns-method", default="standard", choices=("standard", "gram"))
    parser.add_argument("--rounding", default="nearest", choices=("nearest", "stochastic"))
    parser.add_argument("--backend", default="auto", choices=("auto", "p2p", "nccl"))
    parser.add_argument("--out", default=None)
    args = parser.parse_args()
    engine = viola.violaEngine(dict(mixed_precision="bf16", gradient_accumulation_steps=1,
                                    sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True),
                                    precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                                    communication=dict(dtype="fp8", bucket_mb=25, fp8_tile_size=256, backend=args.backend),
                                    ema=dict(decay=0)))
    rank, world, device = engine.rank, engine.world_size, engine.device
    torch.manual_seed(0)
    with torch.device(device):
        model = Stack(args.layers)
    for module in model.modules():
        if isinstance(module, Linear):
            nn.init.normal_(module._initial_weight, std=0.02)
            module.refresh_weight(module._initial_weight)
    model = engine.prepare_model(model)
    matrices = [p for p in model.parameters() if p.ndim == 2]
    vectors = [p for p in model.parameters() if p.ndim == 1]
    engine.prepare_optimizer(lambda _: viola.optim.FP8Muon(
        [dict(params=matrices, use_muon=True), dict(params=vectors, use_muon=False)], lr=1e-3, weight_decay=0.01,
        mode="balanced", ns_method=args.ns_method, rounding=args.rounding))
    state = engine.state
    gradients = state.gradients
    assert gradients.landing is not None
    torch.manual_seed(100 + rank)

    def one_step():
        # "backward": every rank's local gradient lands in the landing buffer (synthetic, ~N(0, 1e-3))
        gradients.begin_backward()
        gradients.landing.normal_(0.0, 1e-3)
        gradients.seen = [True] * len(gradients.records)
        gradients.used = [True] * len(gradients.records)
        with utils.phase("gather"):
            gradients.finish_backward()
        engine._pending_microbatches = 1
        engine.sync_gradients = True
        with utils.phase("step"):
            assert engine.step()

    for _ in range(2):
        one_step()
    torch.cuda.synchronize()
    ops.check_status()
    utils.enable_timing(True)
    dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        one_step()
    stop.record()
    torch.cuda.synchronize()
    total_ms = start.elapsed_time(stop) / args.steps
    phases = utils.phase_times()
    utils.enable_timing(False)
    ops.check_status()
    names = ("gather", "step", "reduce", "optimizer", "writeback")
    values = torch.tensor([total_ms, *(phases.get(name, 0.0) / args.steps for name in names)], device=device,
                          dtype=torch.float64)
    dist.all_reduce(values, op=dist.ReduceOp.MAX)
    owned = [r for r in state.parameters.records if r.owner == rank and len(r.shape) == 2]
    flops = torch.tensor([float(sum(ns_flops(*r.shape) for r in owned))], device=device, dtype=torch.float64)
    dist.all_reduce(flops, op=dist.ReduceOp.MAX)
    if rank == 0:
        values = values.tolist()
        row = dict(op="fp8muon_engine_step", layers=args.layers, parameters=sum(r.numel for r in state.parameters.records),
                   world=world, ns_method=args.ns_method, rounding=args.rounding,
                   transport="peer memory" if engine.transport is not None else ("none" if world == 1 else "nccl"),
                   total_ms_max_over_ranks=values[0],
                   **{f"{name}_ms": value for name, value in zip(names, values[1:])},
                   exposed_comm_ms=values[1] + values[3] + values[5],
                   ns_tflop_busiest_rank=flops.item() / 1e12, ns_tflops_rate=flops.item() / max(values[4], 1e-9) / 1e9)
        report([row], args.out)
    engine.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
