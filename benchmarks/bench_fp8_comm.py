"""FP8 gradient-communication sweep: fused peer-memory kernels against the collective-library path.

Buckets of 1 MB .. 1 GB of fp32 gradients ~N(0, 1e-3) with 0.1 % of the elements scaled x100, e4m3,
tile 128 and 256, reduce-to-owner (sharded gradients) and all-reduce with requantisation
(replicated gradients).  Reports device time (max over ranks), bus bandwidth of the payload that has
to cross NVLink, the fraction of the measured 770 GB/s per-direction peer-copy rate, and the maximum
relative error against the fp32 sum.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_fp8_comm.py --max-mb 256
"""

from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks.common import measure, report  # noqa: E402
import viola_b200 as viola  # noqa: E402
from viola_b200 import ops  # noqa: E402
from viola_b200.parallel.fp8 import FP8Communication  # noqa: E402
from viola_b200.parallel.symm import PeerTransport  # noqa: E402

LINK_GBS = 770.0


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--max-mb", type=int, default=1024)
    parser.add_argument("--out", default=None)
    args = parser.parse_args()
    engine = viola.violaEngine(dict(communication=dict(dtype="fp8", backend="p2p")))
    rank, world, device = engine.rank, engine.world_size, engine.device
    rows = []
    size_mb = 1
    while size_mb <= args.max_mb:
        n = size_mb * (1 << 20) // 4
        torch.manual_seed(rank)
        value = torch.randn(n, device=device) * 1e-3
        value[::1000] *= 100
        exact = value.clone()
        dist.all_reduce(exact)
        for tile in (128, 256):
            wire = n * (1 + 4 / tile)
            # ---- reduce to owner ----
            owner = 0
            transport = PeerTransport(engine, tile_size=tile, overlap=False)   # full-width kernels, as the engine runs them
            accum = torch.zeros(n, device=device) if rank == owner else None
            transport.attach_gradients([(owner, [], n)], [accum], n)
            transport.finalize()
            transport.finalize_gradients()

            def fused_reduce():
                transport.begin_microbatch()
                transport.reduce_to_owner(0, None, n, buffer=value)     # reads the gradient buffer in place
                transport.synchronize()

            library = FP8Communication(n, engine.group, rank, world, engine.global_ranks, device, mode="reduce",
                                       tile_size=tile)
            scratch = value.clone()

            def library_reduce():
                library.reduce(scratch, owner)       # in place on the owner (its buffer becomes the sum)

            fused_ms, library_ms = measure(fused_reduce, repeats=7), measure(library_reduce, repeats=7)
            if rank == owner:
                accum.zero_()
            dist.barrier()
            fused_reduce()
            torch.cuda.synchronize()
            error = ((accum - exact).norm() / exact.norm()).item() if rank == owner else 0.0
            times = torch.tensor([fused_ms, library_ms], device=device)
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
            ingress = (world - 1) * wire            # bytes entering the owner
            if rank == 0:
                rows.append(dict(op="reduce_to_owner", mb=size_mb, tile=tile, world=world, fused_ms=times[0].item(),
                                 library_ms=times[1].item(), fused_owner_ingress_gbs=ingress / times[0].item() / 1e6,
                                 frac_of_link=ingress / times[0].item() / 1e6 / LINK_GBS, rel_error_vs_fp32_sum=error,
                                 note="both paths read the fp32 bucket in place"))
            del transport, library
            # ---- all-reduce with requantisation ----
            transport = PeerTransport(engine, tile_size=tile, overlap=False)
            transport.attach_all_reduce(n)
            transport.finalize()
            transport.finalize_all_reduce()
            library = FP8Communication(n, engine.group, rank, world, engine.global_ranks, device, mode="all_reduce",
                                       tile_size=tile)
            work = value.clone()

            def fused_all_reduce():
                work.copy_(value)
                transport.all_reduce(work)

            def library_all_reduce():
                work.copy_(value)
                library.all_reduce(work)

            def nccl_fp32():
                work.copy_(value)
                dist.all_reduce(work)

            fused_ms, library_ms, nccl_ms = (measure(fn, repeats=7) for fn in (fused_all_reduce, library_all_reduce,
                                                                                 nccl_fp32))
            fused_all_reduce()
            torch.cuda.synchronize()
            error = ((work - exact).norm() / exact.norm()).item()
            times = torch.tensor([fused_ms, library_ms, nccl_ms], device=device)
            dist.all_reduce(times, op=dist.ReduceOp.MAX)
            bus = 2 * (world - 1) / world * wire
            if rank == 0:
                rows.append(dict(op="all_reduce_requant", mb=size_mb, tile=tile, world=world, fused_ms=times[0].item(),
                                 library_ms=times[1].item(), nccl_fp32_ms=times[2].item(),
                                 fused_bus_gbs=bus / times[0].item() / 1e6,
                                 frac_of_link=bus / times[0].item() / 1e6 / LINK_GBS, rel_error_vs_fp32_sum=error))
            del transport, library
            torch.cuda.empty_cache()
        size_mb *= 4
    torch.cuda.synchronize()
    ops.check_status()
    if rank == 0:
        report(rows, args.out)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
