"""DTensor data parallelism with owner-sharded ``FP8Muon`` state and ``ShardedEMA``; no engine, no sharder.

    torchrun --standalone --nproc-per-node 2 examples/train_dtensor.py --ema-decay 0.999

The model's parameters are replicated DTensors.  Each rank feeds its own rows of a ``Shard(0)`` batch, so
the loss is a global mean and autograd hands the optimizer ``Partial`` gradients.  ``FP8Muon`` assigns every
tensor an owner: the owner receives the reduced gradient, keeps the FP8 momentum, runs Newton-Schulz and
writes the new weight back to all ranks.  Masters are disabled, so the bf16 weights are updated in place.
"""
import argparse
import os

import torch
import torch.distributed as dist
from torch import nn
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.tensor import DTensor, Replicate, Shard, distribute_tensor

try:
    import viola_b200 as viola
except ModuleNotFoundError:                          # running from a source checkout that is not installed
    import pathlib
    import sys
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))
    import viola_b200 as viola
from viola_b200.distributed import ShardedEMA


def replicate_parameters(model, mesh):
    for module in model.modules():
        for name, parameter in list(module.named_parameters(recurse=False)):
            module.register_parameter(name, nn.Parameter(distribute_tensor(parameter.detach(), mesh, [Replicate()])))


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--batch-size", type=int, default=32, help="rows per rank")
    parser.add_argument("--ema-decay", type=float, default=0.0, help="0 disables the EMA")
    args = parser.parse_args()
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl" if on_gpu else "gloo")
    kind = "cuda" if on_gpu else "cpu"
    mesh = init_device_mesh(kind, (dist.get_world_size(),))

    viola.set_master_weight_dtype(None)              # update the bf16 weights themselves
    viola.set_gradient_dtype("fp32")
    torch.manual_seed(42)
    model = nn.Sequential(nn.Linear(128, 256), nn.SiLU(), nn.Linear(256, 128)).to(kind).to(torch.bfloat16)
    replicate_parameters(model, mesh)
    optimizer = viola.optim.bind_optimizer(model, viola.optim.FP8Muon(model.parameters(), lr=1e-3))
    ema = ShardedEMA(model, optimizer, decay=args.ema_decay)

    torch.manual_seed(100 + dist.get_rank())
    rows = torch.randn(args.batch_size, 128, device=kind, dtype=torch.bfloat16)
    batch = DTensor.from_local(rows, mesh, [Shard(0)])
    for step in range(1, args.steps + 1):
        optimizer.zero_grad()
        loss = (model(batch).float() - batch.float()).square().mean()
        loss.backward()
        optimizer.step()                              # reduce to owners, update, write back, EMA hook
        if step == 1 or step % 5 == 0:
            value = loss.detach().full_tensor().item()     # a collective: every rank calls it
            if dist.get_rank() == 0:
                print(f"step={step} loss={value:.6f} ema_updates={ema.updates}", flush=True)
    ema.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
