"""Plain PyTorch training loop with ``FP8Muon``; under ``torchrun`` the model is wrapped in DDP.

    python examples/train.py --mode stable --rounding stochastic
    torchrun --standalone --nproc-per-node 2 examples/train.py

Matrices take the Muon update (FP8 momentum + Newton-Schulz), biases the auxiliary AdamW.  No engine,
no master binding: the fp32 model parameters are the masters.
"""
import argparse
import os

import torch
import torch.distributed as dist
from torch import nn

try:
    import viola_b200 as viola
except ModuleNotFoundError:                          # running from a source checkout that is not installed
    import pathlib
    import sys
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))
    import viola_b200 as viola


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--mode", choices=("fast", "balanced", "stable"), default="balanced")
    parser.add_argument("--rounding", choices=("nearest", "stochastic"), default="nearest")
    args = parser.parse_args()
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    on_gpu = torch.cuda.is_available()
    device = torch.device("cuda", local) if on_gpu else torch.device("cpu")
    if on_gpu:
        torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl" if on_gpu else "gloo")
    torch.manual_seed(42)
    net = nn.Sequential(nn.Linear(128, 256), nn.SiLU(), nn.Linear(256, 64)).to(device)
    optimizer = viola.optim.FP8Muon(net.parameters(), lr=3e-3, mode=args.mode, rounding=args.rounding)
    model = nn.parallel.DistributedDataParallel(net, device_ids=[local] if on_gpu else None) if world > 1 else net
    x = torch.randn(128, 128, device=device)
    loss = None
    for step in range(1, args.steps + 1):
        optimizer.zero_grad()
        with torch.autocast(device.type, dtype=torch.bfloat16):
            loss = (model(x).float() - x[:, :64]).square().mean()
        loss.backward()
        optimizer.step()
        if local == 0 and (step == 1 or step % 20 == 0):
            print(f"step={step} loss={loss.item():.6f}", flush=True)
    if world > 1:
        dist.destroy_process_group()
    return loss.item()


if __name__ == "__main__":
    main()
