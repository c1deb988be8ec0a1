"""One FP8 ``Linear`` trained with a stock AdamW through ``bind_optimizer``, with gradient accumulation.

    python examples/linear.py --scaling grouped --mode fast

Shows the single-GPU workflow without the engine: set the precision policy, build the layer, construct the
optimizer, bind it (the optimizer then updates an fp32 master and the layer re-quantises after every step).
Runs on a CPU too (the PyTorch restatement of the kernels), which is slow but needs no GPU.
"""
import argparse

import torch

try:
    import viola_b200 as viola
except ModuleNotFoundError:                          # running from a source checkout that is not installed
    import pathlib
    import sys
    sys.path.insert(0, str(pathlib.Path(__file__).resolve().parent.parent))
    import viola_b200 as viola


def parse():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--mode", choices=("memory", "fast"), default="memory")
    parser.add_argument("--weight-dtype", choices=("fp8", "bf16", "fp16"), default="fp8")
    parser.add_argument("--scaling", choices=("current", "delayed", "grouped", "mxfp8"), default="current")
    parser.add_argument("--forward-dtype", choices=("e4m3", "e5m2"), default="e4m3")
    parser.add_argument("--backward-dtype", choices=("e4m3", "e5m2"), default="e5m2")
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--width", type=int, default=256)
    parser.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    return parser.parse_args()


def main():
    args = parse()
    torch.manual_seed(42)
    viola.set_master_weight_dtype("fp32")
    viola.set_gradient_dtype("bf16")
    layer = viola.nn.Linear(args.width, args.width, mode=args.mode, weight_dtype=args.weight_dtype,
                            scaling=args.scaling, forward_dtype=args.forward_dtype,
                            backward_dtype=args.backward_dtype, device=args.device, dtype=torch.bfloat16)
    optimizer = viola.optim.bind_optimizer(layer, torch.optim.AdamW(layer.parameters(), lr=5e-3))
    inputs = torch.randn(256, args.width, device=args.device, dtype=torch.bfloat16)
    targets = 0.3 * torch.randn_like(inputs)
    chunks = 4
    for step in range(1, args.steps + 1):
        optimizer.zero_grad()
        running = 0.0
        for x, y in zip(inputs.chunk(chunks), targets.chunk(chunks)):
            loss = (layer(x).float() - y.float()).square().mean()
            (loss / chunks).backward()                      # gradients accumulate in bf16 (the policy's dtype)
            running += loss.item() / chunks
        optimizer.step()                                    # master update, then the layer's storage format
        if step == 1 or step % 10 == 0:
            print(f"step={step} loss={running:.5f}", flush=True)
    return running


if __name__ == "__main__":
    main()
