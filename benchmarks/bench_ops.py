"""Single-GPU FP8 op suite: Linear fwd+dgrad+wgrad, fused gated SwiGLU MLP, expert grouped linear.

Shapes of the reference's op benchmarks (checks/benchmark_linear.py, benchmark_fused_mlp.py): bf16
activations ~N(0,1), kaiming-uniform weights, e4m3 forward / e5m2 backward, fp32 scale per 128-element
tile (``scaling="grouped"``) and per-tensor scales (``scaling="current"``), modes fast and memory.
(a) Linear M=8192, K=N=4096 (825 GFLOP per fwd+bwd); (b) MLP 4096 -> 2x11008 -> 4096 at M=8192
(6.65 TFLOP fwd+bwd); (c) 8 experts x (4096 -> 14336), 1024 tokens each (0.96 TFLOP fwd).
Baselines measured in the same run: torch bf16 (cuBLAS) for every shape, and a Python loop of 8
per-expert layers for (c).

    python benchmarks/bench_ops.py [--out results.json]
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from benchmarks.common import measure, peaks, report  # noqa: E402
import viola_b200 as viola  # noqa: E402
from viola_b200.nn import GroupedLinear, Linear, MLP  # noqa: E402

GROUPED = dict(scaling="grouped", weight_group_shape=(128, 128), input_group_shape=(1, 128), grad_group_shape=(1, 128))


def fwd_bwd(module, x, *extra):
    def run():
        y = module(x, *extra)
        y.backward(torch.ones_like(y))
        module.zero_grad(set_to_none=True)
        x.grad = None
    return run


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--out", default=None)
    args = parser.parse_args()
    device = torch.device("cuda")
    peak = peaks()
    rows = []
    torch.manual_seed(0)
    m, k, n = 8192, 4096, 4096
    x = torch.randn(m, k, device=device, dtype=torch.bfloat16, requires_grad=True)
    for name, options in (("grouped128", GROUPED), ("current", dict(scaling="current")), ("mxfp8", dict(scaling="mxfp8"))):
        for mode in ("fast", "memory"):
            layer = Linear(k, n, bias=False, mode=mode, **options).to(device)
            fwd = measure(lambda: layer(x))
            both = measure(fwd_bwd(layer, x))
            rows.append(dict(op="linear", scaling=name, mode=mode, M=m, K=k, N=n, fwd_ms=fwd, fwd_bwd_ms=both,
                             fwd_tflops=2 * m * n * k / fwd / 1e9, fwd_bwd_tflops=6 * m * n * k / both / 1e9))
    reference = torch.nn.Linear(k, n, bias=False, device=device, dtype=torch.bfloat16)
    both = measure(fwd_bwd(reference, x))
    rows.append(dict(op="linear", scaling="bf16 torch.nn.Linear (cuBLAS)", M=m, K=k, N=n, fwd_bwd_ms=both,
                     fwd_bwd_tflops=6 * m * n * k / both / 1e9,
                     frac_of_bf16_peak=6 * m * n * k / both / 1e9 / peak["bf16_tflops"], peak_source=peak["source"]))
    # (b) fused gated MLP
    hidden = 11008
    for name, options in (("grouped128", GROUPED), ("current", dict(scaling="current"))):
        mlp = MLP(k, hidden, activation="silu", bias=False, **options).to(device)
        torch.cuda.reset_peak_memory_stats()
        fwd = measure(lambda: mlp(x), repeats=8)
        both = measure(fwd_bwd(mlp, x), repeats=8)
        flops = 2 * m * k * 2 * hidden + 2 * m * hidden * k
        rows.append(dict(op="gated_mlp", scaling=name, M=m, dims=[k, hidden, k], fwd_ms=fwd, fwd_bwd_ms=both,
                         fwd_tflops=flops / fwd / 1e9, fwd_bwd_tflops=3 * flops / both / 1e9,
                         peak_mib=torch.cuda.max_memory_allocated() / 2 ** 20))
        del mlp
    # (c) expert grouped linear
    experts, per_expert, width = 8, 1024, 14336
    tokens = torch.randn(experts * per_expert, k, device=device, dtype=torch.bfloat16, requires_grad=True)
    offsets = torch.arange(0, experts * per_expert + 1, per_expert, device=device, dtype=torch.int32)
    for scaling in ("grouped", "current"):
        layer = GroupedLinear(experts, k, width, scaling=scaling, dtype=torch.bfloat16).to(device)
        fwd = measure(lambda: layer(tokens, offsets), repeats=8)
        rows.append(dict(op="expert_linear", scaling=scaling, experts=experts, tokens_per_expert=per_expert, K=k, N=width,
                         fwd_ms=fwd, fwd_tflops=2 * experts * per_expert * k * width / fwd / 1e9,
                         note="includes quantising activations and weights each call"))
        del layer
    loop = [Linear(k, width, bias=False, **GROUPED).to(device) for _ in range(experts)]

    def looped():
        return [loop[e](tokens[e * per_expert:(e + 1) * per_expert]) for e in range(experts)]

    fwd = measure(looped, repeats=8)
    rows.append(dict(op="expert_linear", scaling="loop of 8 Linear (baseline shape of the reference)", fwd_ms=fwd,
                     fwd_tflops=2 * experts * per_expert * k * width / fwd / 1e9))
    viola.ops.check_status()
    report(rows, args.out)


if __name__ == "__main__":
    main()
