"""Small, self-terminating workloads for Nsight Compute captures of single kernels.

Each case allocates a few hundred MB (more than the 126 MB L2, far less than a few GB), launches
the kernel of interest a handful of times and exits.  Meant to be run as

    python benchmarks/profile_case.py --case gemm_fp8 &&
    ncu --set full --clock-control none -k regex:gemm_kernel -s 2 -c 1 -o out python benchmarks/profile_case.py --case gemm_fp8
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from viola_b200 import ops  # noqa: E402

E4M3 = torch.float8_e4m3fn


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--case", required=True,
                        choices=("gemm_fp8", "gemm_group", "gemm_ns", "gemm_ns_apply", "gemm_act_bwd", "gemm_wgrad",
                                 "gemm_expert", "quantize", "quantize_rows", "group_quantize", "momentum", "gated",
                                 "gated_bwd", "attention", "attention_library",
                                 "ln_quantize", "gelu_quantize", "ln_backward", "gate_backward", "gemm_mx", "writeback",
                                 "reduce_push", "reduce_accumulate", "gather_pull"))
    parser.add_argument("--launches", type=int, default=4)
    args = parser.parse_args()
    device = torch.device("cuda")
    ops.load()
    torch.manual_seed(0)
    m, n, k = 32768, 3456, 1152
    if args.case in ("gemm_fp8", "gemm_group", "gated"):
        x = torch.randn(m, k, device=device, dtype=torch.bfloat16)
        w = torch.randn(n, k, device=device, dtype=torch.bfloat16) * 0.03
        if args.case == "gemm_fp8":
            sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
            qx, _ = ops.quantize(x, sx)
            qw, _ = ops.quantize(w, sw)
            out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
            run = lambda: ops.gemm(qx, qw, sx, sw, out_dtype=torch.bfloat16, out=out)
        elif args.case == "gemm_group":
            qx, sx = ops.group_quantize(x, E4M3, (1, 128), kmajor=True)
            qw, sw = ops.group_quantize(w, E4M3, (128, 128))
            out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
            run = lambda: ops.group_gemm(qx, qw, sx, sw, (1, 128), (128, 128), out_dtype=torch.bfloat16, sa_kmajor=True,
                                         out=out)
        else:
            sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
            qx, _ = ops.quantize(x, sx)
            qw, _ = ops.quantize(w, sw)
            run = lambda: ops.gated_gemm_forward(qx, qw, sx, sw, activation="silu", out_dtype=torch.bfloat16)
    elif args.case == "gated_bwd":
        # [dGate | dUp] of a gated MLP from the epilogue of dY @ Wdown: M = 32768, hidden 1728, model width 1152
        hidden, width = 1728, 1152
        dy = torch.randn(m, width, device=device, dtype=torch.bfloat16)
        wdown_t = torch.randn(hidden, width, device=device, dtype=torch.bfloat16) * 0.03
        saved = torch.randn(m, 2 * hidden, device=device, dtype=torch.bfloat16)
        sg, st = ops.tensor_scale(dy, fp8_dtype=torch.float8_e5m2), ops.tensor_scale(wdown_t)
        qg, _ = ops.quantize(dy, sg, fp8_dtype=torch.float8_e5m2)
        qt, _ = ops.quantize(wdown_t, st)
        run = lambda: ops.gated_gemm_backward(qg, qt, sg, st, saved, activation="silu", out_dtype=torch.bfloat16)
    elif args.case in ("attention", "attention_library"):
        # DiT-XL/2 attention at 128 images: 256 tokens, 16 heads of 72, packed qkv [B, T, 3, H, D] in bf16
        qkv = torch.randn(128, 256, 3, 16, 72, device=device, dtype=torch.bfloat16)
        if args.case == "attention":
            run = lambda: ops.attention_forward(qkv)
        else:
            from flash_attn import flash_attn_qkvpacked_func
            run = lambda: flash_attn_qkvpacked_func(qkv)
    elif args.case == "gemm_mx":
        # hardware block-scaled MXFP8 product, UE8M0 scale per 32 K elements on both operands
        a = torch.randn(m, k, device=device).to(E4M3)
        b = torch.randn(n, k, device=device).to(E4M3)
        sa = torch.randint(120, 132, (m, k // 32), device=device, dtype=torch.uint8)
        sb = torch.randint(120, 132, (n, k // 32), device=device, dtype=torch.uint8)
        sfa, sfb = ops.mx_pack_scales(sa, m, k), ops.mx_pack_scales(sb, n, k)
        out = torch.empty(m, n, device=device, dtype=torch.bfloat16)
        run = lambda: ops.mx_gemm(a, b, sfa, sfb, out_dtype=torch.bfloat16, out=out)
    elif args.case == "writeback":
        # an owner's write-back of 60 FP8 layers (about 320 MB of fp32 masters) with the EMA folded in; one
        # process, so every "peer" store lands in local memory (the NVLink leg is not exercised)
        shapes = [(1152, 3456), (1152, 1152), (1152, 4608), (4608, 1152), (6912, 1152)] * 12
        masters = [torch.randn(s, device=device) * 0.02 for s in shapes]
        averages = [t.clone() for t in masters]
        codes = [torch.zeros(t.numel(), device=device, dtype=torch.uint8) for t in masters]
        headers = torch.zeros(len(shapes), 32, device=device)
        rows = [dict(master=t, ema=e, n=t.numel(), slab_elems=t.numel(), dst_offset=c.data_ptr(),
                     header_offset=h.data_ptr(), base_index=0, limit=448.0, history_len=16, mode=0, out_dtype=None)
                for t, e, c, h in zip(masters, averages, codes, headers)]
        table = ops.WritebackTable(rows, device)
        calls = iter(range(1 << 30))
        run = lambda: ops.multi_writeback(table, heaps=[0], rank=0, calls=next(calls), decay=0.9999, with_ema=True)
    elif args.case in ("reduce_push", "reduce_accumulate"):
        # one 256 MB fp32 gradient bucket through the FP8 wire codec (e4m3, tile 256); destination / source slots
        # are local buffers, flags are pre-set, so a single process can run the kernels of either side
        count, tile = 64 << 20, 256
        tiles = count // tile
        bucket = torch.randn(count, device=device) * 1e-3
        slot_bytes = tiles * tile + tiles * 4
        slot = torch.zeros(2 * slot_bytes, device=device, dtype=torch.uint8)          # one receive slot per "rank"
        flags = torch.full((4,), 1 << 30, device=device, dtype=torch.int32)
        generation = torch.ones(1, device=device, dtype=torch.int32)
        counter = torch.zeros(1, device=device, dtype=torch.int32)
        status = ops.status_word(device)
        accum = torch.zeros(count, device=device)
        op = torch.ops.viola_b200
        if args.case == "reduce_push":
            run = lambda: op.reduce_push_fp8(bucket, tile, 0, slot.data_ptr(), slot.data_ptr() + tiles * tile,
                                             flags.data_ptr(), flags.data_ptr() + 4, generation, counter, 2_000_000, 296,
                                             status)
        else:
            heap = torch.zeros(1 << 16, device=device, dtype=torch.uint8)
            run = lambda: op.reduce_accumulate_fp8(bucket, tile, 0, slot.data_ptr(), slot_bytes, tiles * tile,
                                                   flags.data_ptr(), [heap.data_ptr(), heap.data_ptr()], 0, 64, generation,
                                                   accum, counter, 2_000_000, 296, status)
    elif args.case == "gather_pull":
        # the pull of one sharding unit (24 MB of FP8 codes in five parameters) with both "ranks" in local memory
        world, sizes = 2, [1152 * 3456, 1152 * 1152, 1152 * 4608, 4608 * 1152, 6912 * 1152]
        shard_bytes = [size // world for size in sizes]
        region = torch.randint(0, 255, (sum(shard_bytes),), device=device, dtype=torch.uint8)
        full = torch.zeros(sum(sizes), device=device, dtype=torch.uint8)
        entries, prefix, total, shard_at, full_at = [], [0], 0, 0, 0
        for nbytes in shard_bytes:
            entries += [shard_at, nbytes, full_at]
            shard_at += nbytes
            full_at += world * nbytes
        for nbytes in shard_bytes:
            for _ in range(world):
                total += (nbytes + 65535) // 65536
                prefix.append(total)
        entries_t = torch.tensor(entries, device=device, dtype=torch.int64)
        prefix_t = torch.tensor(prefix, device=device, dtype=torch.int64)
        counts = torch.zeros(len(shard_bytes) * world, device=device, dtype=torch.int32)
        panel = torch.zeros(len(shard_bytes) * world, device=device, dtype=torch.int32)
        calls = iter(range(1, 1 << 30))
        run = lambda: torch.ops.viola_b200.gather_pull(entries_t, [region.data_ptr()] * world, 0, 0, full, prefix_t,
                                                       counts, panel, next(calls), total, 1184)
    elif args.case == "gemm_ns":
        x = (torch.randn(28, 1152, 4608, device=device) / 68).bfloat16()
        run = lambda: ops.ns_gemm(x, x, symmetric=True)
    elif args.case == "gemm_ns_apply":
        # the third product of a Newton-Schulz step: X' = 3.4445 X + P X for a stack of wide matrices
        x = (torch.randn(14, 1152, 3456, device=device) / 59).bfloat16()
        p = (torch.randn(14, 1152, 1152, device=device) / 34).bfloat16()
        out = torch.empty_like(x)
        run = lambda: ops.ns_gemm(p, x, alpha=1.0, beta=3.4445, resid=x, out=out, b_mn=True)
    elif args.case == "gemm_act_bwd":
        # fc2 dgrad with the activation slope in the epilogue: dZ = (dY W) * act'(z)
        rows = 16384
        dy = torch.randn(rows, 1152, device=device).to(torch.float8_e5m2)
        w = (torch.randn(1152, 4608, device=device) * 0.03).to(E4M3)
        slope = torch.rand(rows, 4608, device=device).bfloat16()
        one = torch.ones(1, device=device)
        amax = ops.amax_word(device)
        run = lambda: ops.activation_backward_gemm(dy, w, one, one, slope, w_mn=True, amax_out=amax)
    elif args.case == "gemm_wgrad":
        # dW = dY^T X for the attention projection: 1152x1152 output, K = 32768 tokens, both operands MN-major
        dy = torch.randn(m, 1152, device=device).to(torch.float8_e5m2)
        xq = torch.randn(m, 1152, device=device).to(E4M3)
        one = torch.ones(1, device=device)
        run = lambda: ops.gemm(dy, xq, one, one, out_dtype=torch.float32, a_mn=True, b_mn=True)
    elif args.case == "gemm_expert":
        experts, tokens, width, hidden = 8, 1024, 4096, 14336
        x = torch.randn(experts * tokens, width, device=device, dtype=torch.bfloat16)
        w = torch.randn(experts, hidden, width, device=device, dtype=torch.bfloat16) * 0.02
        offsets = torch.arange(0, experts * tokens + 1, tokens, device=device, dtype=torch.int32)
        sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
        qx, _ = ops.quantize(x, sx)
        qw, _ = ops.quantize(w.view(-1, width), sw)
        run = lambda: ops.expert_gemm(qx, qw.view(experts, hidden, width), offsets, sx, sw, out_dtype=torch.bfloat16)
    elif args.case == "quantize_rows":
        # output-gradient encode of a linear layer: row-wise e5m2 codes plus the bias gradient (column sums)
        x = torch.randn(m, 4608, device=device, dtype=torch.bfloat16)
        scale = ops.tensor_scale(x, fp8_dtype=torch.float8_e5m2)
        colsum = torch.zeros(4608, device=device)
        run = lambda: ops.quantize(x, scale, fp8_dtype=torch.float8_e5m2, colsum=colsum)
    elif args.case in ("ln_quantize", "ln_backward", "gate_backward"):
        tokens, width = 256, 1152
        x = torch.randn(m, width, device=device)                      # fp32 residual stream
        mod = (torch.randn(m // tokens, 3 * width, device=device) * 0.3).bfloat16()
        shift, scale, gate = mod.chunk(3, dim=-1)
        if args.case == "ln_quantize":
            run = lambda: ops.ln_modulate_quantize(x, shift, scale, tokens)
        elif args.case == "ln_backward":
            _, _, _, mean, rstd = ops.ln_modulate_quantize(x, shift, scale, tokens)
            dh = torch.randn(m, width, device=device, dtype=torch.bfloat16)
            run = lambda: ops.ln_modulate_backward(dh, x, mean, rstd, scale, tokens)
        else:
            y = torch.randn(m, width, device=device, dtype=torch.bfloat16)
            run = lambda: ops.gate_residual_backward(x, gate, y, tokens)
    elif args.case == "gelu_quantize":
        z = torch.randn(m, 4608, device=device, dtype=torch.bfloat16)
        run = lambda: ops.activation_quantize(z, "gelu", slope=True)
    elif args.case == "quantize":
        x = torch.randn(m, 4608, device=device, dtype=torch.bfloat16)
        scale = ops.tensor_scale(x)
        run = lambda: ops.quantize(x, scale, transpose=True)
    elif args.case == "group_quantize":
        x = torch.randn(m, 4608, device=device, dtype=torch.bfloat16)
        run = lambda: ops.group_quantize_pair(x, E4M3, (1, 128), (1, 128), kmajor=True)
    else:
        count = 4096 * 11008
        grad = torch.randn(count, device=device)
        q = torch.zeros(count, device=device, dtype=torch.uint8)
        scale = torch.ones(count // 256, device=device)
        update = torch.empty(count, device=device, dtype=torch.bfloat16)
        run = lambda: ops.momentum_update(grad, q, scale, q, scale, update, beta=0.95)
    run()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.launches - 1):
        run()
    stop.record()
    torch.cuda.synchronize()
    ops.check_status()
    per_call = start.elapsed_time(stop) / max(args.launches - 1, 1)
    print("ok", args.case, f"{per_call * 1000:.1f} us per call (CUDA events, {args.launches - 1} calls after one warm-up)")


if __name__ == "__main__":
    main()
