"""Reference arm of the benchmark: the reference's own engine, layers and optimizer on DiT-XL/2.

Everything on this path comes from the installed reference package (``baseline/_ref``): its
``violaEngine``, ``viola.nn.Linear`` (TileLang kernels), ``viola.optim.FP8Muon`` and its own DiT
definition (``experiments/dit.py``, copied beside the install as ``reference_experiments_dit.py``
because pip installs the package only), resized to XL/2 through its constructor arguments.  The
block matrices are converted with the reference's ``Linear.from_float``.  Nothing from
``viola_b200`` is imported here.
"""

from __future__ import annotations

import json
import os
import time


def run(args, unavailable):
    import torch
    import torch.distributed as dist
    import viola
    try:
        import reference_experiments_dit as reference_dit
    except Exception as error:       # the model definition is not part of the pip-installed package
        return unavailable(f"reference DiT definition missing beside baseline/_ref: {error}")

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    accumulation, global_batch = 2, args.global_batch
    config = dict(num_processes=world, mixed_precision="bf16", gradient_accumulation_steps=accumulation,
                  sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True),
                  precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                  communication=dict(dtype="fp8", bucket_mb=25, fp8_format="e4m3", fp8_tile_size=256),
                  ema=dict(decay=0.9999, dtype="fp32"))
    try:
        engine = viola.violaEngine(config)
        torch.manual_seed(1234)
        model = reference_dit.DiT(width=1152, depth=28, heads=16, patch=2)
        for block in model.blocks:
            block.qkv = viola.nn.Linear.from_float(block.qkv)
            block.proj = viola.nn.Linear.from_float(block.proj)
            block.mlp[0] = viola.nn.Linear.from_float(block.mlp[0])
            block.mlp[2] = viola.nn.Linear.from_float(block.mlp[2])
            block.ada[1] = viola.nn.Linear.from_float(block.ada[1])
        model = engine.prepare_model(model)
        muon, adam = [], []
        for name, param in model.named_parameters():
            (muon if name.startswith("blocks.") and param.ndim == 2 else adam).append(param)
        engine.prepare_optimizer(lambda params: viola.optim.FP8Muon([
            dict(params=muon, use_muon=True, lr=1e-4, momentum=.95, weight_decay=.01, nesterov=True),
            dict(params=adam, use_muon=False, lr=1e-4, betas=(.9, .95), eps=1e-8, weight_decay=.01)],
            mode="balanced", ns_method="standard"))
    except Exception as error:
        return unavailable(f"reference engine set-up failed: {type(error).__name__}: {str(error).splitlines()[0][:160]}")

    device = engine.device
    micro = global_batch // (world * accumulation)
    betas = torch.linspace(1e-4, 2e-2, 1000, dtype=torch.float64, device=device)
    alphas = torch.cumprod(1 - betas, 0)
    sa, sb = alphas.sqrt().float(), (1 - alphas).sqrt().float()
    generator = torch.Generator().manual_seed(100 + rank)
    total = args.warmup + args.steps
    batches = [(torch.randn(micro, 4, 32, 32, generator=generator).to(device),
                torch.randint(0, 1000, (micro,), generator=generator).to(device),
                torch.randint(0, 1000, (micro,), generator=generator).to(device),
                torch.randn(micro, 4, 32, 32, generator=generator).to(device)) for _ in range(total * accumulation)]

    def step(index):
        for latents, labels, timesteps, noise in batches[index * accumulation:(index + 1) * accumulation]:
            noisy = sa[timesteps][:, None, None, None] * latents + sb[timesteps][:, None, None, None] * noise
            with engine.accumulate():
                with engine.autocast():
                    # the reference model multiplies t by 1000 itself
                    loss = torch.nn.functional.mse_loss(model(noisy, timesteps.float() / 1000, labels).float(), noise)
                engine.backward(loss)
        engine.step()
        return loss

    try:
        for index in range(args.warmup):
            step(index)
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for index in range(args.warmup, total):
            loss = step(index)
        stop.record()
        torch.cuda.synchronize()
        elapsed = torch.tensor([start.elapsed_time(stop)], device=device, dtype=torch.float64)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    except Exception as error:
        return unavailable(f"reference training step failed: {type(error).__name__}: {str(error).splitlines()[0][:160]}")
    if rank == 0:
        print(json.dumps({"impl": "reference", "metric": "DiT-XL/2 training images/sec",
                          "value": global_batch * args.steps / (elapsed.item() / 1000), "unit": "images/s",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": elapsed.item() / args.steps, "higher_is_better": True, "scaling": "strong",
                          "dtype": "bf16 autocast + fp8 linears", "data": "synthetic",
                          "config": {"model": "DiT-XL/2", "global_batch": global_batch, "seq_len": 256,
                                     "parallelism": f"dp{world} full sharding"}, "final_loss": float(loss)}), flush=True)
    time.sleep(0)
    return 0
