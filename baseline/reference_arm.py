"""Reference arm of the benchmark: the reference's own engine, layers and optimizer on DiT-XL/2.

Everything on this path comes from the installed reference package (``baseline/_ref``): its
``violaEngine``, ``viola.nn.Linear`` (TileLang kernels), ``viola.optim.FP8Muon`` and its own DiT
definition (``experiments/dit.py``, copied beside the install as ``reference_experiments_dit.py``
because pip installs the package only), resized to XL/2 through its constructor arguments.  The
block matrices are converted with the reference's ``Linear.from_float``.  Nothing from
``viola_b200`` is imported here.

Two measurements of the same K steps are taken, as for the other arm: device-timed with the
inputs resident on the GPU (``value``), and end to end on the host clock with every step's inputs
copied from pinned host memory and the loss read back (``e2e``).
"""

from __future__ import annotations

import json
import os
import time
import traceback


def _first_line(error):
    text = str(error).strip().splitlines()
    return f"{type(error).__name__}: {(text[0] if text else '')[:200]}"


def _where(error):
    """Innermost frame of the reference package that raised, as ``file:line``."""
    frames = [f for f in traceback.extract_tb(error.__traceback__) if "baseline/_ref" in f.filename or "/viola/" in f.filename]
    if not frames:
        return ""
    last = frames[-1]
    return f" at {last.filename.split('_ref/')[-1]}:{last.lineno}"


def run(args, unavailable, shim=None):
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
    named_config = global_batch == 256 and getattr(args, "model", "xl_2") == "xl_2"
    if getattr(args, "ref_microbatch", 0):
        # context runs only: same global batch, smaller microbatches, more accumulation steps
        accumulation = global_batch // (world * args.ref_microbatch)
        named_config = named_config and accumulation == 2
    config = dict(num_processes=world, mixed_precision="bf16", gradient_accumulation_steps=accumulation,
                  sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True),
                  precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                  communication=dict(dtype="fp8", bucket_mb=25, fp8_format="e4m3", fp8_tile_size=256),
                  ema=dict(decay=0.9999, dtype="fp32"))
    widths = dict(xl_2=dict(width=1152, depth=28, heads=16, patch=2), b_4=dict(width=768, depth=12, heads=12, patch=4),
                  tiny=dict(width=256, depth=2, heads=4, patch=4))[getattr(args, "model", "xl_2")]
    try:
        engine = viola.violaEngine(config)
        torch.manual_seed(1234)
        model = reference_dit.DiT(**widths)
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
        return unavailable(f"reference engine set-up failed: {_first_line(error)}{_where(error)}")

    device = engine.device
    micro = global_batch // (world * accumulation)
    betas = torch.linspace(1e-4, 2e-2, 1000, dtype=torch.float64, device=device)
    alphas = torch.cumprod(1 - betas, 0)
    sa, sb = alphas.sqrt().float(), (1 - alphas).sqrt().float()
    generator = torch.Generator().manual_seed(100 + rank)
    total = args.warmup + args.steps
    host = [tuple(t.pin_memory() for t in (torch.randn(micro, 4, 32, 32, generator=generator),
                                           torch.randint(0, 1000, (micro,), generator=generator),
                                           torch.randint(0, 1000, (micro,), generator=generator),
                                           torch.randn(micro, 4, 32, 32, generator=generator)))
            for _ in range(total * accumulation)]
    resident = [tuple(t.to(device) for t in items) for items in host]

    def step(index, from_host):
        source = host if from_host else resident
        for items in source[index * accumulation:(index + 1) * accumulation]:
            if from_host:
                items = tuple(t.to(device, non_blocking=True) for t in items)
            latents, labels, timesteps, noise = items
            noisy = sa[timesteps][:, None, None, None] * latents + sb[timesteps][:, None, None, None] * noise
            with engine.accumulate():
                with engine.autocast():
                    # the reference model multiplies t by 1000 itself
                    loss = torch.nn.functional.mse_loss(model(noisy, timesteps.float() / 1000, labels).float(), noise)
                engine.backward(loss)
        engine.step()
        return loss

    def timed(from_host):
        for index in range(args.warmup):
            loss = step(index, from_host)
            if from_host:
                loss.item()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        wall = time.perf_counter()
        for index in range(args.warmup, total):
            loss = step(index, from_host)
            if from_host:
                loss.item()
        stop.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - wall) * 1000.0
        dist.barrier()
        elapsed = torch.tensor([wall if from_host else start.elapsed_time(stop)], device=device, dtype=torch.float64)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return elapsed.item(), float(loss)

    try:
        began = time.perf_counter()
        device_ms, loss_value = timed(False)
        first_pass_s = time.perf_counter() - began
        e2e_ms, _ = timed(True)
    except Exception as error:
        reason = f"reference training step failed: {_first_line(error)}{_where(error)}"
        if "scalable vector" in str(error) or "eval_vec_" in str(error):
            # second-stage failure under the TileLang of this image (0.1.9; the reference pins 0.1.15): its
            # amax -> scale kernel holds next_pow2(numel / 2048) floats in one fragment and does not lower once a
            # quantised tensor exceeds 2^25 elements, i.e. above 16 images per microbatch for DiT-XL/2
            reason += (f" [microbatch of {micro} images; the reference's _scale_kernel does not lower under TileLang "
                       "0.1.9 for tensors above 2^25 elements; it runs at <= 16 images per microbatch, which the named "
                       "config reaches at 8 GPUs]")
        return unavailable(reason)
    if rank == 0:
        bytes_in = sum(t.numel() * t.element_size() for t in host[0]) * accumulation
        print(json.dumps({"impl": "reference", "metric": "DiT-XL/2 training images/sec",
                          "value": global_batch * args.steps / (device_ms / 1000), "unit": "images/s",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                          "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "bf16 autocast + fp8 linears", "data": "synthetic",
                          "config": {"model": "DiT-XL/2", "global_batch": global_batch, "seq_len": 256,
                                     "parallelism": f"dp{world} full sharding (parameters+gradients+optimizer+ema)",
                                     "grad_accumulation": accumulation, "named_config": named_config,
                                     "engine": "reference violaEngine + viola.nn.Linear (TileLang) + FSDP2 + NCCL"},
                          "shim": shim, "final_loss": loss_value, "first_pass_seconds_incl_jit": first_pass_s,
                          "e2e": {"value": global_batch * args.steps / (e2e_ms / 1000), "unit": "images/s",
                                  "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": bytes_in,
                                  "d2h_bytes_per_step": 4,
                                  "timing": "host wall clock around K steps incl. pinned H2D copies and loss.item(), "
                                            "max over ranks"}}), flush=True)
    engine.close()
    return 0
