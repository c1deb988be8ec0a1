"""Class-conditional latent DiT training through ``violaEngine`` with per-step JSONL logs and optional audits.

    python -m viola_b200 launch --config examples/distributed.yaml experiments/train_dit.py \
        --data /data/latents/mmap --output runs/xl2 --model xl_2 --batch 256
    python experiments/train_dit.py --synthetic 2048 --output runs/smoke --model tiny --max-steps 20

Objective: flow matching with v-prediction, ``z = (1 - t) x + t eps`` with logit-normal ``t``, target
``eps - x``; labels dropped to the unconditional class with probability 0.1; learning rate warmed up linearly
over 1000 updates (the recipe of the reference trainer, experiments/train_dit.py:108-205, which runs DDP;
here the engine provides sharding, gradient accumulation, EMA and checkpoints).

Data: ``--data DIR`` with ``latents.f32`` ([n, 2, 4, 32, 32]: VAE posterior mean and its horizontal flip),
``labels.i64`` and ``metadata.json`` as written by ``prepare_latents.py``; or ``--synthetic N`` for N random
latents (no files needed).  Noise, times and label drops of step s are drawn from one generator seeded with
``seed + 100000 + s`` for the global batch and sliced per rank, so runs with different GPU counts see the
same samples.

Outputs in ``--output``: ``settings.json`` (arguments, model, world size, SHA-256 of the sources),
``steps-rank{r}.jsonl`` (one record per update: loss, lr, seconds, peak memory, audit summary, fixed-probe
loss), ``metrics/`` (with ``--audit``), ``checkpoint/`` (engine checkpoint at the end and every
``--checkpoint-interval`` updates), ``complete.json``.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(Path(__file__).resolve().parent))

import viola_b200 as viola                                              # noqa: E402
from viola_b200.models import DiT, muon_parameter_groups                # noqa: E402

MODELS = {"xl_2": dict(width=1152, depth=28, heads=16, patch=2), "b_4": dict(width=768, depth=12, heads=12, patch=4),
          "tiny": dict(width=128, depth=2, heads=4, patch=4)}
LATENT_SCALE = 0.18215


class Latents:
    """Global batches of (latents, labels) in a fixed, seeded order; every rank takes its slice."""

    def __init__(self, args, rank, world):
        self.batch, self.local, self.rank = args.batch, args.batch // world, rank
        if args.synthetic:
            generator = torch.Generator().manual_seed(args.seed)
            self.count = args.synthetic
            self.data = torch.randn(self.count, 1, 4, 32, 32, generator=generator) / LATENT_SCALE
            self.labels = torch.randint(0, 1000, (self.count,), generator=generator)
            self.description = {"samples": self.count, "source": "synthetic N(0, 1) latents"}
        else:
            import numpy
            root = Path(args.data)
            self.description = json.loads((root / "metadata.json").read_text())
            self.count = self.description["samples"]
            self.data = numpy.memmap(root / "latents.f32", mode="r", dtype="float32", shape=(self.count, 2, 4, 32, 32))
            self.labels = numpy.memmap(root / "labels.i64", mode="r", dtype="int64", shape=(self.count,))
        self.seed = args.seed
        self.steps_per_epoch = self.count // self.batch

    def epoch(self, number):
        generator = torch.Generator().manual_seed(self.seed + number)
        order = torch.randperm(self.count, generator=generator)
        flips = torch.randint(0, self.data.shape[1], (self.count,), generator=generator)
        for index in range(self.steps_per_epoch):                       # an incomplete last batch is dropped
            first = index * self.batch + self.rank * self.local
            chosen = order[first:first + self.local]
            yield self.fetch(chosen, flips[chosen])

    def fetch(self, indices, variants):
        if isinstance(self.data, torch.Tensor):
            return self.data[indices, variants], self.labels[indices]
        rows = indices.numpy()
        import numpy
        return (torch.from_numpy(numpy.ascontiguousarray(self.data[rows, variants.numpy()])),
                torch.from_numpy(numpy.ascontiguousarray(self.labels[rows])))


@torch.no_grad()
def fixed_probe(engine, model, data, samples=1024, chunk=32):
    """Loss on a fixed subset with fixed noise and times (not a held-out set): comparable across runs and GPU counts."""
    device, rank, world = engine.device, engine.rank, engine.world_size
    samples = min(samples, data.count)
    generator = torch.Generator().manual_seed(1701)
    indices = torch.randperm(data.count, generator=generator)[:samples][rank::world]
    noise = torch.randn(samples, 4, 32, 32, generator=generator)[rank::world]
    times = torch.randn(samples, generator=generator).sigmoid()[rank::world]
    totals = torch.zeros(2, device=device, dtype=torch.float64)
    model.eval()
    for first in range(0, len(indices), chunk):
        chosen = indices[first:first + chunk]
        clean, labels = data.fetch(chosen, torch.zeros_like(chosen))
        clean = clean.to(device).float() * LATENT_SCALE
        eps, t = noise[first:first + chunk].to(device), times[first:first + chunk].to(device)
        mixed = (1 - t[:, None, None, None]) * clean + t[:, None, None, None] * eps
        with engine.autocast():
            prediction = model(mixed, t * 1000, labels.to(device)).float()
        totals[0] += (prediction - (eps - clean)).square().flatten(1).mean(1).sum()
        totals[1] += len(chosen)
    model.train()
    totals = engine.reduce(totals, reduction="sum")
    return (totals[0] / totals[1]).item()


def source_digests():
    digests = {}
    for folder in (Path(__file__).resolve().parent, ROOT / "viola_b200"):
        for path in sorted(folder.rglob("*.py")):
            digests[str(path.relative_to(ROOT))] = hashlib.sha256(path.read_bytes()).hexdigest()
    return digests


def parse():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--data", help="directory written by prepare_latents.py")
    source.add_argument("--synthetic", type=int, default=0, help="train on this many random latents instead")
    parser.add_argument("--output", required=True)
    parser.add_argument("--model", choices=sorted(MODELS), default="b_4")
    parser.add_argument("--epochs", type=int, default=10)
    parser.add_argument("--max-steps", type=int, default=0)
    parser.add_argument("--batch", type=int, default=256, help="global batch per update")
    parser.add_argument("--micro-batch", type=int, default=64, help="largest microbatch per rank")
    parser.add_argument("--lr", type=float, default=1e-4)
    parser.add_argument("--warmup", type=int, default=1000)
    parser.add_argument("--mode", default="balanced", choices=("fast", "balanced", "stable"))
    parser.add_argument("--momentum-dtype", default="fp8", choices=("fp8", "bf16"))
    parser.add_argument("--rounding", default="nearest", choices=("nearest", "stochastic"))
    parser.add_argument("--rounding-seed", type=int, default=0)
    parser.add_argument("--granularity", default="tile", choices=("tile", "block"))
    parser.add_argument("--tile-size", type=int)
    parser.add_argument("--block-shape", type=int, nargs=2)
    parser.add_argument("--adam-state-dtype", default="fp32", choices=("fp32", "bf16", "fp16"))
    parser.add_argument("--linear", default="fp8", choices=("fp8", "torch"), help="block matrices: viola Linear or nn.Linear")
    parser.add_argument("--scaling", default="current", choices=("current", "delayed", "grouped", "mxfp8"))
    parser.add_argument("--audit", action="store_true", help="record per-matrix FP8-vs-BF16 momentum diagnostics")
    parser.add_argument("--ns-interval", type=int, default=100)
    parser.add_argument("--probe-interval", type=int, default=500)
    parser.add_argument("--checkpoint-interval", type=int, default=0)
    parser.add_argument("--resume", help="engine checkpoint directory to continue from")
    parser.add_argument("--seed", type=int, default=20261029)
    return parser.parse_args()


def build_model(args, device):
    options = dict(MODELS[args.model])
    if args.linear == "fp8":
        with torch.device(device):
            return DiT(**options, linear_options=dict(scaling=args.scaling))
    model = DiT(**options)
    for block in model.blocks:                                           # plain layers, e.g. for CPU smoke runs
        for name in ("qkv", "proj", "fc1", "fc2", "ada"):
            layer = getattr(block, name)
            plain = torch.nn.Linear(layer.in_features, layer.out_features)
            setattr(block, name, plain)
    model.reset_parameters = lambda: None
    return model.to(device)


def main():
    args = parse()
    engine = viola.violaEngine()
    rank, world, device = engine.rank, engine.world_size, engine.device
    torch.manual_seed(args.seed)
    if device.type == "cuda":
        torch.backends.cuda.matmul.allow_tf32 = False
    local = args.batch // world
    micro = min(args.micro_batch, local)
    if args.batch % world or local % micro:
        raise SystemExit("--batch must divide by the world size and the local batch by the microbatch")
    accumulation = local // micro
    engine.accumulation_steps = accumulation                             # the batch arguments decide, not the YAML
    model = engine.prepare_model(build_model(args, device))
    if args.momentum_dtype == "fp8":
        optimizer_class = viola.optim.FP8Muon
    else:
        from momentum16 import Momentum16 as optimizer_class
    optimizer = engine.prepare_optimizer(lambda _: optimizer_class(
        muon_parameter_groups(model, lr=args.lr), mode=args.mode, ns_method="standard", rounding=args.rounding,
        rounding_seed=args.rounding_seed, granularity=args.granularity, tile_size=args.tile_size,
        block_shape=args.block_shape, adam_state_dtype=args.adam_state_dtype))
    scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: min((step + 1) / max(args.warmup, 1), 1.0))
    output = Path(args.output)
    output.mkdir(parents=True, exist_ok=True)
    audit = None
    if args.audit and args.momentum_dtype == "fp8":
        from audit import MomentumAudit
        audit = MomentumAudit(model, output / "metrics", rank, args.ns_interval)
        for record in engine.state.parameters.records:                   # masters report under the model's names
            master = engine.state.optimizer.parameters.get(record.index)
            if master is not None:
                audit.names[id(master)] = record.name
        optimizer.observer = audit
    if args.resume:
        engine.load_checkpoint(args.resume, scheduler=scheduler)
    data = Latents(args, rank, world)
    total_steps = args.epochs * data.steps_per_epoch
    if rank == 0:
        manifest = dict(vars(args), world_size=world, model_options=MODELS[args.model], accumulation=accumulation,
                        parameters=sum(r.numel for r in engine.state.parameters.records),
                        steps_per_epoch=data.steps_per_epoch, total_steps=total_steps, torch=torch.__version__,
                        sharding=engine.state.sharding, dataset=data.description,
                        objective="flow matching, v-prediction, logit-normal t, label drop 0.1",
                        data_remainder_policy="drop the incomplete global batch of every epoch",
                        comparison=("same-gradient BF16 shadow momentum and Newton-Schulz update" if audit
                                    else "independent run"), source_sha256=source_digests())
        (output / "settings.json").write_text(json.dumps(manifest, indent=2, default=str))
    log = (output / f"steps-rank{rank}.jsonl").open("a", buffering=1)
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats()
    step = engine.global_step
    finished = False
    for epoch in range(step // max(data.steps_per_epoch, 1), args.epochs):
        for index, (clean, labels) in enumerate(data.epoch(epoch)):
            if epoch * data.steps_per_epoch + index < step:
                continue                                                 # already done before the resume point
            begin = time.monotonic()
            if audit is not None:
                audit.step = step + 1
            clean = clean.to(device, non_blocking=True).float() * LATENT_SCALE
            labels = labels.to(device, non_blocking=True)
            generator = torch.Generator().manual_seed(args.seed + 100000 + step)
            window = slice(rank * local, (rank + 1) * local)
            noise = torch.randn(args.batch, 4, 32, 32, generator=generator)[window].to(device)
            times = torch.randn(args.batch, generator=generator).sigmoid()[window].to(device)
            dropped = (torch.rand(args.batch, generator=generator) < 0.1)[window].to(device)
            labels = labels.masked_fill(dropped, 1000)
            running = torch.zeros((), device=device)
            for first in range(0, local, micro):
                part = slice(first, first + micro)
                t = times[part]
                mixed = (1 - t[:, None, None, None]) * clean[part] + t[:, None, None, None] * noise[part]
                with engine.accumulate():
                    with engine.autocast():
                        prediction = model(mixed, t * 1000, labels[part])
                        loss = (prediction.float() - (noise[part] - clean[part])).square().mean()
                    engine.backward(loss)
                running += loss.detach() / accumulation
            updated = engine.step(optimizer, scheduler=scheduler)
            diagnostics = audit.finish(overflow=not updated) if audit is not None else {"momentum_dtype": args.momentum_dtype}
            step = engine.global_step
            record = {"step": step, "epoch": epoch + (index + 1) / data.steps_per_epoch,
                      "loss": engine.reduce(running).item(), "lr": scheduler.get_last_lr()[0], "updated": bool(updated),
                      "seconds": time.monotonic() - begin,
                      "peak_allocated_bytes": torch.cuda.max_memory_allocated() if device.type == "cuda" else 0,
                      **diagnostics}
            if args.probe_interval and step % args.probe_interval == 0:
                record["fixed_probe_loss"] = fixed_probe(engine, model, data)
            log.write(json.dumps(record) + "\n")
            if rank == 0 and (step <= 5 or step % 25 == 0):
                print(json.dumps(record), flush=True)
            if args.checkpoint_interval and step % args.checkpoint_interval == 0:
                engine.save_checkpoint(output / "checkpoint", scheduler=scheduler, extra={"epoch": epoch})
            if args.max_steps and step >= args.max_steps:
                finished = True
                break
        if audit is not None:
            audit.flush()
        if finished:
            break
    engine.save_checkpoint(output / "checkpoint", scheduler=scheduler, extra={"step": step})
    log.close()
    if rank == 0:
        (output / "complete.json").write_text(json.dumps(
            {"steps": step, "epochs_completed": step / max(data.steps_per_epoch, 1), "completed_at": time.time()}, indent=2))
    engine.close()
    if torch.distributed.is_initialized():
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
