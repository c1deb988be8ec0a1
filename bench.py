"""Headline benchmark: DiT-XL/2 class-conditional latent-diffusion training, images per second.

Configuration (the reference's headline workload): 28 blocks x width 1152 x 16 heads, patch 2,
adaLN-Zero; latents 4x32x32; global batch 256 with gradient accumulation 2; bf16 autocast with FP8
linears and FP8 weight storage; FP8Muon on the hidden matrices and AdamW elsewhere; engine with
full parameter / gradient / optimizer / EMA sharding, fp32 masters, FP8 e4m3 gradient
communication (tile 256, 25 MB buckets), EMA 0.9999.  Synthetic data, random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the
inputs already resident on the GPU; ``e2e`` repeats the measurement through the same public API
with every step's inputs copied from pinned host memory and the step's loss read back.  A fresh
batch (larger than nothing but far smaller than L2) is used every step, and the model's ~40 GB of
activations per microbatch cycle through HBM, so no step can be served from L2.

``--impl reference`` runs the unmodified reference package installed under ``baseline/_ref``
through its own engine on the same workload, or reports why it cannot.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 256
ACCUMULATION = 2
CLASSES = 1000


def parse():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--model", default="xl_2", choices=("xl_2", "b_4", "tiny"))
    parser.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    parser.add_argument("--scaling", default="current", choices=("current", "delayed", "grouped"))
    parser.add_argument("--backend", default="auto", choices=("auto", "p2p", "nccl"))
    parser.add_argument("--ref-microbatch", type=int, default=0,
                        help="reference arm only: images per microbatch (raises the accumulation steps above the "
                             "named config's 2 to keep the global batch); 0 = the named config")
    parser.add_argument("--ref-timeout", type=float, default=900.0,
                        help="reference arm: seconds after which it prints an 'unavailable' line and exits 0 "
                             "(its TileLang kernels compile during the first pass, eight ranks at once take long)")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--no-graph", action="store_true", help="run every microbatch eagerly (no CUDA graph)")
    parser.add_argument("--resident", default="auto", choices=("auto", "true", "false"),
                        help="sharding.resident: keep gathered parameters between uses (auto: when one copy is small)")
    parser.add_argument("--overlap", action="store_true", help="communication.overlap: reduce buckets during backward")
    parser.add_argument("--autotune", action="store_true",
                        help="first-use tile search for every GEMM shape during the eager warm-up microbatch")
    parser.add_argument("--no-phases", action="store_true", help="skip the extra untimed steps that measure phase times")
    return parser.parse_args()


class ClockSampler:
    """Samples SM clock, power and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.process, self.lines, self.first = index, None, [], 0

    def mark(self):
        """The timed region starts here: only samples that arrive from now on are reported (the process is started
        earlier, during warm-up, because nvidia-smi needs a few hundred milliseconds before its first sample)."""
        self.first = len(self.lines)

    def start(self):
        try:
            self.process = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                             "--format=csv,noheader,nounits", "-lms", "100"],
                                            stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.process is not None:
            self.process.terminate()
        clocks, maxima, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        lines = self.lines[self.first:] or self.lines[-3:]     # a region shorter than one period: the samples of the
        for line in lines:                                     # identical warm-up steps right before it
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                maxima.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        return dict(sm_mhz=statistics.median(clocks), sm_max_mhz=max(maxima), reasons=sorted(reasons),
                    samples=len(clocks))


def model_options(name):
    if name == "xl_2":
        return dict(width=1152, depth=28, heads=16, patch=2), "DiT-XL/2"
    if name == "b_4":
        return dict(width=768, depth=12, heads=12, patch=4), "DiT-B/4"
    return dict(width=256, depth=2, heads=4, patch=4), "DiT-tiny"


def engine_config(args):
    return dict(num_processes=args.gpus, mixed_precision="bf16", gradient_accumulation_steps=ACCUMULATION,
                sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True,
                              resident={"auto": "auto", "true": True, "false": False}[args.resident]),
                precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                communication=dict(dtype="fp8", bucket_mb=25, fp8_format="e4m3", fp8_tile_size=256,
                                   backend=args.backend, overlap=args.overlap),
                ema=dict(decay=0.9999, dtype="fp32"))


def synthetic_batches(count, micro_batch, seed, pinned):
    """``count`` microbatches of (latents, labels, timesteps, noise) on the host (pinned if asked)."""
    import torch
    generator = torch.Generator().manual_seed(seed)
    batches = []
    for _ in range(count):
        items = (torch.randn(micro_batch, 4, 32, 32, generator=generator),
                 torch.randint(0, CLASSES, (micro_batch,), generator=generator),
                 torch.randint(0, 1000, (micro_batch,), generator=generator),
                 torch.randn(micro_batch, 4, 32, 32, generator=generator))
        batches.append(tuple(t.pin_memory() if pinned else t for t in items))
    return batches


def phase_breakdown(engine, train_step, *, resident_batches, steps, world):
    """Per-phase device milliseconds of a step, from CUDA events around the engine's phases during ``steps`` extra
    steps after the timed regions (these steps are not part of any reported throughput).

    ``fp8muon_ms_per_step`` is the optimizer phase (momentum, Newton-Schulz, weight and AdamW updates);
    ``exposed_comm_ms_per_step`` adds up what communication costs on the compute stream of this rank outside the
    captured microbatches: the step's usage / status exchange and replicated-gradient reduction (``reduce``), the
    owners' write-back with its barriers and the parameter re-gather (``writeback``).  Reduction kernels inside a
    captured microbatch are part of ``microbatch``.  Maxima over ranks."""
    import torch
    import torch.distributed as dist
    from viola_b200 import utils
    from viola_b200.utils.trace import phase
    utils.enable_timing(True)
    for index in range(steps):
        with phase("step_total"):
            train_step(resident_batches[index * ACCUMULATION:(index + 1) * ACCUMULATION], False)
    times = utils.phase_times()
    utils.enable_timing(False)
    names = ("step_total", "microbatch", "backward", "reduce", "optimizer", "writeback", "ema")
    values = torch.tensor([times.get(name, 0.0) / steps for name in names], device=engine.device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(values, op=dist.ReduceOp.MAX)
    per_phase = {name: round(v, 3) for name, v in zip(names, values.tolist()) if v}
    return {"phases_ms_per_step": per_phase, "fp8muon_ms_per_step": per_phase.get("optimizer"),
            "exposed_comm_ms_per_step": round(per_phase.get("reduce", 0.0) + per_phase.get("writeback", 0.0), 3)}


def run_ours(args):
    import torch
    import torch.distributed as dist
    import viola_b200 as viola
    from viola_b200 import ops
    from viola_b200.models import DiT, NoiseSchedule, diffusion_loss, muon_parameter_groups
    from viola_b200.utils.trace import phase

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    if args.autotune:
        from viola_b200 import tuning
        tuning.enable()
    engine = viola.violaEngine(engine_config(args))
    device = engine.device
    options, model_name = model_options(args.model)
    torch.manual_seed(1234)
    linear_options = dict(scaling=args.scaling)
    if args.scaling == "grouped":
        linear_options.update(weight_group_shape=(128, 128), input_group_shape=(1, 128), grad_group_shape=(1, 128))
    with torch.device(device):          # build (and quantise) the weights on the GPU, not on the host
        model = DiT(**options, linear_options=linear_options)
    model = engine.prepare_model(model)
    engine.prepare_optimizer(lambda params: viola.optim.FP8Muon(muon_parameter_groups(model), mode="balanced",
                                                                ns_method="standard"))
    schedule = NoiseSchedule(device=device)
    micro_batch = args.global_batch // (world * ACCUMULATION)
    assert micro_batch * world * ACCUMULATION == args.global_batch

    total_steps = args.warmup + args.steps
    host = synthetic_batches(total_steps * ACCUMULATION, micro_batch, 100 + rank, pinned=True)
    resident_list = [tuple(t.to(device) for t in items) for items in host]

    def microbatch_loss(latents, labels, timesteps, noise):
        return diffusion_loss(model, schedule, latents, labels, timesteps, noise)

    graphed = None if args.no_graph else engine.graph_microbatch(microbatch_loss, *resident_list[0])

    def train_step(microbatches, from_host):
        last = None
        for items in microbatches:
            if graphed is not None:
                with phase("microbatch"):
                    last = graphed(*items)          # pinned host tensors are copied H2D asynchronously inside
                continue
            if from_host:
                items = tuple(t.to(device, non_blocking=True) for t in items)
            with engine.accumulate():
                with engine.autocast():
                    loss = microbatch_loss(*items)
                engine.backward(loss)
            last = loss
        engine.step()
        return last

    def timed(from_host):
        source = host if from_host else resident_list
        sampler = ClockSampler(device.index)
        sampler.start()
        for step in range(args.warmup):
            loss = train_step(source[step * ACCUMULATION:(step + 1) * ACCUMULATION], from_host)
            if from_host:
                loss.item()
        dist.barrier()
        torch.cuda.synchronize()
        launches_before = ops.launch_count
        sampler.mark()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        wall = time.perf_counter()
        for step in range(args.warmup, total_steps):
            loss = train_step(source[step * ACCUMULATION:(step + 1) * ACCUMULATION], from_host)
            if from_host:
                loss.item()                         # device -> host read of the step's result
        stop.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - wall
        dist.barrier()
        clocks = sampler.stop()
        elapsed = torch.tensor([start.elapsed_time(stop) if not from_host else wall * 1000.0], device=device,
                               dtype=torch.float64)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return elapsed.item(), clocks, ops.launch_count - launches_before, float(loss)

    device_ms, clocks, launches, loss_value = timed(from_host=False)
    ops.check_status()
    transport = "peer memory (fused NVLink kernels, no NCCL on the step)" if engine.transport is not None else (
        "none (single GPU)" if world == 1 else f"NCCL collectives ({engine.transport_reason or 'requested'})")
    resident = bool(engine.sharder is not None and engine.sharder.resident)
    result = {
        "metric": "DiT-XL/2 training images/sec" if args.model == "xl_2" else f"{model_name} training images/sec",
        "value": args.global_batch * args.steps / (device_ms / 1000.0),
        "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": device_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16 autocast + fp8 (e4m3 fwd / e5m2 bwd) linears", "data": "synthetic", "impl": "ours",
        "config": {"model": model_name, "global_batch": args.global_batch, "seq_len": 256 if args.model == "xl_2" else None,
                   "parallelism": f"dp{world} full sharding (parameters+gradients+optimizer+ema)",
                   "grad_accumulation": ACCUMULATION, "linear_scaling": args.scaling,
                   "optimizer": "FP8Muon(balanced, standard NS) + AdamW", "ema": 0.9999,
                   "grad_comm": "fp8 e4m3 tile 256, 25 MB buckets",
                   "cache": "fresh inputs every step; per-microbatch activations exceed L2 by >100x",
                   "cuda_graph": graphed is not None, "tile_tuner": bool(args.autotune), "transport": transport,
                   "gathered_parameters_resident": resident, "comm_overlap": bool(args.overlap)},
        "clocks": clocks, "gpu_launches": launches, "final_loss": loss_value,
    }
    if not args.no_e2e:
        e2e_ms, e2e_clocks, _, _ = timed(from_host=True)
        bytes_in = sum(t.numel() * t.element_size() for t in host[0]) * ACCUMULATION
        result["e2e"] = {"value": args.global_batch * args.steps / (e2e_ms / 1000.0), "unit": "images/s",
                         "ms_per_step": e2e_ms / args.steps, "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": 4,
                         "timing": "host wall clock around K steps incl. pinned H2D copies and loss.item(), max over ranks",
                         "clocks": e2e_clocks}
    if not args.no_phases:
        result.update(phase_breakdown(engine, train_step, resident_batches=resident_list,
                                      steps=2, world=world))
    engine.close()
    if rank == 0:
        print(json.dumps(result), flush=True)
    dist.barrier()
    dist.destroy_process_group()


REFERENCE_SHIM = "sys.modules alias tilelang.cuda[.intrinsics] -> tilelang.intrinsics (harness only)"


def alias_tilelang_intrinsics():
    """Make ``tilelang.cuda.intrinsics`` importable on a TileLang that ships the same classes elsewhere.

    The reference's kernel modules do ``from tilelang.cuda.intrinsics import TensorCoreIntrinEmitter``
    (its pinned TileLang 0.1.15 layout); TileLang 0.1.9 exposes that class as
    ``tilelang.intrinsics.TensorCoreIntrinEmitter``.  Two ``sys.modules`` entries in this harness bridge
    the two layouts; nothing under ``baseline/_ref`` is edited.  Returns True when the alias was needed.
    """
    import importlib
    import types
    try:
        importlib.import_module("tilelang.cuda.intrinsics")
        return False
    except ImportError:
        pass
    intrinsics = importlib.import_module("tilelang.intrinsics")
    package = types.ModuleType("tilelang.cuda")
    package.__path__ = []
    package.intrinsics = intrinsics
    sys.modules["tilelang.cuda"] = package
    sys.modules["tilelang.cuda.intrinsics"] = intrinsics
    return True


def run_reference(args):
    """The unmodified reference package from baseline/_ref, driven through its own engine."""
    rank = int(os.environ.get("RANK", 0))
    reference_root = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(reason):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": reason, "shim": REFERENCE_SHIM}), flush=True)
        return 0

    if not os.path.isdir(os.path.join(reference_root, "viola")):
        return unavailable("baseline/_ref is not installed (pip --no-index --no-deps --target baseline/_ref)")
    # JIT results of the reference's TileLang kernels are kept beside the install, so a box that
    # receives this folder with a warm cache does not compile them again
    os.environ.setdefault("TILELANG_CACHE_DIR", os.path.join(reference_root, "tilelang_cache"))
    sys.path.insert(0, reference_root)
    if "RANK" not in os.environ:       # single process without a launcher: the reference engine reads env://
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29534")
        os.environ.update(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    try:
        shimmed = alias_tilelang_intrinsics()
        import viola  # noqa: F401  (the reference package)
    except Exception as error:
        return unavailable(f"import viola failed: {type(error).__name__}: {str(error).splitlines()[0][:160]}")
    from baseline.reference_arm import run

    def give_up():
        unavailable(f"the reference did not finish within {args.ref_timeout:.0f} s on {args.gpus} GPU(s): its first pass "
                    "JIT-compiles the TileLang kernels of this world size's shapes (results are cached under "
                    "baseline/_ref/tilelang_cache for the next run)")
        sys.stdout.flush()
        os._exit(0)

    watchdog = threading.Timer(args.ref_timeout, give_up)
    watchdog.daemon = True
    watchdog.start()
    try:
        return run(args, unavailable, REFERENCE_SHIM if shimmed else None)
    finally:
        watchdog.cancel()


if __name__ == "__main__":
    arguments = parse()
    if arguments.impl == "reference":
        sys.exit(run_reference(arguments) or 0)
    run_ours(arguments)
