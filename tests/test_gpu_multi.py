"""Fused peer-memory communication paths on 2+ GPUs, against the collective-library path and the
fake-quant oracle (bounds of checks/fp8_communication.py:75: reduce-to-owner < 2e-6, all-reduce with
two quantisations < 3e-3 relative L2), plus the bounded-wait failure path on one GPU.
"""
import os
import socket
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import rel_l2

pytestmark = pytest.mark.gpu
GPUS = torch.cuda.device_count() if torch.cuda.is_available() else 0


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def launch(target, world, *args):
    context = mp.get_context("spawn")
    results = context.Queue()
    port = free_port()
    processes = [context.Process(target=target, args=(rank, world, port, *args, results)) for rank in range(world)]
    for process in processes:
        process.start()
    # fail fast: a rank that dies must not leave its peers waiting in a collective
    deadline = time.time() + 300
    while any(process.exitcode is None for process in processes) and time.time() < deadline:
        if any(process.exitcode not in (None, 0) for process in processes):
            break
        time.sleep(0.2)
    for process in processes:
        if process.exitcode is None:
            process.join(timeout=5)
        if process.exitcode is None:
            process.kill()
            process.join()
    codes = [process.exitcode for process in processes]
    assert all(code == 0 for code in codes), codes
    return [results.get(timeout=5) for _ in processes]


def setup(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)


def fake_quant(x, tile, fmt):
    limit = 448.0 if fmt == torch.float8_e4m3fn else 57344.0
    padded = torch.nn.functional.pad(x, (0, (-x.numel()) % tile)).view(-1, tile)
    amax = padded.abs().amax(1, keepdim=True).clamp_min(1e-30)
    scale = amax / torch.full_like(amax, limit)      # tensor / tensor is a true division (scalar divisors are not)
    return ((padded / scale).to(fmt).float() * scale).flatten()[:x.numel()]


def collectives_worker(rank, world, port, results):
    setup(rank, world, port)
    import viola_b200 as viola
    from viola_b200 import ops
    from viola_b200.parallel.symm import PeerTransport
    engine = viola.violaEngine(dict(communication=dict(dtype="fp8", backend="p2p")))
    device = engine.device
    tile, fmt = 256, torch.float8_e4m3fn
    for n in (1000, 70_001, 3_000_000):
        torch.manual_seed(n + rank)
        local = torch.randn(n, device=device) * 1e-3
        local[::997] *= 100
        gathered = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        # ---- path 1: reduce to owner (two generations to exercise the ack flow) ----
        transport = PeerTransport(engine, tile_size=tile)
        owner = 1 % world
        accum = torch.zeros(n, device=device) if rank == owner else None
        transport.attach_gradients([(owner, [], n)], [accum], n)
        transport.finalize()
        transport.finalize_gradients()
        expected = torch.zeros(n, device=device)
        for generation in range(2):
            transport.begin_microbatch()
            index, staging = transport.next_staging()
            staging[:n].copy_(local * (generation + 1))
            transport.reduce_to_owner(0, index, n)
            for source in gathered:
                expected += fake_quant(source * (generation + 1), tile, fmt)
        transport.synchronize()
        torch.cuda.synchronize()
        ops.check_status()
        if rank == owner:
            assert rel_l2(accum, expected) < 2e-6, (n, rel_l2(accum, expected))
        dist.barrier()
        # ---- path 2: all-reduce with requantisation ----
        transport = PeerTransport(engine, tile_size=tile)
        transport.attach_all_reduce(n)
        transport.finalize()
        transport.finalize_all_reduce()
        value = local.clone()
        transport.all_reduce(value)
        again = local.clone()
        transport.all_reduce(again)
        torch.cuda.synchronize()
        ops.check_status()
        exact = torch.stack(gathered).sum(0)
        assert rel_l2(value, exact) < 5e-2
        assert torch.equal(value, again)
        # identical on every rank, and equal to the collective-library implementation
        from viola_b200.parallel.fp8 import FP8Communication
        library = FP8Communication(n, engine.group, rank, world, engine.global_ranks, device, mode="all_reduce",
                                   tile_size=tile)
        reference = local.clone()
        library.all_reduce(reference)
        assert rel_l2(value, reference) < 3e-3
        everyone = [torch.empty_like(value) for _ in range(world)]
        dist.all_gather(everyone, value)
        assert all(torch.equal(everyone[0], other) for other in everyone)
        dist.barrier()
    dist.destroy_process_group()
    results.put(rank)


def training_worker(rank, world, port, backend, directory, results):
    setup(rank, world, port)
    import viola_b200 as viola
    from viola_b200 import ops
    from viola_b200.models import DiT, NoiseSchedule, diffusion_loss, muon_parameter_groups
    label = backend
    backend, _, variant = backend.partition(":")
    resident = False if variant == "gathered-per-use" else "auto"
    config = dict(mixed_precision="bf16", gradient_accumulation_steps=2,
                  sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True, resident=resident),
                  communication=dict(dtype="fp8", backend=backend, bucket_mb=1), ema=dict(decay=0.999))
    engine = viola.violaEngine(config)
    torch.manual_seed(0)
    model = engine.prepare_model(DiT(width=256, depth=3, heads=4, patch=2))
    engine.prepare_optimizer(lambda params: viola.optim.FP8Muon(muon_parameter_groups(model, lr=1e-3)))
    assert (engine.transport is not None) == (backend == "p2p")
    assert engine.sharder.resident == (resident == "auto")
    schedule = NoiseSchedule(device=engine.device)
    losses = []
    for step in range(3):
        for micro in range(2):
            generator = torch.Generator(device=engine.device).manual_seed(100 * step + 10 * micro + rank)
            latents = torch.randn(4, 4, 32, 32, device=engine.device, generator=generator)
            labels = torch.randint(0, 1000, (4,), device=engine.device, generator=generator)
            timesteps = torch.randint(0, 1000, (4,), device=engine.device, generator=generator)
            noise = torch.randn(4, 4, 32, 32, device=engine.device, generator=generator)
            with engine.accumulate():
                with engine.autocast():
                    loss = diffusion_loss(model, schedule, latents, labels, timesteps, noise)
                engine.backward(loss)
        assert engine.step()
        losses.append(loss.item())
    torch.cuda.synchronize()
    ops.check_status()
    weights = engine.state.parameters.model_state_dict()
    store = engine.state.parameters

    def one_step(step):
        for micro in range(2):
            generator = torch.Generator(device=engine.device).manual_seed(100 * step + 10 * micro + rank)
            latents = torch.randn(4, 4, 32, 32, device=engine.device, generator=generator)
            labels = torch.randint(0, 1000, (4,), device=engine.device, generator=generator)
            timesteps = torch.randint(0, 1000, (4,), device=engine.device, generator=generator)
            noise = torch.randn(4, 4, 32, 32, device=engine.device, generator=generator)
            with engine.accumulate():
                with engine.autocast():
                    value = diffusion_loss(model, schedule, latents, labels, timesteps, noise)
                engine.backward(value)
        assert engine.step()
        return value.item()

    # every rank holds the same FP8 codes, scale, amax history and call index after the owners' write-back
    for record in store.records:
        layer = record.layer
        if layer is None or layer.weight_dtype != "fp8":
            continue
        header = torch.cat((layer.weight_scale.reshape(-1).float(), layer.weight_quantizer.history.float(),
                            torch.tensor([float(layer.weight_quantizer.index)], device=engine.device)))
        everyone = [torch.empty_like(header) for _ in range(world)]
        dist.all_gather(everyone, header)
        assert all(torch.equal(everyone[0], other) for other in everyone), record.name
    # the peer-memory gather fills the full buffers with exactly what an all-gather of the shards gives
    if engine.sharder is not None:
        for unit in engine.sharder.units.values():
            unit.stale = True
            unit.unshard()
            for entry in unit.entries:
                shard = unit.shard[entry.shard_offset:entry.shard_offset + entry.shard_bytes].clone()
                expected = torch.empty(world * entry.shard_bytes, device=engine.device, dtype=torch.uint8)
                dist.all_gather_into_tensor(expected, shard)
                got = unit.full[entry.full_offset:entry.full_offset + world * entry.shard_bytes]
                assert torch.equal(got, expected), (unit.name, entry.name)
            unit.reshard()
    # evaluation under the averages leaves the compute weights bit-identical
    before = store.snapshot()
    generator = torch.Generator(device=engine.device).manual_seed(4242)
    probe = [torch.randn(4, 4, 32, 32, device=engine.device, generator=generator),
             torch.randint(0, 1000, (4,), device=engine.device, generator=generator),
             torch.randint(0, 1000, (4,), device=engine.device, generator=generator),
             torch.randn(4, 4, 32, 32, device=engine.device, generator=generator)]
    with engine.ema_scope():
        with engine.autocast():
            averaged_loss = diffusion_loss(model, schedule, *probe).item()
    after = store.snapshot()
    assert all(torch.equal(before[name], after[name]) for name in before)
    # save, run on, reload, run the same step again: identical bits
    path = os.path.join(directory, f"checkpoint-{label.replace(':', '-')}")
    engine.save_checkpoint(path)
    first = one_step(7)
    weights_first = store.snapshot()
    engine.load_checkpoint(path)
    second = one_step(7)
    weights_second = store.snapshot()
    assert first == second
    assert all(torch.equal(weights_first[name], weights_second[name]) for name in weights_first)
    torch.cuda.synchronize()
    ops.check_status()
    if backend == "p2p":
        # a failure code on one rank (put in on the host) reaches every rank with the next step's exchange
        if rank == 1:
            engine.state.monitor.pending = 5
        one_step(8)
        with pytest.raises(RuntimeError, match="rank 1.*peer flag"):
            one_step(9)
        torch.cuda.synchronize()
    engine.close()
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        torch.save((losses + [averaged_loss], {k: v.float() for k, v in weights.items() if isinstance(v, torch.Tensor)}),
                   os.path.join(directory, f"{label}.pt"))
    results.put(rank)


@pytest.mark.skipif(GPUS < 2, reason="needs 2 GPUs")
def test_fused_collectives_match_oracle():
    launch(collectives_worker, min(GPUS, 4))


@pytest.mark.skipif(GPUS < 2, reason="needs 2 GPUs")
def test_engine_peer_backend_matches_collective_backend():
    outputs = {}
    with tempfile.TemporaryDirectory() as directory:
        for backend in ("nccl", "p2p", "p2p:gathered-per-use"):
            launch(training_worker, 2, backend, directory)
            outputs[backend] = torch.load(os.path.join(directory, f"{backend}.pt"), weights_only=False)
    losses_a, weights_a = outputs["nccl"]
    losses_b, weights_b = outputs["p2p"]
    assert losses_a == pytest.approx(losses_b, rel=2e-2)
    for name in weights_a:
        assert rel_l2(weights_b[name], weights_a[name]) < 2e-2, name
    # gathering every unit per use (next unit prefetched on a side stream) computes exactly what resident copies do
    losses_c, weights_c = outputs["p2p:gathered-per-use"]
    assert losses_b == losses_c
    assert all(torch.equal(weights_b[name], weights_c[name]) for name in weights_b)


def test_timed_out_push_leaves_the_ticket_counter_clean():
    """A reduce push whose acknowledgement never comes gives up, reports, and leaves the shared ticket counter at
    zero, so the next push (whose acknowledgement is there) completes and raises its flag."""
    from viola_b200 import ops
    ops.load()
    device = torch.device("cuda", 0)
    n, tile = 300_000, 256
    tiles = (n + tile - 1) // tile
    bucket = torch.randn(n, device=device)
    codes = torch.zeros(tiles * tile, device=device, dtype=torch.uint8)
    scales = torch.zeros(tiles, device=device)
    flag = torch.zeros(1, device=device, dtype=torch.int32)
    ack = torch.zeros(1, device=device, dtype=torch.int32)
    generation = torch.full((1,), 2, device=device, dtype=torch.int32)      # expects ack >= 1, which nobody wrote
    counter = torch.zeros(1, device=device, dtype=torch.int32)
    status = ops.status_word(device)

    def push():
        torch.ops.viola_b200.reduce_push_fp8(bucket, tile, 0, codes.data_ptr(), scales.data_ptr(), flag.data_ptr(),
                                             ack.data_ptr(), generation, counter, 2_000_000, 64, status)
        torch.cuda.synchronize()

    push()
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.check_status(device)
    assert counter.item() == 0 and flag.item() == 0 and not codes.any()
    ack.fill_(1)
    push()
    ops.check_status(device)
    assert counter.item() == 0 and flag.item() == 2 and codes.any()


def test_bounded_wait_reports_and_returns():
    """A wait on a flag nobody sets runs out of its budget, records a status and leaves the GPU usable."""
    from viola_b200 import ops
    ops.load()
    device = torch.device("cuda", 0)
    flags = torch.zeros(4, device=device, dtype=torch.int32)
    status = ops.status_word(device)
    torch.ops.viola_b200.wait_flags(flags.data_ptr(), 4, -1, 1, 2_000_000, status)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="peer flag"):
        ops.check_status(device)
    flags.fill_(1)
    torch.ops.viola_b200.wait_flags(flags.data_ptr(), 4, -1, 1, 2_000_000, status)
    torch.cuda.synchronize()
    ops.check_status(device)
    assert torch.ones(8, device=device).sum().item() == 8
