"""CPU-side API contract: precision policy, config merge, launcher command, dataloader sharding,
ownership packing, master binding round trip, checkpoint layout, and the DTensor owner transfers
(all placements, uneven and empty shards) with a 2-rank Gloo group, mirroring the reference's
checks/dtensor_muon.py:31-54 and checks/optimizer.py semantics.
"""
import json
import os
import socket
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

import viola_b200 as viola
from viola_b200.nn import Linear
from viola_b200.optim import FP8Muon, bind_optimizer
from viola_b200.parallel.config import read_config
from viola_b200.parallel.data import prepare_dataloader
from viola_b200.parallel.launch import build_command
from viola_b200.parallel.partition import assign_owners, owner_rounds


def test_precision_policy_and_public_names():
    assert viola.precision.settings()["master_weight_dtype"] == torch.float32
    viola.set_master_weight_dtype("bf16", rounding="stochastic", seed=7)
    viola.set_gradient_dtype("bf16")
    policy = viola.precision.settings()
    assert policy["master_weight_dtype"] == torch.bfloat16 and policy["master_rounding"] == "stochastic"
    assert policy["gradient_dtype"] == torch.bfloat16 and policy["master_rounding_seed"] == 7
    viola.set_master_weight_dtype(None)
    assert viola.precision.settings()["master_weight_dtype"] is None
    viola.set_master_weight_dtype("fp32")
    viola.set_gradient_dtype("fp32")
    with pytest.raises(ValueError):
        viola.set_master_weight_dtype("fp32", rounding="banker")
    for name in ("nn", "optim", "distributed", "precision", "violaEngine"):
        assert hasattr(viola, name)
    assert viola.distributed.violaEngine is viola.violaEngine


def test_config_defaults_and_one_level_merge(tmp_path):
    config = read_config(dict(sharding=dict(parameters=True), ema=dict(decay=0.5), device="cpu"))
    assert config["sharding"] == dict(parameters=True, gradients=False, optimizer=True, ema=True, blocks=None,
                                      resident="auto")
    assert config["communication"]["bucket_mb"] == 25 and config["communication"]["fp8_tile_size"] == 256
    assert config["ema"] == dict(decay=0.5, dtype="fp32") and config["device"] == "cpu"
    path = tmp_path / "engine.yaml"
    path.write_text("num_processes: 4\ngradient_accumulation_steps: 3\ncommunication:\n  dtype: fp8\n")
    loaded = read_config(str(path))
    assert loaded["num_processes"] == 4 and loaded["gradient_accumulation_steps"] == 3
    assert loaded["communication"]["dtype"] == "fp8" and loaded["communication"]["fp8_format"] == "e4m3"
    command = build_command(str(path), "train.py", ["--flag"], python="python")
    assert command[:3] == ["python", "-m", "torch.distributed.run"] and "--nproc-per-node=4" in command
    assert command[-2:] == ["train.py", "--flag"]


def test_dataloader_preparation():
    dataset = torch.utils.data.TensorDataset(torch.arange(20).float())
    loader = torch.utils.data.DataLoader(dataset, batch_size=2, shuffle=True, drop_last=True)
    assert prepare_dataloader(loader, rank=0, world_size=1) is loader
    sharded = prepare_dataloader(loader, rank=1, world_size=2)
    assert isinstance(sharded.sampler, torch.utils.data.DistributedSampler) and sharded.sampler.rank == 1
    assert sharded.sampler.shuffle and sharded.drop_last and len(sharded) == 5
    assert prepare_dataloader(sharded, rank=1, world_size=2) is sharded
    with pytest.raises(ValueError):
        prepare_dataloader(sharded, rank=0, world_size=2)
    custom = torch.utils.data.DataLoader(dataset, batch_sampler=[[0, 1], [2, 3]])
    with pytest.raises(ValueError):
        prepare_dataloader(custom, rank=0, world_size=2)


def test_greedy_ownership_and_rounds():
    sizes = [100, 100, 50, 400, 10, 400]
    owners = assign_owners(sizes, 2)
    # largest first, ties by index, lightest rank (ties -> lowest): 400(3)->0, 400(5)->1, 100(0)->0, 100(1)->1, 50->0, 10->1
    assert owners == [0, 1, 0, 0, 1, 1]
    assert owner_rounds(owners, 2) == [[0, 1], [2, 4], [3, 5]]
    assert assign_owners(sizes, 1) == [0] * 6


def test_master_binding_round_trip_and_missing_gradients():
    torch.manual_seed(0)
    model = nn.Sequential(Linear(32, 64), nn.GELU(), Linear(64, 32), nn.LayerNorm(32))
    optimizer = bind_optimizer(model, FP8Muon(model.parameters(), lr=1e-2, weight_decay=0.01))
    assert model[0]._initial_weight is None and model[0]._master_ref() is not None
    x = torch.randn(16, 32)
    for _ in range(3):
        model(x).square().mean().backward()
        optimizer.step()
        optimizer.zero_grad()
    assert all(p.grad is None for p in model.parameters())
    saved_model, saved_optimizer = model.state_dict(), optimizer.state_dict()
    masters = saved_optimizer["viola_masters"]
    assert masters["master_dtype"] == torch.float32 and len(masters["weights"]) == len(list(model.parameters()))
    state = saved_optimizer["state"][0]
    assert state["momentum_q"].dtype == torch.uint8 and state["momentum_scale"].dtype == torch.float32
    assert state["momentum_q"].numel() == 32 * 64 and state["momentum_scale"].numel() == 32 * 64 // 256
    clone = nn.Sequential(Linear(32, 64), nn.GELU(), Linear(64, 32), nn.LayerNorm(32))
    clone_optimizer = bind_optimizer(clone, FP8Muon(clone.parameters(), lr=1e-2, weight_decay=0.01))
    clone.load_state_dict(saved_model)
    clone_optimizer.load_state_dict(saved_optimizer)
    assert clone_optimizer.state[clone_optimizer.param_groups[0]["params"][0]]["momentum_q"].dtype == torch.uint8
    outputs = []
    for net, opt in ((model, optimizer), (clone, clone_optimizer)):
        net(x).square().mean().backward()
        opt.step()
        opt.zero_grad()
        outputs.append(net(x))
    assert torch.equal(outputs[0], outputs[1])
    # a parameter without a gradient is left untouched: no decay, no state step
    before = clone[3].weight.detach().clone()
    steps_before = clone_optimizer.state[clone_optimizer.param_groups[0]["params"][-2]].get("step", 0)
    clone[0](x).sum().backward()
    clone_optimizer.step()
    assert torch.equal(clone[3].weight, before)
    assert clone_optimizer.state[clone_optimizer.param_groups[0]["params"][-2]].get("step", 0) == steps_before
    with pytest.raises(RuntimeError):
        bind_optimizer(model, optimizer)


def test_linear_state_dict_contract():
    layer = Linear(64, 32, scaling="delayed")
    keys = set(layer.state_dict().keys())
    assert {"weight", "bias", "weight_scale", "weight_quantizer.history", "weight_quantizer._extra_state",
            "input_quantizer.history", "grad_quantizer._extra_state"} <= keys
    assert "weight_transpose" not in keys
    floating = Linear(64, 32, weight_dtype="bf16")
    assert all(v.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) for v in floating.state_dict().values()
               if isinstance(v, torch.Tensor))
    with pytest.raises(RuntimeError):
        floating.load_state_dict(layer.state_dict())
    converted = Linear.from_float(nn.Linear(64, 32))
    assert converted.weight_quantizer.index == 1 and converted.weight.dtype == torch.float8_e4m3fn
    assert converted.half().weight.dtype == torch.float8_e4m3fn      # dtype casts leave FP8 storage alone


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def run_world(target, world, *args):
    context = mp.get_context("spawn")
    port = free_port()
    processes = [context.Process(target=target, args=(rank, world, port, *args)) for rank in range(world)]
    for process in processes:
        process.start()
    deadline = time.time() + 300
    while any(p.exitcode is None for p in processes) and time.time() < deadline:
        if any(p.exitcode not in (None, 0) for p in processes):
            break
        time.sleep(0.2)
    for process in processes:
        if process.exitcode is None:
            process.join(timeout=5)
        if process.exitcode is None:
            process.kill()
            process.join()
    assert all(p.exitcode == 0 for p in processes), [p.exitcode for p in processes]


def dtensor_worker(rank, world, port):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor, Replicate, Shard, distribute_tensor
    from viola_b200.parallel import MatrixPartition, ShardedEMA, gather_to_owner, partial_gradient, write_from_owner
    from viola_b200.optim import MatrixOptimizer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo")
    mesh = init_device_mesh("cpu", (world,))
    torch.manual_seed(0)
    for shape in ((6, 4), (5, 3), (1, 7)):                      # even, uneven and (for rank 1) empty shards
        full = torch.arange(shape[0] * shape[1], dtype=torch.float32).view(shape)
        for placement in (Replicate(), Shard(0), Shard(1)):
            tensor = distribute_tensor(full.clone(), mesh, [placement])
            for owner in range(world):
                gathered = gather_to_owner(tensor, owner)
                assert (gathered is not None) == (rank == owner)
                if gathered is not None:
                    assert torch.equal(gathered, full)
                target = distribute_tensor(torch.zeros(shape), mesh, [placement])
                write_from_owner(target, full * 2 if rank == owner else None, owner)
                assert torch.equal(target.full_tensor(), full * 2)
        local = torch.full(shape, float(rank + 1))
        total = gather_to_owner(partial_gradient(local, mesh, average=False), 0)
        mean = gather_to_owner(partial_gradient(local, mesh, average=True), 1)
        if rank == 0:
            assert torch.equal(total, torch.full(shape, 3.0))
        if rank == 1:
            assert torch.equal(mean, torch.full(shape, 1.5))

    class OwnerSGD(MatrixOptimizer):
        def __init__(self, params):
            super().__init__(params, dict(lr=0.5))
            self.calls = 0

        def _step_local(self, parameter, gradient, state, group, index):
            self.calls += 1
            parameter.add_(gradient, alpha=-group["lr"])

    weights = [torch.randn(6, 4), torch.randn(5, 3), torch.randn(8)]
    params = [nn.Parameter(distribute_tensor(w.clone(), mesh, [p])) for w, p in
              zip(weights, (Shard(0), Replicate(), Shard(0)))]
    optimizer = OwnerSGD(params)
    ema = ShardedEMA([(f"p{i}", p) for i, p in enumerate(params)], optimizer, decay=0.5)
    grads = [torch.randn_like(w) for w in weights]
    for p, g in zip(params, grads):
        p.grad = distribute_tensor(g.clone(), mesh, p.placements)
    optimizer.step()
    for p, w, g in zip(params, weights, grads):
        torch.testing.assert_close(p.full_tensor(), w - 0.5 * g)
    assert optimizer.calls == sum(1 for p in params if optimizer.partition.owner(p) == rank)
    assert ema.updates == 1
    for (name, average), w, g in zip(ema.weights.items(), weights, grads):
        torch.testing.assert_close(average.full_tensor(), 0.5 * w + 0.5 * (w - 0.5 * g))
    layout = optimizer.state_dict()["viola_dtensor"]
    assert layout["shard_state"] is True and len(layout["partition"]["parameters"]) == 3
    assert isinstance(optimizer.partition, MatrixPartition)
    dist.barrier()
    dist.destroy_process_group()


def test_dtensor_owner_transfers_and_matrix_optimizer():
    run_world(dtensor_worker, 2)


def checkpoint_worker(rank, world, port, directory):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    engine = viola.violaEngine(dict(device="cpu", mixed_precision="no", ema=dict(decay=0.9),
                                    sharding=dict(parameters=True, gradients=True)))
    torch.manual_seed(0)
    model = engine.prepare_model(nn.Sequential(Linear(16, 32), nn.GELU(), Linear(32, 16)))
    engine.prepare_optimizer(lambda params: FP8Muon(params, lr=1e-2))
    x = torch.randn(8, 16)
    engine.backward(model(x).square().mean())
    assert engine.step()
    engine.save_checkpoint(directory, extra={"epoch": 3})
    if rank == 0:
        metadata = json.loads(open(os.path.join(directory, "metadata.json")).read())
        assert metadata == dict(sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True),
                                world_size=world, global_step=1)
        full = torch.load(os.path.join(directory, "model.pt"), weights_only=False)
        assert set(full) == {"model", "global_step"} and full["model"]["0.weight"].dtype == torch.float8_e4m3fn
        assert full["model"]["0.weight"].shape == (32, 16) and "0.weight_scale" in full["model"]
    dist.barrier()
    mine = torch.load(os.path.join(directory, f"rank-{rank}.pt"), weights_only=False)
    assert set(mine) == {"state", "buffers", "rng", "global_step", "micro_step", "scheduler", "extra"}
    state = mine["state"]
    assert set(state) == {"rank", "mesh", "sharding", "parameters", "optimizer", "ema"}
    assert set(state["optimizer"]) == {"optimizer", "precision", "masters"}
    assert set(state["ema"]) == {"decay", "dtype", "shard", "updates", "weights"}
    assert state["parameters"][0]["placement"] == "S(0)" and {"name", "index", "shape", "dtype", "owner"} <= set(state["parameters"][0])
    owned = [entry["name"] for entry in state["parameters"] if entry["owner"] == rank]
    assert sorted(state["optimizer"]["masters"]) == sorted(owned) == sorted(state["ema"]["weights"])
    assert engine.load_checkpoint(directory) == {"epoch": 3}
    with pytest.raises(RuntimeError):
        engine.backward(model(x).square().mean())
        engine.save_checkpoint(directory)                     # mid-accumulation saves are refused
    engine.step(force=True)
    engine.close()
    dist.barrier()
    dist.destroy_process_group()


def test_checkpoint_directory_layout():
    with tempfile.TemporaryDirectory() as directory:
        run_world(checkpoint_worker, 2, directory)


def test_phase_tracing_is_inert_by_default_and_times_when_enabled():
    from viola_b200 import utils
    with utils.phase("anything"):
        pass
    assert utils.phase_times() == {}
    utils.enable_timing(True)
    try:
        with utils.phase("optimizer"):
            sum(range(1000))
        with utils.phase("optimizer"):
            pass
        with utils.phase("ema"):
            pass
        times = utils.phase_times()
        assert set(times) == {"optimizer", "ema"} and times["optimizer"] >= 0.0
        assert utils.phase_times() == {}
    finally:
        utils.enable_timing(False)


def test_packed_attention_and_accumulating_gemm_on_cpu():
    """CPU paths of the two newest ops: packed attention (SDPA) agrees with the fp32 oracle of the tcgen05 kernel,
    and ``ops.gemm(accumulate=True)`` adds the product to its output."""
    from viola_b200 import ops
    from viola_b200.nn.attention import packed_attention
    from viola_b200.ops import reference

    torch.manual_seed(0)
    qkv = torch.randn(2, 256, 3, 4, 16)
    out, lse = ops.attention_forward(qkv)
    want = packed_attention(qkv).view(2, 256, 4, 16)
    assert out.shape == (2, 256, 4, 16) and lse.shape == (2, 4, 256)
    assert torch.allclose(out, want, atol=1e-5)
    scores = torch.einsum("bthd,bshd->bhts", qkv[:, :, 0], qkv[:, :, 1]) * 16 ** -0.5
    assert torch.allclose(lse, torch.logsumexp(scores, dim=-1), atol=1e-5)

    a = torch.randn(24, 32).to(torch.float8_e4m3fn)
    b = torch.randn(40, 32).to(torch.float8_e4m3fn)
    one = torch.ones(1)
    product = ops.gemm(a, b, one, one, out_dtype=torch.float32)
    base = torch.randn(24, 40)
    out = base.clone()
    ops.gemm(a, b, one, one, out_dtype=torch.float32, out=out, accumulate=True)
    assert torch.allclose(out, base + product)
    assert torch.allclose(product, reference.gemm(a, b, one, one, out_dtype=torch.float32))
