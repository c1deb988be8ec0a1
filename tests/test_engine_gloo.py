"""Engine plumbing on a 2-rank CPU/Gloo "cluster": every sharding combination against a replicated
single-copy reference, EMA scope restore, and bit-exact checkpoint resume.

Model and settings of the plumbing configuration: 4 residual blocks Linear(256->1024)->GELU->
Linear(1024->256) in fp32, inputs [16, 256], MSE loss, accumulation 2, fp32 communication, EMA
0.9999, a MatrixOptimizer subclass doing SGD on matrices and AdamW on vectors, 10 steps.
"""
import itertools
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
from viola_b200 import ops
from viola_b200.optim import MatrixOptimizer


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.up, self.act, self.down = nn.Linear(256, 1024), nn.GELU(), nn.Linear(1024, 256)

    def forward(self, x):
        return x + self.down(self.act(self.up(x)))


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.blocks = nn.ModuleList([Block() for _ in range(4)])

    def forward(self, x):
        for block in self.blocks:
            x = block(x)
        return x


class MatrixSGD(MatrixOptimizer):
    """SGD on matrices, AdamW on vectors: exercises the whole-matrix optimizer interface."""

    def __init__(self, params, lr=1e-3):
        super().__init__(params, dict(lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0))

    def _step_local(self, parameter, gradient, state, group, index):
        state.setdefault("step", 0)
        if parameter.ndim >= 2:
            parameter.add_(gradient.to(parameter.dtype), alpha=-group["lr"])
        else:
            if "exp_avg" not in state:
                state["exp_avg"], state["exp_avg_sq"] = torch.zeros_like(parameter), torch.zeros_like(parameter)
            ops.adam_update(parameter, gradient, state["exp_avg"], state["exp_avg_sq"], lr=group["lr"],
                            weight_decay=group["weight_decay"], betas=group["betas"], eps=group["eps"],
                            step=state["step"] + 1)
        state["step"] += 1


def batch(step, micro, rank):
    generator = torch.Generator().manual_seed(1000 * step + 10 * micro + rank)
    return torch.randn(16, 256, generator=generator), torch.randn(16, 256, generator=generator)


def reference_run(world, steps, accumulation):
    torch.manual_seed(7)
    model = Net()
    optimizer = MatrixSGD(model.parameters())
    ema = {name: p.detach().clone() for name, p in model.named_parameters()}
    for step in range(steps):
        for micro in range(accumulation):
            for rank in range(world):
                x, y = batch(step, micro, rank)
                (nn.functional.mse_loss(model(x), y) / (accumulation * world)).backward()
        optimizer.step()
        optimizer.zero_grad()
        for name, p in model.named_parameters():
            ema[name].mul_(0.9999).add_(p.detach(), alpha=1 - 0.9999)
    return {name: p.detach().clone() for name, p in model.named_parameters()}, ema


def engine_steps(engine, model, first, count, accumulation):
    losses = []
    for step in range(first, first + count):
        for micro in range(accumulation):
            x, y = batch(step, micro, engine.rank)
            with engine.accumulate():
                loss = nn.functional.mse_loss(model(x), y)
                engine.backward(loss)
        assert engine.step()
        losses.append(loss.item())
    return losses


def full_weights(engine):
    state = engine.state.parameters.model_state_dict()
    return state


def worker(rank, world, port, flags, directory, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    torch.manual_seed(7 if rank == 0 else 99)       # ranks start different: prepare_model must synchronise
    config = dict(device="cpu", mixed_precision="no", gradient_accumulation_steps=2,
                  sharding=dict(parameters=flags[0], gradients=flags[1], optimizer=flags[2], ema=flags[3],
                                resident=flags[4] if len(flags) > 4 else "auto"),
                  communication=dict(dtype="fp32"), ema=dict(decay=0.9999))
    engine = viola.violaEngine(config)
    model = engine.prepare_model(Net())
    engine.prepare_optimizer(lambda params: MatrixSGD(params))
    engine_steps(engine, model, 0, 10, 2)
    expected, expected_ema = reference_run(world, 10, 2)
    weights = full_weights(engine)
    if rank == 0:
        for name, value in expected.items():
            torch.testing.assert_close(weights[name], value, rtol=1e-5, atol=1e-6, msg=f"{flags} {name}")
    # EMA: evaluate under the average, then the compute weights must come back bit for bit
    before = engine.state.parameters.snapshot()
    with engine.ema_scope() as averaged:
        inside = engine.state.parameters.model_state_dict()
        assert not averaged.training
    if rank == 0:
        for name, value in expected_ema.items():
            torch.testing.assert_close(inside[name], value, rtol=1e-5, atol=1e-6, msg=f"ema {flags} {name}")
    after = engine.state.parameters.snapshot()
    assert all(torch.equal(before[name], after[name]) for name in before) and model.training
    # checkpoint: save, run on, reload, run again -> identical bits
    path = os.path.join(directory, "".join(str(int(f)) for f in flags))
    engine.save_checkpoint(path, extra=dict(note="x"))
    first = engine_steps(engine, model, 10, 2, 2)
    weights_a = full_weights(engine)
    assert engine.load_checkpoint(path) == dict(note="x") and engine.global_step == 10
    second = engine_steps(engine, model, 10, 2, 2)
    weights_b = full_weights(engine)
    assert first == second
    if rank == 0:
        assert all(torch.equal(weights_a[name], weights_b[name]) for name in weights_a)
    # partial flush and "no gradient anywhere" semantics
    x, y = batch(50, 0, rank)
    with engine.accumulate():
        engine.backward(nn.functional.mse_loss(model(x), y))
    assert engine.step() is False and engine.step(force=True) is True
    assert engine.step() is False
    engine.close()
    dist.barrier()
    dist.destroy_process_group()
    results.put((rank, True))


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def run_world(target, world, *args):
    context = mp.get_context("spawn")
    results = context.Queue()
    port = free_port()
    processes = [context.Process(target=target, args=(rank, world, port, *args, results)) for rank in range(world)]
    for process in processes:
        process.start()
    deadline = time.time() + 600
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
    assert all(process.exitcode == 0 for process in processes), [process.exitcode for process in processes]
    return [results.get(timeout=5) for _ in processes]


@pytest.mark.parametrize("flags", [(True, True, True, True), (False, False, False, False), (False, True, True, False),
                                   (True, False, True, True), (False, True, False, True), (True, True, False, False),
                                   (True, True, True, True, True)])      # last: gathered parameters kept resident
def test_two_rank_plumbing(flags):
    with tempfile.TemporaryDirectory() as directory:
        assert len(run_world(worker, 2, flags, directory)) == 2


def test_single_process_engine_matches_reference():
    with tempfile.TemporaryDirectory() as directory:
        assert len(run_world(worker, 1, (True, True, True, True), directory)) == 1


class QuantisedNet(nn.Module):
    """FP8 linears of this package, one of them with the Hadamard rotation (its weight gradient cannot be added into
    a running sum by the GEMM, so the layer hands its landing slot back), plus a torch layer and a tied weight."""

    def __init__(self):
        super().__init__()
        self.first = viola.nn.Linear(128, 128, rotation_size=64)
        self.second = viola.nn.Linear(128, 128)
        self.third = nn.Linear(128, 128)
        self.last = viola.nn.Linear(128, 128, bias=False)
        self.last.weight = self.second.weight

    def forward(self, x):
        return self.last(torch.tanh(self.third(torch.tanh(self.second(torch.tanh(self.first(x)))))))


def landing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    outcomes = []
    for slots in (True, False):
        torch.manual_seed(3)
        config = dict(device="cpu", mixed_precision="no", gradient_accumulation_steps=3,
                      precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                      communication=dict(dtype="fp32", gradient_slots=slots))
        engine = viola.violaEngine(config)
        model = engine.prepare_model(QuantisedNet())
        engine.prepare_optimizer(lambda params: MatrixSGD(params))
        assert engine.state.gradients.summing == slots
        for step in range(3):
            for micro in range(3):
                generator = torch.Generator().manual_seed(100 * step + micro)
                x, y = torch.randn(32, 128, generator=generator), torch.randn(32, 128, generator=generator)
                with engine.accumulate():
                    engine.backward(nn.functional.mse_loss(model(x), y))
            assert engine.step()
        outcomes.append({name: value.clone() for name, value in full_weights(engine).items()
                         if torch.is_tensor(value) and value.is_floating_point()})
        engine.close()
    for name, value in outcomes[0].items():
        torch.testing.assert_close(value.float(), outcomes[1][name].float(), rtol=1e-5, atol=1e-6, msg=name)
    results.put((rank, True))


def test_running_sum_landing_buffer_matches_separate_accumulation():
    """The landing buffer as the step's gradient accumulator (producers add into their slots) against the plain
    per-parameter accumulation: same weights after three steps of three microbatches."""
    assert len(run_world(landing_worker, 1)) == 1
