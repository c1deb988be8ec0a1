"""All 16 combinations of the four sharding switches on a 2-rank CPU/Gloo group, against one unsharded copy.

Covered per combination (the cases of the reference's sharding check, checks/distributed_sharding.py:47-203):
rank-dependent batch sizes with weighted losses, a parameter only rank 0 uses, a parameter no rank uses
(it must keep its value although AdamW decays weights), tied weights across sharding units, activation
checkpointing, a stock ``torch.optim.AdamW`` and a ``MatrixOptimizer`` subclass, the EMA of the masters,
``ema_scope`` restoring the weights bit for bit, a bit-exact checkpoint round trip, and per-rank storage
that adds up to one copy when a switch is on and to ``world`` copies when it is off.  A second test forces
a kernel status code on one rank and expects ``engine.step`` to raise on every rank.
"""
import itertools
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
from torch import nn
from torch.utils.checkpoint import checkpoint

import viola_b200 as viola
from viola_b200.optim import MatrixOptimizer

from test_engine_gloo import run_world

WIDTH = 48


class Residual(nn.Module):
    def __init__(self):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(WIDTH, 2 * WIDTH), nn.SiLU(), nn.Linear(2 * WIDTH, WIDTH))

    def forward(self, x):
        return x + 0.1 * self.net(x)


class Model(nn.Module):
    def __init__(self, *, tied, recompute):
        super().__init__()
        self.blocks = nn.ModuleList([Residual(), Residual(), Residual()])
        if tied:
            self.blocks[2].net[0].weight = self.blocks[0].net[0].weight
        self.recompute = recompute
        self.offset = nn.Parameter(torch.zeros(WIDTH))       # used by rank 0 only
        self.never = nn.Parameter(torch.ones(5))              # used by nobody

    def forward(self, x, with_offset):
        for block in self.blocks:
            x = checkpoint(block, x, use_reentrant=False) if self.recompute else block(x)
        return x + self.offset if with_offset else x


class HeavyBall(MatrixOptimizer):
    def __init__(self, params):
        super().__init__(params, dict(lr=3e-3))

    def _step_local(self, parameter, gradient, state, group, index):
        velocity = state.setdefault("velocity", torch.zeros_like(parameter))
        velocity.mul_(0.9).add_(gradient)
        parameter.add_(velocity, alpha=-group["lr"])


def make_batch(step, micro, rank):
    count = 2 + rank + micro                                  # rank- and microbatch-dependent sizes
    generator = torch.Generator().manual_seed(7919 * step + 31 * micro + rank)
    x = torch.randn(count, 3, WIDTH, generator=generator)
    return x, 0.7 * x, count


def replica_update(replica, optimizer, world, step, micros):
    """What the engine must compute: token-weighted mean gradient over all ranks and microbatches; parameters
    nobody used keep ``grad = None`` (no decay, no state step)."""
    optimizer.zero_grad(set_to_none=True)
    total = 0
    for micro in range(micros):
        for rank in range(world):
            x, y, count = make_batch(step, micro, rank)
            ((replica(x, rank == 0) - y).square().mean() * count).backward()
            total += count
    for parameter in replica.parameters():
        if parameter.grad is not None:
            parameter.grad.div_(total)
    optimizer.step()


def engine_update(engine, model, step, micros):
    for micro in range(micros):
        x, y, count = make_batch(step, micro, engine.rank)
        with engine.accumulate():
            engine.backward((model(x, engine.rank == 0) - y).square().mean(), weight=count)
        if micro + 1 < micros:
            assert engine.step() is False or micros <= micro + 1
    assert engine.step(force=True)


def storage_counts(engine, optimizer):
    state = engine.state
    own = {r.index: r.parameter for r in state.parameters.records}
    counts = dict(
        parameters=sum((r.unit.local_view(r.entry).numel() if r.unit is not None else r.parameter.numel())
                       for r in state.parameters.records),
        gradients=state.gradients.accumulator.numel(),
        ema=sum(v.numel() for v in engine.ema.weights.values()),
        masters=sum(m.numel() for i, m in state.optimizer.parameters.items() if m is not own[i]))
    gathered = [None] * engine.world_size
    dist.all_gather_object(gathered, counts)
    return gathered


def one_combination(engine_config, flags, variant, directory, rank, world):
    tied, recompute, adamw = variant[:3]
    config = dict(engine_config, sharding=dict(zip(("parameters", "gradients", "optimizer", "ema"), flags)))
    engine = viola.violaEngine(config)
    torch.manual_seed(11)
    replica = Model(tied=tied, recompute=recompute)
    torch.manual_seed(11 if rank == 0 else 12)               # rank 1 starts elsewhere; prepare_model aligns it
    model = engine.prepare_model(Model(tied=tied, recompute=recompute))
    factory = (lambda p: torch.optim.AdamW(p, lr=3e-3, weight_decay=0.05)) if adamw else HeavyBall
    optimizer = engine.prepare_optimizer(factory)
    replica_optimizer = factory(replica.parameters())
    ema = {name: p.detach().clone() for name, p in replica.named_parameters()}
    label = f"{flags} tied={tied} recompute={recompute} adamw={adamw}"

    def compare():
        for record in engine.state.parameters.records:
            got = engine.state.parameters.full(record).reshape(record.shape)
            torch.testing.assert_close(got, replica.get_parameter(record.name).detach(), rtol=1e-5, atol=1e-6,
                                       msg=lambda m: f"{label} {record.name}: {m}")
        for name, value in engine.ema.weights.items():
            torch.testing.assert_close(value.reshape(ema[name].shape), ema[name], rtol=1e-5, atol=1e-6,
                                       msg=lambda m: f"{label} ema {name}: {m}")

    for step in range(3):
        engine_update(engine, model, step, 2)
        replica_update(replica, replica_optimizer, world, step, 2)
        for name, p in replica.named_parameters():
            ema[name].mul_(0.9).add_(p.detach(), alpha=0.1)
        compare()
    never = next(r for r in engine.state.parameters.records if r.name == "never")
    assert torch.equal(engine.state.parameters.full(never).reshape(-1), torch.ones(5)), \
        f"{label}: the parameter nobody used was touched"
    # EMA scope: weights inside are the averages; outside they come back bit for bit
    before = engine.state.parameters.snapshot()
    with engine.ema_scope() as averaged:
        averaged(torch.zeros(1, 3, WIDTH), True)
        inside = engine.state.parameters.model_state_dict()
    if rank == 0:
        for name, value in ema.items():
            torch.testing.assert_close(inside[name], value, rtol=1e-5, atol=1e-6)
    after = engine.state.parameters.snapshot()
    assert all(torch.equal(before[name], after[name]) for name in before), label
    # checkpoint: continue one step, reload, repeat that step -> identical local storage
    path = os.path.join(directory, "".join(str(int(f)) for f in flags) + f"{int(tied)}{int(recompute)}{int(adamw)}")
    engine.save_checkpoint(path, extra="round trip")
    engine_update(engine, model, 3, 1)
    expected = engine.state.parameters.snapshot()
    assert engine.load_checkpoint(path) == "round trip"
    engine_update(engine, model, 3, 1)
    again = engine.state.parameters.snapshot()
    assert all(torch.equal(expected[name], again[name]) for name in expected), f"{label}: resume is not exact"
    # storage accounting
    total = sum(p.numel() for p in replica.parameters())
    counts = storage_counts(engine, optimizer)
    for key, flag in (("gradients", flags[1]), ("ema", flags[3])):
        assert sum(c[key] for c in counts) == total * (1 if flag else world), (label, key, counts)
    if not flags[0]:
        assert sum(c["parameters"] for c in counts) == total * world, (label, counts)
    engine.close()


def matrix_worker(rank, world, port, variant, directory, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    base = dict(device="cpu", mixed_precision="no", gradient_accumulation_steps=2,
                precision=dict(master_weight_dtype="fp32", gradient_dtype="fp32"),
                communication=dict(dtype="fp32", bucket_mb=0.02, reduce_once=variant[3]),
                ema=dict(decay=0.9, dtype="fp32"))
    for flags in itertools.product((False, True), repeat=4):
        one_combination(base, flags, variant, directory, rank, world)
    dist.barrier()
    dist.destroy_process_group()
    results.put((rank, True))


# last element: sharded gradients go to their owners once per optimizer step (the default) or in every microbatch
@pytest.mark.parametrize("variant", [(True, True, False, True), (False, True, True, False)],
                         ids=["tied+recompute", "recompute+adamw+reduce-every-microbatch"])
def test_all_sharding_combinations(variant):
    with tempfile.TemporaryDirectory() as directory:
        assert len(run_world(matrix_worker, 2, variant, directory)) == 2


def status_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    engine = viola.violaEngine(dict(device="cpu", mixed_precision="no", communication=dict(dtype="fp32"),
                                    sharding=dict(parameters=True, gradients=True, optimizer=True, ema=True)))
    model = engine.prepare_model(Model(tied=False, recompute=False))
    engine.prepare_optimizer(HeavyBall)
    engine_update(engine, model, 0, 1)                       # a healthy step first
    if rank == 1:
        engine.state.monitor.pending = 5                      # "wait on a peer flag timed out", host-injected
    x, y, count = make_batch(1, 0, rank)
    engine.backward((model(x, rank == 0) - y).square().mean(), weight=count)
    with pytest.raises(RuntimeError, match="peer flag"):
        engine.step(force=True)                               # both ranks must raise, not only rank 1
    with tempfile.TemporaryDirectory() as directory:
        if rank == 1:
            engine.state.monitor.pending = 5
            with pytest.raises(RuntimeError, match="peer flag"):
                engine.state.check_status()                   # what save_checkpoint calls first
    dist.barrier()
    dist.destroy_process_group()
    results.put((rank, True))


def test_kernel_status_of_one_rank_raises_on_every_rank():
    assert len(run_world(status_worker, 2)) == 2
