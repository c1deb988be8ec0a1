"""Failure handling, exercised on the host only: a gradient that is not finite, a checkpoint whose layout does not
match the run, a damaged checkpoint file.  One single-rank Gloo engine per case (the reference's policy:
viola/optim/matrix.py:50-68 for skipped steps, viola/distributed/state.py:66-69 for layout checks)."""
import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
from torch import nn

import viola_b200 as viola
from viola_b200.optim import MatrixOptimizer


class TinyOptimizer(MatrixOptimizer):
    def __init__(self, params, **kwargs):
        super().__init__(params, dict(lr=1e-2), **kwargs)

    def _step_local(self, parameter, gradient, state, group, index):
        parameter.add_(gradient.to(parameter.dtype), alpha=-group["lr"])


def make_engine(sharding, **optimizer_options):
    config = dict(device="cpu", mixed_precision="no", gradient_accumulation_steps=1, sharding=sharding,
                  communication=dict(dtype="fp32"), ema=dict(decay=0.99))
    engine = viola.violaEngine(config)
    torch.manual_seed(3)
    model = engine.prepare_model(nn.Sequential(nn.Linear(16, 32), nn.GELU(), nn.Linear(32, 16)))
    engine.prepare_optimizer(lambda params: TinyOptimizer(params, **optimizer_options))
    return engine, model


def train_step(engine, model, poison=False):
    x = torch.randn(8, 16)
    with engine.accumulate():
        loss = model(x).square().mean()
        if poison:
            loss = loss * float("nan")
        engine.backward(loss)
    return engine.step()


@pytest.fixture(scope="module", autouse=True)
def single_rank_group():
    if not dist.is_initialized():
        with socket.socket() as probe:
            probe.bind(("127.0.0.1", 0))
            port = probe.getsockname()[1]
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
        dist.init_process_group("gloo", rank=0, world_size=1)
    yield


FULL = dict(parameters=True, gradients=True, optimizer=True, ema=True)


def test_nonfinite_gradient_skips_the_step_and_leaves_the_weights():
    engine, model = make_engine(FULL, skip_nonfinite=True)
    assert train_step(engine, model)
    before = {k: v.clone() for k, v in engine.state.parameters.model_state_dict().items()}
    assert not train_step(engine, model, poison=True)
    assert engine.optimizer.step_was_skipped
    after = engine.state.parameters.model_state_dict()
    assert all(torch.equal(before[k], after[k]) for k in before)
    assert train_step(engine, model)                       # training carries on
    engine.close()


def test_checkpoint_from_another_layout_is_refused():
    with tempfile.TemporaryDirectory() as directory:
        engine, model = make_engine(FULL)
        train_step(engine, model)
        engine.save_checkpoint(directory)
        engine.close()
        other, other_model = make_engine(dict(parameters=False, gradients=False, optimizer=True, ema=True))
        with pytest.raises(RuntimeError, match="layout|sharding|differs"):
            other.load_checkpoint(directory)
        other.close()


def test_damaged_checkpoint_file_raises_and_leaves_the_run_usable():
    with tempfile.TemporaryDirectory() as directory:
        engine, model = make_engine(FULL)
        train_step(engine, model)
        engine.save_checkpoint(directory)
        path = os.path.join(directory, "rank-0.pt")
        size = os.path.getsize(path)
        with open(path, "r+b") as handle:
            handle.truncate(size // 2)
        with pytest.raises(Exception):
            engine.load_checkpoint(directory)
        assert train_step(engine, model)
        engine.close()
