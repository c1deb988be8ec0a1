"""Checkpoints of a running engine: a directory with one file per rank, one full model, one manifest.

Layout (identical to the reference's, viola/distributed/checkpoint.py:17-111, so either framework's tools
can read the other's directory):

``rank-{r}.pt`` (every rank)
    ``state``        ``DistributedState.state_dict()``: rank, mesh, sharding flags, record metadata, the
                     optimizer's own state dict plus owner-local masters, EMA weights;
    ``buffers``      ``{"buffers": {name: tensor}, "extra": {module path: extra state}}`` of the model;
    ``rng``          ``{"torch", "python", "cuda"?, "numpy"?}`` generator states;
    ``global_step``, ``micro_step``, ``scheduler`` (its state dict or None), ``extra`` (user payload).
``model.pt`` (rank 0)
    ``{"model": full CPU state dict (FP8 codes, scales, quantizer history and extra state), "global_step"}``.
``metadata.json`` (rank 0, written last)
    ``{"sharding", "world_size", "global_step"}``; its presence marks the checkpoint as complete.

Files are written under a temporary name and renamed.  Loading restores optimizer and EMA state first and
the compute weights from ``model.pt`` afterwards: the FP8 codes and stochastic roundings of the boundary are
taken as saved, never recomputed from the masters, which is what makes a resumed run repeat bit for bit.
"""

from __future__ import annotations

import copy
import json
import random
import sys
from pathlib import Path

import torch
import torch.distributed as dist

from ..nn import Linear
from .parameters import extra_states, restore_extra_states

MANIFEST = "metadata.json"
MODEL_FILE = "model.pt"


def rank_file(rank):
    return f"rank-{rank}.pt"


# ---------------------------------------------------------------------------------------------- model buffers
def capture_buffers(model, *, clone=False):
    """Everything in the model's state dict that is not a parameter, plus the modules' extra states."""
    parameters = {name for name, _ in model.named_parameters(remove_duplicate=False)}
    tensors = {}
    for name, value in model.state_dict(keep_vars=True).items():
        if isinstance(value, torch.Tensor) and name not in parameters:
            tensors[name] = value.detach().clone() if clone else value
    return {"buffers": tensors, "extra": copy.deepcopy(extra_states(model))}


@torch.no_grad()
def restore_buffers(model, state, *, sharded=False):
    live = dict(model.named_buffers(remove_duplicate=False))
    for name, saved in state["buffers"].items():
        live[name].copy_(saved)
    restore_extra_states(model, state["extra"])
    for module in model.modules():
        if not isinstance(module, Linear):
            continue
        # a cached transposed weight belongs to the weights that were just replaced
        if sharded:
            module.clear_weight_cache()
        else:
            module.rebuild_weight_cache()


# ---------------------------------------------------------------------------------------------- random generators
class _Generators:
    """The random generators a training script may draw from, by checkpoint key."""

    @staticmethod
    def sources(device):
        found = {"torch": (torch.get_rng_state, torch.set_rng_state),
                 "python": (random.getstate, random.setstate)}
        if device.type == "cuda":
            found["cuda"] = (lambda: torch.cuda.get_rng_state(device), lambda s: torch.cuda.set_rng_state(s, device))
        numpy = sys.modules.get("numpy")
        if numpy is not None:
            found["numpy"] = (numpy.random.get_state, numpy.random.set_state)
        return found


def rng_state(device):
    return {key: read() for key, (read, _) in _Generators.sources(device).items()}


def restore_rng(state, device):
    if "numpy" in state:
        import numpy  # noqa: F401  (a checkpoint taken with numpy loaded restores its generator too)
    writers = _Generators.sources(device)
    for key, value in state.items():
        if key in writers:
            writers[key][1](value)


# ---------------------------------------------------------------------------------------------- files
def _write_atomically(path, writer):
    scratch = path.with_name(path.name + ".tmp")
    writer(scratch)
    scratch.replace(path)


def _save_tensor_file(payload, path):
    _write_atomically(path, lambda scratch: torch.save(payload, scratch))


def _read_tensor_file(path):
    return torch.load(path, map_location="cpu", weights_only=False)


def save(engine, directory, *, scheduler=None, extra=None):
    if engine._pending_microbatches or engine._in_ema:
        raise RuntimeError("save checkpoints at an update boundary (after engine.step)")
    engine.state.check_status()          # never write a checkpoint after a kernel reported a failed wait
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    step = engine.global_step
    mine = {"state": engine.state.state_dict(), "buffers": capture_buffers(engine.model),
            "rng": rng_state(engine.device), "global_step": step, "micro_step": engine.micro_step,
            "scheduler": None if scheduler is None else scheduler.state_dict(), "extra": extra}
    _save_tensor_file(mine, directory / rank_file(engine.rank))
    full_model = engine.state.parameters.model_state_dict()      # collective: every rank helps gather
    if engine.is_main_process:
        _save_tensor_file({"model": full_model, "global_step": step}, directory / MODEL_FILE)
    dist.barrier(group=engine.group)                              # all tensor files exist ...
    if engine.is_main_process:
        manifest = {"sharding": engine.state.sharding, "world_size": engine.world_size, "global_step": step}
        _write_atomically(directory / MANIFEST, lambda scratch: scratch.write_text(json.dumps(manifest, indent=2) + "\n"))
    dist.barrier(group=engine.group)                              # ... before anyone may treat it as complete


def load(engine, directory, *, scheduler=None):
    directory = Path(directory)
    manifest = json.loads((directory / MANIFEST).read_text())
    if (manifest["sharding"], manifest["world_size"]) != (engine.state.sharding, engine.world_size):
        raise RuntimeError("checkpoint sharding flags / world size differ from this run")
    mine = _read_tensor_file(directory / rank_file(engine.rank))
    if mine["global_step"] != manifest["global_step"]:
        raise RuntimeError("rank file and metadata disagree on the step (incomplete checkpoint)")
    engine.state.load_state_dict(mine["state"])                   # optimizer + EMA first
    full_model = None
    if engine.is_main_process:
        stored = _read_tensor_file(directory / MODEL_FILE)
        if stored["global_step"] != manifest["global_step"]:
            raise RuntimeError("model file and metadata disagree on the step (incomplete checkpoint)")
        full_model = stored["model"]
    engine.state.parameters.load_model_state_dict(full_model)     # then the exact compute weights
    full_model = None
    restore_buffers(engine.model, mine["buffers"], sharded=engine.state.parameters.sharder is not None)
    if scheduler is not None:
        scheduler.load_state_dict(mine["scheduler"])
    engine.global_step, engine.micro_step = mine["global_step"], mine["micro_step"]
    engine._pending_microbatches, engine._loss_weight, engine._weighted = 0, 0.0, None
    engine.sync_gradients = True
    engine.state.zero_grad()
    restore_rng(mine["rng"], engine.device)
    return mine["extra"]
