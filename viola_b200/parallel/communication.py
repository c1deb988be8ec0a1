"""Owner-directed transfers of DTensors on a 1-D mesh (used outside autograd by the optimizers).

API of the reference module (viola/distributed/communication.py:16-147): ``partial_gradient``
annotates an unreduced local gradient, ``replicate_tensor`` materialises a full copy everywhere,
``gather_to_owner`` materialises it on one rank only, ``write_from_owner`` sends an owner's full
tensor back into the existing layout.  FP8 payloads travel as bytes.  Uneven and empty row shards
are padded to ``ceil(rows / world)`` on the wire.  Collectives go through ``torch.distributed``
(NCCL on GPUs, Gloo on CPU); the engine's hot paths use the peer-memory kernels instead.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch.distributed.tensor import DTensor, Partial, Replicate, Shard

_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def partial_gradient(local, mesh, *, average=True):
    """Wrap an unsynchronised local gradient as a Partial DTensor (no copy, no communication).

    ``average=True`` declares equal per-rank sample counts; with unequal counts pre-weight the local
    contributions and pass ``average=False``.  The optimizer performs the reduction.
    """
    if mesh.ndim != 1:
        raise ValueError("partial_gradient supports a 1-D DeviceMesh")
    return DTensor.from_local(local, mesh, [Partial("avg" if average else "sum")])


def wire_tensor(value):
    """Byte view of FP8 tensors so the transport never interprets the codes."""
    return value.view(torch.uint8) if value.dtype in _FP8 else value


def _context(value):
    mesh = value.device_mesh
    if mesh.ndim != 1:
        raise ValueError("owner transfers support a 1-D DeviceMesh")
    return mesh, mesh.get_group(), mesh.get_local_rank()


def _wire_shape(value, dim):
    shape = list(value.shape)
    rows = math.ceil(shape.pop(dim) / value.device_mesh.size())
    return (rows, *shape)


def _padded_local(value, dim):
    """This rank's shard with ``dim`` moved to the front and zero-padded to the wire height."""
    shape = _wire_shape(value, dim)
    moved = value.to_local().movedim(dim, 0)
    if moved.shape[0] == shape[0]:
        return moved.contiguous(), shape
    packed = torch.zeros(shape, device=moved.device, dtype=moved.dtype)
    packed[:moved.shape[0]].copy_(moved)
    return packed, shape


@torch.no_grad()
def replicate_tensor(value):
    """Full tensor on every rank (plain tensors pass through)."""
    if not isinstance(value, DTensor):
        return value.detach()
    mesh, group, _ = _context(value)
    placement, = value.placements
    local = value.to_local()
    if isinstance(placement, Replicate):
        return local
    if isinstance(placement, Partial):
        if placement.reduce_op not in ("sum", "avg"):
            raise ValueError("Partial gradients must be sum or avg")
        total = local.contiguous().clone()
        dist.all_reduce(total, group=group)
        if placement.reduce_op == "avg":
            total.div_(mesh.size())
        return total
    dim = placement.dim % value.ndim
    packed, shape = _padded_local(value, dim)
    gathered = torch.empty((mesh.size(), *shape), device=local.device, dtype=local.dtype)
    dist.all_gather(list(wire_tensor(gathered).unbind(0)), wire_tensor(packed), group=group)
    return gathered.flatten(0, 1)[:value.shape[dim]].movedim(0, dim).contiguous()


@torch.no_grad()
def gather_to_owner(value, owner):
    """Full logical tensor on mesh rank ``owner``; ``None`` elsewhere.

    Replicated values are returned as-is on the owner (the result may alias the input).
    """
    mesh, group, rank = _context(value)
    placement, = value.placements
    local = value.to_local()
    destination = int(mesh.mesh[owner])
    if isinstance(placement, Replicate):
        return local if rank == owner else None
    if isinstance(placement, Partial):
        if placement.reduce_op not in ("sum", "avg"):
            raise ValueError("Partial gradients must be sum or avg")
        total = local.contiguous().clone()
        dist.reduce(total, dst=destination, op=dist.ReduceOp.SUM, group=group)
        if rank != owner:
            return None
        return total.div_(mesh.size()) if placement.reduce_op == "avg" else total
    if not isinstance(placement, Shard):
        raise ValueError(f"unsupported placement {placement}")
    dim = placement.dim % value.ndim
    packed, shape = _padded_local(value, dim)
    received = torch.empty((mesh.size(), *shape), device=local.device, dtype=local.dtype) if rank == owner else None
    dist.gather(wire_tensor(packed), list(wire_tensor(received).unbind(0)) if received is not None else None,
                dst=destination, group=group)
    if received is None:
        return None
    return received.flatten(0, 1)[:value.shape[dim]].movedim(0, dim).contiguous()


@torch.no_grad()
def write_from_owner(target, full, owner):
    """Store the owner's ``full`` tensor into ``target``'s existing (Replicate / Shard) layout."""
    mesh, group, rank = _context(target)
    placement, = target.placements
    local = target.to_local()
    source = int(mesh.mesh[owner])
    if isinstance(placement, Replicate):
        staging = local.contiguous()
        if rank == owner:
            staging.copy_(full)
        dist.broadcast(wire_tensor(staging), src=source, group=group)
        local.copy_(staging)
    elif isinstance(placement, Shard):
        dim = placement.dim % target.ndim
        shape = _wire_shape(target, dim)
        chunks = None
        if rank == owner:
            moved = full.movedim(dim, 0)
            if moved.shape[0] == mesh.size() * shape[0]:
                stacked = moved.contiguous()
            else:
                stacked = torch.zeros((mesh.size() * shape[0], *shape[1:]), device=local.device, dtype=local.dtype)
                stacked[:target.shape[dim]].copy_(moved)
            chunks = list(wire_tensor(stacked.view(mesh.size(), *shape)).unbind(0))
        received = torch.empty(shape, device=local.device, dtype=local.dtype)
        dist.scatter(wire_tensor(received), chunks, src=source, group=group)
        local.copy_(received[:local.movedim(dim, 0).shape[0]].movedim(0, dim))
    else:
        raise ValueError(f"unsupported placement {placement}")
    torch.autograd.graph.increment_version(target)
