"""Whole-tensor ownership: which rank keeps the optimizer state of which parameter.

Muon needs the full logical matrix, so ownership is per tensor, never per row shard.  Assignment
is the reference's deterministic greedy packing (viola/distributed/partition.py:40-53): parameters
sorted by (-numel, index) each go to the currently lightest rank (ties -> lowest rank), and
``batches`` are rounds holding at most one tensor per owner so all ranks update concurrently.
``assign_owners`` is the layout-free core used by the engine; ``MatrixPartition`` is the DTensor
front end of the standalone optimizer path.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist

try:  # DTensor is only needed by the standalone (engine-less) optimizer path
    from torch.distributed.tensor import DTensor, Replicate, Shard
except Exception:  # pragma: no cover
    DTensor = Replicate = Shard = None


def assign_owners(sizes, world_size, costs=None):
    """Greedy balanced ownership.  ``sizes[i]`` = numel of entry i; returns ``owners[i]``.

    ``costs`` (optional) balances on something other than numel, e.g. Newton-Schulz FLOPs.
    """
    weights = list(sizes if costs is None else costs)
    order = sorted(range(len(weights)), key=lambda i: (-sizes[i], i))
    loads = [0] * world_size
    owners = [0] * len(weights)
    for i in order:
        rank = min(range(world_size), key=loads.__getitem__)
        owners[i] = rank
        loads[rank] += weights[i]
    return owners


def owner_rounds(owners, world_size):
    """Rounds of entry indices with at most one entry per owner, in entry order."""
    queues = [[] for _ in range(world_size)]
    for index, owner in enumerate(owners):
        queues[owner].append(index)
    depth = max((len(q) for q in queues), default=0)
    return [[queue[i] for queue in queues if i < len(queue)] for i in range(depth)]


@dataclass(frozen=True)
class MatrixOwner:
    index: int
    rank: int


class MatrixPartition:
    """Ownership of the DTensor parameters among ``parameters`` (plain tensors are ignored)."""

    def __init__(self, parameters):
        self.owners, self.meshes, self.batches = {}, [], []
        by_mesh = {}
        for index, param in enumerate(parameters):
            if DTensor is None or not isinstance(param, DTensor):
                continue
            mesh = param.device_mesh
            if mesh.ndim != 1:
                raise ValueError("matrix ownership supports a 1-D DeviceMesh")
            if not isinstance(param.placements[0], (Replicate, Shard)):
                raise ValueError("parameters must be Replicate or Shard")
            key = (mesh.device_type, tuple(mesh.mesh.tolist()))
            if key not in by_mesh:
                by_mesh[key] = (mesh, [])
                self.meshes.append(mesh)
            by_mesh[key][1].append((index, param))
        for mesh, entries in by_mesh.values():
            owners = assign_owners([p.numel() for _, p in entries], mesh.size())
            # ties are broken by the global parameter index, which is the entry order here
            for (index, param), owner in zip(entries, owners):
                self.owners[param] = MatrixOwner(index, owner)
            for round_ in owner_rounds(owners, mesh.size()):
                self.batches.append([entries[i][1] for i in round_])

    def owner(self, param):
        return self.owners[param].rank

    def is_owner(self, param):
        return param.device_mesh.get_local_rank() == self.owner(param)

    def state_dict(self):
        if not self.owners:
            return {}
        entries = [dict(index=entry.index, shape=tuple(param.shape), placement=str(param.placements[0]),
                        ranks=param.device_mesh.mesh.tolist(), owner=entry.rank)
                   for param, entry in sorted(self.owners.items(), key=lambda item: item[1].index)]
        return dict(rank=dist.get_rank(), parameters=entries)
