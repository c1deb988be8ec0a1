"""Row-wise parameter sharding with explicit gather / free, independent of gradient policy.

Replaces the reference's FSDP2 adapter (viola/distributed/fsdp.py:35-74) with a self-contained
sharder, so nothing depends on FSDP internals.  Unit selection is the same: children of
``ModuleList`` / ``Sequential`` containers (or the ``sharding.blocks`` glob patterns), outermost
first; parameters tied across units stay in the root unit; the root unit holds everything else.

Storage model.  Each unit owns two byte buffers:

* ``shard``  – persistent: this rank's rows ``[rank * h, (rank + 1) * h)`` of every parameter
  (``h = ceil(rows / world)``; padded rows are zero), packed at 16-byte aligned offsets.  Mixed
  dtypes (FP8 codes, bf16 biases, fp32 norms) coexist because the buffer is raw bytes.
* ``full``   – transient: every parameter in full (padded) shape.  The module's parameters are
  permanent views into this buffer; "resharding" resizes its storage to zero bytes and
  "unsharding" resizes it back and fills it, so tensors saved by autograd see the re-gathered
  values in backward.

``unshard`` gathers per parameter straight into its final location (rank ``r``'s rows are the
``r``-th slab of the padded tensor, so there is no copy-out).  The transport is a ``torch.distributed``
all-gather or, when a peer-memory gatherer is installed, one kernel that pulls every peer's slab.
Forward pre/post hooks and a backward pre-hook drive the lifetime; the gradient store frees a unit
once all of its gradients have arrived.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from fnmatch import fnmatchcase

import torch
import torch.distributed as dist
from torch import nn

_ALIGN = 16


def _align(value, alignment=_ALIGN):
    return (value + alignment - 1) // alignment * alignment


@dataclass
class ShardEntry:
    name: str
    parameter: nn.Parameter
    shape: tuple
    dtype: torch.dtype
    rows: int              # extent of dim 0 (1 for scalars)
    shard_rows: int        # h = ceil(rows / world)
    row_bytes: int
    shard_offset: int
    full_offset: int

    @property
    def shard_bytes(self):
        return self.shard_rows * self.row_bytes


@dataclass
class ShardedUnit:
    name: str
    module: nn.Module
    world: int
    rank: int
    group: object
    entries: list = field(default_factory=list)
    shard: torch.Tensor = None
    full: torch.Tensor = None
    unsharded: bool = True
    resident: bool = False         # keep the gathered copy between uses (it is refreshed after every write-back)
    stale: bool = False            # the shards changed since ``full`` was gathered
    pending_gradients: int = 0
    gatherer: object = None        # optional callable(unit) that fills ``full`` from peer memory
    prefetch_event: object = None  # a gather of this unit is in flight on the prefetch stream

    # ------------------------------------------------------------------ views
    def local_view(self, entry):
        """This rank's (padded) rows of ``entry`` inside the shard buffer, in the parameter dtype."""
        raw = self.shard[entry.shard_offset:entry.shard_offset + entry.shard_bytes]
        return raw.view(entry.dtype).view(entry.shard_rows, *entry.shape[1:])

    def full_view(self, entry, padded=False):
        raw = self.full[entry.full_offset:entry.full_offset + self.world * entry.shard_bytes]
        tensor = raw.view(entry.dtype).view(self.world * entry.shard_rows, *entry.shape[1:])
        return tensor if padded else tensor[:entry.rows].view(entry.shape)

    def valid_rows(self, entry, rank=None):
        rank = self.rank if rank is None else rank
        return max(0, min(entry.rows - rank * entry.shard_rows, entry.shard_rows))

    # ------------------------------------------------------------------ lifetime
    def _full_bytes(self):
        return self.full.numel()

    def _join_prefetch(self):
        """Order the current stream after a gather that was started ahead of time on the prefetch stream."""
        if self.prefetch_event is not None:
            torch.cuda.current_stream(self.full.device).wait_event(self.prefetch_event)
            self.prefetch_event = None

    @torch.no_grad()
    def prefetch(self, stream):
        """Start this unit's gather on ``stream`` (a side stream) so that it overlaps the compute in front of the
        unit's use; the storage is allocated on the current stream, which later also frees it."""
        if self.gatherer is None or self.resident or self.prefetch_event is not None or (self.unsharded and not self.stale):
            return
        storage = self.full.untyped_storage()
        if storage.size() == 0:
            storage.resize_(self._full_bytes())
        stream.wait_stream(torch.cuda.current_stream(self.full.device))
        with torch.cuda.stream(stream):
            self.gatherer(self)
            self.prefetch_event = torch.cuda.Event()
            self.prefetch_event.record(stream)
        self.unsharded, self.stale = True, False

    @torch.no_grad()
    def unshard(self):
        if self.unsharded and not self.stale:
            self._join_prefetch()
            return
        storage = self.full.untyped_storage()
        if storage.size() == 0:
            storage.resize_(self._full_bytes())
        if self.gatherer is not None:
            self.gatherer(self)
        else:
            for entry in self.entries:
                target = self.full[entry.full_offset:entry.full_offset + self.world * entry.shard_bytes]
                source = self.shard[entry.shard_offset:entry.shard_offset + entry.shard_bytes]
                if self.world == 1:
                    target.copy_(source)
                else:
                    dist.all_gather_into_tensor(target, source, group=self.group)
        self.unsharded = True
        self.stale = False

    @torch.no_grad()
    def reshard(self):
        if not self.unsharded or self.resident:
            return
        self._join_prefetch()          # never free storage a gather may still be writing
        self.full.untyped_storage().resize_(0)
        self.unsharded = False

    @torch.no_grad()
    def store_local_from_full(self):
        """Copy this rank's rows of the (currently valid) full parameters into the shard buffer."""
        for entry in self.entries:
            padded = self.full_view(entry, padded=True)
            self.local_view(entry).copy_(padded[self.rank * entry.shard_rows:(self.rank + 1) * entry.shard_rows])


def select_units(model, blocks=None):
    """Names of the sub-modules that become sharding units (the root ``""`` is always added last)."""
    modules = dict(model.named_modules())
    if blocks is None:
        candidates = [f"{name}.{child}".lstrip(".") for name, module in modules.items()
                      if isinstance(module, (nn.ModuleList, nn.Sequential)) for child, _ in module.named_children()]
    else:
        candidates = [name for name in modules if name and any(fnmatchcase(name, pattern) for pattern in blocks)]
        if blocks and not candidates:
            raise ValueError("no modules match sharding.blocks")
    candidates.sort(key=lambda name: (name.count("."), name))
    selected = []
    for name in candidates:
        if not any(name.startswith(parent + ".") for parent in selected):
            selected.append(name)
    homes = {}
    for name, param in model.named_parameters(remove_duplicate=False):
        unit = next((p for p in selected if name.startswith(p + ".")), "")
        homes.setdefault(id(param), set()).add(unit)
    tied = set().union(*(units for units in homes.values() if len(units) > 1)) if homes else set()
    selected = [name for name in selected if name not in tied and next(modules[name].parameters(), None) is not None]
    return [*selected, ""]


class ParameterSharder:
    """Shards every parameter of ``model`` by rows across ``group`` and manages gather / free."""

    def __init__(self, model, group, rank, world, *, blocks=None):
        self.model, self.group, self.rank, self.world = model, group, rank, world
        self.in_backward = False
        self.resident = False
        self.prefetch_stream = None    # set by the peer transport: gathers of the next unit run there
        self.units = {}
        self.by_parameter = {}
        self.handles = []
        modules = dict(model.named_modules())
        names = select_units(model, blocks)
        claimed = set()
        for unit_name in names:
            module = modules[unit_name]
            unit = ShardedUnit(unit_name, module, world, rank, group)
            shard_offset = full_offset = 0
            prefix = unit_name + "." if unit_name else ""
            for local_name, param in module.named_parameters():
                if id(param) in claimed:
                    continue
                # selected units are disjoint subtrees; the root unit takes what is left (including
                # parameters tied across units, whose units were dropped from the selection)
                claimed.add(id(param))
                shape = tuple(param.shape)
                rows = shape[0] if shape else 1
                row_elems = 1
                for extent in shape[1:]:
                    row_elems *= extent
                entry = ShardEntry(prefix + local_name, param, shape if shape else (1,), param.dtype, rows,
                                   (rows + world - 1) // world, row_elems * param.element_size(), shard_offset,
                                   full_offset)
                unit.entries.append(entry)
                shard_offset = _align(shard_offset + entry.shard_bytes)
                full_offset = _align(full_offset + world * entry.shard_bytes)
                self.by_parameter[param] = (unit, entry)
            if not unit.entries:
                continue
            device = unit.entries[0].parameter.device
            unit.shard = torch.zeros(max(shard_offset, _ALIGN), device=device, dtype=torch.uint8)
            unit.full = torch.zeros(max(full_offset, _ALIGN), device=device, dtype=torch.uint8)
            with torch.no_grad():
                for entry in unit.entries:
                    padded = unit.full_view(entry, padded=True)
                    padded[:entry.rows].copy_(entry.parameter.detach().reshape(entry.shape))
                    entry.parameter.data = unit.full_view(entry).view(entry.parameter.shape)
                unit.store_local_from_full()
            self.units[unit_name] = unit
            self._install_hooks(unit)
        for unit in self.units.values():
            unit.reshard()

    # ------------------------------------------------------------------ hooks
    def _install_hooks(self, unit):
        is_root = unit.name == ""

        def before_forward(module, args):
            unit.unshard()
            if not self.in_backward:
                self._prefetch_neighbour(unit, +1)

        def after_forward(module, args, output):
            keep = self.in_backward or (is_root and torch.is_grad_enabled())
            if not keep:
                unit.reshard()

        def before_backward(module, grad_output):
            unit.unshard()
            self._prefetch_neighbour(unit, -1)

        self.handles.append(unit.module.register_forward_pre_hook(before_forward))
        self.handles.append(unit.module.register_forward_hook(after_forward))
        self.handles.append(unit.module.register_full_backward_pre_hook(before_backward))

    def enable_prefetch(self, stream):
        """Gather the unit that comes next (forward) or before (backward) on ``stream`` while the current unit
        computes.  Only with a one-sided gatherer: collectives on a side stream would have to be entered in the
        same order by all ranks."""
        self.prefetch_stream = stream
        self._sequence = [unit for name, unit in self.units.items() if name != ""]
        self._position = {id(unit): index for index, unit in enumerate(self._sequence)}

    def _prefetch_neighbour(self, unit, direction):
        if self.prefetch_stream is None or self.resident:
            return
        index = self._position.get(id(unit))
        if index is None:
            return
        index += direction
        if 0 <= index < len(self._sequence):
            self._sequence[index].prefetch(self.prefetch_stream)

    def join_prefetches(self):
        """Make the current stream wait for every gather still in flight (end of a microbatch / graph capture)."""
        for unit in self.units.values():
            unit._join_prefetch()

    def begin_backward(self):
        self.in_backward = True
        for unit in self.units.values():
            unit.pending_gradients = sum(1 for e in unit.entries if e.parameter.requires_grad)

    def gradient_arrived(self, parameter):
        unit, _ = self.by_parameter[parameter]
        unit.pending_gradients -= 1
        if unit.pending_gradients == 0 and unit.name != "":
            unit.reshard()

    def finish_backward(self):
        self.in_backward = False
        for unit in self.units.values():
            unit.reshard()
        self.join_prefetches()

    def set_resident(self, resident=True):
        """Resident mode keeps every unit's gathered parameters allocated: forward and backward of every
        microbatch then read local memory, and the gather runs once per write-back (``refresh``) instead of twice
        per unit per microbatch.  Costs one full copy of the parameters per rank."""
        self.resident = resident
        for unit in self.units.values():
            unit.resident = resident
        if resident:
            self.unshard_all()
        else:
            self.reshard_all()

    def full_bytes(self):
        return sum(unit.full.numel() for unit in self.units.values())

    def invalidate(self):
        """The shards were written (optimizer write-back, EMA swap, state load): gathered copies are out of date."""
        for unit in self.units.values():
            unit.stale = True

    def refresh(self):
        """After a write-back: re-gather right away in resident mode, else leave it to the next use."""
        self.invalidate()
        if self.resident:
            self.unshard_all()
        else:
            for unit in self.units.values():
                if unit.unsharded:
                    unit.unshard()

    def unshard_all(self):
        for unit in self.units.values():
            unit.unshard()

    def reshard_all(self):
        for unit in self.units.values():
            unit.reshard()

    def close(self):
        for handle in self.handles:
            handle.remove()
        self.handles.clear()


def shard_parameters(model, group, rank, world, *, blocks=None):
    return ParameterSharder(model, group, rank, world, blocks=blocks)
