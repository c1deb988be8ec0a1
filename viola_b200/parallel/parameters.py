"""Parameter records, whole-parameter owners and the write-back path from owners to compute storage.

Role of the reference's ``ParameterStore`` (viola/distributed/parameters.py:51-192) on top of this
package's own row sharder instead of FSDP2 / DTensor views: one record per trainable optimizer
parameter with its stable index and owner rank; ``full`` materialises a parameter everywhere;
``write`` takes an owner's full real-valued tensor, derives the storage representation there
(FP8 codes + scale for FP8 layers, a cast otherwise) and delivers it to every rank's storage
(broadcast for replicated parameters, row slabs for sharded ones); ``snapshot`` / ``restore`` and
the model state-dict helpers serve ``ema_scope`` and checkpoints.

Differences from the reference that matter for speed: the FP8 scale and amax history travel in
one small message instead of three collectives, and the quantizer call index is advanced
deterministically on every rank, so no host synchronisation happens per layer per step.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..nn import Linear
from .partition import assign_owners

_FP8 = (torch.float8_e4m3fn, torch.float8_e5m2)


def _wire(tensor):
    return tensor.view(torch.uint8) if tensor.dtype in _FP8 else tensor


@torch.no_grad()
def broadcast_tensor(tensor, source, group):
    """In-place broadcast of any tensor (FP8 as bytes); empty tensors are skipped."""
    if not tensor.numel():
        return
    value = tensor.contiguous()
    dist.broadcast(_wire(value), src=source, group=group)
    if value is not tensor:
        tensor.copy_(value)


def extra_states(model):
    return {name: module.get_extra_state() for name, module in model.named_modules()
            if type(module).get_extra_state is not torch.nn.Module.get_extra_state}


def restore_extra_states(model, states):
    for name, value in states.items():
        model.get_submodule(name).set_extra_state(value)


@torch.no_grad()
def synchronize_model(model, group, source_rank, is_source, *, initial=False):
    """Make every rank's model identical to ``source_rank``'s (tensors, quantizer state, initial masters)."""
    for value in model.state_dict(keep_vars=True).values():
        if isinstance(value, torch.Tensor):
            broadcast_tensor(value.detach() if value.requires_grad else value, source_rank, group)
    payload = [extra_states(model) if is_source else None]
    dist.broadcast_object_list(payload, src=source_rank, group=group)
    restore_extra_states(model, payload[0])
    for module in model.modules():
        if isinstance(module, Linear):
            if initial and module._initial_weight is not None:
                broadcast_tensor(module._initial_weight, source_rank, group)
            module.rebuild_weight_cache()


@dataclass
class ParameterRecord:
    name: str
    parameter: torch.nn.Parameter
    index: int
    owner: int
    layer: Linear | None
    shape: tuple
    numel: int
    dtype: torch.dtype
    unit: object = None       # ShardedUnit when parameters are sharded
    entry: object = None

    @property
    def placement(self):
        return "S(0)" if self.unit is not None else "R"


class ParameterStore:
    def __init__(self, model, optimizer, group, rank, world, global_ranks, gradient_dtype, sharder=None,
                 transport=None):
        self.model, self.group, self.rank, self.world = model, group, rank, world
        self.transport = transport if sharder is not None else None
        self.global_ranks = list(global_ranks)          # mesh rank -> global rank
        self.sharder = sharder
        self.gradient_dtype = gradient_dtype
        names = {id(param): name for name, param in model.named_parameters()}
        layers = {id(m.weight): m for m in model.modules() if isinstance(m, Linear)}
        indexed = [(i, p) for i, p in enumerate(p for g in optimizer.param_groups for p in g["params"])
                   if p.requires_grad]
        owners = assign_owners([p.numel() for _, p in indexed], world)
        self.records = []
        for (index, param), owner in zip(indexed, owners):
            unit, entry = sharder.by_parameter[param] if sharder is not None else (None, None)
            shape = tuple(entry.shape) if entry is not None and param.ndim else tuple(param.shape)
            self.records.append(ParameterRecord(names[id(param)], param, index, owner, layers.get(id(param)),
                                                tuple(param.shape), param.numel(), param.dtype, unit, entry))
            param.grad_dtype = gradient_dtype
        self.by_parameter = {r.parameter: r for r in self.records}
        self.local = [r for r in self.records if r.owner == rank]
        self.hooks = []
        self._tables = {}              # fused write-back tables by purpose ("step", "ema", ...)
        self._local_headers = None     # single process: [scale, amax history] of each FP8 layer, contiguous
        if self.transport is not None:
            self.transport.attach_parameters(sharder, self.records)
        elif sharder is not None and world == 1 and self.records and self.records[0].parameter.is_cuda:
            self._make_local_headers()

    def metadata(self):
        return [dict(name=r.name, index=r.index, shape=r.shape, dtype=r.dtype, owner=r.owner, placement=r.placement)
                for r in self.records]

    # ------------------------------------------------------------------ reads
    @torch.no_grad()
    def full(self, record):
        """The full storage tensor of ``record`` on every rank (a fresh tensor when sharded)."""
        if record.unit is None:
            return record.parameter.detach()
        unit, entry = record.unit, record.entry
        gathered = torch.empty(self.world * entry.shard_bytes, device=unit.shard.device, dtype=torch.uint8)
        local = unit.shard[entry.shard_offset:entry.shard_offset + entry.shard_bytes]
        if self.world == 1:
            gathered.copy_(local)
        else:
            dist.all_gather_into_tensor(gathered, local, group=self.group)
        padded = gathered.view(entry.dtype).view(self.world * entry.shard_rows, *entry.shape[1:])
        return padded[:entry.rows].reshape(record.shape)

    # ------------------------------------------------------------------ writes
    @torch.no_grad()
    def _deliver(self, record, payload, source):
        """Put ``payload`` (storage dtype, full shape, valid on ``source``) into every rank's storage."""
        src = self.global_ranks[source]
        if record.unit is None:
            target = record.parameter.data
            if self.world == 1:
                if payload is not None and payload.data_ptr() != target.data_ptr():
                    target.copy_(payload)
            else:
                staging = target if target.is_contiguous() else target.contiguous()
                if self.rank == source and payload.data_ptr() != staging.data_ptr():
                    staging.copy_(payload)
                dist.broadcast(_wire(staging), src=src, group=self.group)
                if staging is not target:
                    target.copy_(staging)
        else:
            unit, entry = record.unit, record.entry
            local = unit.local_view(entry)
            if self.world == 1:
                local[:entry.rows].copy_(payload.reshape(entry.shape))
            else:
                chunks = None
                if self.rank == source:
                    stacked = torch.zeros((self.world * entry.shard_rows, *entry.shape[1:]), device=local.device,
                                          dtype=entry.dtype)
                    stacked[:entry.rows].copy_(payload.reshape(entry.shape))
                    chunks = list(_wire(stacked.view(self.world, entry.shard_rows, *entry.shape[1:])).unbind(0))
                dist.scatter(_wire(local), chunks, src=src, group=self.group)
            if unit.resident:
                unit.stale = True    # refreshed in one go by end_writes()
            elif unit.unsharded:     # keep a live gathered copy coherent (e.g. inside ema_scope)
                if self.world > 1:
                    unit.full_view(entry).copy_(self.full(record).view(entry.shape))
                else:
                    unit.full_view(entry).copy_(local[:entry.rows].view(entry.shape))
        torch.autograd.graph.increment_version(record.parameter)

    # ------------------------------------------------------------------ fused write-back (one table, two launches)
    def _make_local_headers(self):
        """Single process, sharded storage: give every per-tensor FP8 layer one contiguous ``[scale, history]``
        block so that the table-driven write-back kernel can update both with one address (with several ranks
        the transport keeps these blocks in the symmetric heap)."""
        layers = [r for r in self.records if r.layer is not None and r.layer.weight_dtype == "fp8"
                  and not r.layer._grouped_scaling and r.layer.weight_quantizer.history.numel() + 1 <= 32]
        if not layers:
            return
        block = torch.zeros(len(layers), 32, device=layers[0].parameter.device, dtype=torch.float32)
        self._local_headers = {}
        for row, record in zip(block, layers):
            layer, length = record.layer, record.layer.weight_quantizer.history.numel()
            row[0:1].copy_(layer.weight_scale)
            row[1:1 + length].copy_(layer.weight_quantizer.history)
            layer.weight_scale = row[0:1]
            layer.weight_quantizer.history = row[1:1 + length]
            self._local_headers[record.index] = row.data_ptr()

    def _header_address(self, record):
        if self.transport is not None:
            found = self.transport.header_offset.get(record.index)
            return None if found is None else found[0]
        return None if self._local_headers is None else self._local_headers.get(record.index)

    def _fusable(self, record):
        """True when the table-driven kernels can write this record (same answer on every rank)."""
        from .. import ops
        unit = record.unit
        if unit is None or not record.parameter.is_cuda or (unit.unsharded and not unit.resident):
            return False
        if self.world > 1 and self.transport is None:
            return False
        layer = record.layer
        if layer is not None and layer.weight_dtype == "fp8":
            return (not layer._grouped_scaling and not layer.rotation_size
                    and layer.weight_quantizer.scaling == "current" and self._header_address(record) is not None)
        return record.dtype in ops._DT

    def _table_row(self, record, value, average):
        from .. import ops
        from ..ops.reference import fp8_limit
        unit, entry, layer = record.unit, record.entry, record.layer
        element = torch.empty((), dtype=record.dtype).element_size()
        base = unit.heap_offset if self.transport is not None else unit.shard.data_ptr()
        row = dict(master=value, ema=average, n=value.numel(), slab_elems=entry.shard_rows * (entry.row_bytes // element),
                   dst_offset=base + entry.shard_offset, header_offset=-1, base_index=0, limit=448.0, history_len=0,
                   mode=2, out_dtype=record.dtype)
        if layer is not None and layer.weight_dtype == "fp8":
            limit = layer._quantization_limit(max(layer.in_features, layer.out_features), layer.fp8_dtype)
            row.update(mode=ops._FMT[layer.fp8_dtype], limit=fp8_limit(layer.fp8_dtype, limit),
                       header_offset=self._header_address(record), history_len=layer.weight_quantizer.history.numel(),
                       base_index=layer.weight_quantizer.index)
        return row

    @torch.no_grad()
    def write_many(self, records, values, *, averages=None, decay=0.0, purpose="step"):
        """Write-back of many records at once.  ``values[index]`` is the new real-valued tensor on the owner of
        the record with that index.  Records the fused kernels can handle go through one device table (two
        launches on each owner for all of them, EMA lerp of ``averages[name]`` included when given); the rest
        take :meth:`write`.  Every rank must call this with the same ``records``."""
        from .. import ops
        self.begin_writes()
        fused = [r for r in records if self._fusable(r)]
        fused_ids = {id(r) for r in fused}
        owned = [r for r in fused if r.owner == self.rank and values.get(r.index) is not None
                 and values[r.index].is_contiguous() and values[r.index].dtype in ops._DT]
        if len(owned) != sum(1 for r in fused if r.owner == self.rank):
            fused, fused_ids, owned = [], set(), []          # an owner cannot serve its rows: use the per-record path
        with_ema = bool(averages) and bool(decay)
        if owned:
            rows = [self._table_row(r, values[r.index], averages.get(r.name) if with_ema else None) for r in owned]
            cached = self._tables.get(purpose)
            valid = (cached is not None and cached["table"].matches(rows)
                     and all(row["base_index"] == base + cached["calls"] or row["mode"] == 2
                             for row, base in zip(rows, cached["bases"])))
            if not valid:
                cached = self._tables[purpose] = dict(table=ops.WritebackTable(rows, owned[0].parameter.device),
                                                      bases=[row["base_index"] for row in rows], calls=0)
            if self.transport is not None:
                self.transport.write_table(cached["table"], calls=cached["calls"], decay=decay, with_ema=with_ema)
            else:
                ops.multi_writeback(cached["table"], heaps=[0], rank=0, calls=cached["calls"], decay=decay,
                                    with_ema=with_ema)
            cached["calls"] += 1
        for record in fused:
            layer = record.layer
            if layer is not None and layer.weight_dtype == "fp8":
                layer.weight_quantizer.index += 1
                layer.clear_weight_cache()
            record.unit.stale = True
            torch.autograd.graph.increment_version(record.parameter)
        for record in records:
            if id(record) not in fused_ids:
                self.write(record, values.get(record.index), record.owner)
        self.end_writes()
        return with_ema and len(fused) == len(records)

    # ------------------------------------------------------------------ peer-memory write path
    def begin_writes(self):
        """Cross-rank barrier (on the stream, no host wait) before owners overwrite storage that peers may
        still be reading."""
        if self.transport is not None and self.world > 1:
            self.transport.barrier()

    def end_writes(self):
        """Publish this rank's stores and wait (bounded, on the stream) for every owner's."""
        if self.transport is not None and self.world > 1:
            self.transport.publish_step()
        if self.sharder is not None:
            self.sharder.refresh()

    @torch.no_grad()
    def _write_peer(self, record, value, source):
        """Sharded storage in the symmetric heap: the owner stores into every rank's slab directly."""
        layer, transport = record.layer, self.transport
        fp8_layer = layer is not None and layer.weight_dtype == "fp8"
        if fp8_layer and record.index in transport.header_offset:
            if self.rank == source:
                limit = layer._quantization_limit(max(layer.in_features, layer.out_features), layer.fp8_dtype)
                master = value
                if layer.rotation_size:
                    from .. import ops
                    master = ops.hadamard64(value)
                layer.weight_quantizer.scale(master, layer.fp8_dtype, limit, out=layer.weight_scale)
                from ..ops.reference import fp8_limit
                transport.write_fp8_weight(record, master.contiguous(), layer.weight_scale, fp8_limit(layer.fp8_dtype, limit))
            else:
                layer.weight_quantizer.index += 1
            layer.clear_weight_cache()
            torch.autograd.graph.increment_version(record.parameter)
            return True
        entry = record.entry
        if entry.shard_bytes % 16 or (record.unit.heap_offset + entry.shard_offset) % 16:
            return False
        if fp8_layer:                       # group-scaled FP8: codes by peer stores, scales by a small broadcast
            payload = layer.quantize_master(value) if self.rank == source else None
        else:
            payload = value.to(record.dtype) if self.rank == source else None
        if self.rank == source:
            transport.write_bytes(record, payload)
        if fp8_layer:
            header = layer.weight_scale.reshape(-1).float().contiguous()
            dist.broadcast(header, src=self.global_ranks[source], group=self.group)
            layer.weight_scale.copy_(header.view(layer.weight_scale.shape).to(layer.weight_scale.dtype))
            layer.clear_weight_cache()
        torch.autograd.graph.increment_version(record.parameter)
        return True

    @torch.no_grad()
    def write(self, record, value, source):
        """Owner ``source`` holds the new real-valued ``value``; update the compute storage everywhere."""
        layer = record.layer
        # the shards are the storage of record: write them directly unless a live gathered copy must stay
        # coherent (a resident copy is refreshed in one go by end_writes())
        direct = record.unit is not None and (not record.unit.unsharded or record.unit.resident)
        if self.transport is not None and direct and self.world > 1:
            if self._write_peer(record, value, source):
                record.unit.stale = True
                return
        if self.world == 1 and direct:
            record.unit.stale = True
            # single rank, sharded storage: encode straight into the shard buffer (no staging copy)
            target = record.unit.local_view(record.entry)[:record.entry.rows].view(record.shape)
            if layer is not None and layer.weight_dtype == "fp8":
                layer.quantize_master(value, out=target)
                layer.clear_weight_cache()
            else:
                target.copy_(value)
            torch.autograd.graph.increment_version(record.parameter)
            return
        if layer is not None and layer.weight_dtype == "fp8":
            codes = None
            if self.rank == source:
                codes = layer.quantize_master(value)
            else:
                layer.weight_quantizer.index += 0 if layer._grouped_scaling else 1
            self._deliver(record, codes, source)
            if self.world > 1:
                header = torch.cat((layer.weight_scale.reshape(-1).float(), layer.weight_quantizer.history))
                dist.broadcast(header, src=self.global_ranks[source], group=self.group)
                count = layer.weight_scale.numel()
                layer.weight_scale.copy_(header[:count].view(layer.weight_scale.shape).to(layer.weight_scale.dtype))
                layer.weight_quantizer.history.copy_(header[count:])
            if record.unit is not None:
                layer.clear_weight_cache()
            else:
                layer.rebuild_weight_cache()
        else:
            payload = value.to(record.dtype) if value is not None else None
            self._deliver(record, payload, source)

    def release_initializers(self):
        for module in self.model.modules():
            if isinstance(module, Linear):
                module._initial_weight = None
                if self.sharder is not None:
                    module.clear_weight_cache()

    # ------------------------------------------------------------------ snapshots (ema_scope)
    def _local_storage(self, record):
        if record.unit is None:
            return record.parameter.data
        return record.unit.local_view(record.entry)

    @torch.no_grad()
    def snapshot(self):
        return {r.name: self._local_storage(r).detach().clone() for r in self.records}

    @torch.no_grad()
    def restore(self, values):
        """Put a :meth:`snapshot` back.  With peer-memory storage this is a write like any other: no rank may
        overwrite its slab while a peer still gathers from it, and no rank may gather before every slab is
        back, hence the same barrier / publish bracket as an optimizer write-back."""
        self.begin_writes()
        for record in self.records:
            self._local_storage(record).copy_(values[record.name])
            torch.autograd.graph.increment_version(record.parameter)
        self.end_writes()

    # ------------------------------------------------------------------ full-model state dicts
    @torch.no_grad()
    def model_state_dict(self):
        """Full state dict on CPU (rank 0 only returns it; every rank takes part in the gathers)."""
        if self.sharder is not None:
            self.sharder.unshard_all()
        result = {}
        try:
            for name, value in self.model.state_dict().items():
                if self.rank == 0:
                    result[name] = value.detach().cpu().clone() if isinstance(value, torch.Tensor) else value
        finally:
            if self.sharder is not None:
                self.sharder.reshard_all()
        return result

    @torch.no_grad()
    def load_model_state_dict(self, saved):
        """Rank 0 provides the full CPU state dict; tensors are delivered into every rank's storage."""
        src = self.global_ranks[0]
        sharded = self.sharder.by_parameter if self.sharder is not None else {}
        if self.sharder is not None:
            self.sharder.unshard_all()
        try:
            for name, value in self.model.state_dict(keep_vars=True).items():
                if not isinstance(value, torch.Tensor):
                    continue
                target = value.detach()
                if self.rank == 0:
                    target.copy_(saved[name].to(target.device))
                if self.world > 1:
                    broadcast_tensor(target, src, self.group)
            if self.sharder is not None:
                for unit in self.sharder.units.values():
                    unit.store_local_from_full()
        finally:
            if self.sharder is not None:
                self.sharder.reshard_all()
        if self.sharder is not None and self.world > 1:
            dist.barrier(group=self.group)       # every rank's slab is in place before anyone gathers again
        if self.sharder is not None:
            self.sharder.refresh()
        del sharded
        extras = [dict((name, saved[f"{name}._extra_state" if name else "_extra_state"])
                       for name in extra_states(self.model)) if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(extras, src=src, group=self.group)
        restore_extra_states(self.model, extras[0])
