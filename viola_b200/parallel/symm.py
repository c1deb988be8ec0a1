"""Symmetric peer memory and the fused communication paths built on it.

``SymmetricHeap`` is one allocation per rank, mapped into every rank of the node through
``torch.distributed._symmetric_memory`` (CUDA VMM handles exchanged at rendezvous), with an
identical layout everywhere so that ``(rank, offset)`` names the same object on every GPU.
``PeerTransport`` lays the engine's communication state out in that heap and drives the kernels of
``csrc/comm.cu``; nothing on these paths calls NCCL:

* gradient reduce-to-owner, per bucket and per microbatch: non-owners quantise and store straight
  into the owner's receive slots, the owner dequantises in ascending rank order and adds into its
  accumulator (the FP8 arithmetic is the reference codec's, viola/distributed/fp8.py:67-85);
* replicated-gradient all-reduce with requantisation (viola/distributed/fp8.py:48-65);
* parameter gather: one kernel per sharding unit pulls every peer's row slabs into the local full
  buffers (replaces FSDP2's all-gather + copy-out, viola/distributed/fsdp.py:67);
* owner write-back: updated masters are quantised and stored directly into every rank's shard
  storage; the FP8 scale and amax history of a layer live in the heap too, so the owner's store is
  the broadcast (replaces the scatter plus three small broadcasts and a host sync per layer per
  step of viola/distributed/parameters.py:121-147).

The kernels run on a side stream ordered against the compute stream with events.  Cross-rank
ordering uses generation counters in the heap; every device-side wait is bounded and reports
through the status word (``ops.check_status``).  Each rank's per-step message (its status word and
which parameters produced a gradient) is stored into every rank's heap and followed by a flag; the
bounded on-stream wait for all of those flags doubles as the barrier between "everyone finished reading
the old weights" and "owners overwrite them", so a step contains no NCCL call and no host wait.
"""

from __future__ import annotations

import torch

from .. import ops

_FLAG_BYTES = 1 << 16                      # 16384 int32 flags
_HEADER_FLOATS = 32                        # per FP8 layer: scale + amax history (padded)
_FMT = {"e4m3": 0, "e5m2": 1}
_DEFAULT_WAIT_CLOCKS = 8_000_000_000       # ~4-6 s of SM clocks: peers may be a few steps of skew away


def _align(value, alignment=256):
    return (value + alignment - 1) // alignment * alignment


def probe_peer_memory(group, device):
    """Allocate and rendezvous a small symmetric buffer; raises where peer mapping does not work (ranks on
    different nodes, GPUs without peer access, a torch build without symmetric memory)."""
    import torch.distributed._symmetric_memory as symm_mem
    probe = symm_mem.empty(4096, dtype=torch.uint8, device=device)
    handle = symm_mem.rendezvous(probe, group)
    if len(handle.buffer_ptrs) != handle.world_size:
        raise RuntimeError("symmetric-memory rendezvous returned an incomplete peer table")


class SymmetricHeap:
    def __init__(self, nbytes, group, device):
        import torch.distributed._symmetric_memory as symm_mem
        self.nbytes = _align(nbytes, 1 << 20)
        self.tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]
        self.rank, self.world = int(self.handle.rank), int(self.handle.world_size)
        torch.cuda.synchronize(device)
        self.handle.barrier()

    def view(self, offset, nbytes):
        return self.tensor[offset:offset + nbytes]

    def barrier(self):
        self.handle.barrier()


class PeerTransport:
    """Heap layout + kernel launches for one engine.  Built in ``prepare_optimizer``; the engine then
    calls ``attach_gradients`` / ``attach_parameters`` once the bucket and shard layouts are known."""

    def __init__(self, engine, *, fp8_format="e4m3", tile_size=256, fp8=True, overlap=True, max_blocks=32,
                 wait_clocks=_DEFAULT_WAIT_CLOCKS, prefetch=True):
        if engine.world_size > 16:
            raise RuntimeError("peer transport supports up to 16 ranks on one node")
        self.group, self.rank, self.world, self.device = engine.group, engine.rank, engine.world_size, engine.device
        self.fmt, self.tile, self.fp8 = _FMT[fp8_format], tile_size, fp8
        self.overlap = overlap
        self.prefetch = prefetch           # gather the next sharding unit on a side stream while this one computes
        # Overlapped communication shares the GPU with compute, so its kernels stay narrow; without overlap they
        # run alone after backward and take the whole GPU (a 25 MB bucket then costs microseconds, not hundreds).
        # eight 256-thread CTAs per SM fill the warp slots of a memory-bound kernel (296 CTAs reached a third of
        # the DRAM rate: every warp waits on its own loads)
        self.max_blocks, self.wait_clocks = (max_blocks if overlap else 1184), wait_clocks
        self.stream = torch.cuda.Stream(device=self.device) if overlap else None
        self.status = ops.status_word(self.device)
        self.counters = torch.zeros(64, device=self.device, dtype=torch.int32)
        # microbatch counter in device memory: the generation every bucket of a microbatch signals with
        self.micro_counter = torch.zeros(1, device=self.device, dtype=torch.int32)
        self.heap = None
        self._requests = []                      # (name, nbytes)
        self.offsets = {}
        self.generation = {}
        self.step_generation = 0
        ops.load()
        self._ops = torch.ops.viola_b200

    # ------------------------------------------------------------------ layout
    def request(self, name, nbytes):
        self._requests.append((name, _align(nbytes)))

    def finalize(self):
        offset = _FLAG_BYTES
        for name, nbytes in self._requests:
            self.offsets[name] = offset
            offset += nbytes
        self.heap = SymmetricHeap(offset, self.group, self.device)
        self.pointers = self.heap.pointers
        self._flag_cursor = 0
        self.flag_offsets = {}

    def flags(self, name, count):
        """Reserve ``count`` int32 flags; returns their byte offset in the heap."""
        offset = self._flag_cursor * 4
        self._flag_cursor += count
        if self._flag_cursor * 4 > _FLAG_BYTES:
            raise RuntimeError("flag region exhausted: too many buckets / records for the peer transport")
        self.flag_offsets[name] = offset
        return offset

    def local_pointer(self, offset):
        return self.pointers[self.rank] + offset

    def peer_pointer(self, rank, offset):
        return self.pointers[rank] + offset

    # ------------------------------------------------------------------ stream plumbing
    def _enter(self):
        """Make the side stream wait for everything enqueued on the compute stream so far."""
        if self.stream is None:
            return torch.cuda.current_stream(self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        return self.stream

    def synchronize(self):
        """Compute stream waits for all communication issued so far."""
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)

    # ------------------------------------------------------------------ path 1: reduce to owner
    def attach_gradients(self, buckets, accumulator_slices, capacity):
        """``buckets``: [(owner, pieces, length)]; ``accumulator_slices[b]`` = owner-local fp32 slice of bucket b."""
        self.buckets = buckets
        self.bucket_accum = accumulator_slices
        tile = self.tile
        self.bucket_slot, self.bucket_scales_offset, self.bucket_region = [], [], []
        per_owner = [0] * self.world
        self.owned_index = []
        owned_counts = [0] * self.world
        for owner, _, length in buckets:
            tiles = (length + tile - 1) // tile
            slot = _align(tiles * tile + tiles * 4, 16)
            self.bucket_slot.append(slot)
            self.bucket_scales_offset.append(tiles * tile)
            self.bucket_region.append(per_owner[owner])
            per_owner[owner] += _align(slot * self.world)
            self.owned_index.append(owned_counts[owner])
            owned_counts[owner] += 1
        self.request("grad_receive", max(per_owner) if per_owner else 0)
        self._max_owned = max(owned_counts) if owned_counts else 0
        # staging buffers are only for callers without a landing buffer; they are allocated on first use
        self._staging_capacity = capacity
        self.staging, self.staging_events, self.staging_cursor = [], [], 0

    def finalize_gradients(self):
        self.reduce_flag_offset = self.flags("reduce", max(1, self._max_owned) * self.world)
        self.ack_flag_offset = self.flags("ack", max(1, len(self.buckets)))
        self.many_flag_offset = self.flags("reduce_all", self.world)
        self.many_ack_offset = self.flags("ack_all", self.world)
        self._many = None

    def next_staging(self):
        """A staging buffer whose previous communication has finished (stream-ordered, no host wait)."""
        if not self.staging:
            count = 4 if self.overlap else 1
            self.staging = [torch.empty(self._staging_capacity, device=self.device, dtype=torch.float32) for _ in range(count)]
            self.staging_events = [None] * count
        index = self.staging_cursor
        self.staging_cursor = (index + 1) % len(self.staging)
        event = self.staging_events[index]
        if event is not None:
            torch.cuda.current_stream(self.device).wait_event(event)
        return index, self.staging[index]

    def begin_microbatch(self):
        """Advance the generation all of this microbatch's buckets signal with (captured in CUDA graphs).

        The kernels read the counter when they run, so it may only move once the side stream has finished the
        previous microbatch's kernels."""
        self.synchronize()
        self.micro_counter.add_(1)

    def forget_events(self):
        """Drop cross-stream events recorded outside a CUDA-graph capture (call after a full device sync)."""
        self.staging_events = [None] * len(self.staging_events)

    def reduce_to_owner(self, bucket_index, staging_index, length, buffer=None):
        """Push (non-owners) or accumulate (owner) one bucket; ``buffer`` overrides the rotating staging buffers
        (the gradient landing buffer is read in place)."""
        owner = self.buckets[bucket_index][0]
        generation = self.micro_counter
        if buffer is None:
            buffer = self.staging[staging_index][:length]
        stream = self._enter()
        region = self.offsets["grad_receive"] + self.bucket_region[bucket_index]
        slot = self.bucket_slot[bucket_index]
        scales_offset = self.bucket_scales_offset[bucket_index]
        flag_base = self.reduce_flag_offset + 4 * self.owned_index[bucket_index] * self.world
        ack = self.ack_flag_offset + 4 * bucket_index
        with torch.cuda.stream(stream):
            if self.rank == owner:
                self._ops.reduce_accumulate_fp8(buffer, self.tile, self.fmt, self.local_pointer(region), slot, scales_offset,
                                                self.local_pointer(flag_base), self.pointers, self.rank, ack, generation,
                                                self.bucket_accum[bucket_index], self.counters[0:1], self.wait_clocks,
                                                self.max_blocks, self.status)
            else:
                destination = self.peer_pointer(owner, region + self.rank * slot)
                self._ops.reduce_push_fp8(buffer, self.tile, self.fmt, destination, destination + scales_offset,
                                          self.peer_pointer(owner, flag_base + 4 * self.rank), self.local_pointer(ack),
                                          generation, self.counters[1:2], self.wait_clocks, self.max_blocks, self.status)
            if staging_index is not None:
                event = torch.cuda.Event()
                event.record(stream)
                self.staging_events[staging_index] = event
        ops._count()

    def reduce_all(self, buffers):
        """Reduce every bucket to its owner from ``buffers[b]`` (this rank's fp32 values of bucket ``b``) in two
        launches: one pushes all buckets owned elsewhere, one accumulates all owned buckets.  The generation is the
        one :meth:`begin_microbatch` last set."""
        key = tuple(b.data_ptr() for b in buffers)
        if self._many is None or self._many[0] != key:
            push_rows, push_prefix, own_rows, own_prefix = [], [0], [], [0]
            for index, (owner, _, length) in enumerate(self.buckets):
                tiles = (length + self.tile - 1) // self.tile
                region = self.offsets["grad_receive"] + self.bucket_region[index]
                slot, scales_offset = self.bucket_slot[index], self.bucket_scales_offset[index]
                source = buffers[index].data_ptr()
                if owner == self.rank:
                    own_rows.append([source, length, self.local_pointer(region), 0, self.bucket_accum[index].data_ptr(),
                                     slot, scales_offset, 0])
                    own_prefix.append(own_prefix[-1] + tiles)
                else:
                    codes = self.peer_pointer(owner, region + self.rank * slot)
                    push_rows.append([source, length, codes, codes + scales_offset, 0, 0, 0, 0])
                    push_prefix.append(push_prefix[-1] + tiles)

            def table(rows, prefix):
                rows = rows or [[0] * 8]
                return (torch.tensor(rows, device=self.device, dtype=torch.int64),
                        torch.tensor(prefix, device=self.device, dtype=torch.int64), prefix[-1])

            self._many = (key, table(push_rows, push_prefix), table(own_rows, own_prefix))
        _, push, own = self._many
        stream = self._enter()
        with torch.cuda.stream(stream):
            self._ops.reduce_many(push[0], push[1], push[2], self.tile, self.fmt, self.pointers, self.rank, False,
                                  self.local_pointer(self.many_ack_offset), self.many_flag_offset, self.micro_counter,
                                  self.counters[1:2], self.wait_clocks, self.max_blocks, self.status)
            self._ops.reduce_many(own[0], own[1], own[2], self.tile, self.fmt, self.pointers, self.rank, True,
                                  self.local_pointer(self.many_flag_offset), self.many_ack_offset, self.micro_counter,
                                  self.counters[0:1], self.wait_clocks, self.max_blocks, self.status)
        ops._count(2)

    # ------------------------------------------------------------------ path 2: all-reduce with requantisation
    def attach_all_reduce(self, capacity):
        groups = (capacity + self.world * self.tile - 1) // (self.world * self.tile)
        self.all_reduce_slot = _align(groups * self.tile + groups * 4, 16)
        self.request("a2a", self.all_reduce_slot * self.world)
        self.request("gather", self.all_reduce_slot * self.world)
        self.all_reduce_generation = 0

    def finalize_all_reduce(self):
        self.a2a_flag_offset = self.flags("a2a", self.world)
        self.gather_flag_offset = self.flags("gather", self.world)

    def all_reduce(self, value):
        """In-place FP8 all-reduce (two quantisations) of a contiguous fp32 tensor."""
        self.all_reduce_generation += 1
        groups = (value.numel() + self.world * self.tile - 1) // (self.world * self.tile)
        slot = _align(groups * self.tile + groups * 4, 16)
        assert slot <= self.all_reduce_slot
        self._ops.allreduce_requant_fp8(value, self.tile, self.fmt, self.pointers, self.rank, self.offsets["a2a"],
                                        self.offsets["gather"], slot, self.a2a_flag_offset, self.gather_flag_offset,
                                        self.all_reduce_generation, self.counters[2:4], self.wait_clocks,
                                        max(self.max_blocks, 64), self.status)
        ops._count(3)

    # ------------------------------------------------------------------ paths 3 + 4: sharded parameter storage
    def attach_parameters(self, sharder, records):
        """Reserve heap space for every unit's shard buffer and for the FP8 layer headers."""
        self.sharder = sharder
        self.unit_bytes = {name: unit.shard.numel() for name, unit in sharder.units.items()}
        for name, nbytes in self.unit_bytes.items():
            self.request(f"unit:{name}", nbytes)
        self.header_records = [r for r in records if r.layer is not None and r.layer.weight_dtype == "fp8"
                               and not r.layer._grouped_scaling
                               and r.layer.weight_quantizer.history.numel() + 1 <= _HEADER_FLOATS]
        self.request("headers", max(1, len(self.header_records)) * _HEADER_FLOATS * 4)

    def finalize_parameters(self):
        self.step_flag_offset = self.flags("step", self.world)
        device = self.device
        for name, unit in self.sharder.units.items():
            offset = self.offsets[f"unit:{name}"]
            view = self.heap.view(offset, unit.shard.numel())
            view.copy_(unit.shard)
            unit.shard = view
            unit.heap_offset = offset
            entries, prefix, total = [], [0], 0
            for entry in unit.entries:
                entries.extend([entry.shard_offset, entry.shard_bytes, entry.full_offset])
            for entry in unit.entries:
                for _ in range(self.world):
                    total += (entry.shard_bytes + 65535) // 65536
                    prefix.append(total)
            unit.gather_entries = torch.tensor(entries, device=device, dtype=torch.int64)
            unit.gather_prefix = torch.tensor(prefix, device=device, dtype=torch.int64)
            unit.gather_pieces = total
            unit.piece_counts = torch.zeros(len(unit.entries) * self.world, device=device, dtype=torch.int32)
            unit.panel_flags = torch.zeros(len(unit.entries) * self.world, device=device, dtype=torch.int32)
            unit.gather_generation = 0
            unit.gatherer = self.gather_unit
        if self.prefetch:
            self.gather_stream = torch.cuda.Stream(device=device)
            self.sharder.enable_prefetch(self.gather_stream)
        base = self.offsets["headers"]
        self.header_offset = {}
        for position, record in enumerate(self.header_records):
            layer = record.layer
            offset = base + position * _HEADER_FLOATS * 4
            view = self.heap.view(offset, _HEADER_FLOATS * 4).view(torch.float32)
            length = layer.weight_quantizer.history.numel()
            view[0:1].copy_(layer.weight_scale)
            view[1:1 + length].copy_(layer.weight_quantizer.history)
            layer.weight_scale = view[0:1]
            layer.weight_quantizer.history = view[1:1 + length]
            self.header_offset[record.index] = (offset, (1 + length) * 4)
        torch.cuda.synchronize(device)
        self.heap.barrier()

    def gather_unit(self, unit):
        """Fill ``unit.full`` with every rank's slabs (local rank first) by loads from peer memory."""
        unit.gather_generation += 1
        # a gather running beside compute on the prefetch stream stays narrow (NVLink saturates with a few dozen
        # blocks; more would only take SMs from the GEMMs); a gather the compute stream waits for takes the GPU
        side = getattr(self, "gather_stream", None)
        blocks = 48 if side is not None and torch.cuda.current_stream(self.device) == side else 1184
        self._ops.gather_pull(unit.gather_entries, self.pointers, self.rank, unit.heap_offset, unit.full,
                              unit.gather_prefix, unit.piece_counts, unit.panel_flags, unit.gather_generation,
                              unit.gather_pieces, blocks)
        ops._count()

    def write_fp8_weight(self, record, master, scale, limit):
        """Owner: quantise ``master`` with ``scale`` and store the codes into every rank's slab + header."""
        unit, entry = record.unit, record.entry
        offset = unit.heap_offset + entry.shard_offset
        rows = entry.rows
        cols = entry.row_bytes            # FP8: one byte per element
        self._ops.quantize_push(master.view(rows, cols), scale, float(limit), _FMT_OF[record.dtype], None, 0.0,
                                self.pointers, self.rank, offset, entry.shard_rows, 2368)
        header_offset, header_bytes = self.header_offset[record.index]
        header = self.heap.view(header_offset, _align(header_bytes, 16))
        self._ops.byte_push(header, self.pointers, self.rank, header_offset, 0, 1)
        ops._count(2)

    def write_bytes(self, record, payload):
        """Owner: store an already encoded full tensor into the ranks' slabs (16-byte aligned slabs only)."""
        unit, entry = record.unit, record.entry
        if entry.shard_bytes % 16 or (unit.heap_offset + entry.shard_offset) % 16:
            return False
        padded_bytes = self.world * entry.shard_bytes
        flat = payload.contiguous().view(torch.uint8).reshape(-1)
        if flat.numel() != padded_bytes:
            staged = torch.zeros(padded_bytes, device=flat.device, dtype=torch.uint8)
            staged[:flat.numel()].copy_(flat)
            flat = staged
        self._ops.byte_push(flat, self.pointers, self.rank, unit.heap_offset + entry.shard_offset, entry.shard_bytes,
                            2368)
        ops._count()
        return True

    # ------------------------------------------------------------------ per-step message + barrier
    def attach_usage(self, count):
        """Reserve one message slot per rank: ``[status code, non-finite flag, used[0..count)]`` as int32."""
        self.usage_words = 2 + count
        self.usage_slot = _align(4 * self.usage_words, 16)
        self.request("usage", self.usage_slot * self.world)
        self.usage_generation = 0
        self.barrier_generation = 0

    def finalize_usage(self):
        self.usage_flag_offset = self.flags("usage", self.world)
        self.barrier_flag_offset = self.flags("barrier", self.world)
        self.usage_message = torch.zeros(self.usage_slot // 4, device=self.device, dtype=torch.int32)
        self.usage_staging = torch.zeros(self.usage_words, dtype=torch.int32).pin_memory()
        self.usage_host = torch.zeros(self.world * self.usage_slot // 4, dtype=torch.int32).pin_memory()
        self.usage_event = torch.cuda.Event()
        self.usage_armed = False

    def exchange_usage(self, used, *, bad=None, injected=0):
        """Send this rank's step message to every rank and enqueue the wait for everyone's.

        ``used``: list of bools (one per parameter record); ``bad``: optional device int32[1] non-finite flag;
        ``injected``: a host-side status code to report instead of the device word (fault tests).
        The host first waits for the *previous* step's exchange to land (which bounds how far the host can run
        ahead of the GPU to one step and frees the pinned buffers for reuse) and raises, on every rank alike, if
        any rank reported a kernel failure in it.  It does not wait for this step's exchange; :meth:`read_usage`
        does when the caller needs the answer now."""
        previous = self.read_usage(wait=True)
        if previous is not None:
            self.raise_for_codes(previous[0])
        staging = self.usage_staging
        staging[0] = int(injected)
        staging[1] = 0
        staging[2:] = torch.tensor(used, dtype=torch.int32)
        message = self.usage_message
        message[:self.usage_words].copy_(staging, non_blocking=True)
        if not injected:
            message[0:1].copy_(self.status[0:1])
        if bad is not None:
            message[1:2].copy_(bad.reshape(1))
        self.usage_generation += 1
        base = self.offsets["usage"]
        self._ops.byte_push(message.view(torch.uint8), self.pointers, self.rank, base + self.rank * self.usage_slot, 0, 1)
        self._ops.signal(self.pointers, self.rank, self.usage_flag_offset, self.usage_generation, True)
        self._ops.wait_flags(self.local_pointer(self.usage_flag_offset), self.world, -1, self.usage_generation,
                             self.wait_clocks, self.status)
        self.usage_host.copy_(self.heap.view(base, self.world * self.usage_slot).view(torch.int32), non_blocking=True)
        self.usage_event.record(torch.cuda.current_stream(self.device))
        self.usage_armed = True
        ops._count(3)

    def read_usage(self, *, wait):
        """``(codes, bad, used)`` per rank from the latest completed exchange, or None when it has not landed yet
        (``wait=False``).  ``codes[r]`` is rank r's status code, ``used`` the element-wise OR over ranks."""
        if not self.usage_armed:
            return None
        if wait:
            self.usage_event.synchronize()
        elif not self.usage_event.query():
            return None
        table = self.usage_host.view(self.world, self.usage_slot // 4)
        codes = table[:, 0].tolist()
        bad = bool(table[:, 1].max().item())
        used = table[:, 2:self.usage_words].max(dim=0).values.bool().tolist()
        return codes, bad, used

    def raise_for_codes(self, codes):
        for rank, code in enumerate(codes):
            if code:
                self.usage_armed = False
                raise RuntimeError(f"rank {rank}: {ops.status_message([code, 0, 0, 0], f'rank {rank}')}; the step that "
                                   "followed it did not see that rank's data, stop and resume from a checkpoint")

    def barrier(self):
        """On-stream barrier over all ranks (signal + bounded wait); the host does not wait."""
        self.barrier_generation += 1
        self._ops.signal(self.pointers, self.rank, self.barrier_flag_offset, self.barrier_generation, True)
        self._ops.wait_flags(self.local_pointer(self.barrier_flag_offset), self.world, -1, self.barrier_generation,
                             self.wait_clocks, self.status)
        ops._count(2)

    def write_table(self, table, *, calls, decay=0.0, with_ema=False):
        """Fused owner write-back of a :class:`viola_b200.ops.WritebackTable` whose offsets are heap offsets."""
        ops.multi_writeback(table, heaps=self.pointers, rank=self.rank, calls=calls, decay=decay, with_ema=with_ema)

    def publish_step(self):
        """Owner side done: tell every rank; then wait until every owner's stores for this step landed."""
        self.step_generation += 1
        self._ops.signal(self.pointers, self.rank, self.step_flag_offset, self.step_generation, True)
        self._ops.wait_flags(self.local_pointer(self.step_flag_offset), self.world, -1, self.step_generation,
                             self.wait_clocks, self.status)
        ops._count(2)

    def close(self):
        if self.stream is not None:
            self.stream.synchronize()


_FMT_OF = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
