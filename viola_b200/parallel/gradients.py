"""Gradient accumulation with replicated or whole-parameter-owned placement.

Structure and rules of the reference's ``GradientState`` (viola/distributed/gradients.py:21-156):
a flat accumulator (all parameters, or only the owned ones when gradients are sharded); buckets
that walk the parameters in reverse order, break at every owner change and at ``bucket_mb``; a
post-accumulate hook that steals ``param.grad``; reduce-to-owner per microbatch for sharded
gradients; one all-reduce at the step for replicated gradients; unused parameters contribute
zeros; usage flags agreed with a MAX reduction.

What differs: buckets are drained as soon as their gradients exist even when parameters are
sharded (this package's sharder issues no collectives of its own during backward when the
peer-memory transport is active, so there is no collective-order hazard), the transport is
pluggable (collectives here, fused peer-memory kernels in :mod:`viola_b200.parallel.symm`), and with
a single rank every communication step is skipped.
"""

from __future__ import annotations

from functools import partial

import torch
import torch.distributed as dist

from .config import dtype as to_dtype
from .fp8 import FP8Communication


class GradientState:
    def __init__(self, store, *, gradient_dtype, communication_dtype=None, bucket_mb=25, fp8_format="e4m3",
                 fp8_tile_size=256, shard=False, defer_reduction=False, transport=None, monitor=None, landing=True,
                 reduce_once=True):
        self.store = store
        self.monitor = monitor
        self.mailbox = transport          # per-step usage / status exchange, whatever moves the gradients
        self.records = store.records
        self.rank, self.world, self.group = store.rank, store.world, store.group
        self.shard = shard and self.world > 1
        self.requested_shard = shard
        self.defer_reduction = defer_reduction
        self.gradient_dtype = gradient_dtype
        self.fp8_requested = communication_dtype == "fp8"
        self.dtype = torch.float32 if self.fp8_requested else (to_dtype(communication_dtype) or gradient_dtype)
        device = self.records[0].parameter.device
        if self.fp8_requested and device.type != "cuda" and self.world > 1:
            raise RuntimeError("FP8 gradient communication needs CUDA")
        element = torch.empty((), dtype=self.dtype).element_size()
        total = sum(r.numel for r in self.records)
        capacity = min(max(1, int(bucket_mb * 1024 * 1024) // element), total)
        # buckets: (owner, [(record index, offset in parameter, offset in bucket, length)], filled)
        self.buckets, self.piece_counts = [], [0] * len(self.records)
        pieces, filled, owner = [], 0, None
        for index in reversed(range(len(self.records))):
            record = self.records[index]
            if pieces and record.owner != owner:
                self.buckets.append((owner, pieces, filled))
                pieces, filled = [], 0
            owner, position = record.owner, 0
            while position < record.numel:
                length = min(record.numel - position, capacity - filled)
                pieces.append((index, position, filled, length))
                self.piece_counts[index] += 1
                position += length
                filled += length
                if filled == capacity:
                    self.buckets.append((owner, pieces, filled))
                    pieces, filled = [], 0
        if pieces:
            self.buckets.append((owner, pieces, filled))
        # The accumulator is laid out in bucket order, so every bucket is one contiguous slice of it
        # (a parameter that spans buckets ends one bucket and starts the next, hence stays contiguous).
        kept = [not self.shard or bucket_owner == self.rank for bucket_owner, _, _ in self.buckets]
        self.accumulator = torch.zeros(sum(length for (_, _, length), keep in zip(self.buckets, kept) if keep),
                                       device=device, dtype=gradient_dtype)
        self.local, self.bucket_slices, offset = {}, [], 0
        for (bucket_owner, bucket_pieces, length), keep in zip(self.buckets, kept):
            if not keep:
                self.bucket_slices.append(None)
                continue
            self.bucket_slices.append(self.accumulator[offset:offset + length])
            for index, position, target, size in bucket_pieces:
                if position == 0:
                    self.local[index] = self.accumulator[offset + target:offset + target + self.records[index].numel]
            offset += length
        self.bucket_capacity = max(length for _, _, length in self.buckets)
        # Landing buffer: one wire-dtype slot per parameter, laid out in bucket order, that this microbatch's
        # gradients are written into.  Layers of this package write their weight / bias gradient straight into the
        # slot (``parameter._viola_grad_slot``), so a bucket is ready for the reduction kernels without any
        # per-parameter copy, and replicated / single-rank accumulation is one add over the whole buffer.
        self.landing = torch.zeros(total, device=device, dtype=self.dtype) if landing else None
        self.slots, self.bucket_landing = {}, []
        if self.landing is not None:
            start = 0
            for _, bucket_pieces, length in self.buckets:
                self.bucket_landing.append(self.landing[start:start + length])
                for index, position, target, size in bucket_pieces:
                    if position == 0:
                        record = self.records[index]
                        self.slots[index] = self.landing[start + target:start + target + record.numel].view(record.shape)
                start += length
        # Sharded gradients, reduced once per optimizer step: every microbatch adds its landing buffer into a
        # rank-local fp32 sum (one launch), and the step sends that sum to the owners.  The reduction moves the same
        # bytes whatever the microbatch size, so doing it per microbatch costs the same again for every accumulation
        # step; the price is one more buffer of the gradients' size on every rank.
        self.once = bool(reduce_once) and self.shard and self.landing is not None
        # With fp32 gradients the landing buffer itself can hold the running sum of the step: producers add into
        # their slot (the weight-gradient GEMM's epilogue is a TMA reduce-add), so no pass over the gradients is
        # needed per microbatch.  Replicated / single-rank: the landing buffer IS the accumulator.
        self.summing = (self.landing is not None and self.dtype == torch.float32 and gradient_dtype == torch.float32
                        and (self.once or not self.shard))
        if self.summing and not self.shard:
            self.accumulator = self.landing
            self.bucket_slices = list(self.bucket_landing)
            self.local = {index: slot.view(-1) for index, slot in self.slots.items()}
        self.local_sum = (self.landing if self.summing else torch.zeros_like(self.landing)) if self.once else None
        self.bucket_sum = []
        self.pending_local = False
        if self.once:
            start = 0
            for _, _, length in self.buckets:
                self.bucket_sum.append(self.local_sum[start:start + length])
                start += length
        self.vector_slots = []
        self.claimed = [False] * len(self.records)
        # one-dimensional slots (biases) are accumulated into by atomic column sums: cleared together, one launch per
        # microbatch, instead of one fill per layer
        if not self.summing:
            self.vector_slots = [i for i, slot in self.slots.items() if slot.dim() == 1]
        self.vectors_cleared = False
        self.buffer = (torch.empty(self.bucket_capacity, device=device, dtype=self.dtype)
                       if self.world > 1 and self.landing is None else None)
        self.transport = transport if (transport is not None and self.fp8_requested and self.world > 1
                                       and gradient_dtype == torch.float32) else None
        if self.transport is not None:
            if self.shard:
                self.transport.attach_gradients(self.buckets, self.bucket_slices, self.bucket_capacity)
            else:
                self.transport.attach_all_reduce(self.bucket_capacity)
        transport = self.transport
        self.fp8 = None
        if self.fp8_requested and self.world > 1 and transport is None:
            self.fp8 = FP8Communication(self.bucket_capacity, self.group, self.rank, self.world, store.global_ranks,
                                        device, mode="reduce" if self.shard else "all_reduce", fp8_format=fp8_format,
                                        tile_size=fp8_tile_size)
        self.used = [False] * len(self.records)
        self.pending = [None] * len(self.records)
        self.in_backward = False
        self.hooks = []
        self._bound = set()

    # ------------------------------------------------------------------ hooks
    def bind(self, index, parameter):
        if id(parameter) in self._bound:
            return
        self._bound.add(id(parameter))
        self.hooks.append(parameter.register_post_accumulate_grad_hook(partial(self._ready, index)))
        if index in self.slots and self.dtype == self.gradient_dtype:
            parameter._viola_grad_slot = partial(self._claim, index)

    def _claim(self, index):
        """The landing slot of parameter ``index`` for the layer that is about to produce its gradient, once per
        microbatch (a second producer of a tied parameter gets None and autograd adds the two)."""
        if not self.in_backward or self.claimed[index]:
            return None
        self.claimed[index] = True
        # a fresh view: autograd adopts a gradient tensor as ``.grad`` without copying only when nothing else
        # holds a reference to that tensor object
        slot = self.slots[index].view(self.slots[index].shape)
        if self.summing:
            slot._viola_accumulate = True
            # a producer that cannot add into the running sum hands the slot back and returns its own tensor
            slot._viola_release = partial(self._unclaim, index)
        elif self.vectors_cleared and slot.dim() == 1:
            slot._viola_zeroed = True
        return slot

    def _unclaim(self, index):
        self.claimed[index] = False

    def begin_backward(self):
        self.in_backward = True
        self.seen = [False] * len(self.records)
        self.claimed = [False] * len(self.records)
        self.vectors_cleared = False
        if self.vector_slots and self.landing is not None:
            torch._foreach_zero_([self.slots[i] for i in self.vector_slots])
            self.vectors_cleared = True
        self.remaining = self.piece_counts.copy()
        self.next_bucket = 0
        if self.transport is not None and self.shard and not self.once:
            self.transport.begin_microbatch()
        if self.store.sharder is not None:
            self.store.sharder.begin_backward()

    @torch.no_grad()
    def _ready(self, index, parameter):
        self.seen[index] = self.used[index] = True
        gradient = parameter.grad
        parameter.grad = None
        if self.landing is not None:
            slot = self.slots[index]
            if gradient.data_ptr() != slot.data_ptr():        # produced elsewhere (torch layers, tied weights)
                if self.summing and not self.claimed[index]:
                    slot.add_(gradient.view(slot.shape))      # the slot holds the step's running sum
                else:                                          # (a claimed slot's sum is already part of ``gradient``)
                    slot.copy_(gradient.view(slot.shape))
            if self.shard and not self.defer_reduction and not self.once:
                self._drain()
        elif self.shard:
            self.pending[index] = gradient.contiguous().view(-1)
            if not self.defer_reduction:
                self._drain()
        else:
            self.local[index].add_(gradient.contiguous().view(-1))
        if self.store.sharder is not None:
            self.store.sharder.gradient_arrived(parameter)

    @torch.no_grad()
    def _drain(self, *, final=False):
        while self.next_bucket < len(self.buckets):
            owner, pieces, length = self.buckets[self.next_bucket]
            if not final and any(not self.seen[i] for i, _, _, _ in pieces):
                break
            if self.landing is not None:
                self._reduce_landed(self.next_bucket, owner, pieces, length)
                self.next_bucket += 1
                continue
            if self.transport is not None:
                staging_index, staging = self.transport.next_staging()
                buffer = staging[:length]
            else:
                buffer = self.buffer[:length]
            for index, source, target, size in pieces:
                slot = buffer[target:target + size]
                gradient = self.pending[index]
                if gradient is None:
                    slot.zero_()
                else:
                    slot.copy_(gradient[source:source + size])
                self.remaining[index] -= 1
                if not self.remaining[index]:
                    self.pending[index] = None
            if self.transport is not None:
                self.transport.reduce_to_owner(self.next_bucket, staging_index, length)
            else:
                if self.fp8 is not None:
                    self.fp8.reduce(buffer, owner)
                else:
                    dist.reduce(buffer, dst=self.store.global_ranks[owner], group=self.group)
                if self.rank == owner:
                    for index, target, source, size in pieces:
                        self.local[index][target:target + size].add_(buffer[source:source + size])
            self.next_bucket += 1

    def _reduce_landed(self, bucket_index, owner, pieces, length):
        """Reduce one bucket straight from the landing buffer (no staging copy, no per-piece work)."""
        buffer = self.bucket_landing[bucket_index]
        for index, position, target, size in pieces:
            if not self.seen[index]:
                buffer[target:target + size].zero_()          # unused on this rank: contributes zeros
        if self.transport is not None:
            self.transport.reduce_to_owner(bucket_index, None, length, buffer=buffer)
            return
        if self.fp8 is not None:
            self.fp8.reduce(buffer, owner)
        else:
            dist.reduce(buffer, dst=self.store.global_ranks[owner], group=self.group)
        if self.rank == owner:
            self.bucket_slices[bucket_index].add_(buffer)

    def _accumulate_landed(self):
        """Replicated / single-rank accumulation: one add of the whole landing buffer."""
        if self.summing:
            return                                             # the landing buffer is the accumulator
        if not all(self.seen):
            for index, seen in enumerate(self.seen):
                if not seen and index in self.slots:
                    self.slots[index].zero_()
        self.accumulator.add_(self.landing)

    def _sum_landed(self):
        """Add this microbatch's gradients to the rank-local sum that the step will reduce."""
        self.pending_local = True
        if self.summing:
            return                                             # the producers added into the landing buffer themselves
        if not all(self.seen):
            for index, seen in enumerate(self.seen):
                if not seen and index in self.slots:
                    self.slots[index].zero_()             # unused on this rank in this microbatch: contributes zeros
        self.local_sum.add_(self.landing)
        self.pending_local = True

    def _reduce_summed(self):
        """Send the rank-local sums of all buckets to their owners (once per optimizer step)."""
        if self.transport is not None:
            # one-sided kernels over a table of buckets: one launch pushes everything owned elsewhere, one launch
            # accumulates everything owned here (two rendezvous per step instead of two per bucket)
            self.transport.begin_microbatch()
            self.transport.reduce_all(self.bucket_sum)
            self.transport.synchronize()
            self.local_sum.zero_()
            self.pending_local = False
            return
        for bucket_index, (owner, _, length) in enumerate(self.buckets):
            buffer = self.bucket_sum[bucket_index]
            if self.fp8 is not None:
                self.fp8.reduce(buffer, owner)
            else:
                dist.reduce(buffer, dst=self.store.global_ranks[owner], group=self.group)
            if self.rank == owner:
                self.bucket_slices[bucket_index].add_(buffer)
        self.local_sum.zero_()
        self.pending_local = False

    def finish_backward(self):
        if self.once:
            self._sum_landed()
        elif self.shard:
            self._drain(final=True)
        elif self.landing is not None:
            self._accumulate_landed()
        if self.store.sharder is not None:
            self.store.sharder.finish_backward()
        if self.transport is not None:
            self.transport.synchronize()        # side-stream work joins the compute stream every microbatch
        self.in_backward = False

    # ------------------------------------------------------------------ step-time reduction
    def _agree_on_usage(self):
        """Which records produced a gradient on any rank (``active``), with every rank's kernel status riding
        along so that a recorded failure raises everywhere in the same step.

        Peer-memory transport: each rank stores its message into all heaps and the host does not wait; when
        every local record was used the answer is "all" whatever the peers say, so the host only waits in the
        rare step with locally unused parameters.  Collective transports: one MAX all-reduce.
        """
        count = len(self.records)
        code = self.monitor.local_code() if self.monitor is not None else 0
        if self.world == 1:
            if code:
                self.monitor.raise_for(code)
            return list(self.used)
        if self.mailbox is not None:
            self.mailbox.exchange_usage(self.used, injected=self.monitor.pending if self.monitor is not None else 0)
            if self.monitor is not None:
                self.monitor.pending = 0
            if all(self.used):
                return [True] * count
            codes, _, used = self.mailbox.read_usage(wait=True)
            self.mailbox.raise_for_codes(codes)
            return used
        message = torch.tensor([code, *self.used], device=self.accumulator.device, dtype=torch.int32)
        dist.all_reduce(message, op=dist.ReduceOp.MAX, group=self.group)
        values = message.tolist()
        if values[0]:
            self.monitor.raise_for(values[0], rank="(some)")
        return [bool(v) for v in values[1:]]

    @torch.no_grad()
    def reduce(self, divisor):
        """Agree on which parameters were used anywhere, finish replicated reductions, normalise."""
        if self.once and self.pending_local:
            self._reduce_summed()
        active = self._agree_on_usage()
        if self.world > 1 and not self.shard:
            for bucket in self.bucket_slices:          # bucket-ordered accumulator: reduce in place, no staging
                if self.transport is not None:
                    self.transport.all_reduce(bucket)
                elif self.fp8 is not None and bucket.dtype == torch.float32:
                    self.fp8.all_reduce(bucket)
                elif self.fp8 is None and bucket.dtype == self.dtype:
                    dist.all_reduce(bucket, group=self.group)
                else:                                  # wire dtype differs from the accumulator's
                    staged = self.buffer[:bucket.numel()].copy_(bucket)
                    if self.fp8 is not None:
                        self.fp8.all_reduce(staged)
                    else:
                        dist.all_reduce(staged, group=self.group)
                    bucket.copy_(staged)
        if self.transport is not None:
            self.transport.synchronize()
        self.accumulator.div_(divisor)
        return active

    # ------------------------------------------------------------------ CUDA-graph replays
    def capture_marks(self):
        """Which parameters produced a gradient in the microbatch that was just captured."""
        return [index for index, seen in enumerate(self.seen) if seen]

    def replay_marks(self, marks):
        """A replayed graph runs no Python hooks: restore the bookkeeping those hooks would have done."""
        for index in marks:
            self.used[index] = True
        if self.once:
            self.pending_local = True

    @torch.no_grad()
    def zero_grad(self):
        self.accumulator.zero_()
        if self.once and self.pending_local:
            self.local_sum.zero_()
            self.pending_local = False
        self.used = [False] * len(self.records)
