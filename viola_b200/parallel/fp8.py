"""FP8-on-the-wire gradient communication (collective-library transport).

Two operations with the reference's packet format and arithmetic (viola/distributed/fp8.py:9-85):
``reduce`` (quantise every rank's bucket, deliver to the owner, dequantise and sum in ascending
rank order in fp32 — the owner's own contribution is quantised too) and ``all_reduce`` (quantise,
exchange chunk j with rank j, sum, quantise the partial sum a second time, gather, dequantise).
This class moves the packets with ``torch.distributed`` collectives on ``uint8`` and is both the
portable path and the measured baseline; :mod:`viola_b200.parallel.symm` provides the fused
peer-memory kernels that do the same arithmetic without a packet round trip through HBM.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .. import ops
from ..ops import packet_bytes

_FORMATS = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


class FP8Communication:
    def __init__(self, capacity, group, rank, world, global_ranks, device, *, mode, fp8_format="e4m3", tile_size=256):
        if tile_size < 32 or tile_size & (tile_size - 1):
            raise ValueError("fp8_tile_size must be a power of two >= 32")
        self.fp8_dtype = _FORMATS[fp8_format]
        self.group, self.rank, self.world, self.global_ranks = group, rank, world, list(global_ranks)
        self.tile_size, self.mode, self.device = tile_size, mode, device
        self.send = self.receive = self.partial = None
        if world == 1:
            return
        if mode == "all_reduce":
            groups = math.ceil(capacity / (world * tile_size))
            self.send = torch.empty(world * packet_bytes(groups, tile_size), device=device, dtype=torch.uint8)
            self.receive = torch.empty_like(self.send)
            self.partial = torch.empty(groups * tile_size, device=device, dtype=torch.float32)
        else:
            # bound the owner's gather buffer by about one fp32 bucket rather than world full buckets
            groups = max(1, min(math.ceil(capacity / tile_size), capacity * 4 // (world * (tile_size + 4))))
            self.chunk_size = groups * tile_size
            self.send = torch.empty(packet_bytes(groups, tile_size), device=device, dtype=torch.uint8)

    @property
    def workspace_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.send, self.receive, self.partial) if t is not None)

    @torch.no_grad()
    def all_reduce(self, value):
        if self.world == 1:
            return
        tile, world = self.tile_size, self.world
        groups = math.ceil(value.numel() / (world * tile))
        width, size = groups * tile, packet_bytes(groups, tile)
        send = self.send[:world * size].view(world, size)
        receive = self.receive[:world * size].view(world, size)
        partial = self.partial[:width]
        ops.wire_pack(value, send, tile, self.fp8_dtype)
        dist.all_to_all_single(receive, send, group=self.group)
        ops.wire_unpack(receive, partial, tile, self.fp8_dtype, reduce=True)
        ops.wire_pack(partial, send[:1], tile, self.fp8_dtype)
        dist.all_gather_into_tensor(receive.view(-1), send[0], group=self.group)
        ops.wire_unpack(receive, value, tile, self.fp8_dtype)

    @torch.no_grad()
    def reduce(self, value, owner):
        if self.world == 1:
            return
        tile = self.tile_size
        if self.rank == owner and self.receive is None:
            self.receive = torch.empty(self.world * self.send.numel(), device=self.device, dtype=torch.uint8)
        for offset in range(0, value.numel(), self.chunk_size):
            chunk = value[offset:offset + self.chunk_size]
            groups = math.ceil(chunk.numel() / tile)
            size = packet_bytes(groups, tile)
            send = self.send[:size]
            ops.wire_pack(chunk, send.view(1, -1), tile, self.fp8_dtype)
            receive = self.receive[:self.world * size].view(self.world, size) if self.rank == owner else None
            dist.gather(send, list(receive.unbind(0)) if receive is not None else None,
                        dst=self.global_ranks[owner], group=self.group)
            if receive is not None:
                ops.wire_unpack(receive, chunk, tile, self.fp8_dtype, reduce=True)
