"""FP8 gradient wire format over ``torch.distributed`` collectives (the portable transport).

A *packet* holds ``groups`` tiles of ``tile`` one-byte codes followed by ``groups`` fp32 scales, padded to
16 bytes (``ops.packet_bytes``).  Two operations use it, with the arithmetic of the reference codec
(viola/distributed/fp8.py:9-85):

``reduce(value, owner)``
    every rank encodes its bucket; the packets are gathered on ``owner``, which decodes them and sums in
    ascending rank order in fp32 into ``value`` (its own contribution goes through the codec as well, so the
    result does not depend on who owns the bucket).  Long buckets go in chunks sized so that the owner's
    receive buffer stays near the size of one fp32 bucket instead of ``world`` of them.
``all_reduce(value)``
    rank ``j`` receives everyone's encoding of chunk ``j`` (all-to-all), sums, encodes the sum a second time
    and all ranks gather those packets and decode them into ``value``.

The packets travel as ``uint8`` through NCCL (Gloo has no use for this class: FP8 needs the CUDA codec).
This is the measured baseline of the peer-memory kernels in :mod:`viola_b200.parallel.symm`, which do the
same arithmetic inside the kernels that move the bytes.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops import packet_bytes

_FORMATS = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def _ceil_div(a, b):
    return -(-a // b)


class FP8Communication:
    def __init__(self, capacity, group, rank, world, global_ranks, device, *, mode, fp8_format="e4m3", tile_size=256):
        if tile_size < 32 or tile_size & (tile_size - 1):
            raise ValueError("fp8_tile_size must be a power of two >= 32")
        if mode not in ("reduce", "all_reduce"):
            raise ValueError("mode must be 'reduce' or 'all_reduce'")
        self.fp8_dtype = _FORMATS[fp8_format]
        self.group, self.rank, self.world = group, rank, world
        self.global_ranks = list(global_ranks)
        self.tile_size, self.mode, self.device = tile_size, mode, device
        self._outgoing = self._incoming = self._sum = None
        if world == 1:
            return
        if mode == "all_reduce":
            per_rank = _ceil_div(capacity, world * tile_size)               # tiles each rank reduces
            self._outgoing = self._bytes(world * packet_bytes(per_rank, tile_size))
            self._incoming = torch.empty_like(self._outgoing)
            self._sum = torch.empty(per_rank * tile_size, device=device, dtype=torch.float32)
        else:
            tiles = _ceil_div(capacity, tile_size)
            budget = capacity * 4 // (world * (tile_size + 4))              # tiles whose `world` packets fit one bucket
            self.chunk_tiles = max(1, min(tiles, budget))
            self._outgoing = self._bytes(packet_bytes(self.chunk_tiles, tile_size))

    def _bytes(self, count):
        return torch.empty(count, device=self.device, dtype=torch.uint8)

    # kept for callers that size or report the wire buffers
    @property
    def send(self):
        return self._outgoing

    @property
    def receive(self):
        return self._incoming

    @property
    def chunk_size(self):
        return self.chunk_tiles * self.tile_size

    @property
    def workspace_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self._outgoing, self._incoming, self._sum) if t is not None)

    @torch.no_grad()
    def all_reduce(self, value):
        if self.world == 1:
            return
        tile, world, codec = self.tile_size, self.world, self.fp8_dtype
        per_rank = _ceil_div(value.numel(), world * tile)
        packet = packet_bytes(per_rank, tile)
        outgoing = self._outgoing[:world * packet].view(world, packet)
        incoming = self._incoming[:world * packet].view(world, packet)
        own_sum = self._sum[:per_rank * tile]
        ops.wire_pack(value, outgoing, tile, codec)                         # row j = my encoding of chunk j
        dist.all_to_all_single(incoming, outgoing, group=self.group)        # row r = rank r's encoding of my chunk
        ops.wire_unpack(incoming, own_sum, tile, codec, reduce=True)
        ops.wire_pack(own_sum, outgoing[:1], tile, codec)                   # second quantisation
        dist.all_gather_into_tensor(incoming.view(-1), outgoing[0], group=self.group)
        ops.wire_unpack(incoming, value, tile, codec)

    @torch.no_grad()
    def reduce(self, value, owner):
        if self.world == 1:
            return
        tile, world, codec = self.tile_size, self.world, self.fp8_dtype
        receiving = self.rank == owner
        if receiving and self._incoming is None:
            self._incoming = self._bytes(world * self._outgoing.numel())
        destination = self.global_ranks[owner]
        step = self.chunk_tiles * tile
        for start in range(0, value.numel(), step):
            piece = value[start:start + step]
            packet = packet_bytes(_ceil_div(piece.numel(), tile), tile)
            outgoing = self._outgoing[:packet]
            ops.wire_pack(piece, outgoing.view(1, packet), tile, codec)
            if receiving:
                slots = self._incoming[:world * packet].view(world, packet)
                dist.gather(outgoing, list(slots.unbind(0)), dst=destination, group=self.group)
                ops.wire_unpack(slots, piece, tile, codec, reduce=True)
            else:
                dist.gather(outgoing, None, dst=destination, group=self.group)
