"""CPU tier of the prefix cache: KV blocks evicted from the GPU pool keep living in pinned host memory,
keyed by the same chained block hashes, and come back when a later request's prefix matches them.

The tier is pure bookkeeping on the scheduler side: it decides which host slot a block goes to or comes
from and emits the copy lists of a step — ``stores [(gpu_block, cpu_slot)]`` first, then ``loads
[(cpu_slot, gpu_block)]`` — that the worker executes on its stream before the forward pass (so an evicted
block is saved before its new owner overwrites it, and a loaded block is complete before attention reads
it).  Slots that take part in a step's copies are pinned until the lists are handed out.

Parity: the reference's simple CPU offload (``aphrodite/v1/simple_kv_offload``) and the CPU tier of
``v1/kv_offload`` (LRU over block hashes, store on eviction, load on prefix hit).
"""
from __future__ import annotations

from collections import OrderedDict


class CPUOffloadTier:
    def __init__(self, num_cpu_blocks: int) -> None:
        self.num_slots = num_cpu_blocks
        self.slot_of: OrderedDict[bytes, int] = OrderedDict()     # hash → slot, least recently used first
        self.free_slots = list(range(num_cpu_blocks - 1, -1, -1))
        self.pinned: set[int] = set()
        self.stores: list[tuple[int, int]] = []
        self.loads: list[tuple[int, int]] = []
        self.num_stored = self.num_loaded = self.num_dropped = 0

    # eviction side ----------------------------------------------------------
    def on_evict(self, gpu_block: int, block_hash: bytes) -> None:
        """A cached GPU block is about to be reused: keep its contents in the tier."""
        if block_hash in self.slot_of:
            self.slot_of.move_to_end(block_hash)
            return
        slot = self._take_slot()
        if slot is None:
            self.num_dropped += 1
            return
        self.slot_of[block_hash] = slot
        self.pinned.add(slot)
        self.stores.append((gpu_block, slot))
        self.num_stored += 1

    def _take_slot(self) -> int | None:
        if self.free_slots:
            return self.free_slots.pop()
        for h, slot in self.slot_of.items():           # least recently used first
            if slot not in self.pinned:
                del self.slot_of[h]
                return slot
        return None

    # lookup side --------------------------------------------------------------
    def lookup(self, block_hash: bytes) -> int | None:
        return self.slot_of.get(block_hash)

    def request_load(self, block_hash: bytes, gpu_block: int) -> None:
        slot = self.slot_of[block_hash]
        self.slot_of.move_to_end(block_hash)
        self.pinned.add(slot)
        self.loads.append((slot, gpu_block))
        self.num_loaded += 1

    def take_transfers(self) -> tuple[list[tuple[int, int]], list[tuple[int, int]]]:
        out = (self.stores, self.loads)
        self.stores, self.loads = [], []
        self.pinned.clear()
        return out

    def clear(self) -> None:
        self.slot_of.clear()
        self.free_slots = list(range(self.num_slots - 1, -1, -1))
        self.pinned.clear()
        self.stores, self.loads = [], []
