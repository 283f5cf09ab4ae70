"""Sleep / wake-up memory pools on the CUDA virtual-memory API.

``CuMemAllocator`` routes allocations made inside ``use_memory_pool(tag)`` through the native
allocator in ``_host.so`` (``csrc_host/cumem.cpp``): each allocation is an address range with
separately owned physical memory.  ``sleep(offload_tags)`` gives the physical memory back to the
driver — tags in ``offload_tags`` keep a pinned host copy, other tags are simply dropped — and
``wake_up(tags)`` maps new memory at the same addresses and restores the copies, so tensors and
captured CUDA graphs stay valid.

Parity: ``aphrodite/device_allocator/cumem.py`` (``CuMemAllocator.use_memory_pool/sleep/wake_up``)
over ``csrc/cumem_allocator.cpp``.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

_HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_host.so")


class CuMemAllocator:
    _instance: "CuMemAllocator | None" = None

    @classmethod
    def get_instance(cls) -> "CuMemAllocator":
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def __init__(self) -> None:
        lib = ctypes.CDLL(_HOST)
        lib.sonar_cumem_set_tag.argtypes = [ctypes.c_char_p]
        lib.sonar_cumem_sleep.argtypes = [ctypes.c_char_p, ctypes.c_int]
        lib.sonar_cumem_sleep.restype = ctypes.c_longlong
        lib.sonar_cumem_wake.argtypes = [ctypes.c_char_p]
        lib.sonar_cumem_wake.restype = ctypes.c_longlong
        lib.sonar_cumem_stats.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_longlong)]
        self.lib = lib
        self.available = bool(lib.sonar_cumem_available()) and torch.cuda.is_available()
        self._pools: dict[str, object] = {}
        self._alloc = None
        self.tags: set[str] = set()
        self.sleeping: set[str] = set()

    def _torch_allocator(self):
        if self._alloc is None:
            self._alloc = torch.cuda.memory.CUDAPluggableAllocator(_HOST, "sonar_cumem_malloc", "sonar_cumem_free")
        return self._alloc

    @contextlib.contextmanager
    def use_memory_pool(self, tag: str):
        """Allocations made by torch inside the block belong to ``tag``."""
        if not self.available:
            raise RuntimeError("the CUDA driver's virtual-memory API is not available in this process")
        pool = self._pools.get(tag)
        if pool is None:
            pool = torch.cuda.MemPool(self._torch_allocator().allocator())
            self._pools[tag] = pool
        self.tags.add(tag)
        self.lib.sonar_cumem_set_tag(tag.encode())
        try:
            with torch.cuda.use_mem_pool(pool):
                yield
        finally:
            self.lib.sonar_cumem_set_tag(b"default")

    def sleep(self, offload_tags: tuple[str, ...] | str = ()) -> int:
        """Release the physical memory of every pool.  Returns the bytes released."""
        if isinstance(offload_tags, str):
            offload_tags = (offload_tags,)
        torch.cuda.synchronize()
        total = 0
        for tag in sorted(self.tags - self.sleeping):
            n = self.lib.sonar_cumem_sleep(tag.encode(), int(tag in offload_tags))
            if n < 0:
                raise RuntimeError(f"sleep({tag}) failed: CUDA driver error {self.lib.sonar_cumem_last_error()}")
            total += n
            self.sleeping.add(tag)
        return total

    def wake_up(self, tags: list[str] | None = None) -> int:
        total = 0
        for tag in sorted(self.sleeping if tags is None else set(tags) & self.sleeping):
            n = self.lib.sonar_cumem_wake(tag.encode())
            if n < 0:
                raise RuntimeError(f"wake_up({tag}) failed: CUDA driver error {self.lib.sonar_cumem_last_error()}")
            total += n
            self.sleeping.discard(tag)
        return total

    def stats(self, tag: str | None = None) -> dict[str, int]:
        out = (ctypes.c_longlong * 4)()
        self.lib.sonar_cumem_stats(tag.encode() if tag else None, out)
        return {"allocations": out[0], "mapped_bytes": out[1], "sleeping_bytes": out[2], "host_copy_bytes": out[3]}
