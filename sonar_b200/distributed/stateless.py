"""Process groups that live outside ``torch.distributed``'s global state.

``StatelessProcessGroup`` is a small object-collective layer over a ``TCPStore``: ranks can form,
use and drop a group at any time without touching the default process group — what elastic
expert-parallel resizing, data-parallel coordination and NCCL unique-id exchange need.

Parity: ``aphrodite/distributed/utils.py`` (``StatelessProcessGroup``: ``send_obj / recv_obj /
broadcast_obj / all_gather_obj / barrier``), used by ``pynccl.py:60-145`` to bootstrap communicators.
"""
from __future__ import annotations

import pickle
import time
from datetime import timedelta
from typing import Any

from torch.distributed import TCPStore


class StatelessProcessGroup:
    def __init__(self, rank: int, world_size: int, store: TCPStore, prefix: str = "") -> None:
        self.rank, self.world_size, self.store = rank, world_size, store
        self.prefix = prefix
        self._send_ctr = {r: 0 for r in range(world_size)}
        self._recv_ctr = {r: 0 for r in range(world_size)}
        self._bcast_ctr = {r: 0 for r in range(world_size)}
        self._barrier_ctr = 0
        self._garbage: list[tuple[str, float]] = []

    @classmethod
    def create(cls, host: str, port: int, rank: int, world_size: int, timeout_s: float = 300.0,
               prefix: str = "") -> "StatelessProcessGroup":
        store = TCPStore(host, port, world_size, is_master=(rank == 0), timeout=timedelta(seconds=timeout_s),
                         wait_for_workers=False)
        return cls(rank, world_size, store, prefix)

    # point to point ----------------------------------------------------------
    def send_obj(self, obj: Any, dst: int) -> None:
        self._expire()
        key = f"{self.prefix}send/{self.rank}->{dst}/{self._send_ctr[dst]}"
        self.store.set(key, pickle.dumps(obj))
        self._send_ctr[dst] += 1
        self._garbage.append((key, time.time()))

    def recv_obj(self, src: int) -> Any:
        key = f"{self.prefix}send/{src}->{self.rank}/{self._recv_ctr[src]}"
        obj = pickle.loads(self.store.get(key))
        self._recv_ctr[src] += 1
        return obj

    # collectives ---------------------------------------------------------------
    def broadcast_obj(self, obj: Any, src: int) -> Any:
        key = f"{self.prefix}bcast/{src}/{self._bcast_ctr[src]}"
        self._bcast_ctr[src] += 1
        if self.rank == src:
            self._expire()
            self.store.set(key, pickle.dumps(obj))
            self._garbage.append((key, time.time()))
            return obj
        return pickle.loads(self.store.get(key))

    def all_gather_obj(self, obj: Any) -> list[Any]:
        out = []
        for r in range(self.world_size):
            out.append(self.broadcast_obj(obj if r == self.rank else None, r))
        return out

    def barrier(self, timeout_s: float = 300.0) -> None:
        n = self._barrier_ctr
        self._barrier_ctr += 1
        key = f"{self.prefix}barrier/{n}"
        self.store.add(key, 1)
        deadline = time.time() + timeout_s
        while int(self.store.add(key, 0)) < self.world_size:
            if time.time() > deadline:
                raise TimeoutError(f"barrier {n}: not every rank of {self.world_size} arrived in {timeout_s}s")
            time.sleep(0.002)

    def _expire(self, ttl_s: float = 600.0) -> None:
        now = time.time()
        while self._garbage and now - self._garbage[0][1] > ttl_s:
            key, _ = self._garbage.pop(0)
            try:
                self.store.delete_key(key)
            except Exception:  # noqa: BLE001
                pass
