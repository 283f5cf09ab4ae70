"""Symmetric device memory across the ranks of a process group.

Every rank allocates a buffer of the same size; after ``rendezvous`` each rank
holds a device address for every peer's buffer (NVLink peer mapping), which
kernels use for plain loads/stores, ``red`` and flag words.  The allocator is
PyTorch's symmetric-memory pool (CUDA VMM handles exchanged through the group's
store; also yields an NVSwitch multicast address when the fabric supports it);
if that is unavailable the buffer is a regular allocation shared through CUDA
IPC handles.

Parity: the IPC buffer registration of the reference's custom all-reduce
(``distributed/device_communicators/custom_all_reduce.py:476``,
``csrc/custom_all_reduce.cuh:138-225``) and its torch symmetric-memory
communicator (``device_communicators/symm_mem.py:25``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from sonar_b200.logger import init_logger

logger = init_logger(__name__)


class SymmetricBuffer:
    """``nbytes`` of zero-initialised device memory on every rank of ``group``."""

    def __init__(self, nbytes: int, device: torch.device, group, group_ranks: list[int]) -> None:
        self.nbytes = (nbytes + 255) // 256 * 256
        self.device = device
        self.world = len(group_ranks)
        self.rank = group_ranks.index(dist.get_rank())
        self.multicast_ptr = 0
        self.backend = "symm_mem"
        self._keep = []
        try:
            self._init_symm_mem(group)
        except Exception as e:  # noqa: BLE001 - any failure of the optional allocator falls back to IPC
            logger.warning("symmetric-memory allocator unavailable (%s); using CUDA IPC", e)
            self.backend = "ipc"
            self._init_ipc(group, group_ranks)
        self.local_ptr = self.peer_ptrs[self.rank]

    def _init_symm_mem(self, group) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        self.local = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.local.zero_()
        hdl = symm_mem.rendezvous(self.local, group=group)
        self.peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        try:
            self.multicast_ptr = int(hdl.multicast_ptr or 0)
        except Exception:  # noqa: BLE001
            self.multicast_ptr = 0
        self._keep.append(hdl)
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def _init_ipc(self, group, group_ranks: list[int]) -> None:
        self.local = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
        torch.cuda.synchronize()
        shared = self.local.untyped_storage()._share_cuda_()
        gathered: list = [None] * self.world
        dist.all_gather_object(gathered, shared, group=group)
        self.peer_ptrs = []
        for r, args in enumerate(gathered):
            if r == self.rank:
                self.peer_ptrs.append(self.local.data_ptr())
                continue
            storage = torch.UntypedStorage._new_shared_cuda(*args)
            t = torch.empty(0, dtype=torch.uint8, device=torch.device("cuda", args[0])).set_(storage)
            self._keep.append(t)
            self.peer_ptrs.append(t.data_ptr())
        dist.barrier(group=group)

    def view(self, offset: int, shape, dtype: torch.dtype) -> torch.Tensor:
        """Typed view of the local buffer starting ``offset`` bytes in."""
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def ptr_table(self, offset: int, extra_per_peer=None) -> torch.Tensor:
        """Device int64 array: ``peer_ptrs[d] + offset (+ extra_per_peer(d))``."""
        vals = [p + offset + (extra_per_peer(d) if extra_per_peer else 0) for d, p in enumerate(self.peer_ptrs)]
        return torch.tensor(vals, dtype=torch.int64, device=self.device)
