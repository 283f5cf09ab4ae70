"""In-place weight updates for a running engine (RLHF loops: the trainer pushes new policy weights between
generation phases, the engine keeps its KV pool, graphs and allocator state).

A *weight transfer engine* lives in every worker.  ``init_transfer_engine(info)`` sets up the transport once;
``receive(update_info)`` yields ``(checkpoint name, tensor)`` pairs, which the worker feeds through the same
name mapping and shard slicing as checkpoint loading (``loader.weights.load_weights_from``), followed by the
layers' post-load processing (fp8 re-quantisation, fused-weight repacking).  The engine core then drops the
prefix cache, whose blocks were computed with the old weights.

Backends:

* ``checkpoint`` — the update names a directory of safetensors files every worker can read.
* ``store``      — the trainer and the workers form a stateless group over a TCP store (no
  ``torch.distributed`` world in common); tensors travel as store values.  For CPU runs and small models.
* ``nccl``       — same rendezvous, tensors are broadcast from the trainer's GPU (rank 0) over an NCCL
  communicator created outside the engine's own process groups; the update message carries names, dtypes
  and shapes so that receivers allocate matching buffers.  ``packed=True`` coalesces tensors into
  buffers of ``packed_buffer_bytes`` per broadcast.

The trainer side uses ``TrainerSender`` with the same backend name.

Parity: ``aphrodite/distributed/weight_transfer/base.py:172`` (``WeightTransferEngine``: init / receive),
``nccl_engine.py`` (trainer at rank 0, broadcast per tensor or packed), ``factory.py`` (registry by backend
name), ``entrypoints/serve/rlhf`` routes (``/init_weight_transfer_engine``, ``/update_weights``).
"""
from __future__ import annotations

from typing import Any, Iterator

import torch

from sonar_b200.logger import init_logger

logger = init_logger(__name__)

_DTYPES = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16,
           "float8_e4m3fn": torch.float8_e4m3fn, "int32": torch.int32, "int64": torch.int64, "uint8": torch.uint8}
_BACKENDS: dict[str, type] = {}


def register_backend(name: str):
    def deco(cls):
        _BACKENDS[name] = cls
        cls.backend = name
        return cls
    return deco


def create_engine(backend: str, device: torch.device, rank: int, world_size: int) -> "WeightTransferEngine":
    if backend not in _BACKENDS:
        raise ValueError(f"unknown weight transfer backend {backend!r}; known: {sorted(_BACKENDS)}")
    return _BACKENDS[backend](device, rank, world_size)


class WeightTransferEngine:
    """Worker half.  ``rank`` / ``world_size``: this worker's place among the engine's workers."""
    backend = "?"

    def __init__(self, device: torch.device, rank: int, world_size: int) -> None:
        self.device, self.rank, self.world_size = device, rank, world_size

    def init_transfer_engine(self, info: dict[str, Any]) -> None:
        pass

    def receive(self, info: dict[str, Any]) -> Iterator[tuple[str, torch.Tensor]]:
        raise NotImplementedError

    def shutdown(self) -> None:
        pass


@register_backend("checkpoint")
class CheckpointTransfer(WeightTransferEngine):
    def receive(self, info):
        from sonar_b200.loader.weights import _iter_checkpoint
        yield from _iter_checkpoint(info["path"])


class _GroupTransfer(WeightTransferEngine):
    """Rendezvous shared by the store and NCCL backends: trainer = rank 0, engine worker r = rank 1 + r
    (+ ``rank_offset`` when several engines listen to one trainer)."""

    def init_transfer_engine(self, info):
        from sonar_b200.distributed.stateless import StatelessProcessGroup
        offset = int(info.get("rank_offset", 1))
        self.group = StatelessProcessGroup.create(info["master_address"], int(info["master_port"]),
                                                  offset + self.rank, int(info["world_size"]),
                                                  timeout_s=float(info.get("timeout_s", 300.0)))

    @staticmethod
    def _meta(info) -> list[tuple[str, torch.dtype, tuple[int, ...]]]:
        return [(n, _DTYPES[d], tuple(s)) for n, d, s in zip(info["names"], info["dtype_names"], info["shapes"])]


@register_backend("store")
class StoreTransfer(_GroupTransfer):
    def receive(self, info):
        for name, dtype, shape in self._meta(info):
            raw = self.group.broadcast_obj(None, src=0)
            t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype).reshape(shape)
            yield name, t


@register_backend("nccl")
class NcclTransfer(_GroupTransfer):
    def init_transfer_engine(self, info):
        from sonar_b200.distributed.pynccl import PyNcclCommunicator
        super().init_transfer_engine(info)
        self.comm = PyNcclCommunicator(self.group, self.device)

    def receive(self, info):
        meta = self._meta(info)
        if not info.get("packed", False):
            for name, dtype, shape in meta:
                t = torch.empty(shape, dtype=dtype, device=self.device)
                self.comm.broadcast(t, src=0)
                yield name, t
            return
        for chunk in pack_plan(meta, int(info.get("packed_buffer_bytes", 1 << 30))):
            buf = torch.empty(sum(_nbytes_aligned(d, s) for _, d, s in chunk), dtype=torch.uint8, device=self.device)
            self.comm.broadcast(buf, src=0)
            torch.cuda.current_stream().synchronize()
            yield from unpack(buf, chunk)

    def shutdown(self):
        comm = getattr(self, "comm", None)
        if comm is not None:
            comm.destroy()
            self.comm = None


# ---- packing: several tensors per broadcast, each at a 16-byte aligned offset ------------------------------
def _nbytes_aligned(dtype: torch.dtype, shape) -> int:
    n = torch.empty((), dtype=dtype).element_size()
    for s in shape:
        n *= s
    return (n + 15) // 16 * 16


def pack_plan(meta, limit: int) -> list[list[tuple[str, torch.dtype, tuple[int, ...]]]]:
    """Split the tensor list into consecutive groups of at most ``limit`` bytes (a tensor larger than the
    limit gets a group of its own)."""
    groups, cur, size = [], [], 0
    for item in meta:
        n = _nbytes_aligned(item[1], item[2])
        if cur and size + n > limit:
            groups.append(cur)
            cur, size = [], 0
        cur.append(item)
        size += n
    if cur:
        groups.append(cur)
    return groups


def pack(tensors: dict[str, torch.Tensor], chunk, device) -> torch.Tensor:
    buf = torch.zeros(sum(_nbytes_aligned(d, s) for _, d, s in chunk), dtype=torch.uint8, device=device)
    off = 0
    for name, dtype, shape in chunk:
        t = tensors[name].to(device=device, dtype=dtype).contiguous().view(-1).view(torch.uint8)
        buf[off:off + t.numel()].copy_(t)
        off += _nbytes_aligned(dtype, shape)
    return buf


def unpack(buf: torch.Tensor, chunk) -> Iterator[tuple[str, torch.Tensor]]:
    off = 0
    for name, dtype, shape in chunk:
        n = torch.empty((), dtype=dtype).element_size()
        for s in shape:
            n *= s
        yield name, buf[off:off + n].view(dtype).reshape(shape)
        off += _nbytes_aligned(dtype, shape)


# ---- trainer side ---------------------------------------------------------------------------------------
class TrainerSender:
    """What the training process runs: joins the rendezvous as rank 0 and pushes named tensors.

        sender = TrainerSender("nccl", "10.0.0.1", 29600, world_size=1 + tp, device="cuda:0")
        # meanwhile: POST /init_weight_transfer_engine {"backend": "nccl", "init_info": sender.init_info()}
        sender.connect()
        info = sender.update_info(state_dict)       # POST /update_weights {"update_info": info} …
        sender.send(state_dict)                     # … while this runs
    """

    def __init__(self, backend: str, master_address: str, master_port: int, world_size: int, device="cpu",
                 packed: bool = False, packed_buffer_bytes: int = 1 << 30) -> None:
        assert backend in ("store", "nccl")
        self.backend, self.addr, self.port, self.world = backend, master_address, master_port, world_size
        self.device = torch.device(device)
        self.packed, self.limit = packed, packed_buffer_bytes
        self.group = self.comm = None

    def init_info(self, rank_offset: int = 1) -> dict[str, Any]:
        return {"master_address": self.addr, "master_port": self.port, "world_size": self.world,
                "rank_offset": rank_offset}

    def connect(self) -> None:
        from sonar_b200.distributed.stateless import StatelessProcessGroup
        self.group = StatelessProcessGroup.create(self.addr, self.port, 0, self.world)
        if self.backend == "nccl":
            from sonar_b200.distributed.pynccl import PyNcclCommunicator
            self.comm = PyNcclCommunicator(self.group, self.device)

    def update_info(self, tensors: dict[str, torch.Tensor]) -> dict[str, Any]:
        return {"names": list(tensors), "dtype_names": [str(t.dtype).replace("torch.", "") for t in tensors.values()],
                "shapes": [list(t.shape) for t in tensors.values()], "packed": self.packed,
                "packed_buffer_bytes": self.limit}

    def send(self, tensors: dict[str, torch.Tensor]) -> None:
        if self.backend == "store":
            for t in tensors.values():
                raw = t.detach().cpu().contiguous().view(-1).view(torch.uint8).numpy().tobytes()
                self.group.broadcast_obj(raw, src=0)
            return
        if not self.packed:
            for t in tensors.values():
                self.comm.broadcast(t.detach().to(self.device).contiguous(), src=0)
            return
        meta = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
        for chunk in pack_plan(meta, self.limit):
            self.comm.broadcast(pack(tensors, chunk, self.device), src=0)
            torch.cuda.current_stream().synchronize()
