"""NCCL through ctypes: a communicator that does not depend on ``torch.distributed``'s process-group
machinery (so it can be created from a stateless group, e.g. while resizing an expert-parallel job)
and that launches on a stream of the caller's choice (so collectives can be captured in CUDA graphs).

The library is the NCCL that ships with PyTorch (``nvidia/nccl/lib/libnccl.so.2``), found next to the
torch package; ``SONAR_NCCL_SO_PATH`` overrides it.

Parity: ``aphrodite/distributed/device_communicators/pynccl_wrapper.py:165-345`` (function table) and
``pynccl.py:60-316`` (communicator, v-collectives via grouped send/recv).
"""
from __future__ import annotations

import ctypes
import glob
import os

import torch

ncclResult_t = ctypes.c_int
ncclComm_t = ctypes.c_void_p
cudaStream_t = ctypes.c_void_p
buffer_t = ctypes.c_void_p


class ncclUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


_DTYPES = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
           torch.float64: 8, torch.bfloat16: 9, torch.float8_e4m3fn: 1}
_OPS = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}


def find_nccl_library() -> str:
    env = os.environ.get("SONAR_NCCL_SO_PATH")
    if env:
        return env
    site = os.path.dirname(os.path.dirname(torch.__file__))
    hits = sorted(glob.glob(os.path.join(site, "nvidia", "nccl", "lib", "libnccl.so*")))
    return hits[0] if hits else "libnccl.so.2"


class NCCLLibrary:
    _FUNCS = [
        ("ncclGetErrorString", ctypes.c_char_p, [ncclResult_t]),
        ("ncclGetVersion", ncclResult_t, [ctypes.POINTER(ctypes.c_int)]),
        ("ncclGetUniqueId", ncclResult_t, [ctypes.POINTER(ncclUniqueId)]),
        ("ncclCommInitRank", ncclResult_t, [ctypes.POINTER(ncclComm_t), ctypes.c_int, ncclUniqueId, ctypes.c_int]),
        ("ncclAllReduce", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                        cudaStream_t]),
        ("ncclReduce", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                     ncclComm_t, cudaStream_t]),
        ("ncclAllGather", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ncclComm_t, cudaStream_t]),
        ("ncclReduceScatter", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int,
                                            ncclComm_t, cudaStream_t]),
        ("ncclBroadcast", ncclResult_t, [buffer_t, buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t,
                                        cudaStream_t]),
        ("ncclSend", ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        ("ncclRecv", ncclResult_t, [buffer_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, ncclComm_t, cudaStream_t]),
        ("ncclGroupStart", ncclResult_t, []),
        ("ncclGroupEnd", ncclResult_t, []),
        ("ncclCommDestroy", ncclResult_t, [ncclComm_t]),
    ]

    def __init__(self, path: str | None = None) -> None:
        self.path = path or find_nccl_library()
        self.lib = ctypes.CDLL(self.path)
        for name, res, args in self._FUNCS:
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args

    def check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError(f"NCCL error {rc}: {self.lib.ncclGetErrorString(rc).decode()}")

    def version(self) -> str:
        v = ctypes.c_int()
        self.check(self.lib.ncclGetVersion(ctypes.byref(v)))
        n = v.value
        return f"{n // 10000}.{n // 100 % 100}.{n % 100}"

    def unique_id(self) -> ncclUniqueId:
        uid = ncclUniqueId()
        self.check(self.lib.ncclGetUniqueId(ctypes.byref(uid)))
        return uid


class PyNcclCommunicator:
    """One NCCL communicator over the ranks of ``group`` (a ``StatelessProcessGroup`` or anything with
    ``rank``, ``world_size`` and ``broadcast_obj``)."""

    def __init__(self, group, device: torch.device | int, library: NCCLLibrary | None = None) -> None:
        self.nccl = library or NCCLLibrary()
        self.rank, self.world_size = group.rank, group.world_size
        self.device = torch.device("cuda", device) if isinstance(device, int) else device
        uid = self.nccl.unique_id() if self.rank == 0 else None
        raw = group.broadcast_obj(bytes(uid.internal) if uid is not None else None, 0)
        uid = ncclUniqueId()
        ctypes.memmove(uid.internal, raw, 128)
        self.comm = ncclComm_t()
        with torch.cuda.device(self.device):
            self.nccl.check(self.nccl.lib.ncclCommInitRank(ctypes.byref(self.comm), self.world_size, uid, self.rank))
            warm = torch.zeros(1, device=self.device)
            self.all_reduce(warm)
            torch.cuda.current_stream().synchronize()

    def _stream(self, stream) -> cudaStream_t:
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        return cudaStream_t(s.cuda_stream)

    def all_reduce(self, t: torch.Tensor, op: str = "sum", out: torch.Tensor | None = None, stream=None):
        out = t if out is None else out
        self.nccl.check(self.nccl.lib.ncclAllReduce(t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype], _OPS[op],
                                                    self.comm, self._stream(stream)))
        return out

    def all_gather(self, out: torch.Tensor, t: torch.Tensor, stream=None):
        self.nccl.check(self.nccl.lib.ncclAllGather(t.data_ptr(), out.data_ptr(), t.numel(), _DTYPES[t.dtype],
                                                    self.comm, self._stream(stream)))
        return out

    def reduce_scatter(self, out: torch.Tensor, t: torch.Tensor, op: str = "sum", stream=None):
        self.nccl.check(self.nccl.lib.ncclReduceScatter(t.data_ptr(), out.data_ptr(), out.numel(), _DTYPES[t.dtype],
                                                        _OPS[op], self.comm, self._stream(stream)))
        return out

    def all_gatherv(self, out: torch.Tensor, t: torch.Tensor, sizes: list[int], stream=None):
        """Rows per rank differ: rank r contributes ``sizes[r]`` rows (grouped broadcasts)."""
        s = self._stream(stream)
        row = t[0].numel() if t.dim() > 1 else 1
        self.nccl.check(self.nccl.lib.ncclGroupStart())
        off = 0
        for r, n in enumerate(sizes):
            dst = out[off:off + n]
            src = t if r == self.rank else dst
            self.nccl.check(self.nccl.lib.ncclBroadcast(src.data_ptr(), dst.data_ptr(), n * row, _DTYPES[t.dtype], r,
                                                        self.comm, s))
            off += n
        self.nccl.check(self.nccl.lib.ncclGroupEnd())
        return out

    def reduce_scatterv(self, out: torch.Tensor, t: torch.Tensor, sizes: list[int], op: str = "sum", stream=None):
        s = self._stream(stream)
        row = t[0].numel() if t.dim() > 1 else 1
        self.nccl.check(self.nccl.lib.ncclGroupStart())
        off = 0
        for r, n in enumerate(sizes):
            chunk = t[off:off + n]
            self.nccl.check(self.nccl.lib.ncclReduce(chunk.data_ptr(), out.data_ptr(), n * row, _DTYPES[t.dtype],
                                                     _OPS[op], r, self.comm, s))
            off += n
        self.nccl.check(self.nccl.lib.ncclGroupEnd())
        return out

    def send(self, t: torch.Tensor, dst: int, stream=None) -> None:
        self.nccl.check(self.nccl.lib.ncclSend(t.data_ptr(), t.numel(), _DTYPES[t.dtype], dst, self.comm,
                                               self._stream(stream)))

    def recv(self, t: torch.Tensor, src: int, stream=None) -> None:
        self.nccl.check(self.nccl.lib.ncclRecv(t.data_ptr(), t.numel(), _DTYPES[t.dtype], src, self.comm,
                                               self._stream(stream)))

    def broadcast(self, t: torch.Tensor, src: int, stream=None) -> None:
        self.nccl.check(self.nccl.lib.ncclBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), _DTYPES[t.dtype], src,
                                                    self.comm, self._stream(stream)))

    def destroy(self) -> None:
        if self.comm:
            self.nccl.lib.ncclCommDestroy(self.comm)
            self.comm = ncclComm_t()
