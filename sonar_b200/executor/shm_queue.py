"""Python face of the native shared-memory ring (``csrc_host/shm_ring.cpp``).

``MessageQueue.create(n_readers)`` makes a ring and returns a picklable handle;
``MessageQueue.attach(handle, reader_index)`` joins it from another process.
Objects are pickled (the ring only connects processes of one engine on one
host).  Parity: ``distributed/device_communicators/shm_broadcast.py:454``.
"""
from __future__ import annotations

import ctypes
import os
import pickle
import uuid
from ctypes import c_char_p, c_int, c_long, c_void_p
from dataclasses import dataclass

_LIB = None


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_host.so")
        if not os.path.exists(path):
            from sonar_b200.ops.build import build_host_extension
            build_host_extension()
        lib = ctypes.CDLL(path)
        lib.ring_create.argtypes, lib.ring_create.restype = [c_char_p, c_int, c_int, c_int], c_void_p
        lib.ring_open.argtypes, lib.ring_open.restype = [c_char_p], c_void_p
        lib.ring_close.argtypes, lib.ring_close.restype = [c_void_p], None
        lib.ring_write.argtypes, lib.ring_write.restype = [c_void_p, c_char_p, c_long, c_long], c_int
        lib.ring_read.argtypes, lib.ring_read.restype = [c_void_p, c_int, c_void_p, c_long, c_long], c_long
        lib.ring_next_len.argtypes, lib.ring_next_len.restype = [c_void_p, c_int, c_long], c_long
        _LIB = lib
    return _LIB


class QueueTimeout(TimeoutError):
    pass


@dataclass
class QueueHandle:
    name: str
    n_readers: int
    slot_bytes: int
    n_slots: int


class MessageQueue:
    def __init__(self, ptr: int, handle: QueueHandle, reader: int | None) -> None:
        self._ptr, self.handle, self.reader = ptr, handle, reader
        self._buf = ctypes.create_string_buffer(handle.slot_bytes * 4)

    @classmethod
    def create(cls, n_readers: int, slot_bytes: int = 1 << 20, n_slots: int = 8) -> "MessageQueue":
        h = QueueHandle(f"/sonar-{os.getpid()}-{uuid.uuid4().hex[:10]}", n_readers, slot_bytes, n_slots)
        ptr = _lib().ring_create(h.name.encode(), n_readers, slot_bytes, n_slots)
        if not ptr:
            raise OSError(f"could not create shared-memory ring {h.name}")
        return cls(ptr, h, None)

    @classmethod
    def attach(cls, handle: QueueHandle, reader: int | None) -> "MessageQueue":
        ptr = _lib().ring_open(handle.name.encode())
        if not ptr:
            raise OSError(f"could not open shared-memory ring {handle.name}")
        return cls(ptr, handle, reader)

    def put(self, obj, timeout_s: float | None = None) -> None:
        data = pickle.dumps(obj, protocol=pickle.HIGHEST_PROTOCOL)
        rc = _lib().ring_write(self._ptr, data, len(data), -1 if timeout_s is None else int(timeout_s * 1000))
        if rc == -2:
            raise QueueTimeout("a reader did not drain the ring in time")
        if rc != 0:
            raise OSError(f"ring_write failed ({rc})")

    def get(self, timeout_s: float | None = None):
        assert self.reader is not None, "this end of the queue is the writer"
        ms = -1 if timeout_s is None else int(timeout_s * 1000)
        while True:
            n = _lib().ring_read(self._ptr, self.reader, self._buf, len(self._buf), ms)
            if n >= 0:
                return pickle.loads(self._buf.raw[:n] if n < len(self._buf) else self._buf.raw)
            if n == -2:
                raise QueueTimeout("no message")
            if n == -4:
                raise OSError("message larger than the receive buffer was dropped; raise slot_bytes")
            raise OSError(f"ring_read failed ({n})")

    def grow_buffer(self, nbytes: int) -> None:
        if nbytes > len(self._buf):
            self._buf = ctypes.create_string_buffer(nbytes)

    def close(self) -> None:
        if self._ptr:
            _lib().ring_close(self._ptr)
            self._ptr = None
