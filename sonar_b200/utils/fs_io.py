"""Whole-buffer file IO outside the interpreter lock (native ``sonar_fs_*`` in ``_host.so``).

Used by the filesystem KV-offload tier: a tensor's bytes go to / come from one file with a few
threads of positional IO, the write is renamed into place atomically.

Parity: ``csrc/fs_io.cpp`` of the reference (``fs_io_C`` extension).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

_lib = None


def _host():
    global _lib
    if _lib is None:
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "_host.so")
        if not os.path.exists(path):
            from sonar_b200.ops.build import build_host_extension
            build_host_extension()
        lib = ctypes.CDLL(path)
        lib.sonar_fs_write.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int, ctypes.c_int]
        lib.sonar_fs_read.argtypes = [ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
        lib.sonar_fs_size.argtypes = [ctypes.c_char_p]
        lib.sonar_fs_size.restype = ctypes.c_longlong
        _lib = lib
    return _lib


def _buffer(t) -> tuple[int, int]:
    if isinstance(t, torch.Tensor):
        assert t.device.type == "cpu" and t.is_contiguous()
        return t.data_ptr(), t.numel() * t.element_size()
    assert isinstance(t, np.ndarray) and t.flags.c_contiguous
    return t.ctypes.data, t.nbytes


def write_file(path: str, data, threads: int = 4, fsync: bool = False) -> None:
    ptr, n = _buffer(data)
    err = _host().sonar_fs_write(os.fsencode(path), ptr, n, threads, int(fsync))
    if err:
        raise OSError(err, os.strerror(err), path)


def read_file_into(path: str, out, threads: int = 4) -> None:
    ptr, n = _buffer(out)
    err = _host().sonar_fs_read(os.fsencode(path), ptr, n, threads)
    if err:
        raise OSError(err, os.strerror(err), path)


def file_size(path: str) -> int:
    return int(_host().sonar_fs_size(os.fsencode(path)))
