"""msgpack codec for the frontend ⇄ engine-core wire.

Registered dataclasses travel as ``{"__t": tag, ...fields}`` maps, enums as
ints, sets as tagged lists, exceptions as their message, torch tensors as raw
bytes with dtype and shape.  Nothing is pickled, so a frame can only rebuild
the known wire types.  Parity: ``aphrodite/v1/serial_utils.py`` (581).
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any

import msgpack
import numpy as np
import torch

from sonar_b200 import request as _rq
from sonar_b200 import sampling_params as _sp
from sonar_b200.core import kv_cache_manager as _kv

_TYPES: dict[str, type] = {}
_ENUMS: dict[str, type] = {}

for _cls in (_rq.EngineCoreRequest, _rq.EngineCoreOutput, _rq.EngineCoreOutputs, _rq.SchedulerStats,
             _sp.SamplingParams, _sp.PoolingParams, _sp.StructuredOutputsParams, _kv.KVCacheSpec,
             _kv.KVCacheConfig):
    _TYPES[_cls.__name__] = _cls
for _cls in (_rq.FinishReason, _sp.RequestOutputKind):
    _ENUMS[_cls.__name__] = _cls


def register_wire_type(cls: type) -> None:
    _TYPES[cls.__name__] = cls


def _default(obj: Any) -> Any:
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        d = {"__t": type(obj).__name__}
        for f in dataclasses.fields(obj):
            d[f.name] = getattr(obj, f.name)
        return d
    if isinstance(obj, enum.Enum):
        return {"__e": type(obj).__name__, "v": int(obj.value)}
    if isinstance(obj, (set, frozenset)):
        return {"__s": list(obj)}
    if isinstance(obj, tuple):
        return list(obj)
    if isinstance(obj, torch.Tensor):
        t = obj.detach().cpu().contiguous()
        return {"__T": str(t.dtype).replace("torch.", ""), "s": list(t.shape),
                "b": t.view(torch.uint8).numpy().tobytes() if t.numel() else b""}
    if isinstance(obj, np.ndarray):
        return {"__N": str(obj.dtype), "s": list(obj.shape), "b": np.ascontiguousarray(obj).tobytes()}
    if isinstance(obj, (np.integer,)):
        return int(obj)
    if isinstance(obj, (np.floating,)):
        return float(obj)
    if isinstance(obj, Exception):
        return {"__x": f"{type(obj).__name__}: {obj}"}
    raise TypeError(f"cannot serialise {type(obj)!r}")


def _hook(d: dict) -> Any:
    if "__t" in d:
        cls = _TYPES.get(d.pop("__t"))
        if cls is None:
            raise ValueError("unknown wire type")
        obj = cls.__new__(cls)
        for k, v in d.items():
            if k == "_all_stop_token_ids" and isinstance(v, list):
                v = set(v)
            object.__setattr__(obj, k, v)
        return obj
    if "__e" in d:
        return _ENUMS[d["__e"]](d["v"])
    if "__s" in d:
        return set(d["__s"])
    if "__T" in d:
        dt = getattr(torch, d["__T"])
        if not d["b"]:
            return torch.empty(d["s"], dtype=dt)
        return torch.frombuffer(bytearray(d["b"]), dtype=torch.uint8).view(dt).reshape(d["s"])
    if "__N" in d:
        return np.frombuffer(d["b"], dtype=d["__N"]).reshape(d["s"]).copy()
    if "__x" in d:
        return RuntimeError(d["__x"])
    return d


def encode(obj: Any) -> bytes:
    return msgpack.packb(obj, default=_default, use_bin_type=True, strict_types=False)


def decode(buf: bytes) -> Any:
    return msgpack.unpackb(buf, object_hook=_hook, raw=False, strict_map_key=False)
