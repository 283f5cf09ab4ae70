"""Weight-only int4 checkpoints (AWQ and GPTQ layouts), widened when they are loaded.

Both formats store, per linear layer, ``qweight`` (eight 4-bit values per int32), ``qzeros`` (packed zero
points per group of input channels) and ``scales`` (fp16, per group and output channel); the weight is
``(q - z) · s``.  This build has no int4 GEMM: the loader rebuilds the 16-bit ``weight`` tensor and hands it
to the ordinary bf16/fp16 path.  Such checkpoints load and produce the numbers of their quantised weights;
the memory saving of int4-resident weights is not provided.

Layouts (as written by the AutoAWQ and AutoGPTQ / GPTQModel exporters):

* AWQ ("gemm" version): ``qweight [in, out/8]`` packs along the OUTPUT dimension with the nibble order
  0,2,4,6,1,3,5,7; ``qzeros [in/g, out/8]`` likewise; ``scales [in/g, out]``.
* GPTQ: ``qweight [in/8, out]`` packs along the INPUT dimension in natural order; ``qzeros [in/g, out/8]``
  packs along the output dimension in natural order and, in the classic ``gptq`` checkpoint format, stores
  ``z - 1``; ``scales [in/g, out]``; optional ``g_idx [in]`` maps input channels to groups (act-order).

* compressed-tensors ``pack-quantized`` (llm-compressor W4A16): ``weight_packed [out, in/8]`` packs along the
  INPUT dimension in natural order, values stored offset by 8 when symmetric; ``weight_scale [out, in/g]``;
  optional ``weight_zero_point [out/8, in/g]`` packed along the output dimension; ``weight_shape``.

Parity: ``aphrodite/model_executor/layers/quantization/{awq,gptq}.py``, ``compressed_tensors/`` (tensor layouts and the dequantisation
formula; the reference keeps the weights packed and runs Marlin / exllama kernels).
"""
from __future__ import annotations

from typing import Iterator

import torch

_AWQ_REVERSE = [0, 4, 1, 5, 2, 6, 3, 7]          # position in the int32 → column inside the group of eight
_SHIFTS = torch.arange(0, 32, 4, dtype=torch.int32)


def _unpack_cols(packed: torch.Tensor) -> torch.Tensor:
    """[r, c] int32 → [r, c * 8] nibbles, the eight values of a word side by side (natural order)."""
    x = (packed.to(torch.int32)[:, :, None] >> _SHIFTS[None, None, :]) & 0xF
    return x.reshape(packed.shape[0], -1)


def _unpack_rows(packed: torch.Tensor) -> torch.Tensor:
    """[r, c] int32 → [r * 8, c] nibbles, the eight values of a word below one another."""
    x = (packed.to(torch.int32)[:, None, :] >> _SHIFTS[None, :, None]) & 0xF
    return x.reshape(-1, packed.shape[1])


def dequantize_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor,
                   group_size: int) -> torch.Tensor:
    """→ ``[out, in]`` in the dtype of ``scales``."""
    n_in, n_out = qweight.shape[0], qweight.shape[1] * 8
    q = _unpack_cols(qweight).reshape(n_in, n_out // 8, 8)[:, :, _AWQ_REVERSE].reshape(n_in, n_out)
    z = _unpack_cols(qzeros).reshape(-1, n_out // 8, 8)[:, :, _AWQ_REVERSE].reshape(-1, n_out)
    g = n_in if group_size in (-1, 0) else group_size
    grp = torch.arange(n_in) // g
    w = (q - z[grp]).to(scales.dtype) * scales[grp]
    return w.t().contiguous()


def dequantize_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int,
                    g_idx: torch.Tensor | None = None, zero_offset: int = 1) -> torch.Tensor:
    """→ ``[out, in]``.  ``zero_offset``: 1 for the classic format (zero points stored minus one), 0 for
    ``checkpoint_format: gptq_v2``."""
    q = _unpack_rows(qweight)
    n_in, n_out = q.shape
    z = _unpack_cols(qzeros)[:, :n_out] + zero_offset
    g = n_in if group_size in (-1, 0) else group_size
    grp = g_idx.long() if g_idx is not None and g_idx.numel() == n_in else torch.arange(n_in) // g
    w = (q - z[grp]).to(scales.dtype) * scales[grp]
    return w.t().contiguous()


def dequantize_compressed_tensors(packed: torch.Tensor, scale: torch.Tensor, zero_point: torch.Tensor | None,
                                  group_size: int, shape: tuple[int, int] | None = None) -> torch.Tensor:
    """→ ``[out, in]``.  Symmetric checkpoints (no zero point) store ``q + 8``."""
    q = _unpack_cols(packed)                                   # [out, in]
    n_out, n_in = (int(shape[0]), int(shape[1])) if shape is not None else tuple(q.shape)
    q = q[:n_out, :n_in]
    g = n_in if group_size in (-1, 0, None) else group_size
    grp = torch.arange(n_in) // g
    if zero_point is None:
        z = torch.full((n_out, scale.shape[1]), 8, dtype=torch.int32)
    else:
        z = _unpack_rows(zero_point)[:n_out] if zero_point.dtype == torch.int32 else zero_point.to(torch.int32)
    return ((q - z[:, grp]).to(scale.dtype) * scale[:, grp]).contiguous()


def widen_compressed_tensors(weights: Iterator[tuple[str, torch.Tensor]], qcfg: dict) -> Iterator[tuple[str, torch.Tensor]]:
    """``weight_packed`` / ``weight_scale`` / ``weight_shape`` (/ ``weight_zero_point``) → ``weight``."""
    group, sym = 128, True
    for grp_cfg in (qcfg.get("config_groups") or {}).values():
        w = grp_cfg.get("weights") or {}
        if w.get("num_bits", 4) != 4:
            raise ValueError("compressed-tensors pack-quantized checkpoints are supported for 4-bit weights only")
        group = w.get("group_size") or -1
        sym = bool(w.get("symmetric", True))
    need = {"weight_packed", "weight_scale", "weight_shape"} | (set() if sym else {"weight_zero_point"})
    pending: dict[str, dict[str, torch.Tensor]] = {}
    for name, t in weights:
        prefix, _, leaf = name.rpartition(".")
        if leaf not in ("weight_packed", "weight_scale", "weight_shape", "weight_zero_point", "weight_g_idx"):
            yield name, t
            continue
        parts = pending.setdefault(prefix, {})
        parts[leaf] = t
        if need <= parts.keys():
            yield prefix + ".weight", dequantize_compressed_tensors(
                parts["weight_packed"], parts["weight_scale"], parts.get("weight_zero_point"), group,
                tuple(parts["weight_shape"].tolist()))
            del pending[prefix]
    if pending:
        raise ValueError(f"incomplete pack-quantized tensors for {sorted(pending)[:3]}")


def widen_int4_checkpoint(weights: Iterator[tuple[str, torch.Tensor]], qcfg: dict) -> Iterator[tuple[str, torch.Tensor]]:
    """Wrap a checkpoint iterator: ``qweight`` / ``qzeros`` / ``scales`` (/ ``g_idx``) triples come out as one
    ``weight`` tensor; everything else passes through."""
    method = qcfg.get("quant_method")
    if method == "compressed-tensors":
        yield from widen_compressed_tensors(weights, qcfg)
        return
    bits = int(qcfg.get("bits", qcfg.get("w_bit", 4)))
    if bits != 4:
        raise ValueError(f"{method} checkpoints with {bits}-bit weights are not supported (4-bit only)")
    group = int(qcfg.get("group_size", qcfg.get("q_group_size", 128)))
    zero_offset = 0 if qcfg.get("checkpoint_format") == "gptq_v2" else 1
    need = {"qweight", "qzeros", "scales"}
    pending: dict[str, dict[str, torch.Tensor]] = {}
    for name, t in weights:
        prefix, _, leaf = name.rpartition(".")
        if leaf not in ("qweight", "qzeros", "scales", "g_idx"):
            yield name, t
            continue
        parts = pending.setdefault(prefix, {})
        parts[leaf] = t
        # exporters of the GPTQ layout always write g_idx; a layer without one is flushed at the end
        if need <= parts.keys() and (method == "awq" or "g_idx" in parts):
            yield prefix + ".weight", _widen(method, parts, group, zero_offset)
            del pending[prefix]
    for prefix, parts in pending.items():          # GPTQ layers whose g_idx never came
        if need <= parts.keys():
            yield prefix + ".weight", _widen(method, parts, group, zero_offset)
        else:
            raise ValueError(f"incomplete int4 tensors for {prefix}: {sorted(parts)}")


def _widen(method: str, p: dict[str, torch.Tensor], group: int, zero_offset: int) -> torch.Tensor:
    if method == "awq":
        return dequantize_awq(p["qweight"], p["qzeros"], p["scales"], group)
    return dequantize_gptq(p["qweight"], p["qzeros"], p["scales"], group, p.get("g_idx"), zero_offset)


# ---- packers (tests and tools: write checkpoints in these layouts) --------------------------------------------
def pack_awq(q: torch.Tensor) -> torch.Tensor:
    """[r, c] nibbles → [r, c/8] int32 in AWQ order."""
    order = [0, 2, 4, 6, 1, 3, 5, 7]
    g = q.to(torch.int64).reshape(q.shape[0], -1, 8)[:, :, order]
    word = (g << torch.arange(0, 32, 4, dtype=torch.int64)).sum(-1)
    return _to_i32(word)


def pack_cols(q: torch.Tensor) -> torch.Tensor:
    g = q.to(torch.int64).reshape(q.shape[0], -1, 8)
    return _to_i32((g << torch.arange(0, 32, 4, dtype=torch.int64)).sum(-1))


def pack_rows(q: torch.Tensor) -> torch.Tensor:
    g = q.to(torch.int64).reshape(-1, 8, q.shape[1])
    return _to_i32((g << torch.arange(0, 32, 4, dtype=torch.int64)[None, :, None]).sum(1))


def _to_i32(word: torch.Tensor) -> torch.Tensor:
    return torch.where(word >= 2**31, word - 2**32, word).to(torch.int32)
