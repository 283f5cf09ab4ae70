"""Multi-adapter LoRA: adapters live in fixed slots of stacked per-layer tensors, every token row of a
step names its slot, and each targeted linear layer adds ``B[slot] · (A[slot] · x)`` with two
batched-gather kernels (``ops.lora_shrink`` / ``ops.lora_expand``).

* ``LoRARequest`` — what a user passes to ``LLM.generate`` / the server (name, id, path).
* ``load_adapter`` — reads a PEFT checkpoint (``adapter_config.json`` + ``adapter_model.safetensors``).
* ``LoRALayer`` — the per-linear-layer slot tensors; ``apply`` is called from ``LinearBase.apply``.
* ``LoRAManager`` — per worker: finds the target layers of a model, loads adapters into slots
  (least-recently-used eviction), and publishes the step's token → slot map.

Tensor-parallel layout: column-parallel targets shard ``B`` along the output rows exactly like the base
weight and replicate ``A``; row-parallel targets shard ``A`` along the input columns and add their
partial ``B · v`` to the partial output, so the layer's existing all-reduce completes the sum.

Parity: ``aphrodite/lora/model_manager.py`` (slots, LRU), ``lora/layers/*`` (per-layer wrappers),
``lora/punica_wrapper`` (token → adapter index mapping), ``csrc/punica`` (bgmv kernels).
"""
from __future__ import annotations

import json
import os
from collections import OrderedDict
from dataclasses import dataclass

import torch

from sonar_b200 import ops
from sonar_b200.config import LoRAConfig
from sonar_b200.logger import init_logger

logger = init_logger(__name__)


@dataclass
class LoRARequest:
    lora_name: str
    lora_int_id: int = 0
    lora_path: str = ""


# HF module name → (packed layer attribute, sub-matrix index)
PACKED = {
    "q_proj": ("qkv_proj", 0), "k_proj": ("qkv_proj", 1), "v_proj": ("qkv_proj", 2),
    "gate_proj": ("gate_up_proj", 0), "up_proj": ("gate_up_proj", 1),
    "o_proj": ("o_proj", 0), "down_proj": ("down_proj", 0),
}


def load_adapter(path: str) -> tuple[dict[str, tuple[torch.Tensor, torch.Tensor]], float, int]:
    """→ ({module path like ``model.layers.0.self_attn.q_proj``: (A [r, K], B [N, r])}, α/r, r)."""
    from sonar_b200.loader.weights import read_safetensors
    with open(os.path.join(path, "adapter_config.json")) as f:
        cfg = json.load(f)
    r = int(cfg["r"])
    scaling = float(cfg.get("lora_alpha", r)) / r
    if cfg.get("use_rslora"):
        scaling = float(cfg.get("lora_alpha", r)) / (r ** 0.5)
    tensors = dict(read_safetensors(os.path.join(path, "adapter_model.safetensors")))
    pairs: dict[str, dict[str, torch.Tensor]] = {}
    for name, t in tensors.items():
        key = name
        for pre in ("base_model.model.",):
            if key.startswith(pre):
                key = key[len(pre):]
        if ".lora_A" in key:
            mod, which = key.split(".lora_A")[0], "A"
        elif ".lora_B" in key:
            mod, which = key.split(".lora_B")[0], "B"
        else:
            continue
        pairs.setdefault(mod, {})[which] = t
    out = {}
    for mod, ab in pairs.items():
        if "A" not in ab or "B" not in ab:
            raise ValueError(f"adapter {path}: module {mod} lacks lora_A or lora_B")
        out[mod] = (ab["A"], ab["B"])
    return out, scaling, r


class LoRALayer:
    """Slot tensors of one (possibly packed) linear layer."""

    def __init__(self, layer, max_loras: int, max_rank: int, dtype: torch.dtype, device) -> None:
        from sonar_b200.layers.linear import ColumnParallelLinear, RowParallelLinear
        self.layer = layer
        self.rank = max_rank
        self.row_parallel = isinstance(layer, RowParallelLinear)
        if isinstance(layer, ColumnParallelLinear):
            self.sub_sizes = list(layer.local_sizes)
        else:
            self.sub_sizes = [layer.weight.shape[0]]
        k_local = layer.weight.shape[1]
        n_sub = len(self.sub_sizes)
        # one A per sub-matrix (q, k and v adapters have different A's)
        self.A = torch.zeros(n_sub, max_loras, max_rank, k_local, dtype=dtype, device=device)
        self.B = [torch.zeros(max_loras, n, max_rank, dtype=dtype, device=device) for n in self.sub_sizes]
        self.used = [[False] * n_sub for _ in range(max_loras)]
        self.manager: "LoRAManager | None" = None

    def set(self, slot: int, sub: int, a: torch.Tensor, b: torch.Tensor, scaling: float) -> None:
        """``a`` [r, K_full], ``b`` [N_full, r]: shard like the base weight, pad the rank, fold the scale in."""
        layer = self.layer
        tp, rank = getattr(layer, "tp_size", 1), getattr(layer, "tp_rank", 0)
        r = a.shape[0]
        if r > self.rank:
            raise ValueError(f"adapter rank {r} exceeds max_lora_rank {self.rank}")
        if self.row_parallel:
            k = layer.k_local
            a = a[:, rank * k:(rank + 1) * k]
        elif tp > 1:
            n = self.sub_sizes[sub]
            shard = rank
            if hasattr(layer, "kv_replicas") and sub > 0:
                shard = rank // layer.kv_replicas
            b = b[shard * n:(shard + 1) * n]
        self.A[sub, slot].zero_()
        self.B[sub][slot].zero_()
        self.A[sub, slot, :r].copy_(a)
        self.B[sub][slot, :, :r].copy_(b.float() * scaling)
        self.used[slot][sub] = True

    def clear(self, slot: int) -> None:
        for sub in range(len(self.sub_sizes)):
            if self.used[slot][sub]:
                self.A[sub, slot].zero_()
                self.B[sub][slot].zero_()
                self.used[slot][sub] = False

    def apply(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        m = self.manager
        if m is None or not m.any_active:
            return y
        slots = m.token_slots[: x.shape[0]]
        off = 0
        for sub, n in enumerate(self.sub_sizes):
            if any(self.used[s][sub] for s in m.active_slots):
                v = ops.lora_shrink(x, self.A[sub], slots)
                ops.lora_expand(v, self.B[sub], slots, y, off)
            off += n
        return y


class LoRAManager:
    def __init__(self, model: torch.nn.Module, cfg: LoRAConfig, dtype: torch.dtype, device, max_tokens: int) -> None:
        from sonar_b200.layers.linear import LinearBase
        self.cfg = cfg
        self.device = device
        self.layers: dict[str, LoRALayer] = {}
        targets = {v[0] for v in PACKED.values()}
        for name, mod in model.named_modules():
            if isinstance(mod, LinearBase) and name.rsplit(".", 1)[-1] in targets:
                ll = LoRALayer(mod, cfg.max_loras, cfg.max_lora_rank, dtype, device)
                ll.manager = self
                mod.lora = ll
                self.layers[name] = ll
        self.slot_of: OrderedDict[str, int] = OrderedDict()       # adapter name → slot, LRU order
        self.paths: dict[str, str] = {}
        self.token_slots = torch.full((max_tokens,), -1, dtype=torch.int32, device=device)
        self.any_active = False
        self.active_slots: list[int] = []
        logger.info("LoRA: %d target layers, %d slots, max rank %d", len(self.layers), cfg.max_loras,
                    cfg.max_lora_rank)

    # registry -------------------------------------------------------------
    def register(self, name: str, path: str) -> None:
        if not os.path.exists(os.path.join(path, "adapter_config.json")):
            raise ValueError(f"LoRA adapter {name!r}: no adapter_config.json under {path}")
        self.paths[name] = path
        if name in self.slot_of:               # reloaded from a new path
            self._evict(name)

    def unregister(self, name: str) -> bool:
        if name in self.slot_of:
            self._evict(name)
        return self.paths.pop(name, None) is not None

    def list_adapters(self) -> list[str]:
        return sorted(self.paths)

    def _evict(self, name: str) -> int:
        slot = self.slot_of.pop(name)
        for ll in self.layers.values():
            ll.clear(slot)
        return slot

    def _ensure_loaded(self, name: str, pinned: set[str]) -> int:
        if name in self.slot_of:
            self.slot_of.move_to_end(name)
            return self.slot_of[name]
        if name not in self.paths:
            raise ValueError(f"unknown LoRA adapter {name!r}")
        if len(self.slot_of) >= self.cfg.max_loras:
            victim = next((n for n in self.slot_of if n not in pinned), None)
            if victim is None:
                raise RuntimeError(f"a step needs more than max_loras={self.cfg.max_loras} adapters")
            slot = self._evict(victim)
        else:
            slot = next(i for i in range(self.cfg.max_loras) if i not in self.slot_of.values())
        tensors, scaling, _ = load_adapter(self.paths[name])
        n_set = 0
        for mod, (a, b) in tensors.items():
            parent, leaf = mod.rsplit(".", 1)
            if leaf not in PACKED:
                continue
            attr, sub = PACKED[leaf]
            ll = self.layers.get(f"{parent}.{attr}")
            if ll is None:
                continue              # a layer of another pipeline stage
            ll.set(slot, sub, a.to(self.device), b.to(self.device), scaling)
            n_set += 1
        self.slot_of[name] = slot
        logger.info("LoRA adapter %s → slot %d (%d modules)", name, slot, n_set)
        return slot

    # per step -------------------------------------------------------------
    def set_step(self, names_per_token_run: list[tuple[str | None, int]]) -> None:
        """``[(adapter name or None, number of consecutive token rows), …]`` in batch order."""
        wanted = {n for n, _ in names_per_token_run if n}
        self.any_active = bool(wanted)
        if not wanted:
            self.active_slots = []
            return
        slots = {n: self._ensure_loaded(n, wanted) for n in wanted}
        self.active_slots = sorted(slots.values())
        host = torch.empty(sum(c for _, c in names_per_token_run), dtype=torch.int32)
        pos = 0
        for n, c in names_per_token_run:
            host[pos:pos + c] = slots[n] if n else -1
            pos += c
        self.token_slots[:pos].copy_(host, non_blocking=False)
