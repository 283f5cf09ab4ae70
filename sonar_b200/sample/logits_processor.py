"""Custom logits processors: user code that edits the logits of a step before sampling.

A processor is a class constructed once per worker with ``(engine_config, device)``.  Each step the runner
hands it the logits rows about to be sampled, ``[n, vocab]`` on the device, together with one ``RowView`` per
row (request id, sampling parameters incl. ``extra_args``, and — when the class sets ``needs_history`` — the
prompt and output token ids).  ``apply`` edits the tensor in place or returns a replacement.  Processors run
after grammar masks and before the built-in chain (penalties, temperature, top-k/p …), in the order given.
``is_active(params)`` lets a processor skip requests that did not ask for it (typically via
``SamplingParams.extra_args``); a step none of whose rows is active does not call ``apply``.

Processors are named by ``"package.module:Class"`` / ``"package.module.Class"`` strings, passed as classes,
or installed under the entry-point group ``sonar.logits_processors``.  While any is configured the engine
steps in lock-step (no run-ahead), so ``output_token_ids`` is always complete.

Parity: ``aphrodite/v1/sample/logits_processor/interface.py`` (``LogitsProcessor``: construct with config and
device, per-step ``apply(logits)``; ``--logits-processors`` fully-qualified names and entry points).
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any

import torch

from sonar_b200.logger import init_logger
from sonar_b200.sampling_params import SamplingParams

logger = init_logger(__name__)
ENTRY_POINT_GROUP = "sonar.logits_processors"


@dataclass
class RowView:
    req_id: str
    params: SamplingParams
    prompt_token_ids: list[int] = field(default_factory=list)
    output_token_ids: list[int] = field(default_factory=list)


class LogitsProcessor:
    needs_history = False

    def __init__(self, engine_config, device: torch.device) -> None:
        self.engine_config, self.device = engine_config, device

    def is_active(self, params: SamplingParams) -> bool:
        return True

    def apply(self, logits: torch.Tensor, rows: list[RowView]) -> torch.Tensor | None:
        """``rows[i]`` describes ``logits[i]``; rows of inactive requests are not passed (the tensor then is a
        gathered copy that is scattered back afterwards)."""
        raise NotImplementedError


def _resolve(spec: Any) -> type:
    if isinstance(spec, type):
        return spec
    if not isinstance(spec, str):
        raise TypeError(f"logits processor must be a class or a qualified name, got {spec!r}")
    mod, sep, name = spec.partition(":")
    if not sep:
        mod, _, name = spec.rpartition(".")
    cls = getattr(importlib.import_module(mod), name)
    if not (isinstance(cls, type) and issubclass(cls, LogitsProcessor)):
        raise TypeError(f"{spec} is not a LogitsProcessor subclass")
    return cls


def any_configured(engine_config) -> bool:
    """True when the engine will run custom processors (configured ones or installed entry points)."""
    if engine_config.logits_processors:
        return True
    try:
        from importlib.metadata import entry_points
        return any(True for _ in entry_points(group=ENTRY_POINT_GROUP))
    except Exception:  # noqa: BLE001
        return False


def load_logits_processors(specs: list | None, engine_config, device: torch.device) -> list[LogitsProcessor]:
    classes = [_resolve(s) for s in (specs or [])]
    try:
        from importlib.metadata import entry_points
        for ep in entry_points(group=ENTRY_POINT_GROUP):
            cls = ep.load()
            if cls not in classes:
                classes.append(cls)
    except Exception as e:  # noqa: BLE001 - a broken third-party entry point must not stop the engine
        logger.warning("logits-processor entry points not loaded: %s", e)
    return [cls(engine_config, device) for cls in classes]


def run_logits_processors(procs: list[LogitsProcessor], logits: torch.Tensor, rows: list[RowView]) -> torch.Tensor:
    for p in procs:
        active = [i for i, r in enumerate(rows) if p.is_active(r.params)]
        if not active:
            continue
        if len(active) == len(rows):
            out = p.apply(logits, rows)
            logits = out if out is not None else logits
            continue
        idx = torch.tensor(active, device=logits.device)
        sub = logits.index_select(0, idx)
        out = p.apply(sub, [rows[i] for i in active])
        logits.index_copy_(0, idx, out if out is not None else sub)
    return logits
