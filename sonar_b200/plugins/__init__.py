"""Plugin loading through Python entry points.

Groups:
  * ``sonar_b200.general_plugins`` — callables run once in every process (engine core, workers, API
    server) before the model is built; the place to register model architectures
    (``sonar_b200.models.registry.register_model``), tool / reasoning parsers, or samplers.
  * ``sonar_b200.endpoint_plugins`` — callables ``f(app, state)`` that add routes to the HTTP server.
  * ``sonar_b200.lora_resolvers`` — callables ``f(name) -> path | None`` that find an adapter by name
    when a request names one that is not loaded.

``SONAR_PLUGINS`` (comma-separated entry-point names) restricts which plugins load; unset loads all.
The reference's group names (``aphrodite.general_plugins`` …) are searched too, so its plugins load.

Parity: ``aphrodite/plugins/__init__.py`` (``load_general_plugins``, ``load_plugins_by_group``).
"""
from __future__ import annotations

import os
from importlib.metadata import entry_points
from typing import Any, Callable

from sonar_b200.logger import init_logger

logger = init_logger(__name__)

GENERAL = "general_plugins"
ENDPOINT = "endpoint_plugins"
LORA_RESOLVER = "lora_resolvers"
_PREFIXES = ("sonar_b200", "aphrodite")
_loaded_general = False
_extra: dict[str, dict[str, Callable[..., Any]]] = {}


def register_plugin(group: str, name: str, fn: Callable[..., Any]) -> None:
    """In-process registration (tests, embedding applications) — same effect as an entry point."""
    _extra.setdefault(group, {})[name] = fn


def load_plugins_by_group(group: str) -> dict[str, Callable[..., Any]]:
    allowed = os.environ.get("SONAR_PLUGINS")
    allow = None if allowed is None else {a.strip() for a in allowed.split(",") if a.strip()}
    found: dict[str, Callable[..., Any]] = {}
    for prefix in _PREFIXES:
        try:
            eps = entry_points(group=f"{prefix}.{group}")
        except Exception:  # noqa: BLE001
            eps = []
        for ep in eps:
            if allow is not None and ep.name not in allow:
                continue
            try:
                found[ep.name] = ep.load()
            except Exception:  # noqa: BLE001
                logger.exception("plugin %s (%s) failed to load", ep.name, group)
    for name, fn in _extra.get(group, {}).items():
        if allow is None or name in allow:
            found[name] = fn
    return found


def load_general_plugins(force: bool = False) -> list[str]:
    """Run every general plugin once per process.  Returns the names that ran."""
    global _loaded_general
    if _loaded_general and not force:
        return []
    _loaded_general = True
    ran = []
    for name, fn in load_plugins_by_group(GENERAL).items():
        try:
            fn()
            ran.append(name)
        except Exception:  # noqa: BLE001
            logger.exception("general plugin %s raised", name)
    if ran:
        logger.info("general plugins: %s", ", ".join(ran))
    return ran


def resolve_lora(name: str) -> str | None:
    for fn in load_plugins_by_group(LORA_RESOLVER).values():
        path = fn(name)
        if path:
            return path
    return None
