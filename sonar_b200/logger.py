"""Process-wide logging setup.

One ``logging`` hierarchy rooted at ``sonar_b200``; the level comes from the
``SONAR_LOG_LEVEL`` environment variable.  Parity: the reference configures its
own hierarchy in ``aphrodite/logger.py``.
"""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(levelname)s %(asctime)s [%(name)s:%(lineno)d] %(message)s"
_configured = False


def _configure() -> None:
    global _configured
    if _configured:
        return
    root = logging.getLogger("sonar_b200")
    level = os.environ.get("SONAR_LOG_LEVEL", "INFO").upper()
    root.setLevel(getattr(logging, level, logging.INFO))
    if not root.handlers:
        handler = logging.StreamHandler(sys.stderr)
        handler.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d %H:%M:%S"))
        root.addHandler(handler)
    root.propagate = False
    _configured = True


def init_logger(name: str) -> logging.Logger:
    _configure()
    if not name.startswith("sonar_b200"):
        name = "sonar_b200." + name
    return logging.getLogger(name)
