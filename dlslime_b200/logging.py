"""Logging namespace ``slime.*`` with one stderr handler, as in the reference (``dlslime/logging.py:20-59``)."""

from __future__ import annotations

import logging
import sys

_ROOT = "slime"
_installed = False


def _install() -> None:
    global _installed
    if _installed:
        return
    root = logging.getLogger(_ROOT)
    if not root.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter("%(asctime)s %(levelname)s %(name)s: %(message)s"))
        root.addHandler(h)
        root.setLevel(logging.WARNING)
        root.propagate = False
    _installed = True


def get_logger(name: str = "") -> logging.Logger:
    _install()
    return logging.getLogger(f"{_ROOT}.{name}" if name else _ROOT)


def set_log_level(level: int | str) -> None:
    _install()
    logging.getLogger(_ROOT).setLevel(level if isinstance(level, int) else getattr(logging, str(level).upper()))
