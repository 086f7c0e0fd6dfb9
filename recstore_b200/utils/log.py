"""Logging of the Python half: one format everywhere (``LEVEL [pid file:line] message``), a debug form that prefixes the
rank and colours it (rank 0 red, the others green) so interleaved output of several workers can be told apart, and a
print for rank 0 only.  Role of ``XLOG`` / ``XLOG.cdebug`` / ``print_rank0`` in src/python/pytorch/recstore/utils.py:
24-32, 183-219.  ``RECSTORE_LOG_LEVEL`` (``DEBUG``, ``INFO``, ...) sets the level; nothing is configured until
``get_logger`` is first called, so importing the package does not touch an application's logging set-up."""
from __future__ import annotations

import logging
import os
import sys

_FORMAT = "%(levelname)-2s [%(process)d %(filename)s:%(lineno)d] %(message)s"
_logger = None


def _rank():
    try:
        import torch.distributed as dist
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else None
    except Exception:
        return None


def get_logger() -> logging.Logger:
    global _logger
    if _logger is None:
        lg = logging.getLogger("recstore_b200")
        if not lg.handlers:
            h = logging.StreamHandler(sys.stderr)
            h.setFormatter(logging.Formatter(_FORMAT, datefmt="%m-%d:%H:%M:%S"))
            lg.addHandler(h)
            lg.propagate = False
        lg.setLevel(getattr(logging, os.environ.get("RECSTORE_LOG_LEVEL", "INFO").upper(), logging.INFO))
        _logger = lg
    return _logger


def cdebug(msg, colour: bool = True) -> None:
    """Debug line prefixed with the rank; rank 0 (or no process group) in red, other ranks in green."""
    r = _rank()
    text = f"{msg}" if r is None else f"{r}:{msg}"
    if colour:
        text = f"\033[{31 if r in (None, 0) else 32}m{text}\033[0m"
    get_logger().debug(text, stacklevel=2)


def print_rank0(msg) -> None:
    if _rank() in (None, 0):
        print(msg, flush=True)


class _XLog:
    """``XLOG.info(...)``, ``XLOG.debug(...)``, ``XLOG.cdebug(...)``: the reference's spelling."""

    def __getattr__(self, name):
        if name == "cdebug":
            return cdebug
        return getattr(get_logger(), name)


XLOG = _XLog()
