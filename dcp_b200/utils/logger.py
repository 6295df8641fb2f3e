"""Logging helpers: per-component log files under ``$DCP_LOGGING_DEBUG_DIR`` (default ./debug) when
``DCP_DEBUG`` is set, a quiet stderr logger otherwise (dcp/utils/logger.py:129-207)."""
from __future__ import annotations

import logging
import os
import sys
from typing import Optional

_LEVELS = {"DEBUG": logging.DEBUG, "INFO": logging.INFO, "WARNING": logging.WARNING, "ERROR": logging.ERROR}


def read_env_bool(name: str, default: bool = False) -> bool:
    v = os.environ.get(name)
    if v is None:
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")


def debug_level() -> int:
    v = os.environ.get("DCP_DEBUG", "")
    if not v:
        return logging.WARNING
    return _LEVELS.get(v.upper(), logging.DEBUG)


def log_dir() -> str:
    return os.environ.get("DCP_LOGGING_DEBUG_DIR", "./debug")


class _Formatter(logging.Formatter):
    def __init__(self, prefix: Optional[str] = None):
        p = f"[{prefix}] " if prefix else ""
        super().__init__(f"%(asctime)s {p}%(name)s %(levelname)s: %(message)s", "%H:%M:%S")


def create_logger(name: Optional[str] = None, prefix: Optional[str] = None, level: Optional[int] = None,
                  log_file: Optional[str] = None, file_level: int = logging.DEBUG,
                  override_existing: bool = True) -> logging.Logger:
    """A logger that writes to stderr at ``level`` and, when DCP_DEBUG is set and ``log_file`` is
    given, to ``<log_dir>/<log_file>`` at ``file_level``."""
    level = debug_level() if level is None else level
    logger = logging.getLogger(f"dcp_b200.{name}" if name else "dcp_b200")
    if override_existing:
        for h in list(logger.handlers):
            logger.removeHandler(h)
            h.close()
    if not logger.handlers:
        logger.setLevel(min(level, file_level) if (log_file and os.environ.get("DCP_DEBUG")) else level)
        sh = logging.StreamHandler(sys.stderr)
        sh.setLevel(level)
        sh.setFormatter(_Formatter(prefix))
        logger.addHandler(sh)
        if log_file and os.environ.get("DCP_DEBUG"):
            path = os.path.join(log_dir(), log_file)
            os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
            fh = logging.FileHandler(path, mode="a")
            fh.setLevel(file_level)
            fh.setFormatter(_Formatter(prefix))
            logger.addHandler(fh)
        logger.propagate = False
    return logger


logger = create_logger(override_existing=False)
