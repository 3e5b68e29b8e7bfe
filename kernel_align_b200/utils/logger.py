"""Process-wide logger with once-only and rank-filtered helpers.

Same surface as the reference's ``rl_engine/utils/logger.py:9-67`` (``init_logger``, the
``logger`` singleton, ``info_once`` / ``warn_once`` / ``info_on_rank``, the
``"%(levelname)s %(asctime)s [%(name)s]: %(message)s"`` line format), built as a
``logging.Logger`` subclass instead of methods patched onto an instance, and with
``info_on_rank`` reading the real distributed rank.

Environment: ``RL_ENGINE_LOG_LEVEL`` (default ``INFO``).
"""
from __future__ import annotations

import logging
import os
import sys
import threading
from typing import Any

LINE_FORMAT = "%(levelname)s %(asctime)s [%(name)s]: %(message)s"
DATE_FORMAT = "%m-%d %H:%M:%S"


def current_rank() -> int:
    """Rank of this process: torch.distributed if initialised, else ``RANK``, else 0."""
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank()
    except Exception:  # torch missing or half-initialised: fall through to the environment
        pass
    try:
        return int(os.environ.get("RANK", "0"))
    except ValueError:
        return 0


class RLEngineLogger(logging.Logger):
    """``logging.Logger`` plus message de-duplication and rank filtering."""

    def __init__(self, name: str, level: int = logging.NOTSET) -> None:
        super().__init__(name, level)
        self._seen: set[tuple] = set()
        self._seen_lock = threading.Lock()

    def _once(self, level: int, msg: str, args: tuple) -> None:
        key = (level, msg, args)
        with self._seen_lock:
            if key in self._seen:
                return
            self._seen.add(key)
        if self.isEnabledFor(level):
            self._log(level, msg, args, stacklevel=3)

    def info_once(self, msg: str, *args: Any) -> None:
        """Log at INFO the first time this exact (message, args) pair is seen."""
        self._once(logging.INFO, msg, args)

    def warn_once(self, msg: str, *args: Any) -> None:
        """Log at WARNING the first time this exact (message, args) pair is seen."""
        self._once(logging.WARNING, msg, args)

    def info_on_rank(self, msg: str, rank: int = 0, *args: Any) -> None:
        """Log at INFO only in the process whose distributed rank is ``rank``."""
        if current_rank() == rank and self.isEnabledFor(logging.INFO):
            self._log(logging.INFO, msg, args, stacklevel=2)

    def reset_once_cache(self) -> None:
        with self._seen_lock:
            self._seen.clear()


def init_logger(name: str) -> RLEngineLogger:
    """Create (or fetch) the named logger writing one formatted line per record to stdout."""
    manager = logging.Logger.manager
    existing = manager.loggerDict.get(name)
    if isinstance(existing, RLEngineLogger):
        return existing
    log = RLEngineLogger(name)
    log.parent = logging.getLogger()
    manager.loggerDict[name] = log
    level = getattr(logging, os.environ.get("RL_ENGINE_LOG_LEVEL", "INFO").upper(), logging.INFO)
    log.setLevel(level)
    handler = logging.StreamHandler(sys.stdout)
    handler.setFormatter(logging.Formatter(LINE_FORMAT, datefmt=DATE_FORMAT))
    log.addHandler(handler)
    log.propagate = False
    return log


logger = init_logger("RL-Engine")
