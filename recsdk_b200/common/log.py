"""Logging proxy: one library logger whose level comes from the environment (``RECSDK_LOG_LEVEL`` or, like the
reference's native logger, ``GLOG_stderrthreshold`` 0..3 = info, warning, error, fatal).
Reference: ``training/common/python/log/log.py:24-69``."""
from __future__ import annotations

import logging
import os

_GLOG = {0: logging.INFO, 1: logging.WARNING, 2: logging.ERROR, 3: logging.CRITICAL}


def _level_from_env() -> int:
    name = os.environ.get("RECSDK_LOG_LEVEL")
    if name:
        return getattr(logging, name.upper(), logging.INFO)
    try:
        return _GLOG.get(int(os.environ.get("GLOG_stderrthreshold", "0")), logging.INFO)
    except ValueError:
        return logging.INFO


class LoggingProxy:
    """Forwards ``debug/info/warning/error/critical`` to a lazily configured logger; ``set_level`` at any time."""

    def __init__(self, name: str = "recsdk_b200") -> None:
        self._logger = logging.getLogger(name)
        if not self._logger.handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("[%(asctime)s][%(levelname)s][%(name)s] %(message)s"))
            self._logger.addHandler(h)
            self._logger.propagate = False
        self._logger.setLevel(_level_from_env())

    def set_level(self, level) -> None:
        self._logger.setLevel(getattr(logging, level.upper()) if isinstance(level, str) else level)

    def __getattr__(self, item):
        return getattr(self._logger, item)


logger = LoggingProxy()
