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

    # -- the reference's class-level form: ``LoggingProxy.set_instance("INFO"); LoggingProxy.error("...")`` -------------
    _instance = None

    @classmethod
    def set_instance(cls, log_level: str = "INFO") -> None:
        level = str(log_level).upper()
        if level not in ("DEBUG", "INFO", "WARNING", "ERROR", "CRITICAL"):
            raise ValueError("log level is not valid, only DEBUG / INFO / WARNING / ERROR / CRITICAL are allowed, but got %s" % log_level)
        proxy = cls("recsdk_b200")
        proxy.set_level(level)
        cls._instance = proxy._logger


def _class_level(name: str, **fixed):
    def call(cls, msg, *args, **kwargs):
        if cls._instance is None:
            cls.set_instance(logging.getLevelName(_level_from_env()))
        for k, v in fixed.items():
            kwargs.setdefault(k, v)
        getattr(cls._instance, name)(msg, *args, **kwargs)
    return call


class _ClassOrInstance:
    """``LoggingProxy.info(...)`` on the class goes to the shared logger, ``proxy.info(...)`` on an object to that object's."""

    def __init__(self, name: str, method: str, **fixed) -> None:
        self.name, self.method, self.fixed = name, method, fixed

    def __get__(self, obj, cls):
        if obj is None:
            return _class_level(self.method, **self.fixed).__get__(cls, type(cls))
        target = getattr(obj._logger, self.method)
        if not self.fixed:
            return target
        return lambda msg, *a, **k: target(msg, *a, **{**self.fixed, **k})


for _n, _m, _kw in (("info", "info", {}), ("debug", "debug", {}), ("error", "error", {}), ("warning", "warning", {}),
                    ("critical", "critical", {}), ("exception", "error", {"exc_info": True})):
    setattr(LoggingProxy, _n, _ClassOrInstance(_n, _m, **_kw))


logger = LoggingProxy()
