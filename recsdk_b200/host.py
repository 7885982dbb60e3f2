"""Loader of the native host engines (``_C_host``): builds the pybind11 module in-tree when its
sources are newer than the binary, then imports it."""
from __future__ import annotations

import importlib
import os

from . import _build

_mod = None


def host():
    global _mod
    if _mod is None:
        if os.environ.get("RECSDK_B200_NO_BUILD", "0") != "1":
            try:
                _build.build_host()
            except Exception:
                if not _build.HOST_SO.exists():
                    raise
        _mod = importlib.import_module("recsdk_b200._C_host")
    return _mod
