"""Imports the C++ host runtime (cache manager, scheduler), building it at first use."""

from __future__ import annotations

import importlib.util
import sys

from ..ops import build

_mod = None


def host():
    global _mod
    if _mod is None:
        path = build.build_host()
        spec = importlib.util.spec_from_file_location("_rlis_host", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules.setdefault("_rlis_host", mod)
        _mod = mod
    return _mod
