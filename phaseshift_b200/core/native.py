"""Loader for the C++ host runtime (pybind11 module ``ps_runtime`` built in-tree by ``phaseshift_b200.build``)."""
from __future__ import annotations

import importlib.util
import sys

_MOD = None


def runtime():
    """The ``ps_runtime`` extension module (built on first use when missing)."""
    global _MOD
    if _MOD is None:
        from ..build import build_runtime, runtime_lib_path
        p = runtime_lib_path()
        if not p.exists():
            build_runtime()
        spec = importlib.util.spec_from_file_location("ps_runtime", str(p))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules["ps_runtime"] = mod
        _MOD = mod
    return _MOD
