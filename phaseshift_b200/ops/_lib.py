"""ctypes binding to ``libps_kernels.so`` (the hand-written sm_100a kernels).

Every launcher is ``extern "C" int ps_xxx(..., cudaStream_t)`` and returns a ``cudaError_t`` value.
There is no fallback: if the library is missing on a machine with a GPU the import raises, so a test
run can never silently pass on PyTorch eager code.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None


class KernelLibraryError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        from ..build import kernels_lib_path, build_kernels
        checked = os.environ.get("PS_CHECKED", "0") == "1"
        p = kernels_lib_path(checked)
        override = os.environ.get("PS_KERNELS_LIB")            # load this library file instead (A/B runs of two builds)
        if override:
            from pathlib import Path
            p = Path(override)
        if not p.exists():
            try:
                build_kernels(checked=checked)
            except Exception as e:  # pragma: no cover - build environment problem
                raise KernelLibraryError(f"libps_kernels.so is not built and nvcc failed: {e}") from e
        _LIB = ctypes.CDLL(str(p))
        ms = os.environ.get("PS_WAIT_BUDGET_MS")
        if ms:
            # budget of every bounded device-side wait (peer flags, mbarriers), in milliseconds at ~1.9 GHz
            _LIB.ps_set_wait_budget.restype = ctypes.c_longlong
            _LIB.ps_set_wait_budget(ctypes.c_longlong(int(float(ms) * 1.9e6)))
    return _LIB


def checked_build() -> bool:
    """Whether the loaded kernel library is the checked variant (PS_CHECKED=1)."""
    L = lib()
    L.ps_checked_build.restype = ctypes.c_int
    return bool(L.ps_checked_build())


def set_limits(max_slots: int, max_rows: int, status) -> None:
    """Checked build: register the descriptor limits and the status word with every kernel file that asserts on them."""
    L = lib()
    for tag in ("gdn_recurrent", "gdn_chunked"):
        fn = getattr(L, "ps_set_limits_" + tag, None)
        if fn is not None:
            fn.restype = ctypes.c_int
            check(fn(ctypes.c_int(max_slots), ctypes.c_int(max_rows), ptr(status)), "ps_set_limits_" + tag)


def ptr(t) -> ctypes.c_void_p:
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(err: int, what: str) -> None:
    if err != 0:
        raise KernelLibraryError(f"{what} failed with cudaError {err}")


def call(name: str, *args) -> None:
    """Call launcher ``name`` with pre-converted ctypes args and the current stream appended."""
    fn = getattr(lib(), name)
    fn.restype = ctypes.c_int
    check(fn(*args, stream()), name)


c_int = ctypes.c_int
c_float = ctypes.c_float
c_ll = ctypes.c_longlong
