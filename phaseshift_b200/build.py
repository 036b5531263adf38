"""In-tree native build for phaseshift_b200.

Two shared objects are produced under ``phaseshift_b200/_C``:

* ``libps_kernels.so`` -- every CUDA kernel (``csrc/kernels/*.cu``), compiled by
  nvcc for ``sm_100a`` only, exposing plain ``extern "C"`` launchers that take raw
  device pointers and a ``cudaStream_t``.  Loaded with ``ctypes``.
* ``ps_runtime<abi>.so`` -- the host runtime (``csrc/runtime/*.cpp``: safetensors
  IO, quantisation codecs, pools, scheduler, KV banker, batcher, prefix-cache
  index, speculative-decode bookkeeping), a pybind11 module compiled by g++.

The build is incremental (per-object mtime check) and runs without a GPU: nvcc
cross-compiles.  ``python -m phaseshift_b200.build`` rebuilds from the shell.
"""
from __future__ import annotations

import concurrent.futures as _cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_C"
OBJ = OUT / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
    "-I", str(CSRC / "include"),
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-sign-compare",
             "-ffp-contract=off", "-I", str(CSRC / "include")]


def _nvcc() -> str:
    for cand in (os.environ.get("PS_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src: Path, dst: Path, extra_deps) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    if src.stat().st_mtime > t:
        return True
    return any(d.stat().st_mtime > t for d in extra_deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(map(str, cmd)) + "\n" + p.stdout + p.stderr)
    return p.stdout + p.stderr


def kernels_lib_path(checked: bool = False) -> Path:
    return OUT / ("libps_kernels_checked.so" if checked else "libps_kernels.so")


def runtime_lib_path() -> Path:
    return OUT / ("ps_runtime" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_kernels(verbose: bool = False, force: bool = False, ptxas_info: bool = False, checked: bool = False) -> Path:
    """``checked``: the -DPS_CHECKED variant (descriptor assertions that report through a status word), built beside
    the normal library; ``PS_CHECKED=1`` in the environment makes the op set load it."""
    obj_dir = OBJ / "checked" if checked else OBJ
    obj_dir.mkdir(parents=True, exist_ok=True)
    headers = list((CSRC / "include").rglob("*.h")) + list((CSRC / "include").rglob("*.cuh")) + \
        list((CSRC / "kernels").glob("*.cuh"))
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if force or _newer(s, o, headers):
            cmd = [nvcc, *NVCC_FLAGS, *(["-DPS_CHECKED=1"] if checked else []), "-c", str(s), "-o", str(o)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    logs = []
    if jobs:
        with _cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(lambda c: _run(c, verbose), jobs):
                logs.append(out)
    lib = kernels_lib_path(checked)
    if jobs or not lib.exists():
        _run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-lcudart", "-lcuda",
              "-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    if ptxas_info:
        print("\n".join(logs))
    return lib


def build_runtime(verbose: bool = False, force: bool = False) -> Path:
    import pybind11
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list((CSRC / "include").rglob("*.h")) + list((CSRC / "runtime").glob("*.h"))
    srcs = sorted((CSRC / "runtime").glob("*.cpp"))
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    cxx = os.environ.get("CXX", "g++")
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / ("rt_" + s.stem + ".o")
        objs.append(o)
        if force or _newer(s, o, headers):
            jobs.append([cxx, *CXX_FLAGS, *inc, "-c", str(s), "-o", str(o)])
    if jobs:
        with _cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = runtime_lib_path()
    if jobs or not lib.exists():
        _run([cxx, "-shared", "-o", str(lib), *map(str, objs), "-lpthread"], verbose)
    return lib


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_runtime(verbose, force)
    build_kernels(verbose, force)
    build_kernels(verbose, force, checked=True)


if __name__ == "__main__":
    v = "-v" in sys.argv
    f = "-f" in sys.argv
    if "--ptxas" in sys.argv:
        build_kernels(v, True, True)
    else:
        build_all(v, f)
    print("built:", kernels_lib_path(), runtime_lib_path())
