"""Source-level rules of the package, checked by scanning the tree (the reference keeps a similar scanner,
tests/unit/test_architecture_boundaries.cpp:53-185): no compatibility layers on the engine's paths, no calls that are
closed on the target machines, nothing committed depends on working files, kernels keep their waits bounded."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "phaseshift_b200"


def _sources(exts):
    for p in list(PKG.rglob("*")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"] + list((ROOT / "tests").glob("*.py")):
        if p.suffix in exts and "_C" not in p.parts and p.name != "test_architecture_cpu.py":
            yield p


def test_no_compatibility_layers_or_tracing_compilers():
    bad = []
    for p in _sources({".py"}):
        if "tests" in p.parts:
            continue
        txt = p.read_text()
        for pat in (r"^\s*import triton", r"^\s*from triton", r"torch\.compile\(", r"import tilelang", r"^\s*import jax"):
            if re.search(pat, txt, re.M):
                bad.append((str(p.relative_to(ROOT)), pat))
    assert not bad, bad


def test_library_gemm_only_in_reference_and_optional_paths():
    """`@` / matmul / einsum on activations is allowed in the CPU reference ops, the fp32 oracle, quantiser tooling, the
    optional torch drafters and tests -- not in the CUDA op set, the engine, the native drafter or the transport."""
    hot = ["ops/cuda_ops.py", "runtime/engine.py", "runtime/serving.py", "runtime/spec_serving.py", "parallel/tp.py",
           "models/dflash2/native.py", "models/qwen35/model.py"]
    bad = []
    for rel in hot:
        txt = (PKG / rel).read_text()
        code = "\n".join(l.split("#")[0] for l in txt.splitlines() if "W.dense()" not in l)
        for pat in (r"torch\.matmul", r"torch\.einsum", r"F\.linear", r"\.mm\(", r"torch\.bmm"):
            if re.search(pat, code):
                bad.append((rel, pat))
    assert not bad, bad


def test_closed_calls_and_cluster_multicast_loads_never_appear():
    closed = ["cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync", "cuMemcpy" + "BatchAsync", "cuMemcpy3D" + "BatchAsync"]
    bad = []
    for p in _sources({".py", ".cu", ".cuh", ".h", ".cpp"}):
        txt = p.read_text(errors="ignore")
        for name in closed:
            if name in txt:
                bad.append((str(p.relative_to(ROOT)), name))
        for m in re.finditer(r"cp\.async\.bulk[\w\.:]*", txt):
            if ("multi" + "cast::cluster") in m.group(0):      # (spelled in two pieces: this file only tests for the qualifier)
                bad.append((str(p.relative_to(ROOT)), m.group(0)))
    assert not bad, bad


def test_nothing_committed_depends_on_working_files_or_machine_paths():
    bad = []
    for p in _sources({".py", ".cu", ".cuh", ".h", ".cpp"}):
        txt = p.read_text(errors="ignore")
        for pat in (r"_work/", r"gpurun", r"/root/"):
            if re.search(pat, txt):
                bad.append((str(p.relative_to(ROOT)), pat))
    assert not bad, bad


def test_device_spin_waits_are_bounded():
    """Every `do { ... } while (true)` / `while (true)` spin in a kernel file mentions a budget inside its body."""
    bad = []
    for p in (PKG / "csrc").rglob("*.cu*"):
        txt = p.read_text()
        for m in re.finditer(r"\bdo\s*\{(.*?)\}\s*while\s*\(\s*true\s*\)", txt, re.S):
            if "budget" not in m.group(1):
                bad.append((p.name, m.group(1)[:80]))
        for m in re.finditer(r"while\s*\(\s*(true|1)\s*\)\s*\{(.*?)\}", txt, re.S):
            if "budget" not in m.group(2) and "break" in m.group(2):
                bad.append((p.name, m.group(2)[:80]))
    assert not bad, bad
