"""The allocation-free attention entry point, called through its exported C symbol, must reproduce the
regular entry point (which takes caller-provided scratch) on consecutive calls.  It exists for callers
that cannot obtain device memory at call time (stream capture, real-time loops, foreign runtimes); see
csrc/include/ps_noalloc.h.  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(q, k, v, bt, slot, pos, rows, Hq, Hkv, D, split, max_splits, vis, gate, out, status, scratch=None):
    P = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    I, F = ctypes.c_int, ctypes.c_float
    a = [P(q), P(k), P(v), P(None), P(None), P(bt), I(bt.shape[1]), I(16), I(k.shape[0]), P(slot), P(pos), I(rows),
         I(Hq), I(Hkv), I(D), F(D ** -0.5), I(0), I(split), I(max_splits), I(vis)]
    if scratch is not None:
        a += [P(scratch[0]), P(scratch[1])]
    a += [P(gate), I(gate.stride(0)), I(2 * D), I(D), P(out), P(status), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)]
    return a


def test_noalloc_entry_matches_regular_entry_twice():
    from phaseshift_b200.build import kernels_lib_path
    lib = ctypes.CDLL(str(kernels_lib_path()))
    lib.ps_paged_attention.restype = ctypes.c_int
    lib.ps_paged_attention_noalloc.restype = ctypes.c_int
    lib.ps_noalloc_last_error.restype = ctypes.c_char_p
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    rows, Hq, Hkv, D, pages, split, max_splits = 2, 12, 2, 256, 40, 128, 4
    for call in range(2):
        k = torch.randn(pages, Hkv, 16, D, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(pages, Hkv, 16, D, device=dev, generator=g).to(torch.bfloat16)
        q = torch.randn(rows, Hq * D, device=dev, generator=g).to(torch.bfloat16)
        gate = torch.randn(rows, 2 * Hq * D, device=dev, generator=g).to(torch.bfloat16)
        bt = torch.stack([torch.randperm(pages - 1, device=dev, generator=g)[:20] + 1 for _ in range(2)]).int().contiguous()
        slot = torch.tensor([0, 1], dtype=torch.int32, device=dev)
        pos = torch.tensor([300 - 37 * call, 150 + 11 * call], dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        vis = int(pos.max()) + 1
        ref = torch.empty(rows, Hq * D, dtype=torch.bfloat16, device=dev)
        got = torch.full_like(ref, float("nan"))
        pacc = torch.empty(rows * Hq * max_splits * D, dtype=torch.float32, device=dev)
        pml = torch.empty(rows * Hq * max_splits * 2, dtype=torch.float32, device=dev)
        assert lib.ps_paged_attention(*_args(q, k, v, bt, slot, pos, rows, Hq, Hkv, D, split, max_splits, vis, gate, ref,
                                             status, (pacc, pml))) == 0
        assert lib.ps_paged_attention_noalloc(*_args(q, k, v, bt, slot, pos, rows, Hq, Hkv, D, split, max_splits, vis, gate,
                                                     got, status)) == 0
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, ref)          # both entry points launch the same kernels: bit for bit
    # a problem larger than the built-in scratch is refused with a message, nothing is launched
    rc = lib.ps_paged_attention_noalloc(*_args(q, k, v, bt, slot, pos, rows, Hq, Hkv, D, split, 4096, vis, gate, got, status))
    assert rc == -2 and b"exceeds" in lib.ps_noalloc_last_error()
