"""Block-scaled tcgen05 projection (csrc/kernels/gemm_bs.cu) against a plain PyTorch fp32 restatement of the
same op: RMSNorm -> activation block quantisation (quant/act_quant.py) -> product with the dequantised weights
-> epilogue.  Covers both formats, the resident (<= 32 rows) and streamed paths, ragged shapes, the 27B
projection shapes, every epilogue, stream-K partitions of several grid sizes, batch invariance, and the bounded
wait of the tensor-parallel combine."""
import ctypes

import pytest
import torch
import torch.nn.functional as F

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.weights import LinearW
from phaseshift_b200.quant.act_quant import fake_quant, pack_sf_atoms, unpack_sf_atoms
from phaseshift_b200.quant.formats import quantize

pytestmark = pytest.mark.gpu

SHAPES_27B = [(16384, 5120), (14336, 5120), (5120, 6144), (34816, 5120), (5120, 17408), (151936, 5120)]


def _ops(grid_override=0):
    from phaseshift_b200.ops.cuda_ops import CudaOps
    ops = CudaOps(tiny_config(), torch.device("cuda:0"))
    ops.bs_grid_override = grid_override
    ops.BS_RESIDENT_MAX_ROWS = 32          # the kernel's own limit (the engine switches to the streamed path above 8 rows)
    return ops


def _make(N, K, fmt, seed, act_scale=None):
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(N, K, device="cuda", generator=g) * 0.02
    W = LinearW(quantize(w, fmt)).make_umma()
    if act_scale is not None:
        W.act_scale = act_scale
    return W, g


def _reference(x, W, norm_w=None, eps=1e-6, residual=None, swiglu=False):
    xf = x.float()
    inv = None
    if norm_w is not None:
        # the kernel quantises x (1 + w) and applies the row factor 1/rms after the product
        inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps).double()
        xf = xf * (1.0 + norm_w.float())
    xq = fake_quant(xf, W.fmt, W.act_scale)
    y = xq.double() @ W.dense().double().T
    if inv is not None:
        y = y * inv
    if swiglu:
        yb = y.float().to(torch.bfloat16).float()
        return F.silu(yb[:, 0::2]) * yb[:, 1::2]
    if residual is not None:
        return y.float().to(torch.bfloat16).float() + residual.float()
    return y.float()


def _rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / (b.norm() + 1e-30))


def test_sf_atom_layout_round_trip():
    s = torch.randint(0, 255, (300, 40), dtype=torch.uint8, device="cuda")
    a = pack_sf_atoms(s, "nvfp4", 640)
    assert a.shape == (3, 12, 512)
    assert torch.equal(unpack_sf_atoms(a, 300, 40), s)
    # row 37 of tile 1 (global row 165), block 9 -> atom 2, j = 1
    assert int(a[1, 2, (37 % 32) * 16 + (37 // 32) * 4 + 1]) == int(s[165, 9])


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("M", [1, 3, 16, 17, 32])
@pytest.mark.parametrize("shape", [(256, 512), (200, 328), (1024, 5120), (640, 17408)])
def test_resident_plain(fmt, M, shape):
    N, K = shape
    ops = _ops()
    W, g = _make(N, K, fmt, N + K + M)
    x = (torch.randn(M, K, device="cuda", generator=g) * 1.5).to(torch.bfloat16)
    assert ops.bs_resident_ok(W, M)
    y = ops.linear(x, W, name="t", out_f32=True)
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0
    assert _rel(y, _reference(x, W)) < 2e-4


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("grid", [1, 3, 7, 40, 148])
def test_stream_k_partitions(fmt, grid):
    """Any grid size gives the same result up to fp32 summation order: head / middle / tail segments, tiles
    split over several CTAs and CTAs spanning several tiles."""
    ops = _ops(grid)
    W, g = _make(384, 2304, fmt, 77 + grid)
    x = torch.randn(5, 2304, device="cuda", generator=g).to(torch.bfloat16)
    y = ops.linear(x, W, name="t", out_f32=True)
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0 and int(ops.bs_flags.abs().sum()) == 0
    assert _rel(y, _reference(x, W)) < 2e-4


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("M", [2, 8])
def test_resident_fused_norm_and_epilogues(fmt, M):
    ops = _ops()
    N, K = 768, 1024
    W, g = _make(N, K, fmt, 5 + M)
    x = (torch.randn(M, K, device="cuda", generator=g) * 3).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    xn = torch.empty(M, K, dtype=torch.bfloat16, device="cuda")
    y = ops.linear(x, W, name="a", norm_w=nw, eps=1e-6, out_f32=True, xn_out=xn)
    assert _rel(y, _reference(x, W, nw)) < 2e-4
    xf = x.float()
    xn_ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + nw.float())).to(torch.bfloat16)
    assert _rel(xn, xn_ref) < 4e-3
    y = ops.linear(x, W, name="b", norm_w=nw, eps=1e-6, residual=res)
    assert _rel(y, _reference(x, W, nw, residual=res)) < 6e-3
    y = ops.linear(x, W, name="c", norm_w=nw, eps=1e-6, swiglu=True)
    assert _rel(y, _reference(x, W, nw, swiglu=True)) < 1e-2
    assert int(ops.status[0]) == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("M", [1, 5, 20])
def test_row_statistics_hand_over(fmt, M):
    """A residual epilogue leaves per-tile sums of squares of what it stores; the next projection's fused RMSNorm
    built from them matches the one that sweeps the rows itself."""
    ops = _ops()
    H, K = 640, 1024
    W1, g = _make(H, K, fmt, 31 + M)
    W2, _ = _make(384, H, fmt, 32 + M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    res = torch.randn(M, H, device="cuda", generator=g).to(torch.bfloat16)
    nw = (torch.randn(H, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    ssq = ops.ssq_buf("t", M)
    ssq.fill_(float("nan"))
    r = ops.linear(x, W1, name="r", residual=res, ssq_out=ssq)
    n = -(-H // 128)
    torch.cuda.synchronize()
    want = r.float().pow(2).sum(-1)
    assert _rel(ssq[:, :n].sum(-1), want) < 1e-5
    y_a = ops.linear(r, W2, name="a", norm_w=nw, eps=1e-6, out_f32=True, ssq_in=(ssq, n)).clone()
    y_b = ops.linear(r, W2, name="b", norm_w=nw, eps=1e-6, out_f32=True)
    assert _rel(y_a, y_b) < 1e-5
    assert _rel(y_a, _reference(r, W2, nw)) < 2e-4


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("M", [33, 64, 300, 1000])
def test_streamed(fmt, M):
    ops = _ops()
    N, K = 640, 1536
    W, g = _make(N, K, fmt, 11 + M)
    x = (torch.randn(M, K, device="cuda", generator=g) * 2).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
    y = ops.linear(x, W, name="a", out_f32=True)
    assert _rel(y, _reference(x, W)) < 2e-4
    y = ops.linear(x, W, name="b", norm_w=nw, eps=1e-6, residual=res)
    assert _rel(y, _reference(x, W, nw, residual=res)) < 6e-3
    y = ops.linear(x, W, name="c", norm_w=nw, eps=1e-6, swiglu=True)
    assert _rel(y, _reference(x, W, nw, swiglu=True)) < 1e-2
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("shape", SHAPES_27B[:5])
@pytest.mark.parametrize("M", [2, 8, 64, 300, 2048])
def test_27b_shapes(fmt, shape, M):
    N, K = shape
    ops = _ops()
    W, g = _make(N, K, fmt, N // 128 + K + M)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    if N == 34816:
        y = ops.linear(x, W, name="s", norm_w=nw, eps=1e-6, swiglu=True)
        assert _rel(y, _reference(x, W, nw, swiglu=True)) < 1e-2
    elif N == 5120:
        res = torch.randn(M, N, device="cuda", generator=g).to(torch.bfloat16)
        y = ops.linear(x, W, name="r", residual=res)
        assert _rel(y, _reference(x, W, residual=res)) < 6e-3
    else:
        y = ops.linear(x, W, name="p", norm_w=nw, eps=1e-6, out_f32=True)
        assert _rel(y, _reference(x, W, nw)) < 2e-4
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0


def test_lm_head_shape_mxfp8():
    N, K = SHAPES_27B[5]
    ops = _ops()
    W, g = _make(N, K, "mxfp8", 3)
    x = torch.randn(2, K, device="cuda", generator=g).to(torch.bfloat16)
    nw = (torch.randn(K, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    y = ops.linear(x, W, name="l", norm_w=nw, eps=1e-6, out_f32=True)
    assert _rel(y, _reference(x, W, nw)) < 2e-4


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
def test_rows_are_batch_invariant(fmt):
    """Row r of an M-row launch equals the same row of a 1-row launch bit for bit (Exact verification), on the
    16-row and on the 32-row instruction shape, and the two shapes agree with each other."""
    ops = _ops()
    W, g = _make(640, 5120, fmt, 9)
    x = torch.randn(24, 5120, device="cuda", generator=g).to(torch.bfloat16)
    nw = (torch.randn(5120, device="cuda", generator=g) * 0.1).to(torch.bfloat16)
    y8 = ops.linear(x[:8], W, name="i8", norm_w=nw, eps=1e-6, out_f32=True).clone()
    y24 = ops.linear(x, W, name="i24", norm_w=nw, eps=1e-6, out_f32=True).clone()
    for r in (0, 3, 7):
        y1 = ops.linear(x[r:r + 1], W, name="i1", norm_w=nw, eps=1e-6, out_f32=True)
        assert torch.equal(y1[0], y8[r])
        assert torch.equal(y1[0], y24[r])


def test_tp_combine_wait_runs_out_and_kernel_returns():
    """A two-rank combine whose peer never raises its flag: the bounded wait expires, the kernel reports
    PS_DEV_WAIT_TIMEOUT in the status word and returns; the next launch works."""
    from phaseshift_b200.ops import _lib
    from phaseshift_b200.parallel.tp import TpCombineStruct
    ops = _ops()
    N, K, M = 256, 512, 2
    W, g = _make(N, K, "nvfp4", 21)
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    res = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
    c = TpCombineStruct()
    c.size, c.rank, c.max_rows, c.n_pad = 2, 0, 32, N
    recv = torch.zeros(2 * 2 * 32 * N, dtype=torch.float32, device="cuda")
    flags_mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags_peer = torch.zeros(64, dtype=torch.int32, device="cuda")     # the "peer" writes nothing here
    counter = torch.zeros(64, dtype=torch.int32, device="cuda")
    c.recv[0] = c.recv[1] = recv.data_ptr()
    c.flags[0], c.flags[1] = flags_mine.data_ptr(), flags_peer.data_ptr()
    c.counter = counter.data_ptr()
    L = _lib.lib()
    L.ps_set_wait_budget.restype = ctypes.c_longlong
    prev = L.ps_set_wait_budget(ctypes.c_longlong(2_000_000))          # about a millisecond
    try:
        ops.linear(x, W, name="tp", residual=res, tp_combine=c)
        torch.cuda.synchronize()
        assert int(ops.status[0]) == 2                                  # PS_DEV_WAIT_TIMEOUT
    finally:
        L.ps_set_wait_budget(ctypes.c_longlong(prev))
    ops.reset_after_error()
    y = ops.linear(x, W, name="ok", out_f32=True)
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0
    assert _rel(y, _reference(x, W)) < 2e-4
