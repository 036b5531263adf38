"""Offline-tooling kernels: the CUDA row quantisers must reproduce the C++ CPU quantisers bit for bit (with
and without importance weights); KLD / NLL / imatrix reductions against plain PyTorch fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _cpu_quant(w, fmt, search, imp, ts):
    from phaseshift_b200.core.native import runtime
    rt = runtime()
    n, k = w.shape
    kp = -(-k // 32) * 32
    wf = w.float().contiguous()
    codes = torch.empty(n, kp // 2 if fmt == "nvfp4" else kp, dtype=torch.uint8)
    scales = torch.empty(n, kp // (16 if fmt == "nvfp4" else 32), dtype=torch.uint8)
    ip = imp.float().contiguous() if imp is not None else None
    if fmt == "nvfp4":
        rt.quantize_rows_nvfp4(wf.data_ptr(), n, k, kp, ts, search, ip.data_ptr() if ip is not None else 0, codes.data_ptr(), scales.data_ptr())
    else:
        rt.quantize_rows_mxfp8(wf.data_ptr(), n, k, kp, search, ip.data_ptr() if ip is not None else 0, codes.data_ptr(), scales.data_ptr())
    return codes, scales


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("with_imp", [False, True])
def test_cuda_quantiser_is_bit_equal_to_cpu(fmt, with_imp):
    from phaseshift_b200.quant import formats
    g = torch.Generator().manual_seed(5)
    w = torch.randn(37, 600, generator=g) * 0.05
    w[3, :40] = 0.0
    w[5, 7] = 9.0                                        # outlier block
    w[6] *= 1e-4
    imp = (torch.rand(600, generator=g) + 0.05) if with_imp else None
    search = 2 if fmt == "nvfp4" else 1
    q = formats.quantize_nvfp4(w.cuda(), imp, search) if fmt == "nvfp4" else formats.quantize_mxfp8(w.cuda(), imp, search)
    ts = float(torch.tensor(q.tensor_scale, dtype=torch.float32))
    codes, scales = _cpu_quant(w, fmt, search, imp, ts)
    assert torch.equal(q.scales.cpu(), scales)
    assert torch.equal(q.codes.cpu(), codes)
    # and the torch implementation (used on CPU tensors) agrees on the reconstruction
    formats.USE_CUDA_KERNELS = False
    try:
        qt = formats.quantize_nvfp4(w.cuda(), imp, search) if fmt == "nvfp4" else formats.quantize_mxfp8(w.cuda(), imp, search)
    finally:
        formats.USE_CUDA_KERNELS = True
    assert torch.allclose(formats.dequantize(qt).cpu(), formats.dequantize(q).cpu(), atol=0, rtol=0) or \
        float((formats.dequantize(qt) - formats.dequantize(q)).abs().max()) < 1e-3


def test_kld_nll_imatrix_kernels():
    import ctypes
    from phaseshift_b200.ops import _lib
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(3)
    rows, vocab = 6, 5000
    base = torch.randn(rows, vocab, device=dev, generator=g) * 3
    cand = base + torch.randn(rows, vocab, device=dev, generator=g) * 0.3
    cand[2] = base[2]
    kld = torch.empty(rows, device=dev); agree = torch.empty(rows, dtype=torch.int32, device=dev)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.call("ps_kld_rows", vp(base), vp(cand), ctypes.c_int(rows), ctypes.c_int(vocab), ctypes.c_longlong(vocab), vp(kld), vp(agree))
    lp, lq = torch.log_softmax(base.double(), -1), torch.log_softmax(cand.double(), -1)
    ref = (lp.exp() * (lp - lq)).sum(-1)
    assert torch.allclose(kld.double(), ref, rtol=2e-3, atol=1e-5) and float(kld[2]) < 1e-6
    assert agree.tolist() == (base.argmax(-1) == cand.argmax(-1)).int().tolist()
    tgt = torch.randint(0, vocab, (rows,), device=dev, generator=g).int()
    nll = torch.empty(rows, device=dev)
    _lib.call("ps_nll_rows", vp(base), vp(tgt), ctypes.c_int(rows), ctypes.c_int(vocab), ctypes.c_longlong(vocab), vp(nll))
    refn = -lp[torch.arange(rows), tgt.long()]
    assert torch.allclose(nll.double(), refn, rtol=1e-3, atol=1e-4)
    x = torch.randn(33, 1000, device=dev, generator=g).to(torch.bfloat16)
    acc = torch.ones(1000, device=dev)
    _lib.call("ps_imatrix_accumulate", vp(x), ctypes.c_longlong(1000), ctypes.c_int(33), ctypes.c_int(1000), vp(acc))
    assert torch.allclose(acc, 1.0 + x.float().pow(2).sum(0), rtol=1e-5)
