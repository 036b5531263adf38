"""Host codec of the NVFP4 key/value pages, and the configuration plumbing around the 4-bit cache."""
import pytest
import torch

from phaseshift_b200.quant.kv_formats import bits_per_value, decode_nvfp4_rows, encode_nvfp4_rows, nvfp4_row_bytes
from phaseshift_b200.runtime.state import KV_DTYPE_ALIASES, KV_DTYPES, StateConfig, kv_row_bytes


@pytest.mark.parametrize("D", [64, 128, 256])
def test_row_layout_and_size(D):
    assert nvfp4_row_bytes(D) % 16 == 0 and nvfp4_row_bytes(D) >= D // 2 + D // 16
    assert kv_row_bytes("nvfp4", D) == nvfp4_row_bytes(D)
    assert kv_row_bytes("fp8_e4m3", D) == D and kv_row_bytes("bf16", D) == 2 * D
    x = torch.randn(3, 5, D, generator=torch.Generator().manual_seed(D))
    rows, ts = encode_nvfp4_rows(x)
    assert rows.shape == (3, 5, nvfp4_row_bytes(D)) and rows.dtype == torch.uint8 and ts.shape == (3, 5)
    assert int(rows[..., D // 2 + D // 16:].sum()) == 0                       # padding stays zero
    assert bits_per_value("nvfp4", 256) == pytest.approx(4.625) and bits_per_value("fp8_e4m3", 256) == pytest.approx(8.125)


def test_round_trip_error_is_that_of_a_four_bit_float():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(64, 256, generator=g) * torch.logspace(-3, 3, 64).unsqueeze(1)      # rows of very different size
    rows, ts = encode_nvfp4_rows(x)
    y = decode_nvfp4_rows(rows, ts, 256)
    # E2M1 has steps of at most one third of the value above the smallest binade; within a block of 16 the error of every
    # value is bounded by half a step at the block's maximum, i.e. a quarter of (block max / 6) * 2 ... measured against
    # the block maximum this is < 1/6 (+ the rounding of the E4M3 block scale, 1/16)
    blk = x.reshape(64, 16, 16)
    err = (y.reshape(64, 16, 16) - blk).abs().amax(-1)
    assert bool((err <= blk.abs().amax(-1) * (1 / 6 + 1 / 16) + 1e-30).all())
    rel = ((y - x).norm(dim=1) / x.norm(dim=1))
    assert float(rel.max()) < 0.12, float(rel.max())
    # representable rows come back up to the rounding of the fp32 row scale: values on the E2M1 grid, every block at the top code
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    z = grid[torch.randint(0, 8, (4, 256), generator=g)] * torch.where(torch.rand(4, 256, generator=g) < 0.5, -1.0, 1.0)
    z[:, ::16] = 6.0                                                           # every block reaches the top code
    rz, tz = encode_nvfp4_rows(z)
    torch.testing.assert_close(decode_nvfp4_rows(rz, tz, 256), z, rtol=1e-6, atol=0)


def test_zero_rows_and_sign():
    x = torch.zeros(2, 64)
    x[1, 3] = -2.5
    rows, ts = encode_nvfp4_rows(x)
    y = decode_nvfp4_rows(rows, ts, 64)
    assert float(ts[0]) == 1.0 and torch.equal(y[0], torch.zeros(64))
    assert float(y[1, 3]) == pytest.approx(-2.5, rel=1e-6) and float(y[1].abs().sum()) == pytest.approx(2.5, rel=1e-6)


def test_state_config_accepts_the_four_bit_cache_and_the_upstream_names():
    assert "nvfp4" in KV_DTYPES and KV_DTYPE_ALIASES == {"psq4": "nvfp4", "psq8": "fp8_e4m3"}
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.runtime.state import ModelState
    st = ModelState(tiny_config(), StateConfig(max_slots=1, max_seq_len=32, kv_dtype="nvfp4"), torch.device("cpu"), act_dtype=torch.float32)
    assert st.kv_fmt == 0                                                      # the fp32 oracle keeps full-precision pages
    with pytest.raises(ValueError):
        ModelState(tiny_config(), StateConfig(kv_dtype="int3"), torch.device("cpu"), act_dtype=torch.float32)


def test_native_codec_matches_the_tensor_codec_byte_for_byte():
    from phaseshift_b200.core.native import runtime
    rt = runtime()
    g = torch.Generator().manual_seed(7)
    for D in (64, 128, 256):
        x = (torch.randn(37, D, generator=g) * torch.logspace(-2, 2, 37).unsqueeze(1)).contiguous()
        x[5] = 0
        x[6, ::3] = 0
        rows_t, ts_t = encode_nvfp4_rows(x)
        rb = rt.kv_nvfp4_row_bytes(D)
        assert rb == nvfp4_row_bytes(D)
        rows_n = torch.empty(37, rb, dtype=torch.uint8)
        ts_n = torch.empty(37, dtype=torch.float32)
        rt.kv_nvfp4_encode_rows(x.data_ptr(), 37, D, rows_n.data_ptr(), ts_n.data_ptr())
        assert torch.equal(ts_n, ts_t) and torch.equal(rows_n, rows_t)
        out = torch.empty(37, D, dtype=torch.float32)
        rt.kv_nvfp4_decode_rows(rows_n.data_ptr(), ts_n.data_ptr(), 37, D, out.data_ptr())
        assert torch.equal(out, decode_nvfp4_rows(rows_t, ts_t, D))
