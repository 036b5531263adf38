"""Kernel-selection rules as pure functions (the reference tests each of its selectors this way,
tests/unit/test_qwen35_linear_selector.cpp): no GPU, no kernel library."""
import types

import pytest

from phaseshift_b200.ops.cuda_ops import CudaOps, SMALL_M_MAX


def _ops(force_tc=False, exact=False, use_tc_gemm=True):
    o = object.__new__(CudaOps)          # selection reads three attributes only
    o.force_tc, o.exact_rows, o.use_tc_gemm = force_tc, exact, use_tc_gemm
    return o


def _w(tc=False, tiled=False):
    return types.SimpleNamespace(sf_atoms=object() if tc else None, tiled=object() if tiled else None)


@pytest.mark.parametrize("M", [2, 8, 9, 33, 2048])
def test_block_scaled_weights_use_tensor_cores_for_multi_row_steps(M):
    assert CudaOps.select_linear(_ops(), _w(tc=True, tiled=True), M) == "tc"
    assert CudaOps.select_linear(_ops(exact=True), _w(tc=True, tiled=True), M) == "tc"


def test_single_row_streams_only_when_both_layouts_are_resident():
    assert CudaOps.select_linear(_ops(), _w(tc=True, tiled=True), 1) == "stream"
    assert CudaOps.select_linear(_ops(), _w(tc=True, tiled=False), 1) == "tc"
    # speculative decoding: one arithmetic for plain and verification steps
    assert CudaOps.select_linear(_ops(force_tc=True), _w(tc=True, tiled=True), 1) == "tc"


def test_weights_without_tensor_core_layout():
    w = _w(tc=False, tiled=True)
    for M in range(1, SMALL_M_MAX + 1):
        assert CudaOps.select_linear(_ops(), w, M) == "stream"
    assert CudaOps.select_linear(_ops(), w, SMALL_M_MAX + 1) == "gemm"
    assert CudaOps.select_linear(_ops(exact=True), w, 64) == "stream"         # Exact verification never leaves the row kernel
    assert CudaOps.select_linear(_ops(use_tc_gemm=False), w, 64) == "stream"
