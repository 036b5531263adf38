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


def test_step_batch_marks_rows_of_short_and_long_sequences():
    """The descriptor block a step uploads: positions of every row, and a second copy for the per-row attention kernel in
    which rows of sequences with more than SHORT_SEQ_ROWS rows carry -2 (another kernel owns them) and padding rows -1."""
    import torch
    from phaseshift_b200.runtime.batch import SeqRows, StepBatch
    b = StepBatch(64, 4, torch.device("cpu"), pinned=False)
    n_long = StepBatch.SHORT_SEQ_ROWS + 4
    b.fill([SeqRows(2, 100, [7], (0,)), SeqRows(0, 10, list(range(n_long)), ()), SeqRows(1, 5, [1, 2, 3], (2,))])
    b.upload()
    pos, short = b.row_pos.tolist(), b.row_pos_short.tolist()
    assert pos[0] == 100 and short[0] == 100
    assert pos[1:1 + n_long] == list(range(10, 10 + n_long)) and short[1:1 + n_long] == [-2] * n_long
    assert pos[1 + n_long:4 + n_long] == [5, 6, 7] and short[1 + n_long:4 + n_long] == [5, 6, 7]
    assert set(pos[4 + n_long:]) == {-1} and set(short[4 + n_long:]) == {-1}
    assert b.seq_desc[:3].tolist() == [[0, 1, 2, 100], [1, n_long, 0, 10], [1 + n_long, 3, 1, 5]]
    assert b.out_rows[:2].tolist() == [0, 1 + n_long + 2] and b.n_out == 2 and not b.identity_out


def test_graph_keys_separate_greedy_steps_and_keep_the_bucket_readable():
    from phaseshift_b200.runtime.engine import Engine
    keys = {Engine.graph_key(bk, n, ident, g) for bk in (1, 4, 16, 64) for n in (1, 4) for ident in (False, True) for g in (False, True)}
    assert len(keys) == 4 * 2 * 2 * 2
    for bk in (1, 16, 64):
        assert Engine.graph_key_bucket(Engine.graph_key(bk, 1, True, True)) == bk
        assert Engine.graph_key_bucket((Engine.graph_key(bk, 3, False), (1, 2), 0, False, True)) == bk
