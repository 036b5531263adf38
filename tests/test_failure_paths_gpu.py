"""Bounded device waits that actually run out, on ONE GPU: a two-rank collective whose "peer" never raises its flag
(all buffers local, nothing faults, nothing hangs).  Every kernel must return within its budget, report
PS_DEV_WAIT_TIMEOUT (2) through the status word, leave the context usable, and the engine must poison the step's
sequences and serve a fresh one afterwards."""
import ctypes

import pytest
import torch

from phaseshift_b200.models.qwen35.config import tiny_config
from phaseshift_b200.models.qwen35.weights import LinearW, build_engine_weights, random_hf_weights
from phaseshift_b200.quant.formats import quantize
from phaseshift_b200.runtime.batch import SeqRows
from phaseshift_b200.runtime.state import StateConfig

pytestmark = pytest.mark.gpu
TIMEOUT = 2            # PS_DEV_WAIT_TIMEOUT


class _Budget:
    """About a millisecond of wait budget while the block runs."""

    def __enter__(self):
        from phaseshift_b200.ops import _lib
        self.L = _lib.lib()
        self.L.ps_set_wait_budget.restype = ctypes.c_longlong
        self.prev = self.L.ps_set_wait_budget(ctypes.c_longlong(2_000_000))
        return self

    def __exit__(self, *exc):
        torch.cuda.synchronize()
        self.L.ps_set_wait_budget(ctypes.c_longlong(self.prev))
        return False


def _dead_peer_combine(n, keep):
    """TpCombineStruct of rank 0 of 2 whose peer flags stay zero."""
    from phaseshift_b200.parallel.tp import MAX_ROWS, TpCombineStruct
    c = TpCombineStruct()
    n_pad = -(-n // 4) * 4
    c.size, c.rank, c.max_rows, c.n_pad = 2, 0, MAX_ROWS, n_pad
    recv = torch.zeros(2 * 2 * MAX_ROWS * n_pad, dtype=torch.float32, device="cuda")
    mine = torch.zeros(256 * 2, dtype=torch.int32, device="cuda")
    peer = torch.zeros(256 * 2, dtype=torch.int32, device="cuda")
    counter = torch.zeros(256, dtype=torch.int32, device="cuda")
    c.recv[0] = c.recv[1] = recv.data_ptr()
    c.flags[0], c.flags[1] = mine.data_ptr(), peer.data_ptr()
    c.counter = counter.data_ptr()
    keep += [recv, mine, peer, counter]
    return c


def test_streaming_projection_combine_wait_expires():
    from phaseshift_b200.ops.cuda_ops import CudaOps
    ops = CudaOps(tiny_config(), torch.device("cuda:0"))
    g = torch.Generator(device="cuda").manual_seed(3)
    W = LinearW(quantize(torch.randn(256, 512, device="cuda", generator=g) * 0.05, "bf16"))
    x = torch.randn(2, 512, device="cuda", generator=g).to(torch.bfloat16)
    res = torch.zeros(2, 256, dtype=torch.bfloat16, device="cuda")
    keep = []
    with _Budget():
        ops.linear(x, W, name="dead", residual=res, tp_combine=_dead_peer_combine(256, keep))
        torch.cuda.synchronize()
        assert int(ops.status[0]) == TIMEOUT
    ops.reset_after_error()
    y = ops.linear(x, W, name="alive", out_f32=True)
    torch.cuda.synchronize()
    assert int(ops.status[0]) == 0
    ref = x.float() @ W.dense().T
    assert float((y - ref).norm() / ref.norm()) < 1e-2


@pytest.mark.parametrize("kernel", ["peer", "reduce_gather"])
def test_collective_kernels_give_up_on_a_silent_peer(kernel):
    from phaseshift_b200.ops import _lib
    from phaseshift_b200.parallel.tp import AR_GRID, RG_GRID, ArStruct, RgStruct
    rows, n = 64, 256
    part = torch.ones(rows, n, dtype=torch.bfloat16, device="cuda")
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    grid = AR_GRID if kernel == "peer" else RG_GRID
    mine = torch.zeros(2 * grid * 2, dtype=torch.int32, device="cuda")
    peer = torch.zeros(2 * grid * 2, dtype=torch.int32, device="cuda")
    counter = torch.zeros(grid, dtype=torch.int32, device="cuda")
    with _Budget():
        if kernel == "peer":
            a = ArStruct()
            a.size, a.rank, a.rows, a.n = 2, 0, rows, n
            a.inp[0] = a.inp[1] = part.data_ptr()
            a.flags[0], a.flags[1] = mine.data_ptr(), peer.data_ptr()
            a.counter, a.out, a.ldo, a.status = counter.data_ptr(), out.data_ptr(), n, status.data_ptr()
            _lib.call("ps_allreduce", ctypes.byref(a), ctypes.c_int(0), ctypes.c_int(grid))
        else:
            recv = torch.zeros(2 * rows * n, dtype=torch.bfloat16, device="cuda")
            a = RgStruct()
            a.size, a.rank, a.rows, a.n, a.rpr, a.ld = 2, 0, rows, n, rows // 2, n
            a.src_row0 = 0
            for r in range(2):
                a.src[r] = recv.data_ptr() + r * (rows // 2) * n * 2
                a.recv[r] = recv.data_ptr()
                a.out[r] = out.data_ptr()
                a.flags[r] = (mine if r == 0 else peer).data_ptr()
            a.partial, a.ld_partial = part.data_ptr(), n
            a.counter, a.ldo, a.status = counter.data_ptr(), n, status.data_ptr()
            _lib.call("ps_tp_reduce_gather", ctypes.byref(a), ctypes.c_int(grid))
        torch.cuda.synchronize()
        assert int(status[0]) == TIMEOUT
    assert torch.all(out == 7.0)                # a collective that gave up wrote no result
    assert int(torch.zeros(1, device="cuda").sum()) == 0      # the context still works


@pytest.mark.parametrize("preset", ["bf16", "nvfp4"])
def test_engine_poisons_the_step_and_serves_a_fresh_sequence(preset):
    """Engine.step on rank 0 of a two-rank job whose peer is silent: device status -> SequenceError, the sequences of
    the step are poisoned (and refuse further steps), the status words and stream-K flags are clean again, and a new
    sequence steps normally once the transport is gone."""
    from phaseshift_b200.runtime.engine import Engine, SequenceError
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], preset, "cuda", tp_rank=0, tp_size=2)
    eng = Engine(ew, "cuda", StateConfig(max_slots=2, max_seq_len=64))
    keep = []

    class SilentPeer:
        size, rank, transport = 2, 0, "fused"
        stats = {"fused": 0}
        combines = {}

        def assert_alive(self):
            pass

        def max_fused_rows(self, W):
            return 8

        def combine_for(self, n):
            if n not in self.combines:
                self.combines[n] = _dead_peer_combine(n, keep)
            return self.combines[n]
    eng.tp = eng.runner.tp = SilentPeer()
    s = eng.open_sequence()
    with _Budget():
        with pytest.raises(SequenceError):
            eng.step([SeqRows(s.slot, 0, [5, 6, 7], (2,))], [s])
    assert s.poisoned and eng.status_errors == 1
    with pytest.raises(SequenceError):
        eng.step([SeqRows(s.slot, 0, [5], (0,))], [s])
    assert int(eng.ops.status[0]) == 0 and int(eng.state.status[0]) == 0
    eng.close_sequence(s)
    eng.tp = eng.runner.tp = None                     # the job continues on this rank alone (its weights are a TP slice)
    eng.graphs.clear(); eng.graph_out.clear()         # captured steps have the dead transport baked in
    s2 = eng.open_sequence()
    toks, _ = eng.step([SeqRows(s2.slot, 0, [5, 6, 7], (2,))], [s2])
    toks2, _ = eng.step([SeqRows(s2.slot, 3, [toks[0]], (0,))], [s2])
    assert len(toks) == 1 and len(toks2) == 1 and not s2.poisoned and int(eng.ops.status[0]) == 0
