"""VMM arena: stable addresses, on-demand commitment, reuse after reset."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_arena_grows_keeps_addresses_and_is_usable_by_kernels():
    from phaseshift_b200.core.arena import ArenaSet, GpuArena
    a = GpuArena(4 << 30, chunk_bytes=64 << 20, name="t")
    assert a.committed == 0 and a.reserved >= (4 << 30)
    x = a.alloc((1024, 1024), torch.float32)
    c1 = a.committed
    assert 0 < c1 <= (128 << 20)
    x.fill_(3.0)
    y = a.alloc((300 << 20,), torch.uint8)            # forces more chunks; x must stay where it is
    assert a.committed > c1
    p = x.data_ptr()
    y.zero_()
    z = a.alloc((1024, 1024), torch.float32)
    torch.matmul(x, x, out=z)                          # library kernels accept arena memory
    torch.cuda.synchronize()
    assert x.data_ptr() == p and float(z[0, 0]) == 3.0 * 3.0 * 1024
    assert y.data_ptr() % 256 == 0 and z.data_ptr() > y.data_ptr()
    with pytest.raises(MemoryError):
        a.alloc((8 << 30,), torch.uint8)
    a.reset(release=True)
    assert a.committed == 0
    w = a.alloc((16,), torch.int32)
    assert w.data_ptr() == a.base
    a.close()
    s = ArenaSet(1 << 30)
    s.get("kv", 512 << 20)
    with pytest.raises(MemoryError):
        s.get("ws", 768 << 20)
    s.close()


def test_engine_state_lives_in_the_arenas_and_the_budget_is_enforced():
    """--arena-gib: KV pages and recurrent state are carved from the VMM arenas (same tokens as with the framework
    allocator, committed bytes match the configuration), and a budget the configuration does not fit is refused."""
    import pytest
    from phaseshift_b200.models.qwen35.config import tiny_config
    from phaseshift_b200.models.qwen35.weights import build_engine_weights, random_hf_weights
    from phaseshift_b200.runtime.engine import Engine
    from phaseshift_b200.runtime.state import StateConfig
    cfg = tiny_config()
    hf = random_hf_weights(cfg, seed=0)
    ew = build_engine_weights(cfg, lambda n: hf[n], "nvfp4", "cuda")
    prompt = list(range(11, 60))
    sc = StateConfig(max_slots=4, max_seq_len=512, kv_dtype="fp8_e4m3")
    plain = Engine(ew, "cuda", sc).generate(prompt, 16, prefill_chunk=32)
    eng = Engine(ew, "cuda", sc, arena_gib=1.0)
    assert eng.generate(prompt, 16, prefill_chunk=32) == plain
    st = eng.state
    assert set(eng.arenas.arenas) == {"kv", "state"}
    kv = eng.arenas.arenas["kv"]
    assert kv.base <= st.kv[3].k.data_ptr() < kv.base + kv.reserved
    need = st.kv_bytes()
    assert need <= kv.committed <= need + (64 << 20)           # exactly what the configuration needs, rounded to chunks
    assert eng.arenas.committed() < (1 << 30)
    with pytest.raises(MemoryError):
        Engine(ew, "cuda", StateConfig(max_slots=64, max_seq_len=65536, kv_dtype="bf16"), arena_gib=0.05)
