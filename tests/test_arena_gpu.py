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
