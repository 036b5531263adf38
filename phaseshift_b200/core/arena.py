"""Device arenas: stable-address, growable memory regions for the pools whose addresses are baked into
CUDA graphs and peer mappings (KV pages, recurrent state, workspaces).

`GpuArena` wraps the native VMM arena (csrc/kernels/vmm_arena.cu): a virtual range of ``reserve_bytes`` is
reserved once, physical chunks are committed behind it on demand, and tensors are bump-allocated views
into the range.  `ArenaSet` keeps the named arenas of one engine under a common budget, the role of the
reference's ArenaSet / `--arena-gib` (include/phaseshift/core/memory/arena.h:14-120,
src/phaseshift/core/memory/arena.hip:48-138).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Tuple

import torch


class _CudaView:
    """Minimal __cuda_array_interface__ carrier so torch can adopt arena memory without copying."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}
        self._owner = owner


class GpuArena:
    def __init__(self, reserve_bytes: int, device: int = 0, chunk_bytes: int = 0, name: str = "arena"):
        from ..ops import _lib
        self._lib = _lib.lib()
        self.name, self.device = name, device
        h = ctypes.c_void_p()
        fn = self._lib.ps_arena_create
        fn.restype = ctypes.c_int
        rc = fn(ctypes.c_ulonglong(reserve_bytes), ctypes.c_ulonglong(chunk_bytes), ctypes.c_int(device), ctypes.byref(h))
        if rc != 0:
            raise RuntimeError(f"arena '{name}': virtual-memory reservation failed (code {rc})")
        self._h = h
        for f in ("ps_arena_base", "ps_arena_committed", "ps_arena_reserved", "ps_arena_chunk"):
            getattr(self._lib, f).restype = ctypes.c_ulonglong
        self.base = int(self._lib.ps_arena_base(h))
        self.top = 0                      # bump pointer (bytes)

    @property
    def reserved(self) -> int:
        return int(self._lib.ps_arena_reserved(self._h))

    @property
    def committed(self) -> int:
        return int(self._lib.ps_arena_committed(self._h))

    def alloc(self, shape: Tuple[int, ...], dtype: torch.dtype, align: int = 256) -> torch.Tensor:
        """Bump-allocate a tensor; commits more physical memory when needed.  Raises MemoryError when the
        reservation is exhausted (the arena never moves, so it cannot grow past it)."""
        n = 1
        for d in shape:
            n *= int(d)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = (self.top + align - 1) // align * align
        if off + nbytes > self.reserved:
            raise MemoryError(f"arena '{self.name}': {off + nbytes} bytes needed, {self.reserved} reserved")
        fn = self._lib.ps_arena_grow
        fn.restype = ctypes.c_int
        rc = fn(self._h, ctypes.c_ulonglong(off + nbytes))
        if rc != 0:
            raise MemoryError(f"arena '{self.name}': committing {off + nbytes} bytes failed (code {rc})")
        self.top = off + nbytes
        if nbytes == 0:
            return torch.empty(shape, dtype=dtype, device=f"cuda:{self.device}")
        t = torch.as_tensor(_CudaView(self.base + off, nbytes, self), device=f"cuda:{self.device}")
        return t.view(dtype).reshape(shape)

    def reset(self, release: bool = False) -> None:
        """Forget all allocations (tensors handed out earlier must no longer be used); optionally give
        the physical memory back."""
        self.top = 0
        if release:
            fn = self._lib.ps_arena_shrink
            fn.restype = ctypes.c_int
            fn(self._h, ctypes.c_ulonglong(0))

    def close(self) -> None:
        if self._h:
            fn = self._lib.ps_arena_destroy
            fn.restype = ctypes.c_int
            fn(self._h)
            self._h = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


class ArenaSet:
    """Named arenas under one byte budget (`--arena-gib`)."""

    def __init__(self, budget_bytes: int, device: int = 0):
        self.budget, self.device = budget_bytes, device
        self.arenas: Dict[str, GpuArena] = {}

    def get(self, name: str, reserve_bytes: int) -> GpuArena:
        a = self.arenas.get(name)
        if a is None:
            if sum(x.reserved for x in self.arenas.values()) + reserve_bytes > self.budget:
                raise MemoryError(f"arena budget exceeded while reserving '{name}'")
            # physical memory is committed in chunks: small arenas get small chunks so that the commitment tracks the need
            chunk = 2 << 20
            while chunk < (256 << 20) and chunk * 16 < reserve_bytes:
                chunk *= 2
            a = GpuArena(reserve_bytes, self.device, chunk_bytes=chunk, name=name)
            self.arenas[name] = a
        return a

    def committed(self) -> int:
        return sum(a.committed for a in self.arenas.values())

    def close(self) -> None:
        for a in self.arenas.values():
            a.close()
        self.arenas.clear()
