// Growable device arena on the CUDA virtual-memory API: one virtual address range is reserved up front
// (cheap: no physical memory), physical chunks are created and mapped behind it as the arena grows and
// are unmapped/released from the tail when it shrinks, so tensors placed in the arena keep their
// addresses for the life of the process (CUDA graphs and peer mappings stay valid) while HBM is only
// spent on what is in use.  The reference's GpuArena reserves `--arena-gib` with one hipMalloc and bump
// allocates inside it (include/phaseshift/core/memory/arena.h:14-62, src/phaseshift/core/memory/arena.hip:48-138); on a 180 GB part the reservation can be the
// whole address budget while the commitment follows the KV cache.
//
// Host-only code; the driver entry points are resolved through the runtime, so the library needs no
// direct link against libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "ps_common.cuh"

namespace ps {

struct DriverVmm {
    CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    bool ok = false;
};

static DriverVmm& driver() {
    static DriverVmm d;
    static std::once_flag once;
    std::call_once(once, [] {
        auto get = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess;
        };
        d.ok = get("cuMemAddressReserve", (void**)&d.reserve) && get("cuMemAddressFree", (void**)&d.addr_free) &&
               get("cuMemCreate", (void**)&d.create) && get("cuMemRelease", (void**)&d.release) &&
               get("cuMemMap", (void**)&d.map) && get("cuMemUnmap", (void**)&d.unmap) &&
               get("cuMemSetAccess", (void**)&d.set_access) &&
               get("cuMemGetAllocationGranularity", (void**)&d.granularity);
    });
    return d;
}

struct Arena {
    int device = 0;
    CUdeviceptr base = 0;
    size_t reserved = 0, committed = 0, chunk = 0;
    std::vector<CUmemGenericAllocationHandle> chunks;
    CUmemAllocationProp prop{};
};

}  // namespace ps

// Error codes: 0 ok, -1 driver VMM entry points unavailable, otherwise the CUresult of the failing call.
PS_API int ps_arena_create(unsigned long long reserve_bytes, unsigned long long chunk_bytes, int device, void** out) {
    using namespace ps;
    DriverVmm& d = driver();
    if (!d.ok) return -1;
    if (cudaSetDevice(device) != cudaSuccess) return (int)cudaErrorInvalidDevice;
    cudaFree(nullptr);                                   // make sure the primary context exists
    Arena* a = new Arena();
    a->device = device;
    a->prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    a->prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a->prop.location.id = device;
    size_t gran = 0;
    CUresult r = d.granularity(&gran, &a->prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS || gran == 0) { delete a; return (int)r ? (int)r : -1; }
    size_t chunk = chunk_bytes ? chunk_bytes : (size_t)256 << 20;
    chunk = (chunk + gran - 1) / gran * gran;
    a->chunk = chunk;
    a->reserved = (reserve_bytes + chunk - 1) / chunk * chunk;
    r = d.reserve(&a->base, a->reserved, 0, 0, 0);
    if (r != CUDA_SUCCESS) { delete a; return (int)r; }
    *out = a;
    return 0;
}

// Commit physical memory so that at least `bytes` from the base are usable (never shrinks).
PS_API int ps_arena_grow(void* h, unsigned long long bytes) {
    using namespace ps;
    Arena* a = (Arena*)h;
    DriverVmm& d = driver();
    if (bytes > a->reserved) return (int)CUDA_ERROR_OUT_OF_MEMORY;
    while (a->committed < bytes) {
        CUmemGenericAllocationHandle mh;
        CUresult r = d.create(&mh, a->chunk, &a->prop, 0);
        if (r != CUDA_SUCCESS) return (int)r;
        r = d.map(a->base + a->committed, a->chunk, 0, mh, 0);
        if (r != CUDA_SUCCESS) { d.release(mh); return (int)r; }
        CUmemAccessDesc acc{};
        acc.location = a->prop.location;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        r = d.set_access(a->base + a->committed, a->chunk, &acc, 1);
        if (r != CUDA_SUCCESS) { d.unmap(a->base + a->committed, a->chunk); d.release(mh); return (int)r; }
        a->chunks.push_back(mh);
        a->committed += a->chunk;
    }
    return 0;
}

// Release whole chunks beyond `bytes` (the caller guarantees nothing on the device still uses them).
PS_API int ps_arena_shrink(void* h, unsigned long long bytes) {
    using namespace ps;
    Arena* a = (Arena*)h;
    DriverVmm& d = driver();
    while (!a->chunks.empty() && a->committed - a->chunk >= bytes) {
        a->committed -= a->chunk;
        CUresult r = d.unmap(a->base + a->committed, a->chunk);
        if (r != CUDA_SUCCESS) { a->committed += a->chunk; return (int)r; }
        d.release(a->chunks.back());
        a->chunks.pop_back();
    }
    return 0;
}

PS_API unsigned long long ps_arena_base(void* h) { return (unsigned long long)((ps::Arena*)h)->base; }
PS_API unsigned long long ps_arena_committed(void* h) { return ((ps::Arena*)h)->committed; }
PS_API unsigned long long ps_arena_reserved(void* h) { return ((ps::Arena*)h)->reserved; }
PS_API unsigned long long ps_arena_chunk(void* h) { return ((ps::Arena*)h)->chunk; }

PS_API int ps_arena_destroy(void* h) {
    using namespace ps;
    Arena* a = (Arena*)h;
    if (a == nullptr) return 0;
    int rc = ps_arena_shrink(h, 0);
    if (a->base) driver().addr_free(a->base, a->reserved);
    delete a;
    return rc;
}
