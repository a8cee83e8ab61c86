// KV cache pool that grows in place (include/pa_b200.h: pa_b200_cache_pool_*).
//
// KVCacheManager::allocate_cache_if_needed grows a layer's cache by allocating a larger tensor and copying
// every block over (src/cpp/src/continuous_batching/cache/kv_cache_manager.hpp:159-262), which doubles
// the memory for the time of the copy and moves the pointers the compiled model was bound to.  Here the
// pool reserves the virtual address range of its largest size once and maps physical memory into it
// as it grows (CUDA virtual memory management): key_cache / value_cache never move, blocks written
// before a growth keep their bytes, and nothing is copied.  The driver entry points are looked up at
// run time, so the library has no link-time dependency on libcuda.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <string>
#include <vector>

#include "../../../include/pa_b200.h"
#include "../pa_common.cuh"

namespace {

thread_local std::string g_pool_error;
int pfail(int code, const std::string& msg) { g_pool_error = msg; return code; }

struct Driver {
    CUresult (*AddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*GetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    bool ok = false;
};

Driver& driver() {
    static Driver d = [] {
        Driver x;
        auto get = [&](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn;
        };
        x.ok = get("cuMemAddressReserve", (void**)&x.AddressReserve) && get("cuMemAddressFree", (void**)&x.AddressFree) &&
               get("cuMemCreate", (void**)&x.Create) && get("cuMemRelease", (void**)&x.Release) && get("cuMemMap", (void**)&x.Map) &&
               get("cuMemUnmap", (void**)&x.Unmap) && get("cuMemSetAccess", (void**)&x.SetAccess) &&
               get("cuMemGetAllocationGranularity", (void**)&x.GetGranularity);
        return x;
    }();
    return d;
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

struct pa_cache_pool {
    int device = 0;
    size_t block_bytes = 0;      // one block of one cache tensor
    size_t granularity = 0;
    int64_t max_blocks = 0, num_blocks = 0;
    size_t reserved = 0;         // bytes of each of the two ranges
    size_t mapped = 0;           // bytes mapped so far in each range
    CUdeviceptr base[2] = {0, 0};   // key, value
    std::vector<CUmemGenericAllocationHandle> chunks[2];
    std::vector<size_t> chunk_bytes;
};

extern "C" {

const char* pa_b200_cache_pool_last_error(void) { return g_pool_error.c_str(); }

int pa_b200_cache_pool_destroy(pa_cache_pool* p) {
    if (!p) return PA_OK;
    Driver& d = driver();
    cudaSetDevice(p->device);
    cudaDeviceSynchronize();
    for (int t = 0; t < 2; ++t) {
        if (p->base[t] && p->mapped) d.Unmap(p->base[t], p->mapped);
        for (CUmemGenericAllocationHandle hnd : p->chunks[t]) d.Release(hnd);
        if (p->base[t]) d.AddressFree(p->base[t], p->reserved);
    }
    delete p;
    return PA_OK;
}

int pa_b200_cache_pool_grow(pa_cache_pool* p, int64_t num_blocks) {
    if (!p) return pfail(PA_ERR_INVALID_ARG, "NULL pool");
    if (num_blocks <= p->num_blocks) return PA_OK;   // allocate_cache_if_needed: never shrinks
    if (num_blocks > p->max_blocks) return pfail(PA_ERR_TOO_LARGE, "the pool reserved address space for " + std::to_string(p->max_blocks) + " blocks");
    Driver& d = driver();
    if (cudaSetDevice(p->device) != cudaSuccess) return pfail(PA_ERR_CUDA, "cudaSetDevice failed");
    const size_t want = round_up((size_t)num_blocks * p->block_bytes, p->granularity);
    if (want > p->mapped) {
        const size_t add = want - p->mapped;
        CUmemAllocationProp prop;
        std::memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = p->device;
        CUmemAccessDesc acc;
        std::memset(&acc, 0, sizeof(acc));
        acc.location = prop.location;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        CUmemGenericAllocationHandle made[2] = {0, 0};
        for (int t = 0; t < 2; ++t) {
            CUresult r = d.Create(&made[t], add, &prop, 0);
            if (r == CUDA_SUCCESS) {
                r = d.Map(p->base[t] + p->mapped, add, 0, made[t], 0);
                if (r == CUDA_SUCCESS) r = d.SetAccess(p->base[t] + p->mapped, add, &acc, 1);
                if (r != CUDA_SUCCESS) { d.Unmap(p->base[t] + p->mapped, add); d.Release(made[t]); made[t] = 0; }
            }
            if (r != CUDA_SUCCESS) {
                if (t == 1) { d.Unmap(p->base[0] + p->mapped, add); d.Release(made[0]); }
                return pfail(PA_ERR_CUDA, r == CUDA_ERROR_OUT_OF_MEMORY ? "Requested KV-cache size is larger than available memory size on the system."
                                                                        : "mapping " + std::to_string(add) + " bytes failed with CUresult " + std::to_string((int)r));
            }
        }
        // fresh blocks start as zeros, as a freshly created cache tensor does
        if (cudaMemset((void*)(p->base[0] + p->mapped), 0, add) != cudaSuccess || cudaMemset((void*)(p->base[1] + p->mapped), 0, add) != cudaSuccess)
            return pfail(PA_ERR_CUDA, "clearing the new blocks failed");
        p->chunks[0].push_back(made[0]);
        p->chunks[1].push_back(made[1]);
        p->chunk_bytes.push_back(add);
        p->mapped = want;
    }
    p->num_blocks = num_blocks;
    return PA_OK;
}

int pa_b200_cache_pool_create(const pa_model_desc* desc, int device, int64_t max_blocks, int64_t initial_blocks, pa_cache_pool** out) {
    if (!out || !desc) return pfail(PA_ERR_INVALID_ARG, "NULL argument");
    pa_cache_layout lay;
    lay.struct_size = sizeof(lay);
    const int rc = pa_b200_query_cache_layout(desc, &lay);
    if (rc != PA_OK) return pfail(rc, pa_b200_last_error());
    if (max_blocks <= 0 || initial_blocks < 0 || initial_blocks > max_blocks) return pfail(PA_ERR_INVALID_ARG, "0 <= initial_blocks <= max_blocks and max_blocks > 0");
    Driver& d = driver();
    if (!d.ok) return pfail(PA_ERR_NO_DEVICE, "the CUDA driver's virtual memory management entry points are not available");
    if (cudaSetDevice(device) != cudaSuccess || cudaFree(0) != cudaSuccess) return pfail(PA_ERR_CUDA, "cudaSetDevice failed");
    pa_cache_pool* p = new pa_cache_pool();
    p->device = device;
    p->block_bytes = (size_t)lay.key_block_bytes;
    p->max_blocks = max_blocks;
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    if (d.GetGranularity(&p->granularity, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || p->granularity == 0) {
        delete p;
        return pfail(PA_ERR_CUDA, "cuMemGetAllocationGranularity failed");
    }
    p->reserved = round_up((size_t)max_blocks * p->block_bytes, p->granularity);
    for (int t = 0; t < 2; ++t)
        if (d.AddressReserve(&p->base[t], p->reserved, p->granularity, 0, 0) != CUDA_SUCCESS) {
            if (t == 1) d.AddressFree(p->base[0], p->reserved);
            delete p;
            return pfail(PA_ERR_CUDA, "reserving " + std::to_string(p->reserved) + " bytes of address space failed");
        }
    const int grc = pa_b200_cache_pool_grow(p, initial_blocks);
    if (grc != PA_OK) { pa_b200_cache_pool_destroy(p); return grc; }
    *out = p;
    return PA_OK;
}

int pa_b200_cache_pool_get(pa_cache_pool* p, void** key_cache, void** value_cache, int64_t* num_blocks) {
    if (!p) return pfail(PA_ERR_INVALID_ARG, "NULL pool");
    if (key_cache) *key_cache = (void*)p->base[0];
    if (value_cache) *value_cache = (void*)p->base[1];
    if (num_blocks) *num_blocks = p->num_blocks;
    return PA_OK;
}

}  // extern "C"
