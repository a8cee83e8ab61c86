// The exchange step of a sharded engine step (include/exchange_b200.h): an in-place ncclAllGather
// of the sampled token ids, issued from the host layer on the sampler's stream.  NCCL is bound with
// dlopen so that the library has no link-time dependency on it.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "../../../include/exchange_b200.h"

namespace {

thread_local std::string g_error;
int xfail(int code, const std::string& msg) { g_error = msg; return code; }

// the few NCCL declarations used here, spelled out so that no NCCL header is needed at build time
struct NcclUniqueId { char internal[EXCHANGE_B200_ID_BYTES]; };
typedef struct ncclComm* NcclComm;
enum { kNcclSuccess = 0, kNcclInt64 = 4 };
struct Nccl {
    int (*GetUniqueId)(NcclUniqueId*) = nullptr;
    int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
    int (*CommDestroy)(NcclComm) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string why;
};

Nccl& nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) { n.why = std::string("dlopen(libnccl.so.2): ") + dlerror(); return; }
        auto sym = [&](const char* name) {
            void* p = dlsym(lib, name);
            if (!p && n.why.empty()) n.why = std::string("libnccl.so.2 lacks ") + name;
            return p;
        };
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
        n.ok = n.why.empty();
    });
    return n;
}

__global__ void pad_row_kernel(int64_t* row, int n_local, int cap) {
    for (int i = n_local + blockIdx.x * blockDim.x + threadIdx.x; i < cap; i += gridDim.x * blockDim.x) row[i] = -1;
}

}  // namespace

struct exchange_handle {
    NcclComm comm = nullptr;
    int rank = 0, world = 1, device = 0, cap = 0;
    int64_t* rows = nullptr;   // [world][cap]
};

extern "C" {

const char* exchange_b200_last_error(void) { return g_error.c_str(); }

int exchange_b200_unique_id(uint8_t id[EXCHANGE_B200_ID_BYTES]) {
    if (!id) return xfail(EXCHANGE_ERR_INVALID_ARG, "NULL id");
    Nccl& n = nccl();
    if (!n.ok) return xfail(EXCHANGE_ERR_NO_NCCL, n.why);
    NcclUniqueId u;
    const int rc = n.GetUniqueId(&u);
    if (rc != kNcclSuccess) return xfail(EXCHANGE_ERR_NCCL, std::string("ncclGetUniqueId: ") + n.GetErrorString(rc));
    std::memcpy(id, u.internal, EXCHANGE_B200_ID_BYTES);
    return EXCHANGE_OK;
}

int exchange_b200_create(const uint8_t id[EXCHANGE_B200_ID_BYTES], int32_t rank, int32_t world, int32_t device, int32_t cap, exchange_handle** out) {
    if (!id || !out || world < 1 || rank < 0 || rank >= world || cap < 1) return xfail(EXCHANGE_ERR_INVALID_ARG, "bad rank / world / cap or NULL pointer");
    Nccl& n = nccl();
    if (!n.ok) return xfail(EXCHANGE_ERR_NO_NCCL, n.why);
    if (cudaSetDevice(device) != cudaSuccess) return xfail(EXCHANGE_ERR_CUDA, "cudaSetDevice failed");
    exchange_handle* h = new exchange_handle();
    h->rank = rank; h->world = world; h->device = device; h->cap = cap;
    cudaError_t e = cudaMalloc((void**)&h->rows, (size_t)world * cap * sizeof(int64_t));
    if (e == cudaSuccess) e = cudaMemset(h->rows, 0xff, (size_t)world * cap * sizeof(int64_t));
    if (e != cudaSuccess) { delete h; return xfail(EXCHANGE_ERR_CUDA, std::string("exchange buffer: ") + cudaGetErrorString(e)); }
    NcclUniqueId u;
    std::memcpy(u.internal, id, EXCHANGE_B200_ID_BYTES);
    const int rc = n.CommInitRank(&h->comm, world, u, rank);
    if (rc != kNcclSuccess) {
        cudaFree(h->rows);
        delete h;
        return xfail(EXCHANGE_ERR_NCCL, std::string("ncclCommInitRank: ") + n.GetErrorString(rc));
    }
    *out = h;
    return EXCHANGE_OK;
}

int exchange_b200_destroy(exchange_handle* h) {
    if (!h) return EXCHANGE_OK;
    cudaSetDevice(h->device);
    cudaDeviceSynchronize();
    if (h->comm) nccl().CommDestroy(h->comm);
    if (h->rows) cudaFree(h->rows);
    delete h;
    return EXCHANGE_OK;
}

int64_t* exchange_b200_local_row(exchange_handle* h) { return h ? h->rows + (size_t)h->rank * h->cap : nullptr; }
int64_t* exchange_b200_all_rows(exchange_handle* h) { return h ? h->rows : nullptr; }

int exchange_b200_all_gather_ids(exchange_handle* h, int32_t n_local, void* stream) {
    if (!h || n_local < 0 || n_local > h->cap) return xfail(EXCHANGE_ERR_INVALID_ARG, "NULL handle or n_local outside [0, cap]");
    if (cudaSetDevice(h->device) != cudaSuccess) return xfail(EXCHANGE_ERR_CUDA, "cudaSetDevice failed");
    cudaStream_t s = (cudaStream_t)stream;
    int64_t* mine = h->rows + (size_t)h->rank * h->cap;
    if (n_local < h->cap) {
        pad_row_kernel<<<1, 256, 0, s>>>(mine, n_local, h->cap);
        if (cudaGetLastError() != cudaSuccess) return xfail(EXCHANGE_ERR_CUDA, "pad launch failed");
    }
    // in place: this rank's share already sits at rows + rank * cap
    const int rc = nccl().AllGather(mine, h->rows, (size_t)h->cap, kNcclInt64, h->comm, s);
    if (rc != kNcclSuccess) return xfail(EXCHANGE_ERR_NCCL, std::string("ncclAllGather: ") + nccl().GetErrorString(rc));
    return EXCHANGE_OK;
}

}  // extern "C"
