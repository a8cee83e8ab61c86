// Eviction scoring on the device (include/eviction_b200.h): the score manager and the block selection of
// src/cpp/src/continuous_batching/cache/cache_eviction.cpp for the SUM / NORM_SUM modes, one CTA per
// sequence.  Every double is produced by the operation the host code performs, in its order, so the
// evicted block lists are the reference's.
//   register  max_pool (:51-66) -> accumulate (:130-224) -> counters (:204-224)
//   evict     block sums (:457-483) -> lowest (score, index) (:485-519) -> removal of their tokens (:14-48)
#include <cuda_runtime.h>

#include <cstring>
#include <string>

#include "../../include/eviction_b200.h"

namespace {

thread_local std::string g_error;
int efail(int code, const std::string& msg) { g_error = msg; return code; }
#define E_CUDA(expr)                                                                               \
    do {                                                                                           \
        cudaError_t _e = (expr);                                                                   \
        if (_e != cudaSuccess) return efail(EVICTION_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

constexpr int kThreads = 256;

struct Cfg {
    int start_size, recent_size, max_cache_size, bs, aggregation, snapkv_window, pool, layers, slots, max_tokens, max_evicted;
};

struct StepArgs {
    Cfg c;
    int layer, num_sequences, do_evict;
    const float* scores;
    const long long* span_begin;
    const int* span_len;
    const int* slot;
    const int* num_snapkv;
    int* evicted_count;
    int* evicted_blocks;
    double* acc;        // [layers][slots][max_tokens]
    unsigned* counter;  // [layers][slots][max_tokens]
    int* length;        // [layers][slots]
    int* snap;          // [layers][slots] SnapKV rows registered so far
    unsigned* status;
};

__global__ void __launch_bounds__(kThreads) eviction_step_kernel(StepArgs a) {
    extern __shared__ unsigned char smem[];
    const Cfg& c = a.c;
    const int s = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) a.evicted_count[s] = 0;
    const int slot = a.slot[s];
    if (slot < 0 || slot >= c.slots) {
        if (tid == 0) atomicOr(a.status, 2u);
        return;
    }
    const size_t rec = (size_t)a.layer * c.slots + slot;
    double* acc = a.acc + rec * c.max_tokens;
    unsigned* cnt = a.counter + rec * c.max_tokens;
    const int n = a.span_len[s];
    const int start_off = (c.start_size / c.bs) * c.bs;
    int len = a.length[rec];
    __syncthreads();

    // ---- register_new_token_scores -------------------------------------------------------------------
    if (n > start_off) {
        const int m = n - start_off;
        const float* hh = a.scores + a.span_begin[s] + start_off;
        const int num_snap = a.num_snapkv[s];
        int registered = a.snap[rec];
        if (registered < c.snapkv_window) {
            if (num_snap + registered > c.snapkv_window) { if (tid == 0) atomicOr(a.status, 4u); }
            registered += num_snap;
        }
        const bool initial = len == 0;
        const bool skip_initial = initial && c.snapkv_window != 0 && num_snap == 0;   // window not reached: nothing to accumulate yet
        if (m > c.max_tokens) {
            if (tid == 0) atomicOr(a.status, 1u);
        } else if (!initial && m < len) {
            if (tid == 0) atomicOr(a.status, 8u);
        } else if (!skip_initial) {
            for (int i = tid; i < m; i += kThreads) {
                float mx = hh[i];
                const int w = min(c.pool, m - i);
                for (int k = 1; k < w; ++k) mx = fmaxf(hh[i + k], mx);   // std::max(val, max_val): NaN handling aside, the larger one
                const double pooled = (double)mx;
                acc[i] = (!initial && i < len) ? __dadd_rn(acc[i], pooled) : (initial ? pooled : __dadd_rn(0.0, pooled));
            }
            if (c.aggregation == EVICTION_AGG_NORM_SUM) {
                if (initial) {
                    for (int i = tid; i < m; i += kThreads) {
                        unsigned v;
                        if (c.snapkv_window == 0) v = (unsigned)(m - i);
                        else v = i < m - num_snap ? (unsigned)num_snap : (unsigned)(m - i);
                        cnt[i] = v;
                    }
                } else {
                    const int num_new = m - len;
                    if (c.snapkv_window == 0 || registered == c.snapkv_window) {
                        for (int i = tid; i < m; i += kThreads) cnt[i] = i < len ? cnt[i] + (unsigned)num_new : (unsigned)(num_new - (i - len));
                    } else {
                        for (int i = tid; i < m; i += kThreads) cnt[i] = i < m - registered ? (unsigned)registered : (unsigned)(m - i);
                    }
                }
            }
            len = m;
        }
        __syncthreads();
        if (tid == 0) { a.length[rec] = len; a.snap[rec] = registered; }
    }
    if (!a.do_evict) return;

    // ---- evict_logical_blocks -------------------------------------------------------------------------
    if ((long long)len + c.start_size <= (long long)c.max_cache_size + c.bs - 1) return;   // cache not yet filled
    const int seq_len = c.start_size + len;
    const int start_blocks = c.start_size / c.bs;
    const int num_evictable = seq_len / c.bs - c.recent_size / c.bs - start_blocks;
    const int evictable_size = c.max_cache_size - c.start_size - c.recent_size;
    const int keep = (evictable_size + c.bs - 1) / c.bs;
    const int to_evict = num_evictable >= keep ? num_evictable - keep : 0;
    if (to_evict <= 0 || num_evictable <= 0) return;
    if (to_evict > c.max_evicted) { if (tid == 0) atomicOr(a.status, 1u); return; }
    double* bscore = reinterpret_cast<double*>(smem);                       // [num_evictable]
    unsigned char* evict = smem + (size_t)num_evictable * sizeof(double);   // [num_evictable]
    for (int i = tid; i < num_evictable; i += kThreads) {
        double sum = 0.0;
        for (int j = 0; j < c.bs; ++j) {
            const int t = c.bs * i + j;
            sum = c.aggregation == EVICTION_AGG_NORM_SUM ? __dadd_rn(sum, __ddiv_rn(acc[t], (double)cnt[t])) : __dadd_rn(sum, acc[t]);
        }
        bscore[i] = sum;
    }
    __syncthreads();
    // the to_evict lowest by (score, index): a block's rank is the number of blocks ordered before it
    for (int i = tid; i < num_evictable; i += kThreads) {
        const double si = bscore[i];
        int rank = 0;
        for (int j = 0; j < num_evictable; ++j) {
            const double sj = bscore[j];
            rank += (sj < si || (sj == si && j < i)) ? 1 : 0;
        }
        evict[i] = rank < to_evict ? 1 : 0;
    }
    __syncthreads();
    // ascending list, and the tokens of the kept blocks moved down over the evicted ones (chunk by chunk: a
    // token only ever moves to a lower index, so a chunk's destinations lie in what has been read already)
    __shared__ int sh_scan[kThreads];
    __shared__ int sh_base;
    if (tid == 0) sh_base = 0;
    __syncthreads();
    for (int base = 0; base < num_evictable; base += kThreads) {
        const int i = base + tid;
        const int e = i < num_evictable ? evict[i] : 0;
        sh_scan[tid] = e;
        __syncthreads();
        for (int o = 1; o < kThreads; o <<= 1) {
            const int v = tid >= o ? sh_scan[tid - o] : 0;
            __syncthreads();
            sh_scan[tid] += v;
            __syncthreads();
        }
        if (e) a.evicted_blocks[(size_t)s * c.max_evicted + sh_base + sh_scan[tid] - 1] = i + start_blocks;
        __syncthreads();
        if (tid == kThreads - 1) sh_base += sh_scan[tid];
        __syncthreads();
    }
    // removal: token t of block b moves down by bs * (evicted blocks before b); blocks past the evictable range keep all
    __shared__ int sh_shift;   // evicted blocks before the current chunk's first block
    if (tid == 0) sh_shift = 0;
    __syncthreads();
    for (int base = 0; base < len; base += kThreads) {
        const int t = base + tid;
        double v = 0.0;
        unsigned cv = 0;
        int dst = -1;
        if (t < len) {
            const int b = t / c.bs;
            int before = 0;
            const int upto = min(b, num_evictable);
            for (int j = 0; j < upto; ++j) before += evict[j];   // short lists: a few hundred blocks
            const bool gone = b < num_evictable && evict[b];
            if (!gone) { dst = t - before * c.bs; v = acc[t]; cv = c.aggregation == EVICTION_AGG_NORM_SUM ? cnt[t] : 0u; }
        }
        __syncthreads();
        if (dst >= 0) { acc[dst] = v; if (c.aggregation == EVICTION_AGG_NORM_SUM) cnt[dst] = cv; }
        __syncthreads();
    }
    if (tid == 0) {
        a.evicted_count[s] = to_evict;
        a.length[rec] = len - to_evict * c.bs;
    }
}

__global__ void reset_slot_kernel(int* length, int* snap, int layers, int slots, int slot) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l < layers) { length[(size_t)l * slots + slot] = 0; snap[(size_t)l * slots + slot] = 0; }
}

}  // namespace

struct eviction_handle {
    Cfg c{};
    int device = 0;
    cudaStream_t stream = nullptr;
    double* acc = nullptr;
    unsigned* counter = nullptr;
    int* length = nullptr;
    int* snap = nullptr;
    unsigned* status = nullptr;
};

extern "C" {

const char* eviction_b200_last_error(void) { return g_error.c_str(); }

int eviction_b200_create(const eviction_config_b200* cfg, int device, eviction_handle** out) {
    if (!cfg || !out || cfg->struct_size != sizeof(eviction_config_b200)) return efail(EVICTION_ERR_INVALID_ARG, "eviction_config_b200: NULL or struct_size mismatch");
    if (cfg->block_size <= 0 || cfg->start_size < 0 || cfg->recent_size < 0 || cfg->max_cache_size <= 0 || cfg->start_size % cfg->block_size ||
        cfg->recent_size % cfg->block_size || cfg->max_cache_size % cfg->block_size || cfg->start_size + cfg->recent_size > cfg->max_cache_size)
        return efail(EVICTION_ERR_INVALID_ARG, "sizes must be multiples of block_size and start + recent <= max_cache_size");
    if (cfg->aggregation != EVICTION_AGG_SUM && cfg->aggregation != EVICTION_AGG_NORM_SUM) return efail(EVICTION_ERR_UNSUPPORTED, "only SUM and NORM_SUM run on the device");
    if (cfg->max_pool_window < 1 || cfg->num_layers < 1 || cfg->num_slots < 1 || cfg->max_tracked_tokens < 1 || cfg->max_evicted_blocks < 1 || cfg->snapkv_window_size < 0)
        return efail(EVICTION_ERR_INVALID_ARG, "bad capacity");
    E_CUDA(cudaSetDevice(device));
    eviction_handle* h = new eviction_handle();
    h->device = device;
    h->c = Cfg{cfg->start_size, cfg->recent_size, cfg->max_cache_size, cfg->block_size, cfg->aggregation, cfg->snapkv_window_size, cfg->max_pool_window,
               cfg->num_layers, cfg->num_slots, cfg->max_tracked_tokens, cfg->max_evicted_blocks};
    const size_t recs = (size_t)cfg->num_layers * cfg->num_slots;
    cudaError_t e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->acc, recs * cfg->max_tracked_tokens * sizeof(double));
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->counter, recs * cfg->max_tracked_tokens * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->length, recs * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->snap, recs * sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->length, 0, recs * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->snap, 0, recs * sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 256);
    if (e != cudaSuccess) {
        eviction_b200_destroy(h);
        return efail(EVICTION_ERR_CUDA, std::string("eviction_b200_create: ") + cudaGetErrorString(e));
    }
    *out = h;
    return EVICTION_OK;
}

int eviction_b200_destroy(eviction_handle* h) {
    if (!h) return EVICTION_OK;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    cudaFree(h->acc); cudaFree(h->counter); cudaFree(h->length); cudaFree(h->snap); cudaFree(h->status);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return EVICTION_OK;
}

int eviction_b200_reset_slot(eviction_handle* h, int32_t slot, void* stream) {
    if (!h || slot < 0 || slot >= h->c.slots) return efail(EVICTION_ERR_INVALID_ARG, "NULL handle or slot out of range");
    E_CUDA(cudaSetDevice(h->device));
    reset_slot_kernel<<<(h->c.layers + 127) / 128, 128, 0, stream ? (cudaStream_t)stream : h->stream>>>(h->length, h->snap, h->c.layers, h->c.slots, slot);
    E_CUDA(cudaGetLastError());
    return EVICTION_OK;
}

int eviction_b200_step(eviction_handle* h, const eviction_step_args* a) {
    if (!h || !a || a->struct_size != sizeof(eviction_step_args)) return efail(EVICTION_ERR_INVALID_ARG, "NULL argument or struct_size mismatch");
    if (a->layer < 0 || a->layer >= h->c.layers || a->num_sequences < 0) return efail(EVICTION_ERR_INVALID_ARG, "layer or num_sequences out of range");
    if (a->num_sequences == 0) return EVICTION_OK;
    if (!a->scores || !a->span_begin || !a->span_len || !a->slot || !a->num_snapkv_scores || !a->evicted_count || !a->evicted_blocks)
        return efail(EVICTION_ERR_INVALID_ARG, "NULL pointer");
    E_CUDA(cudaSetDevice(h->device));
    StepArgs k{};
    k.c = h->c; k.layer = a->layer; k.num_sequences = a->num_sequences; k.do_evict = a->do_evict;
    k.scores = a->scores; k.span_begin = reinterpret_cast<const long long*>(a->span_begin); k.span_len = a->span_len; k.slot = a->slot;
    k.num_snapkv = a->num_snapkv_scores; k.evicted_count = a->evicted_count; k.evicted_blocks = a->evicted_blocks;
    k.acc = h->acc; k.counter = h->counter; k.length = h->length; k.snap = h->snap; k.status = h->status;
    // block scores and flags of the evictable blocks
    const size_t blocks = (size_t)(h->c.max_tokens + h->c.start_size) / h->c.bs + 2;
    const size_t smem = blocks * (sizeof(double) + 1) + 16;
    if (smem > 200 * 1024) return efail(EVICTION_ERR_TOO_LARGE, "max_tracked_tokens / block_size too large for one CTA's shared memory");
    E_CUDA(cudaFuncSetAttribute(eviction_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    eviction_step_kernel<<<a->num_sequences, kThreads, smem, a->stream ? (cudaStream_t)a->stream : h->stream>>>(k);
    E_CUDA(cudaGetLastError());
    return EVICTION_OK;
}

int eviction_b200_last_device_status(eviction_handle* h, uint32_t* bits) {
    if (!h || !bits) return efail(EVICTION_ERR_INVALID_ARG, "NULL argument");
    E_CUDA(cudaSetDevice(h->device));
    E_CUDA(cudaDeviceSynchronize());
    E_CUDA(cudaMemcpy(bits, h->status, 4, cudaMemcpyDeviceToHost));
    if (*bits) E_CUDA(cudaMemset(h->status, 0, 4));
    return EVICTION_OK;
}

int eviction_b200_read_slot(eviction_handle* h, int32_t layer, int32_t slot, double* scores, uint32_t* counters, int32_t* length) {
    if (!h || !length || layer < 0 || layer >= h->c.layers || slot < 0 || slot >= h->c.slots) return efail(EVICTION_ERR_INVALID_ARG, "bad argument");
    E_CUDA(cudaSetDevice(h->device));
    E_CUDA(cudaDeviceSynchronize());
    const size_t rec = (size_t)layer * h->c.slots + slot;
    E_CUDA(cudaMemcpy(length, h->length + rec, 4, cudaMemcpyDeviceToHost));
    if (scores) E_CUDA(cudaMemcpy(scores, h->acc + rec * h->c.max_tokens, (size_t)h->c.max_tokens * sizeof(double), cudaMemcpyDeviceToHost));
    if (counters) E_CUDA(cudaMemcpy(counters, h->counter + rec * h->c.max_tokens, (size_t)h->c.max_tokens * sizeof(unsigned), cudaMemcpyDeviceToHost));
    return EVICTION_OK;
}

}  // extern "C"
