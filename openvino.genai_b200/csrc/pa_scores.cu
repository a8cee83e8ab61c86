// SnapKV-style score output of the PagedAttention operator.
//
// scores[off_s + pos] = sum over q heads h and over the last W rows j of sequence s's chunk of
//                       exp(scale * q[j,h].k[pos] - lse[j,h])          (pos <= past + j)
// where lse is the log-sum-exp the attention kernels exported for every (token, q head).
// The sum is taken in a fixed order (kv head, then q head inside the group, then row) so the
// f32 result does not depend on scheduling: block selection downstream compares these values
// (src/cpp/src/continuous_batching/cache/cache_eviction.cpp:486-519).
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

// Builds the per-sequence offsets into `scores` (prefix sum of past_len + new tokens) with one warp.
__global__ void score_offsets_kernel(KernelArgs a) {
    long long run = 0;
    const int lane = threadIdx.x;
    for (int base = 0; base < a.num_sequences; base += 32) {
        const int s = base + lane;
        long long len = 0;
        if (s < a.num_sequences) len = (long long)max(a.past_lens[s], 0) + max(a.subsequence_begins[s + 1] - a.subsequence_begins[s], 0);
        long long incl = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            long long v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (s < a.num_sequences) a.score_offsets[s] = run + incl - len;
        run += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) a.score_offsets[a.num_sequences] = run;
}

// One warp per (sequence, context position); lane l owns dims {l + 32*i}.
template <int D>
__global__ void __launch_bounds__(256) scores_kernel(KernelArgs a) {
    constexpr int PER = D / 32;
    const int s = blockIdx.y;
    const int t0 = a.subsequence_begins[s];
    const int n = a.subsequence_begins[s + 1] - t0;
    const int past = a.past_lens[s];
    if (n <= 0 || past < 0) return;
    const int ctx = past + n;
    const int W = min(max(a.score_aggregation_window[s], 0), n);
    const int tb = a.block_indices_begins[s];
    const int nb = a.block_indices_begins[s + 1] - tb;
    const int lane = threadIdx.x & 31;
    const int G = a.g.Hq / a.g.Hkv;
    const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)D);
    float* out = a.scores + a.score_offsets[s];
    for (int pos = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); pos < ctx; pos += gridDim.x * (blockDim.x >> 5)) {
        float total = 0.f;
        if (W > 0 && pos / a.g.bs < nb) {
            int block = a.block_indices[tb + pos / a.g.bs];
            if (block < 0 || block >= a.num_blocks) block = 0;  // flagged by the attention kernel
            const int slot = pos % a.g.bs;
            for (int hk = 0; hk < a.g.Hkv; ++hk) {
                const uint8_t* rec = (const uint8_t*)a.key_cache + (long long)block * a.g.block_bytes + (long long)hk * a.g.head_bytes;
                float k[PER];
                if (a.g.cache == PA_DTYPE_U8) {
                    const float* params = (const float*)(rec + (long long)a.g.bs * D);
                    const float sc = params[slot], zp = params[a.g.bs + slot];
#pragma unroll
                    for (int i = 0; i < PER; ++i) k[i] = dequant_one(rec[(long long)slot * D + lane + 32 * i], sc, zp);
                } else {
                    const uint16_t* p = (const uint16_t*)rec + (long long)slot * D;
#pragma unroll
                    for (int i = 0; i < PER; ++i)
                        k[i] = a.g.cache == PA_DTYPE_F16 ? __half2float(__ushort_as_half(p[lane + 32 * i]))
                                                         : __bfloat162float(__ushort_as_bfloat16(p[lane + 32 * i]));
                }
                for (int hq = hk * G; hq < (hk + 1) * G; ++hq)
                    for (int j = max(n - W, pos - past); j < n; ++j) {  // rows that can see `pos`
                        const long long row = (long long)(t0 + j) * a.g.Hq + hq;
                        float dot = 0.f;
#pragma unroll
                        for (int i = 0; i < PER; ++i) dot += load_act(a.query, row * D + lane + 32 * i, a.g.act) * k[i];
                        dot = warp_sum(dot);
                        total += __expf(dot * sm_scale - a.lse[row]);
                    }
            }
        }
        if (lane == 0) out[pos] = total;
    }
}

}  // namespace

cudaError_t launch_scores(const KernelArgs& a, cudaStream_t stream, int* launches) {
    if (!a.scores || !a.score_aggregation_window || a.num_sequences <= 0) return cudaSuccess;
    score_offsets_kernel<<<1, 32, 0, stream>>>(a);
    ++*launches;
    const int per_block = 8;
    int gx = (a.max_context_len + per_block - 1) / per_block;
    gx = max(1, min(gx, 2048));
    dim3 grid(gx, a.num_sequences);
    if (a.g.D == 128) scores_kernel<128><<<grid, 256, 0, stream>>>(a);
    else scores_kernel<64><<<grid, 256, 0, stream>>>(a);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace pa
