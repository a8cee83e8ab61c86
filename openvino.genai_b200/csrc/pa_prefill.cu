// Prefill-chunk attention (rows with more than one new token) of the PagedAttention operator.
//
// Generic CUDA-core kernel: one warp per (new token, q head), lane l owns dims {l + 32*i},
// online softmax over the causal context read back from the paged cache.  It is the
// any-shape fallback and the cross-check for the tensor-core chunk kernel.
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

__device__ __forceinline__ int find_sequence(const int32_t* begins, int num_seq, int t) {
    int lo = 0, hi = num_seq;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (begins[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

template <int D>
__global__ void __launch_bounds__(256) prefill_generic_kernel(KernelArgs a) {
    constexpr int PER = D / 32;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (long long)a.num_tokens * a.g.Hq) return;
    const int t = (int)(warp / a.g.Hq), hq = (int)(warp % a.g.Hq);
    const int s = find_sequence(a.subsequence_begins, a.num_sequences, t);
    SeqView sv;
    if (!seq_view(a, s, sv)) return;
    const int t0 = sv.t0, n = sv.n, past = sv.past, tb = sv.tb;
    if (n <= 1 || t < t0 || t >= t0 + n) return;  // decode rows are handled by the split-K kernel
    const int visible = past + (t - t0) + 1;
    const int hk = hq / (a.g.Hq / a.g.Hkv);
    const float sm_scale = (a.scale != 0.f ? a.scale : rsqrtf((float)D)) * 1.4426950408889634f;
    float q[PER], acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        q[i] = load_act(a.query, ((long long)t * a.g.Hq + hq) * D + lane + 32 * i, a.g.act);
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int pos = 0; pos < visible; ++pos) {
        int block = a.block_indices[tb + pos / a.g.bs];
        if (block < 0 || block >= a.num_blocks) {
            if (lane == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
            block = 0;
        }
        const int slot = pos % a.g.bs;
        const long long off = (long long)block * a.g.block_bytes + (long long)hk * a.g.head_bytes;
        const uint8_t* kr = (const uint8_t*)a.key_cache + off;
        const uint8_t* vr = (const uint8_t*)a.value_cache + off;
        float k[PER], v[PER];
        if (a.g.cache == PA_DTYPE_U8) {
            const float* kp = (const float*)(kr + (long long)a.g.bs * D);
            const float* vp = (const float*)(vr + (long long)a.g.bs * D);
            const float ks = kp[slot], kz = kp[a.g.bs + slot], vs = vp[slot], vz = vp[a.g.bs + slot];
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                k[i] = dequant_one(kr[(long long)slot * D + d], ks, kz);
                v[i] = dequant_one(vr[(long long)d * a.g.bs + slot], vs, vz);
            }
        } else {
            const uint16_t* kp = (const uint16_t*)kr + (long long)slot * D;
            const uint16_t* vp = (const uint16_t*)vr + (long long)slot * D;
#pragma unroll
            for (int i = 0; i < PER; ++i) {
                const int d = lane + 32 * i;
                if (a.g.cache == PA_DTYPE_F16) {
                    k[i] = __half2float(__ushort_as_half(kp[d]));
                    v[i] = __half2float(__ushort_as_half(vp[d]));
                } else {
                    k[i] = __bfloat162float(__ushort_as_bfloat16(kp[d]));
                    v[i] = __bfloat162float(__ushort_as_bfloat16(vp[d]));
                }
            }
        }
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) dot += q[i] * k[i];
        dot = warp_sum(dot) * sm_scale;
        const float m_new = fmaxf(m, dot);
        const float alpha = exp2f(m - m_new), p = exp2f(dot - m_new);
        l = l * alpha + p;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] = acc[i] * alpha + p * v[i];
        m = m_new;
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) store_act(a.output, ((long long)t * a.g.Hq + hq) * D + lane + 32 * i, a.g.act, acc[i] / l);
    if (lane == 0 && a.lse) a.lse[(long long)t * a.g.Hq + hq] = (m + log2f(l)) * 0.6931471805599453f;
}

}  // namespace

cudaError_t launch_prefill(const KernelArgs& a, cudaStream_t stream, int* launches) {
    if (a.num_tokens <= 0) return cudaSuccess;
    const long long warps = (long long)a.num_tokens * a.g.Hq;
    const int grid = (int)((warps * 32 + 255) / 256);
    if (a.g.D == 128) prefill_generic_kernel<128><<<grid, 256, 0, stream>>>(a);
    else prefill_generic_kernel<64><<<grid, 256, 0, stream>>>(a);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace pa
