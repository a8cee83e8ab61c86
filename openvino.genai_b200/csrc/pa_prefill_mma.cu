// Prefill-chunk attention for the f16 / bf16 caches (head size 64 or 128) on mma.sync m16n8k16.
//
// The u8 cache has its tcgen05 kernel (pa_prefill_tc.cu); the other cache types went through the
// one-warp-per-row CUDA-core kernel (pa_prefill.cu), which reads the whole context once per
// (token, q head) and is two orders of magnitude slower.  This kernel is the tensor-core path for
// them: a CTA of eight warps takes half of a 256-row work item of the plan - rows are (new token, q
// head of one GQA group) pairs of one (sequence, kv head), token-major - and every warp keeps 16 rows.
// The key / value blocks of the context are brought 32 tokens at a time into a double buffer in shared
// memory with 16-byte cp.async (XOR-swizzled rows, read with ldmatrix), once for all eight warps; each
// warp runs S = Q.K^T, the online softmax with its rows' own causal limits, and O += P.V, skipping the
// tiles that lie beyond the limit of all of its rows.  K and V of a chunk are read back from the cache,
// so a chunk sees its own keys at cache precision, as the operator's contract says.
// Tensor-bound in principle: 4 * Hq * D flops per (new token, context token) pair.
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kMmaWarps = 8;
constexpr int kMmaRows = 16 * kMmaWarps;   // rows of a CTA: half of a work item
constexpr int kPTile = 32;                 // context tokens per tile
constexpr float kLog2eM = 1.4426950408889634f;
constexpr float kLn2M = 0.6931471805599453f;
constexpr float kLazyM = 8.f;
static_assert(2 * kMmaRows == kPrefillItemRows, "two CTAs per work item");

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void store_pair_m(void* out, long long idx, int act, float v0, float v1) {
    if (act == PA_DTYPE_F32) *reinterpret_cast<float2*>((float*)out + idx) = make_float2(v0, v1);
    else if (act == PA_DTYPE_F16) *reinterpret_cast<__half2*>((__half*)out + idx) = __floats2half2_rn(v0, v1);
    else *reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)out + idx) = __floats2bfloat162_rn(v0, v1);
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kMmaWarps * 32, 1) prefill_mma_kernel(KernelArgs a) {
    constexpr int NKK = D / 16;    // k-steps of Q.K^T
    constexpr int NDT = D / 8;     // n-tiles of P.V
    constexpr int CPR = D / 8;     // 16-byte chunks of a token row
    constexpr int HALF = kPTile * D * 2;   // bytes of the key (or value) part of a stage
    extern __shared__ __align__(128) uint8_t smem[];   // [2 stages][K | V]
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int Hkv = a.g.Hkv, G = a.g.Hq / Hkv, BS = a.g.bs;

    // ---- the work item of this CTA ---------------------------------------------------------------------
    const int item = blockIdx.x >> 1, half = blockIdx.x & 1;
    const int total = a.plan->total_ptiles;
    if (item >= total * Hkv) return;
    const int qt = item / Hkv, hk = item % Hkv;
    int s;
    {
        int lo = 0, hi = a.num_sequences;   // ptile_prefix[lo] <= qt < ptile_prefix[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (a.ptile_prefix[mid] <= qt) lo = mid; else hi = mid;
        }
        s = lo;
    }
    SeqView sv;
    if (!seq_view(a, s, sv) || sv.n <= 1) return;
    const int pairs = sv.n * G;
    const int first = (qt - a.ptile_prefix[s]) * kPrefillItemRows + half * kMmaRows;   // first (token, head) pair of the CTA
    if (first >= pairs) return;
    const int last = min(first + kMmaRows, pairs) - 1;
    const int cta_ctx = sv.past + last / G + 1;          // keys the CTA's last row sees

    // ---- this warp's rows: g and g + 8 of its 16 ---------------------------------------------------------
    const float sm_scale = (a.scale != 0.f ? a.scale : rsqrtf((float)D)) * kLog2eM;
    int limit[2];          // keys row r sees (0: the row does not exist)
    long long orow[2];     // token * Hq + q head
    float unscale[2];      // f16 operands: the exact power of two a row of large queries was divided by
    uint32_t qa[NKK][4];
    uint32_t qlo[BF16 ? NKK : 1][4];   // bf16 operands: what the rounding of the query to 8 significant bits left over
    bool any_lo = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int pi = first + 16 * warp + g + 8 * r;
        const bool live = pi < pairs;
        const int tok = live ? pi / G : 0, head = live ? pi % G : 0;
        limit[r] = live ? sv.past + tok + 1 : 0;
        orow[r] = (long long)(sv.t0 + tok) * a.g.Hq + hk * G + head;
        float q[NKK][4];
        float amax = 0.f;
#pragma unroll
        for (int ks = 0; ks < NKK; ++ks)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int dd = 16 * ks + 2 * c + (e & 1) + 8 * (e >> 1);
                // f16 operands: Q carries the softmax scale; bf16 operands: the scale is applied to S, so that bf16 queries go in exactly
                q[ks][e] = live ? load_act(a.query, orow[r] * D + dd, a.g.act) * (BF16 ? 1.f : sm_scale) : 0.f;
                amax = fmaxf(amax, fabsf(q[ks][e]));
            }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        float qmul = 1.f;
        if (!BF16 && amax > 32768.f && amax < INFINITY) {   // keep the row inside the f16 range; taken back out of S
            int ex;
            frexpf(amax, &ex);
            qmul = ldexpf(1.f, 15 - ex);
        }
        unscale[r] = BF16 ? sm_scale : 1.f / qmul;
#pragma unroll
        for (int ks = 0; ks < NKK; ++ks) {
            if constexpr (BF16) {
                const uint32_t h0 = pack_bf2(q[ks][0], q[ks][1]), h1 = pack_bf2(q[ks][2], q[ks][3]);
                qa[ks][r] = h0; qa[ks][r + 2] = h1;
                qlo[ks][r] = pack_bf2(q[ks][0] - __uint_as_float(h0 << 16), q[ks][1] - __uint_as_float(h0 & 0xffff0000u));
                qlo[ks][r + 2] = pack_bf2(q[ks][2] - __uint_as_float(h1 << 16), q[ks][3] - __uint_as_float(h1 & 0xffff0000u));
                any_lo |= ((qlo[ks][r] | qlo[ks][r + 2]) & 0x7fff7fffu) != 0u;
            } else {
                qa[ks][r] = pack_h2(q[ks][0] * qmul, q[ks][1] * qmul);
                qa[ks][r + 2] = pack_h2(q[ks][2] * qmul, q[ks][3] * qmul);
            }
        }
    }
    const bool use_lo = BF16 && __any_sync(0xffffffffu, any_lo);   // f32 / f16 queries with a bf16 cache
    int wmax = max(limit[0], limit[1]);   // keys the warp's last row sees
#pragma unroll
    for (int o = 16; o; o >>= 1) wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, o));

    float oacc[NDT][4];
#pragma unroll
    for (int i = 0; i < NDT; ++i) { oacc[i][0] = 0.f; oacc[i][1] = 0.f; oacc[i][2] = 0.f; oacc[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    // ---- loader: tile k of the context into stage k & 1, all threads ----------------------------------------
    const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)hk * a.g.head_bytes;
    const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)hk * a.g.head_bytes;
    bool bad_index = false;
    auto load_tile = [&](int k) {
        uint8_t* st = smem + (k & 1) * 2 * HALF;
        for (int i = tid; i < kPTile * CPR; i += kMmaWarps * 32) {
            const int row = i / CPR, ch = i % CPR;
            const int tok = k * kPTile + row;
            if (tok < cta_ctx) {
                const int bi = tok / BS;
                int blk = bi < sv.nb ? a.block_indices[sv.tb + bi] : 0;
                if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                const long long off = (long long)blk * a.g.block_bytes + ((long long)(tok % BS) * D + 8 * ch) * 2;
                const int dst = row * (2 * D) + ((ch ^ (row & 7)) << 4);
                cp_async16(st + dst, kc + off);
                cp_async16(st + HALF + dst, vc + off);
            } else {   // beyond the context: zeros (a stale value row could hold NaN bit patterns)
                const int dst = row * (2 * D) + ((ch ^ (row & 7)) << 4);
                *reinterpret_cast<uint4*>(st + dst) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(st + HALF + dst) = make_uint4(0, 0, 0, 0);
            }
        }
        cp_async_commit();
    };

    const int ntiles = (cta_ctx + kPTile - 1) / kPTile;
    load_tile(0);
    for (int k = 0; k < ntiles; ++k) {
        if (k + 1 < ntiles) load_tile(k + 1);
        else cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint8_t* st = smem + (k & 1) * 2 * HALF;
        const int tok0 = k * kPTile;
        if (tok0 < wmax) {   // some row of this warp sees keys of the tile
            // ---- S = Q.K^T over four 8-token n-tiles -----------------------------------------------------------------
            float sacc[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                sacc[j][0] = 0.f; sacc[j][1] = 0.f; sacc[j][2] = 0.f; sacc[j][3] = 0.f;
#pragma unroll
                for (int p = 0; p < NKK / 2; ++p) {
                    const int row = 8 * j + (lane & 7), ch = 4 * p + (lane >> 3);
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(st + row * 2 * D + ((ch ^ (row & 7)) << 4)));
                    mma16816<BF16, true>(sacc[j], qa[2 * p], b[0], b[1]);
                    mma16816<BF16, true>(sacc[j], qa[2 * p + 1], b[2], b[3]);
                    if constexpr (BF16) {
                        if (use_lo) {
                            mma16816<BF16, true>(sacc[j], qlo[2 * p], b[0], b[1]);
                            mma16816<BF16, true>(sacc[j], qlo[2 * p + 1], b[2], b[3]);
                        }
                    }
                }
            }
            // ---- causal mask, online softmax ------------------------------------------------------------------
            float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int pos = tok0 + 8 * j + 2 * c + e;
                        const float v = pos < limit[r] ? sacc[j][2 * r + e] * unscale[r] : -INFINITY;
                        sacc[j][2 * r + e] = v;
                        tmax[r] = fmaxf(tmax[r], v);
                    }
            bool grow = false;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
                tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
                grow |= tmax[r] > m_run[r] + kLazyM;
            }
            if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    const float m_new = fmaxf(m_run[r], tmax[r]);
                    const float alpha = m_new == -INFINITY ? 1.f : ex2(m_run[r] - m_new);   // 0 on the first tile with a visible key
                    m_run[r] = m_new;
                    l_run[r] *= alpha;
#pragma unroll
                    for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] *= alpha; oacc[i][2 * r + 1] *= alpha; }
                }
            }
            // P as the A operand of the second product.  bf16 has 8 significant bits: there P goes in as two pieces
            // (rounded value and remainder), so that the kernel's own error stays below that of the cache's values.
            uint32_t pa_frag[2][4], pa_low[2][4];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float mref = m_run[r] == -INFINITY ? 0.f : m_run[r];   // a row that has seen no key yet: every p is 0
                float lsum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = ex2(sacc[j][2 * r] - mref), p1 = ex2(sacc[j][2 * r + 1] - mref);
                    lsum += p0 + p1;
                    if constexpr (BF16) {
                        const uint32_t hi = pack_bf2(p0, p1);
                        pa_frag[j >> 1][r + 2 * (j & 1)] = hi;
                        pa_low[j >> 1][r + 2 * (j & 1)] = pack_bf2(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
                    } else {
                        pa_frag[j >> 1][r + 2 * (j & 1)] = pack_h2(p0, p1);
                    }
                }
                l_run[r] += lsum;
            }
            // ---- O += P.V ---------------------------------------------------------------------------------------
#pragma unroll
            for (int kt = 0; kt < 2; ++kt)
#pragma unroll
                for (int q = 0; q < NDT / 2; ++q) {
                    const int row = 16 * kt + 8 * ((lane >> 3) & 1) + (lane & 7), ch = 2 * q + (lane >> 4);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(st + HALF + row * 2 * D + ((ch ^ (row & 7)) << 4)));
                    mma16816<BF16, true>(oacc[2 * q], pa_frag[kt], b[0], b[1]);
                    mma16816<BF16, true>(oacc[2 * q + 1], pa_frag[kt], b[2], b[3]);
                    if constexpr (BF16) {
                        mma16816<BF16, true>(oacc[2 * q], pa_low[kt], b[0], b[1]);
                        mma16816<BF16, true>(oacc[2 * q + 1], pa_low[kt], b[2], b[3]);
                    }
                }
        }
        __syncthreads();   // every warp is done with the stage before it is refilled
    }
    cp_async_wait<0>();

    // ---- normalise and write --------------------------------------------------------------------------------
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = l_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (limit[r] == 0) continue;
        const float inv = 1.f / l;
#pragma unroll
        for (int i = 0; i < NDT; ++i) store_pair_m(a.output, orow[r] * D + 8 * i + 2 * c, a.g.act, oacc[i][2 * r] * inv, oacc[i][2 * r + 1] * inv);
        if (c == 0 && a.lse) a.lse[orow[r]] = (m_run[r] + log2f(l)) * kLn2M;
    }
    if (__any_sync(0xffffffffu, bad_index) && lane == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
}

template <int D, bool BF16>
cudaError_t launch_mma_t(const KernelArgs& a, cudaStream_t stream, long long max_items) {
    constexpr int smem = 2 * 2 * kPTile * D * 2;
    static bool set = false;
    if (!set) {
        const cudaError_t e = cudaFuncSetAttribute(prefill_mma_kernel<D, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        set = true;
    }
    prefill_mma_kernel<D, BF16><<<(unsigned)(2 * max_items), kMmaWarps * 32, smem, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

bool prefill_mma_supported(const CacheGeom& g) {
    return (g.cache == PA_DTYPE_F16 || g.cache == PA_DTYPE_BF16) && (g.D == 64 || g.D == 128) && (g.bs == 16 || g.bs == 32);
}

cudaError_t launch_prefill_mma(const KernelArgs& a, cudaStream_t stream, long long max_items, int* launches) {
    if (a.num_tokens <= 0 || max_items <= 0) return cudaSuccess;
    cudaError_t e;
    const bool bf = a.g.cache == PA_DTYPE_BF16;
    if (a.g.D == 128) e = bf ? launch_mma_t<128, true>(a, stream, max_items) : launch_mma_t<128, false>(a, stream, max_items);
    else e = bf ? launch_mma_t<64, true>(a, stream, max_items) : launch_mma_t<64, false>(a, stream, max_items);
    if (e == cudaSuccess) ++*launches;
    return e;
}

}  // namespace pa
