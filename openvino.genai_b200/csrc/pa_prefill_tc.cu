// Prefill-chunk attention on the 5th-generation tensor cores (tcgen05 + TMEM) for the u8 cache,
// head size 128.
//
// One CTA (128 threads) owns a q tile of 128 rows = (new token, q head of one GQA group) pairs of
// one (sequence, kv head), so a K/V byte is read once for the whole group.  Per 64-token KV tile:
//   1. lane 0 of the CTA has the TMA engine copy the tile's (block, head) records (u8 data +
//      per-token scale / zero-point) into a raw staging buffer (bulk copy, mbarrier completion);
//   2. all threads turn the bytes into f16 (byte | 0x6400 = 1024 + byte, the offset is removed
//      algebraically with the zero-point) and write them into 128-byte-swizzled operand tiles:
//      K as [64 tokens][128 dims] (K-major B operand), V^T as [128 dims][64 tokens] (the cache keeps
//      value bytes token-minor, so V^T is K-major for P.V as well);
//   3. one thread issues tcgen05.mma: S[128 x 64] = Q.K^T into TMEM, commit -> mbarrier;
//   4. thread r reads row r of S from TMEM (tcgen05.ld 32x32b), applies per-token scale,
//      zero-point, causal mask and the online softmax, and stores P' = P * v_scale as f16 into a
//      swizzled A-operand tile;
//   5. one thread issues tcgen05.mma: PV[128 x 128] = P'.V into TMEM; every thread folds its row of
//      PV into register accumulators (O = O * alpha + PV), so TMEM is never read-modify-written.
// Tensor-bound for long contexts: 4 * Hq * D flops per (new token, context token) pair.
#include <algorithm>

#include "pa_common.cuh"
#include "pa_kernels.h"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kRows = 128;     // q-tile rows = UMMA M
constexpr int kD = 128;        // head size
constexpr int kKv = 64;        // context tokens per KV tile = UMMA N of Q.K^T
constexpr int kTmemCols = 256; // S: columns [0, 64), PV: columns [64, 192)
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLn2P = 0.6931471805599453f;

template <int BS>
struct PrefillSmem {
    static constexpr int REC = BS * (kD + 8);
    static constexpr int NREC = kKv / BS;
    alignas(1024) uint8_t q[kRows * kD * 2];       // 2 swizzle atoms of [128 rows][64 dims]
    alignas(1024) uint8_t k[kKv * kD * 2];         // 2 atoms of [64 tokens][64 dims]
    alignas(1024) uint8_t vt[kD * kKv * 2];        // 1 atom of [128 dims][64 tokens]
    alignas(1024) uint8_t p[kRows * kKv * 2];      // 1 atom of [128 rows][64 tokens]
    alignas(128) uint8_t raw_k[NREC * REC];        // staged key records
    alignas(128) uint8_t raw_v[NREC * REC];        // staged value records
    alignas(16) float k_scale[kKv];
    alignas(16) float k_zp[kKv];
    alignas(16) float v_scale[kKv];
    alignas(16) float v_zp[kKv];
    alignas(8) uint64_t bar_raw;
    alignas(8) uint64_t bar_s;
    alignas(8) uint64_t bar_o;
    uint32_t tmem_base;
    int failed;
};

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int BS>
__global__ void __launch_bounds__(kRows, 2) prefill_tc_kernel(KernelArgs a) {
    using Smem = PrefillSmem<BS>;
    extern __shared__ uint8_t smem_raw_[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw_) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5;
    const int G = a.g.Hq / a.g.Hkv;
    const int Hkv = a.g.Hkv;
    const int total_items = a.plan->total_ptiles * Hkv;
    const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)kD);

    if (tid == 0) {
        mbar_init(&sm.bar_raw, 1);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_fence_init();
        sm.failed = 0;
    }
    if (warp == 0) tc05::tmem_alloc(&sm.tmem_base, kTmemCols);
    tc05::fence_before_thread_sync();
    __syncthreads();
    tc05::fence_after_thread_sync();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + kKv;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;   // this warp's TMEM lanes

    constexpr uint32_t idesc_s = tc05::instr_desc_f16(kRows, kKv, 0, 0, 0);   // f16, A and B K-major
    constexpr uint32_t idesc_o = tc05::instr_desc_f16(kRows, kD, 0, 0, 0);
    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), vt_addr = smem_u32(sm.vt), p_addr = smem_u32(sm.p);

    uint32_t phase_raw = 0, phase_s = 0, phase_o = 0;
    bool bad_index = false;

    for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
        // ---- which q tile -------------------------------------------------------------------------
        const int gq = item / Hkv, hk = item % Hkv;
        int lo = 0, hi = a.num_sequences;  // ptile_prefix[lo] <= gq < ptile_prefix[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (__ldcg(a.ptile_prefix + mid) <= gq) lo = mid; else hi = mid;
        }
        const int s = lo;
        const int p0 = __ldcg(a.ptile_prefix + s), ntile_s = __ldcg(a.ptile_prefix + s + 1) - p0;
        const int qt = ntile_s - 1 - (gq - p0);           // heavy (late) tiles first
        const int t0 = a.subsequence_begins[s];
        const int n_new = a.subsequence_begins[s + 1] - t0;
        const int past = a.past_lens[s];
        const int tb = a.block_indices_begins[s];
        const int32_t* table = a.block_indices + tb;

        // ---- this thread's row ---------------------------------------------------------------------
        const int flat = qt * kRows + tid;
        const int tok = flat / G, hq = hk * G + flat % G;
        const bool row_live = tok < n_new;
        const int tok_lo = (qt * kRows) / G;
        const int tok_hi = min(n_new - 1, (qt * kRows + kRows - 1) / G);
        const int ctx_hi = past + tok_hi + 1;             // context the last row of the tile sees
        const int ntiles = (ctx_hi + kKv - 1) / kKv;
        const int my_ctx = row_live ? past + tok + 1 : ctx_hi;

        // ---- Q -> f16 swizzled A operand; sum of the row for the zero-point term ------------------
        float qsum = 0.f, qscale;
        {
            const long long qoff = ((long long)(t0 + (row_live ? tok : 0)) * a.g.Hq + hq) * kD;
            float amax = 0.f;
            for (int c = 0; c < kD / 8; ++c) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) { v[e] = row_live ? load_act(a.query, qoff + 8 * c + e, a.g.act) : 0.f; amax = fmaxf(amax, fabsf(v[e])); }
                uint4 w;
                w.x = pack_h2(v[0], v[1]); w.y = pack_h2(v[2], v[3]); w.z = pack_h2(v[4], v[5]); w.w = pack_h2(v[6], v[7]);
                const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e) qsum += __low2float(h[e]) + __high2float(h[e]);
                *reinterpret_cast<uint4*>(sm.q + (c / 8) * (kRows * 128) + sw128(tid, c % 8)) = w;
            }
            (void)amax;  // no power-of-two prescale here: |q| is assumed to stay inside the f16 range
            qscale = sm_scale * kLog2eP;
        }

        float o[kD];
#pragma unroll
        for (int d = 0; d < kD; ++d) o[d] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, z_run = 0.f;

        auto issue_raw = [&](int j) {   // thread 0: TMA-engine copies of tile j's records
            uint32_t bytes = 0;
            int blocks[Smem::NREC];
#pragma unroll
            for (int r = 0; r < Smem::NREC; ++r) {
                const int bi = j * Smem::NREC + r;
                int blk = -1;
                if (bi * BS < ctx_hi) {
                    blk = table[bi];
                    if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                    bytes += 2 * Smem::REC;
                }
                blocks[r] = blk;
            }
            mbar_expect_tx(&sm.bar_raw, bytes);
            const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)hk * a.g.head_bytes;
            const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)hk * a.g.head_bytes;
#pragma unroll
            for (int r = 0; r < Smem::NREC; ++r)
                if (blocks[r] >= 0) {
                    bulk_g2s(sm.raw_k + r * Smem::REC, kc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.bar_raw);
                    bulk_g2s(sm.raw_v + r * Smem::REC, vc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.bar_raw);
                }
        };

        __syncthreads();                 // Q tile written; previous item's operand buffers are free
        if (tid == 0) issue_raw(0);

        // A wait that runs out sets `failed`; the flag is made uniform at the next block barrier so
        // that every thread leaves the loop at the same place.
        bool failed = false;
        for (int j = 0; j < ntiles; ++j) {
            // ---- 1-2. raw records -> f16 operand tiles -------------------------------------------
            if (!failed && !mbar_wait_bounded(&sm.bar_raw, phase_raw)) { failed = true; }
            phase_raw ^= 1;
            const int live_tokens = min(kKv, ctx_hi - j * kKv);
            if (!failed) {
                // K: unit u = 16 dims of one token
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int u = tid + kRows * i;
                    const int token = u >> 3, seg = u & 7;
                    uint4 lo4 = make_uint4(0x64006400u, 0x64006400u, 0x64006400u, 0x64006400u), hi4 = lo4;  // 1024.0: cancels with the offset term
                    if (token < live_tokens) {
                        const uint4 w = *reinterpret_cast<const uint4*>(sm.raw_k + (token / BS) * Smem::REC + (token % BS) * kD + 16 * seg);
                        lo4.x = __byte_perm(w.x, 0x64646464u, 0x4140); lo4.y = __byte_perm(w.x, 0x64646464u, 0x4342);
                        lo4.z = __byte_perm(w.y, 0x64646464u, 0x4140); lo4.w = __byte_perm(w.y, 0x64646464u, 0x4342);
                        hi4.x = __byte_perm(w.z, 0x64646464u, 0x4140); hi4.y = __byte_perm(w.z, 0x64646464u, 0x4342);
                        hi4.z = __byte_perm(w.w, 0x64646464u, 0x4140); hi4.w = __byte_perm(w.w, 0x64646464u, 0x4342);
                    }
                    uint8_t* atom = sm.k + (seg >> 2) * (kKv * 128);
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg) & 7)) = lo4;
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg + 1) & 7)) = hi4;
                }
                // V^T: thread = dim row, 64 token bytes from the tile's records
                {
                    const int d = tid;
#pragma unroll
                    for (int r = 0; r < Smem::NREC; ++r) {
#pragma unroll
                        for (int q16 = 0; q16 < BS / 16; ++q16) {
                            const int tbase = r * BS + 16 * q16;   // first of 16 tokens
                            uint4 lo4 = make_uint4(0x64006400u, 0x64006400u, 0x64006400u, 0x64006400u), hi4 = lo4;
                            if (tbase < live_tokens) {
                                const uint4 w = *reinterpret_cast<const uint4*>(sm.raw_v + r * Smem::REC + d * BS + 16 * q16);
                                lo4.x = __byte_perm(w.x, 0x64646464u, 0x4140); lo4.y = __byte_perm(w.x, 0x64646464u, 0x4342);
                                lo4.z = __byte_perm(w.y, 0x64646464u, 0x4140); lo4.w = __byte_perm(w.y, 0x64646464u, 0x4342);
                                hi4.x = __byte_perm(w.z, 0x64646464u, 0x4140); hi4.y = __byte_perm(w.z, 0x64646464u, 0x4342);
                                hi4.z = __byte_perm(w.w, 0x64646464u, 0x4140); hi4.w = __byte_perm(w.w, 0x64646464u, 0x4342);
                            }
                            *reinterpret_cast<uint4*>(sm.vt + sw128(d, (tbase >> 3))) = lo4;
                            *reinterpret_cast<uint4*>(sm.vt + sw128(d, (tbase >> 3) + 1)) = hi4;
                        }
                    }
                }
                // per-token parameters outlive the raw buffer
                if (tid < kKv) {
                    const int token = tid;
                    const bool ok = token < live_tokens;
                    const float* kp = reinterpret_cast<const float*>(sm.raw_k + (token / BS) * Smem::REC + BS * kD);
                    const float* vp = reinterpret_cast<const float*>(sm.raw_v + (token / BS) * Smem::REC + BS * kD);
                    sm.k_scale[token] = ok ? kp[token % BS] : 0.f;
                    sm.k_zp[token] = ok ? kp[BS + token % BS] + 1024.f : 0.f;
                    sm.v_scale[token] = ok ? vp[token % BS] : 0.f;
                    sm.v_zp[token] = ok ? vp[BS + token % BS] + 1024.f : 0.f;
                }
            }
            tc05::fence_proxy_async_smem();
            tc05::fence_before_thread_sync();
            failed = __syncthreads_or(failed ? 1 : 0) != 0;
            if (failed) break;
            // ---- 3. S = Q.K^T ------------------------------------------------------------------------
            if (tid == 0) {
                tc05::fence_after_thread_sync();
                if (j + 1 < ntiles) issue_raw(j + 1);   // the raw buffers are free again
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint64_t da = tc05::smem_desc_sw128(q_addr + (kk >> 2) * (kRows * 128) + (kk & 3) * 32, 1024);
                    const uint64_t db = tc05::smem_desc_sw128(k_addr + (kk >> 2) * (kKv * 128) + (kk & 3) * 32, 1024);
                    tc05::mma_ss(tmem_s, da, db, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc05::commit(&sm.bar_s);
            }
            if (!mbar_wait_bounded(&sm.bar_s, phase_s)) failed = true;
            phase_s ^= 1;
            tc05::fence_after_thread_sync();

            // ---- 4. softmax of this thread's row ------------------------------------------------------
            float alpha = 1.f;
            if (!failed) {
                uint32_t sreg[2][32];
                tc05::ld_32x32b_x32(tmem_s + lane_base, sreg[0]);
                tc05::ld_32x32b_x32(tmem_s + lane_base + 32, sreg[1]);
                tc05::wait_ld();
                float sv[kKv];
                float mx = -INFINITY;
                const int col0 = j * kKv;
#pragma unroll
                for (int c = 0; c < kKv; ++c) {
                    const float raw = __uint_as_float(sreg[c >> 5][c & 31]);
                    float v = (raw - sm.k_zp[c] * qsum) * (sm.k_scale[c] * qscale);
                    v = (col0 + c < my_ctx) ? v : -INFINITY;
                    sv[c] = v;
                    mx = fmaxf(mx, v);
                }
                const float m_new = fmaxf(m_run, mx);      // finite: column 0 of every tile is visible to every row
                alpha = ex2(m_run - m_new);
                m_run = m_new;
                float lsum = 0.f, zsum = 0.f;
#pragma unroll
                for (int c = 0; c < kKv; c += 8) {
                    uint32_t packed[4];
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float p0 = ex2(sv[c + e] - m_new), p1 = ex2(sv[c + e + 1] - m_new);
                        lsum += p0 + p1;
                        const uint32_t pk = pack_h2(p0 * sm.v_scale[c + e], p1 * sm.v_scale[c + e + 1]);
                        const __half2 h = *reinterpret_cast<const __half2*>(&pk);
                        zsum += __low2float(h) * sm.v_zp[c + e] + __high2float(h) * sm.v_zp[c + e + 1];
                        packed[e >> 1] = pk;
                    }
                    *reinterpret_cast<uint4*>(sm.p + sw128(tid, c >> 3)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
                l_run = l_run * alpha + lsum;
                z_run = z_run * alpha + zsum;
            }
            tc05::fence_proxy_async_smem();
            tc05::fence_before_thread_sync();
            failed = __syncthreads_or(failed ? 1 : 0) != 0;
            if (failed) break;
            // ---- 5. PV = P'.V, folded into the register accumulators ------------------------------------
            if (tid == 0) {
                tc05::fence_after_thread_sync();
#pragma unroll
                for (int kk = 0; kk < kKv / 16; ++kk) {
                    const uint64_t da = tc05::smem_desc_sw128(p_addr + kk * 32, 1024);
                    const uint64_t db = tc05::smem_desc_sw128(vt_addr + kk * 32, 1024);
                    tc05::mma_ss(tmem_o, da, db, idesc_o, kk > 0 ? 1u : 0u);
                }
                tc05::commit(&sm.bar_o);
            }
            if (!mbar_wait_bounded(&sm.bar_o, phase_o)) failed = true;
            phase_o ^= 1;
            tc05::fence_after_thread_sync();
            if (!failed) {
#pragma unroll
                for (int q4 = 0; q4 < kD / 32; ++q4) {
                    uint32_t oreg[32];
                    tc05::ld_32x32b_x32(tmem_o + lane_base + 32 * q4, oreg);
                    tc05::wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[32 * q4 + c] = o[32 * q4 + c] * alpha + __uint_as_float(oreg[c]);
                }
            }
            tc05::fence_before_thread_sync();
        }
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        if (failed) {
            if (tid == 0) { atomicOr(a.status, 0x40000000u); sm.failed = 1; }
            break;
        }
        // ---- epilogue: out = (O - z) / l -----------------------------------------------------------
        if (row_live) {
            const float inv = 1.f / l_run;
            const long long ooff = ((long long)(t0 + tok) * a.g.Hq + hq) * kD;
            for (int d = 0; d < kD; ++d) store_act(a.output, ooff + d, a.g.act, (o[d] - z_run) * inv);
            if (a.lse) a.lse[(long long)(t0 + tok) * a.g.Hq + hq] = (m_run + log2f(l_run)) * kLn2P;
        }
        (void)tok_lo;
    }
    if (__syncthreads_or(bad_index ? 1 : 0) && tid == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
    tc05::fence_before_thread_sync();
    __syncthreads();
    if (warp == 0) tc05::tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool prefill_tc_supported(const CacheGeom& g) {
    return g.cache == PA_DTYPE_U8 && g.D == kD && (g.bs == 32 || g.bs == 16) && g.Hq % g.Hkv == 0;
}

cudaError_t launch_prefill_tc(const KernelArgs& a, cudaStream_t stream, int sm_count, long long max_items, int* launches) {
    if (max_items <= 0) return cudaSuccess;
    const int grid = (int)std::min<long long>(max_items, 2LL * sm_count);
    cudaError_t e;
    if (a.g.bs == 32) {
        const int bytes = (int)sizeof(PrefillSmem<32>) + 1024;
        e = cudaFuncSetAttribute(prefill_tc_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        prefill_tc_kernel<32><<<grid, kRows, bytes, stream>>>(a);
    } else {
        const int bytes = (int)sizeof(PrefillSmem<16>) + 1024;
        e = cudaFuncSetAttribute(prefill_tc_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return e;
        prefill_tc_kernel<16><<<grid, kRows, bytes, stream>>>(a);
    }
    ++*launches;
    return cudaGetLastError();
}

}  // namespace pa
