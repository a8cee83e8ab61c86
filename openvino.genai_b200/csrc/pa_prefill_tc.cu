// Prefill-chunk attention on the 5th-generation tensor cores (tcgen05 + TMEM) for the u8 cache,
// head size 128.
//
// One CTA (128 threads) owns a q tile of 128 rows = (new token, q head of one GQA group) pairs of
// one (sequence, kv head), so a K/V byte is read once for the whole group.  Per 64-token KV tile:
//   1. one thread has the TMA engine copy the tile's (block, head) records (u8 data + per-token
//      scale / zero-point) into a raw staging buffer (bulk copy, mbarrier completion);
//   2. all threads turn the bytes into f16 (byte | 0x6400 = 1024 + byte) and write them into
//      128-byte-swizzled operand tiles: K as [64 tokens][128 dims] (K-major B operand), V^T as
//      [128 dims][64 tokens] (the cache keeps value bytes token-minor, so V^T is K-major for P.V too);
//   3. one thread issues tcgen05.mma: S[128 x 64] = Q.K^T into TMEM, commit -> mbarrier;
//   4. thread r reads row r of S from TMEM (tcgen05.ld 32x32b), applies the per-token scale, the
//      causal mask (diagonal tiles only) and the online softmax, and stores P' = P * v_scale as f16
//      into a swizzled A-operand tile;
//   5. one thread issues tcgen05.mma: O[128 x 144] += P'.V in TMEM; it runs while the CTA converts
//      the next tile's keys.
// The zero-points ride on the tensor core: Q and K carry 16 extra dims holding the row's sum of q
// and minus (1024 + k zero-point), split into f16 pieces, so S comes out with the offset term
// already subtracted; V^T carries 16 extra rows holding 1024 + v zero-point, whose P'.V columns
// are subtracted from O in the epilogue.  The running maximum is lazy: O in TMEM is rescaled only
// when a row's maximum grows by more than 2^4, so most tiles never touch the accumulator.
// Tensor-bound for long contexts: 4 * Hq * D flops per (new token, context token) pair.
#include <algorithm>

#include "pa_common.cuh"
#include "pa_kernels.h"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kRows = 128;     // q-tile rows = UMMA M
constexpr int kD = 128;        // head size
constexpr int kDx = 16;        // extra dims / extra V^T rows that carry the zero-point terms
constexpr int kKv = 64;        // context tokens per KV tile = UMMA N of Q.K^T
constexpr int kNo = kD + kDx;  // UMMA N of P.V
constexpr int kTmemCols = 256; // S: columns [0, 64), O: columns [64, 208)
constexpr float kLazy = 4.f;   // log2 of the growth of a row maximum that forces a rescale of O
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLn2P = 0.6931471805599453f;

template <int BS>
struct PrefillSmem {
    static constexpr int REC = BS * (kD + 8);
    static constexpr int NREC = kKv / BS;
    static constexpr int RSTRIDE = REC + 64;       // records 64 bytes out of phase: conflict-free 16-byte reads across records
    alignas(1024) uint8_t q[kRows * kD * 2];       // 2 swizzle atoms of [128 rows][64 dims]
    alignas(1024) uint8_t k[kKv * kD * 2];         // 2 atoms of [64 tokens][64 dims]
    alignas(1024) uint8_t vt[kNo * kKv * 2];       // [144 dims][64 tokens], 18 groups of 8 rows
    alignas(1024) uint8_t p[kRows * kKv * 2];      // 1 atom of [128 rows][64 tokens]
    alignas(128) uint8_t qx[kRows * kDx * 2];      // unswizzled [128 rows][16 dims]
    alignas(128) uint8_t kx[kKv * kDx * 2];        // unswizzled [64 tokens][16 dims]
    alignas(128) uint8_t raw_k[NREC * RSTRIDE];    // staged key records
    alignas(128) uint8_t raw_v[NREC * RSTRIDE];    // staged value records
    alignas(16) uint2 v_tab[kRows / 32][kKv / 2];  // per warp: (scale, -1024 * scale) as f16 pairs of two tokens
    alignas(8) uint64_t bar_raw;
    alignas(8) uint64_t bar_s;
    alignas(8) uint64_t bar_o;
    uint32_t tmem_base;
};

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }
// unswizzled K-major tile of 16 dims: 8-row groups 256 bytes apart, the two 8-dim halves 128 apart
__device__ __forceinline__ uint32_t plain16(uint32_t row, uint32_t half) { return (row >> 3) * 256u + half * 128u + (row & 7u) * 16u; }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
// z = h + m + l up to 2^-33 |z|, every piece an f16
__device__ __forceinline__ void split3(float z, __half& h, __half& m, __half& l) {
    h = __float2half_rn(z);
    const float r = z - __half2float(h);
    m = __float2half_rn(r);
    l = __float2half_rn(r - __half2float(m));
}
__device__ __forceinline__ uint32_t h2_bits(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}
__device__ __forceinline__ uint32_t ex2_h2(uint32_t x) {
    uint32_t y;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t y;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(y) : "r"(a), "r"(b), "r"(c));
    return y;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}
// 16 cache bytes -> 16 f16 values 1024 + byte
__device__ __forceinline__ void bytes16_to_h(const uint4 w, uint4& lo4, uint4& hi4) {
    lo4.x = __byte_perm(w.x, 0x64646464u, 0x4140); lo4.y = __byte_perm(w.x, 0x64646464u, 0x4342);
    lo4.z = __byte_perm(w.y, 0x64646464u, 0x4140); lo4.w = __byte_perm(w.y, 0x64646464u, 0x4342);
    hi4.x = __byte_perm(w.z, 0x64646464u, 0x4140); hi4.y = __byte_perm(w.z, 0x64646464u, 0x4342);
    hi4.z = __byte_perm(w.w, 0x64646464u, 0x4140); hi4.w = __byte_perm(w.w, 0x64646464u, 0x4342);
}
// (1024 + byte) -> byte * scale, rounded once.  The fused form needs -1024 * scale inside the f16
// range; scales of 32 and more take the two-step form.
__device__ __forceinline__ void scale16(uint4& lo4, uint4& hi4, __half sc) {
    const uint32_t s2 = h2_bits(sc, sc);
    uint32_t* w0 = reinterpret_cast<uint32_t*>(&lo4);
    uint32_t* w1 = reinterpret_cast<uint32_t*>(&hi4);
    if (fabsf(__half2float(sc)) < 32.f) {
        const uint32_t c2 = hmul2_bits(s2, 0xE400E400u);   // -1024 * scale, exact
#pragma unroll
        for (int k = 0; k < 4; ++k) { w0[k] = hfma2_bits(w0[k], s2, c2); w1[k] = hfma2_bits(w1[k], s2, c2); }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) { w0[k] = hmul2_bits(hadd2_bits(w0[k], 0xE400E400u), s2); w1[k] = hmul2_bits(hadd2_bits(w1[k], 0xE400E400u), s2); }
    }
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
    const float qscale = (a.scale != 0.f ? a.scale : rsqrtf((float)kD)) * kLog2eP;

    if (tid == 0) {
        mbar_init(&sm.bar_raw, 1);
        mbar_init(&sm.bar_s, 1);
        mbar_init(&sm.bar_o, 1);
        mbar_fence_init();
    }
    // rows 132..143 of V^T stay zero for the whole kernel
    if (tid < (kNo - kD - 4) * 8) *reinterpret_cast<uint4*>(sm.vt + (kD + 4) * 128 + tid * 16) = make_uint4(0, 0, 0, 0);
    if (warp == 0) tc05::tmem_alloc(&sm.tmem_base, kTmemCols);
    tc05::fence_before_thread_sync();
    __syncthreads();
    tc05::fence_after_thread_sync();
    const uint32_t tmem = sm.tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + kKv;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;   // this warp's TMEM lanes

    constexpr uint32_t idesc_s = tc05::instr_desc_f16(kRows, kKv, 0, 0, 0);   // f16, A and B K-major
    constexpr uint32_t idesc_o = tc05::instr_desc_f16(kRows, kNo, 0, 0, 0);
    const uint32_t q_addr = smem_u32(sm.q), k_addr = smem_u32(sm.k), vt_addr = smem_u32(sm.vt), p_addr = smem_u32(sm.p);
    const uint32_t qx_addr = smem_u32(sm.qx), kx_addr = smem_u32(sm.kx);

    uint32_t phase_raw = 0, phase_s = 0, phase_o = 0;
    bool bad_index = false;
    bool failed = false;

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
        const int32_t* table = a.block_indices + a.block_indices_begins[s];

        // ---- this thread's row ---------------------------------------------------------------------
        const int flat = qt * kRows + tid;
        const int tok = flat / G, hq = hk * G + flat % G;
        const bool row_live = tok < n_new;
        const int tok_hi = min(n_new - 1, (qt * kRows + kRows - 1) / G);
        const int ctx_hi = past + tok_hi + 1;             // context the last row of the tile sees
        const int ntiles = (ctx_hi + kKv - 1) / kKv;
        const int my_ctx = row_live ? past + tok + 1 : ctx_hi;

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
                    bulk_g2s(sm.raw_k + r * Smem::RSTRIDE, kc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.bar_raw);
                    bulk_g2s(sm.raw_v + r * Smem::RSTRIDE, vc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.bar_raw);
                }
        };
        // every tensor-core read of the previous item has completed (its waits sit in program order
        // before this point) and every thread has finished reading the raw buffers
        if (tid == 0) issue_raw(0);

        // ---- Q -> f16 swizzled A operand; the row's sum goes into the extra dims ------------------
        {
            const long long qoff = ((long long)(t0 + (row_live ? tok : 0)) * a.g.Hq + hq) * kD;
            float qsum = 0.f;
#pragma unroll 4
            for (int c = 0; c < kD / 8; ++c) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
                if (row_live) load_act_vec<8>(a.query, qoff + 8 * c, a.g.act, v);
                uint4 w;
                w.x = pack_h2(v[0], v[1]); w.y = pack_h2(v[2], v[3]); w.z = pack_h2(v[4], v[5]); w.w = pack_h2(v[6], v[7]);
                const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e) qsum += __low2float(h[e]) + __high2float(h[e]);
                *reinterpret_cast<uint4*>(sm.q + (c / 8) * (kRows * 128) + sw128(tid, c % 8)) = w;
            }
            // |q| is assumed to stay inside the f16 range (no power-of-two prescale here)
            const __half qh = __float2half_rn(qsum), ql = __float2half_rn(qsum - __half2float(qh));
            const __half zero = __ushort_as_half(0);
            *reinterpret_cast<uint4*>(sm.qx + plain16(tid, 0)) = make_uint4(h2_bits(qh, qh), h2_bits(qh, ql), h2_bits(ql, zero), 0u);
            *reinterpret_cast<uint4*>(sm.qx + plain16(tid, 1)) = make_uint4(0u, 0u, 0u, 0u);
        }

        float m_run = -INFINITY;   // running maximum of q.k' (before the softmax scale)

        // A wait that runs out sets `failed`; the flag is made uniform at the next block barrier so
        // that every thread leaves the loop at the same place.
        for (int j = 0; j < ntiles; ++j) {
            const int col0 = j * kKv;
            const int live_tokens = min(kKv, ctx_hi - col0);
            // ---- 1-2. raw records -> f16 operand tiles -------------------------------------------
            if (!mbar_wait_bounded(&sm.bar_raw, phase_raw)) failed = true;
            phase_raw ^= 1;
            if (!failed) {
                // K' = byte * f16(k scale): unit u = 16 dims of one token.  S of the previous tile has completed.
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int u = tid + kRows * i;
                    const int token = u >> 3, seg = u & 7;
                    uint4 lo4 = make_uint4(0u, 0u, 0u, 0u), hi4 = lo4;
                    if (token < live_tokens) {
                        const uint8_t* rec = sm.raw_k + (token / BS) * Smem::RSTRIDE;
                        const __half ksh = __float2half_rn(*reinterpret_cast<const float*>(rec + BS * kD + 4 * (token % BS)));
                        bytes16_to_h(*reinterpret_cast<const uint4*>(rec + (token % BS) * kD + 16 * seg), lo4, hi4);
                        scale16(lo4, hi4, ksh);
                    }
                    uint8_t* atom = sm.k + (seg >> 2) * (kKv * 128);
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg) & 7)) = lo4;
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg + 1) & 7)) = hi4;
                }
                if (tid < kKv) {
                    const int token = tid;
                    const bool ok = token < live_tokens;
                    const float* kp = reinterpret_cast<const float*>(sm.raw_k + (token / BS) * Smem::RSTRIDE + BS * kD);
                    const float ksf = __half2float(__float2half_rn(kp[token % BS]));
                    __half zh, zm, zl;
                    split3(ok ? -(ksf * kp[BS + token % BS]) : 0.f, zh, zm, zl);
                    const __half zero = __ushort_as_half(0);
                    *reinterpret_cast<uint4*>(sm.kx + plain16(token, 0)) = make_uint4(h2_bits(zh, zm), h2_bits(zl, zh), h2_bits(zm, zero), 0u);
                    *reinterpret_cast<uint4*>(sm.kx + plain16(token, 1)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            if (j > 0) {   // P.V of the previous tile still reads V^T and P
                if (!failed && !mbar_wait_bounded(&sm.bar_o, phase_o)) failed = true;
                phase_o ^= 1;
                tc05::fence_after_thread_sync();
            }
            failed = __any_sync(0xffffffffu, failed);
            if (!failed) {
                // this warp's table of (scale, -1024 * scale) for the tile's token pairs
                const int lane = tid & 31;
                __syncwarp();
                float vs0 = 0.f, vs1 = 0.f;
                {
                    const int t0k = 2 * lane, t1k = 2 * lane + 1;
                    if (t0k < live_tokens) vs0 = *reinterpret_cast<const float*>(sm.raw_v + (t0k / BS) * Smem::RSTRIDE + BS * kD + 4 * (t0k % BS));
                    if (t1k < live_tokens) vs1 = *reinterpret_cast<const float*>(sm.raw_v + (t1k / BS) * Smem::RSTRIDE + BS * kD + 4 * (t1k % BS));
                }
                const uint32_t s2 = pack_h2(vs0, vs1);
                sm.v_tab[warp][lane] = make_uint2(s2, hmul2_bits(s2, 0xE400E400u));
                const bool big = __any_sync(0xffffffffu, !(fabsf(vs0) < 32.f) || !(fabsf(vs1) < 32.f));
                __syncwarp();
                // V'^T = byte * f16(v scale): unit = 16 tokens of one dim
                const int tg = tid & 3;
                uint2 tab[8];
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    const uint4 t4 = *reinterpret_cast<const uint4*>(&sm.v_tab[warp][8 * tg + k]);
                    tab[k] = make_uint2(t4.x, t4.y);
                    tab[k + 1] = make_uint2(t4.z, t4.w);
                }
                constexpr int UPR = BS / 16;   // 16-token units per record
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int d = (tid >> 2) + 32 * i;
                    uint4 lo4, hi4;
                    bytes16_to_h(*reinterpret_cast<const uint4*>(sm.raw_v + (tg / UPR) * Smem::RSTRIDE + d * BS + 16 * (tg % UPR)), lo4, hi4);
                    uint32_t w[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
                    if (!big) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) w[k] = hfma2_bits(w[k], tab[k].x, tab[k].y);
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) w[k] = hmul2_bits(hadd2_bits(w[k], 0xE400E400u), tab[k].x);
                    }
                    *reinterpret_cast<uint4*>(sm.vt + sw128(d, 2 * tg)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(sm.vt + sw128(d, 2 * tg + 1)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
                if (tid < kKv) {
                    const int token = tid;
                    const bool ok = token < live_tokens;
                    const float* vp = reinterpret_cast<const float*>(sm.raw_v + (token / BS) * Smem::RSTRIDE + BS * kD);
                    const float vsf = __half2float(__float2half_rn(vp[token % BS]));
                    __half zh, zm, zl;
                    split3(ok ? vsf * vp[BS + token % BS] : 0.f, zh, zm, zl);
                    const uint32_t off = (token & 7) * 2;
                    *reinterpret_cast<__half*>(sm.vt + sw128(kD + 0, token >> 3) + off) = zh;
                    *reinterpret_cast<__half*>(sm.vt + sw128(kD + 1, token >> 3) + off) = zm;
                    *reinterpret_cast<__half*>(sm.vt + sw128(kD + 2, token >> 3) + off) = zl;
                    *reinterpret_cast<__half*>(sm.vt + sw128(kD + 3, token >> 3) + off) = __float2half_rn(ok ? 1.f : 0.f);
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
                tc05::mma_ss(tmem_s, tc05::smem_desc_plain(qx_addr, 128, 256), tc05::smem_desc_plain(kx_addr, 128, 256), idesc_s, 1u);
                tc05::commit(&sm.bar_s);
            }
            if (!mbar_wait_bounded(&sm.bar_s, phase_s)) failed = true;
            phase_s ^= 1;
            failed = __any_sync(0xffffffffu, failed);   // the TMEM accesses below are warp-collective
            tc05::fence_after_thread_sync();

            // ---- 4. softmax of this thread's row ------------------------------------------------------
            if (!failed) {
                float sv[kKv];   // q.k' in units of 1 / qscale
                {
                    uint32_t s0[32], s1[32];
                    tc05::ld_32x32b_x32(tmem_s + lane_base, s0);
                    tc05::ld_32x32b_x32(tmem_s + lane_base + 32, s1);
                    tc05::wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) { sv[c] = __uint_as_float(s0[c]); sv[32 + c] = __uint_as_float(s1[c]); }
                }
                if (col0 + kKv > my_ctx) {   // diagonal tile: hide what this row cannot see
                    const int nvis = my_ctx - col0;   // may be <= 0
#pragma unroll
                    for (int c = 0; c < kKv; ++c) sv[c] = c < nvis ? sv[c] : -INFINITY;
                }
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < kKv; c += 2) mx = max3(mx, sv[c], sv[c + 1]);
                if (j == 0) {
                    m_run = mx;      // finite: column 0 of tile 0 is visible to every row
                } else {
                    const bool grow = (mx - m_run) * qscale > kLazy;
                    if (__any_sync(0xffffffffu, grow)) {
                        // rescale this warp's rows of O in TMEM; P.V of the previous tile has completed
                        const float alpha = grow ? ex2((m_run - mx) * qscale) : 1.f;
                        if (grow) m_run = mx;
#pragma unroll
                        for (int q4 = 0; q4 < kD / 32; ++q4) {
                            uint32_t r[32];
                            tc05::ld_32x32b_x32(tmem_o + lane_base + 32 * q4, r);
                            tc05::wait_ld();
#pragma unroll
                            for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                            tc05::st_32x32b_x32(tmem_o + lane_base + 32 * q4, r);
                        }
                        uint32_t r[16];
                        tc05::ld_32x32b_x16(tmem_o + lane_base + kD, r);
                        tc05::wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
                        tc05::st_32x32b_x16(tmem_o + lane_base + kD, r);
                        tc05::wait_st();
                    }
                }
                // P = 2^(qscale * (s - m)) in f16 pairs: the exponent is rounded to f16 first, which costs
                // at most 2^-12 of the exponent's magnitude in relative error of p
                const float mq = m_run * qscale;
#pragma unroll
                for (int c = 0; c < kKv; c += 8) {
                    uint4 w;
                    w.x = ex2_h2(pack_h2(fmaf(sv[c], qscale, -mq), fmaf(sv[c + 1], qscale, -mq)));
                    w.y = ex2_h2(pack_h2(fmaf(sv[c + 2], qscale, -mq), fmaf(sv[c + 3], qscale, -mq)));
                    w.z = ex2_h2(pack_h2(fmaf(sv[c + 4], qscale, -mq), fmaf(sv[c + 5], qscale, -mq)));
                    w.w = ex2_h2(pack_h2(fmaf(sv[c + 6], qscale, -mq), fmaf(sv[c + 7], qscale, -mq)));
                    *reinterpret_cast<uint4*>(sm.p + sw128(tid, c >> 3)) = w;
                }
            }
            tc05::fence_proxy_async_smem();
            tc05::fence_before_thread_sync();
            failed = __syncthreads_or(failed ? 1 : 0) != 0;
            if (failed) break;
            // ---- 5. O += P'.V; overlaps the next tile's key conversion -----------------------------------
            if (tid == 0) {
                tc05::fence_after_thread_sync();
#pragma unroll
                for (int kk = 0; kk < kKv / 16; ++kk) {
                    const uint64_t da = tc05::smem_desc_sw128(p_addr + kk * 32, 1024);
                    const uint64_t db = tc05::smem_desc_sw128(vt_addr + kk * 32, 1024);
                    tc05::mma_ss(tmem_o, da, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tc05::commit(&sm.bar_o);
            }
        }
        if (!failed && !mbar_wait_bounded(&sm.bar_o, phase_o)) failed = true;
        phase_o ^= 1;
        tc05::fence_after_thread_sync();
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        if (failed) {
            if (tid == 0) atomicOr(a.status, 0x40000000u);
            break;
        }
        // ---- epilogue: out = (O - z) / l, z = the three zero-point columns ---------------------------
        {
            uint32_t zr[16];
            tc05::ld_32x32b_x16(tmem_o + lane_base + kD, zr);
            tc05::wait_ld();
            const float z = __uint_as_float(zr[0]) + __uint_as_float(zr[1]) + __uint_as_float(zr[2]);
            const float l_run = __uint_as_float(zr[3]);   // the all-ones row of V^T sums the probabilities
            const float inv = 1.f / l_run;
            const long long ooff = ((long long)(t0 + (row_live ? tok : 0)) * a.g.Hq + hq) * kD;
#pragma unroll
            for (int q4 = 0; q4 < kD / 32; ++q4) {
                uint32_t r[32];
                tc05::ld_32x32b_x32(tmem_o + lane_base + 32 * q4, r);
                tc05::wait_ld();
                if (row_live) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = (__uint_as_float(r[c + e]) - z) * inv;
                        store_act_vec8(a.output, ooff + 32 * q4 + c, a.g.act, v);
                    }
                }
            }
            if (row_live && a.lse) a.lse[(long long)(t0 + tok) * a.g.Hq + hq] = (m_run * qscale + log2f(l_run)) * kLn2P;
        }
        tc05::fence_before_thread_sync();
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
