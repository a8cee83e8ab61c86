// SnapKV-style score output of the PagedAttention operator.
//
// scores[off_s + pos] = sum over q heads h and over the last W rows j of sequence s's chunk of
//                       exp(scale * q[j,h].k[pos] - lse[j,h])          (pos <= past + j)
// where lse is the log-sum-exp the attention kernels exported for every (token, q head).
//
// Three launches: (1) one warp builds the per-sequence offsets into `scores` and the prefix sum of
// 32-token key tiles of the sequences that want scores; (2) a persistent kernel in which every warp
// takes an equal slice of the global (sequence, kv head, tile) sequence, stages the key records with
// TMA bulk copies (u8) or cp.async (f16 / bf16), recomputes Q.K^T on mma.sync with the window rows
// and the GQA group as the M dimension, and writes the per-kv-head column sums of the
// probabilities; (3) a reduction that adds the kv heads in a fixed order, so the f32 result does
// not depend on scheduling - block selection downstream compares these values
// (src/cpp/src/continuous_batching/cache/cache_eviction.cpp:486-519).
// HBM-bound: Hkv*(D+8) key bytes per position (u8).
#include <algorithm>

#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kTileS = kScoreTile;
constexpr int kScoreWarps = 4;
constexpr float kLog2eS = 1.4426950408889634f;

template <int D, int BS, int CACHE>
struct ScoreCfg {
    static constexpr bool U8 = CACHE == PA_DTYPE_U8;
    static constexpr bool BF16 = CACHE == PA_DTYPE_BF16;
    static constexpr int REC = U8 ? BS * (D + 8) : BS * D * 2;
    static constexpr int NREC = kTileS / BS;
    static constexpr int STAGE = NREC * REC;   // keys only
    static constexpr int NSTAGE = 3;
    static constexpr int RING = NSTAGE * STAGE;
    // rounded to 128 bytes: every warp's ring must start 16-byte aligned for bulk copies and 16-byte loads
    static constexpr int WARP_SMEM = (RING + NSTAGE * 16 + NSTAGE * 8 + 127) / 128 * 128;
    static constexpr int SMEM = kScoreWarps * WARP_SMEM;
    static_assert(WARP_SMEM % 16 == 0 && STAGE % 16 == 0 && REC % 16 == 0, "bulk copies and 16-byte loads need 16-byte aligned stages");
};

// What the loader records per ring stage.
struct __align__(16) ScoreDesc {
    int s;       // sequence, -1 = end of this worker's slice
    int hk;      // kv head
    int tile;    // tile index inside the sequence
    int first;   // first tile of a run: reload the per-run state
};

__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int D, int BS, int CACHE>
__global__ void __launch_bounds__(kScoreWarps * 32) score_kernel(KernelArgs a) {
    using Cfg = ScoreCfg<D, BS, CACHE>;
    constexpr bool U8 = Cfg::U8;
    constexpr bool BF16 = Cfg::BF16;
    constexpr int NKK = D / 16;
    constexpr int NS = Cfg::NSTAGE;

    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    uint8_t* ring = smem + warp * Cfg::WARP_SMEM;
    ScoreDesc* descs = reinterpret_cast<ScoreDesc*>(ring + Cfg::RING);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + Cfg::RING + NS * 16);
    if constexpr (U8) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NS; ++i) mbar_init(&bars[i], 1);
            mbar_fence_init();
        }
        __syncwarp();
    }
    const int Hkv = a.g.Hkv, G = a.g.Hq / a.g.Hkv;
    const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)D);

    // ---- this worker's slice --------------------------------------------------------------------------
    // Cost space: sequence s occupies [P[s]*Hkv, P[s+1]*Hkv) with P = stile_prefix, kv head hk the
    // hk-th equal part of it, and tile t of that part starts at t * weight(s).  A worker owns the
    // tiles whose start lies in its equal slice [c_pos, c_end) of the cost range.
    const long long total_cost = (long long)a.stile_prefix[a.num_sequences] * Hkv;
    const long long all_workers = (long long)gridDim.x * kScoreWarps;
    const long long workers = max(1LL, min(all_workers, (total_cost + 3) / 4));
    const long long per_worker = (total_cost + workers - 1) / workers;
    const long long wid = (long long)blockIdx.x * kScoreWarps + warp;
    long long c_pos = min(total_cost, wid * per_worker);
    const long long c_end = min(total_cost, c_pos + per_worker);

    // ---- loader state (warp-uniform) ------------------------------------------------------------------
    int r_s = -1, r_hk = 0, r_tile = 0, r_tile_end = 0, r_ctx = 0, r_tb = 0, r_nb = 0;
    int w_blk0 = 0, tbl = 0;
    bool r_first = false;

    auto load_window = [&](int first_block) {
        w_blk0 = first_block;
        const int bi = first_block + lane;
        int blk = 0;
        if (bi < r_nb) {
            blk = a.block_indices[r_tb + bi];
            if (blk < 0 || blk >= a.num_blocks) blk = 0;  // flagged by the attention kernels
        }
        tbl = blk;
    };
    // Finds the next run of tiles of one (sequence, kv head) inside the slice; false when the slice is done.
    auto next_run = [&]() -> bool {
        while (c_pos < c_end) {
            const int key = (int)(c_pos / Hkv);
            int lo = 0, hi = a.num_sequences;
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (a.stile_prefix[mid] <= key) lo = mid; else hi = mid;
            }
            const int p0 = a.stile_prefix[lo];
            const long long seq_cost = a.stile_prefix[lo + 1] - p0;
            const int n = a.subsequence_begins[lo + 1] - a.subsequence_begins[lo];
            const int ctx = a.past_lens[lo] + n;
            const int tiles = (ctx + kTileS - 1) / kTileS;
            const long long weight = seq_cost / tiles;
            const long long off = c_pos - (long long)p0 * Hkv;
            const int hk = (int)(off / seq_cost);
            const long long head_base = (long long)p0 * Hkv + hk * seq_cost;
            const int tile0 = (int)((c_pos - head_base + weight - 1) / weight);
            const int tile1 = (int)((min(c_end, head_base + seq_cost) - head_base + weight - 1) / weight);
            c_pos = min(c_end, head_base + seq_cost);
            if (tile0 >= tile1) continue;
            r_s = lo;
            r_hk = hk;
            r_tile = tile0;
            r_tile_end = tile1;
            r_ctx = ctx;
            r_tb = a.block_indices_begins[lo];
            r_nb = a.block_indices_begins[lo + 1] - r_tb;
            r_first = true;
            load_window(tile0 * kTileS / BS);
            return true;
        }
        return false;
    };
    auto produce = [&](int slot) {
        if (r_tile >= r_tile_end && !next_run()) {
            if (lane == 0) descs[slot] = ScoreDesc{-1, 0, 0, 0};
            if constexpr (!U8) cp_async_commit();
            return;
        }
        uint8_t* st = ring + slot * Cfg::STAGE;
        const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)r_hk * a.g.head_bytes;
        const int bi0 = r_tile * kTileS / BS;
        if (bi0 + Cfg::NREC - 1 - w_blk0 >= 32) load_window(bi0);
        int blocks[Cfg::NREC];
        bool live[Cfg::NREC];
#pragma unroll
        for (int r = 0; r < Cfg::NREC; ++r) {
            live[r] = (bi0 + r) * BS < r_ctx;
            blocks[r] = __shfl_sync(0xffffffffu, tbl, (bi0 + r - w_blk0) & 31);
        }
        if constexpr (U8) {
            if (lane == 0) {
                uint32_t bytes = 0;
#pragma unroll
                for (int r = 0; r < Cfg::NREC; ++r) bytes += live[r] ? Cfg::REC : 0;
                mbar_expect_tx(&bars[slot], bytes);
#pragma unroll
                for (int r = 0; r < Cfg::NREC; ++r)
                    if (live[r]) bulk_g2s(st + r * Cfg::REC, kc + (long long)blocks[r] * a.g.block_bytes, Cfg::REC, &bars[slot]);
            }
        } else {
            constexpr int CPR = D / 8;
#pragma unroll
            for (int r = 0; r < Cfg::NREC; ++r)
                if (live[r]) {
                    const uint8_t* ksrc = kc + (long long)blocks[r] * a.g.block_bytes;
#pragma unroll
                    for (int i = lane; i < BS * CPR; i += 32) {
                        const int row = r * BS + i / CPR, ch = i % CPR;
                        cp_async16(st + row * (2 * D) + ((ch ^ (row & 7)) << 4), ksrc + (long long)i * 16);
                    }
                }
            cp_async_commit();
        }
        if (lane == 0) descs[slot] = ScoreDesc{r_s, r_hk, r_tile, r_first ? 1 : 0};
        r_first = false;
        ++r_tile;
    };

    // ---- consumer state ----------------------------------------------------------------------------
    uint32_t qa[NKK][4];
    float qsum[2], qsc[2], lse2[2];
    int vis[2];                 // first position the row cannot see (0 for padding rows)
    int t0 = 0, n_new = 0, past = 0, W = 0, rows = 0, row_tiles = 0, hk = 0;
    float* out = nullptr;
    long long out_room = 0;     // floats left in `scores` from the sequence's offset on

    // Loads the Q fragments and per-row constants of row tile `rt` (rows 16*rt + g and + 8).
    // Row r of the run is (chunk row n - W + r / G, q head hk*G + r % G).
    auto load_q = [&](int rt) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int rr = 16 * rt + g + 8 * r;
            const bool live = rr < rows;
            const int j = n_new - W + (live ? rr / G : 0), h = hk * G + (live ? rr % G : 0);
            const long long grow = (long long)(t0 + j) * a.g.Hq + h;
            float q[D / 4];
            float amax = 0.f;
            if constexpr (U8) {
                // element e is dimension 64*(e/16) + 16*c + e%16: runs of 16
#pragma unroll
                for (int h = 0; h < D / 64; ++h) {
                    float v[16];
                    if (live) load_act_vec<16>(a.query, grow * D + 64 * h + 16 * c, a.g.act, v);
#pragma unroll
                    for (int e = 0; e < 16; ++e) q[16 * h + e] = live ? v[e] : 0.f;
                }
            } else {
                // element e is dimension 16*(e/4) + 8*((e>>1)&1) + 2*c + (e&1): pairs
#pragma unroll
                for (int e = 0; e < D / 4; e += 2) {
                    float v[2];
                    if (live) load_act_vec<2>(a.query, grow * D + 16 * (e / 4) + 8 * ((e >> 1) & 1) + 2 * c, a.g.act, v);
                    q[e] = live ? v[0] : 0.f;
                    q[e + 1] = live ? v[1] : 0.f;
                }
            }
#pragma unroll
            for (int e = 0; e < D / 4; ++e) amax = fmaxf(amax, fabsf(q[e]));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            float qmul = 1.f;
            if (!BF16 && amax > 32768.f && amax < INFINITY) {
                int ex;
                frexpf(amax, &ex);
                qmul = ldexpf(1.f, 15 - ex);
            }
            float sum = 0.f;
#pragma unroll
            for (int e = 0; e < D / 4; e += 2) {
                uint32_t packed;
                if constexpr (BF16) {
                    packed = pack_bf2(q[e], q[e + 1]);
                } else {
                    packed = pack_h2(q[e] * qmul, q[e + 1] * qmul);
                    __half2 hh = *reinterpret_cast<__half2*>(&packed);
                    sum += __low2float(hh) + __high2float(hh);
                }
                qa[e / 4][r + 2 * ((e >> 1) & 1)] = packed;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            qsum[r] = sum;
            qsc[r] = sm_scale * kLog2eS / qmul;
            lse2[r] = live ? a.lse[grow] * kLog2eS : 0.f;
            vis[r] = live ? past + j + 1 : 0;
        }
    };

#pragma unroll
    for (int p = 0; p < NS - 1; ++p) produce(p);

    for (int it = 0;; ++it) {
        __syncwarp();
        produce((it + NS - 1) % NS);
        __syncwarp();
        const int slot = it % NS;
        const ScoreDesc d = descs[slot];
        if (d.s < 0) break;
        if constexpr (U8) {
            if (!mbar_wait_bounded(&bars[slot], (it / NS) & 1)) {
                if (lane == 0) atomicOr(a.status, PA_DEV_WAIT_TIMEOUT_SCORES);
                break;
            }
        } else {
            cp_async_wait<NS - 1>();
            __syncwarp();
        }
        const uint8_t* st = ring + slot * Cfg::STAGE;
        if (d.first) {
            hk = d.hk;
            t0 = a.subsequence_begins[d.s];
            n_new = a.subsequence_begins[d.s + 1] - t0;
            past = a.past_lens[d.s];
            W = min(max(a.score_aggregation_window[d.s], 0), n_new);
            rows = W * G;
            row_tiles = (rows + 15) / 16;
            out = a.score_part + (long long)hk * a.scores_len + a.score_offsets[d.s];
            out_room = a.scores_len - a.score_offsets[d.s];
            if (row_tiles == 1) load_q(0);
        }
        const int tile_base = d.tile * kTileS;
        const int valid = min(kTileS, past + n_new - tile_base);
        float csum[4][2];
#pragma unroll
        for (int j = 0; j < 4; ++j) { csum[j][0] = 0.f; csum[j][1] = 0.f; }

        for (int rt = 0; rt < row_tiles; ++rt) {
            if (row_tiles > 1) load_q(rt);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float acc4[4] = {0.f, 0.f, 0.f, 0.f};
                if constexpr (U8) {
                    const int row = 8 * (g >> 1) + 2 * j + (g & 1);
                    const uint8_t* kp = st + (row / BS) * Cfg::REC + (row % BS) * D + 16 * c;
#pragma unroll
                    for (int h = 0; h < D / 64; ++h) {
                        const uint4 w = *reinterpret_cast<const uint4*>(kp + 64 * h);
                        const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            mma16816<false, true>(acc4, qa[4 * h + i], __byte_perm(ww[i], 0x64646464u, 0x4140), __byte_perm(ww[i], 0x64646464u, 0x4342));
                    }
                } else {
#pragma unroll
                    for (int p = 0; p < NKK / 2; ++p) {
                        const int row = 8 * j + (lane & 7), ch = 4 * p + (lane >> 3);
                        uint32_t b[4];
                        ldmatrix_x4(b, smem_u32(st + row * 2 * D + ((ch ^ (row & 7)) << 4)));
                        mma16816<BF16, true>(acc4, qa[2 * p], b[0], b[1]);
                        mma16816<BF16, true>(acc4, qa[2 * p + 1], b[2], b[3]);
                    }
                }
                const int tk = U8 ? 8 * c + 2 * j : 8 * j + 2 * c;   // tile token of accumulator column 0
                float ks0 = 1.f, ks1 = 1.f, kz0 = 0.f, kz1 = 0.f;
                if constexpr (U8) {
                    const uint8_t* pp = st + (tk / BS) * Cfg::REC + BS * D;
                    const float2 ks = *reinterpret_cast<const float2*>(pp + 4 * (tk % BS));
                    const float2 kz = *reinterpret_cast<const float2*>(pp + 4 * BS + 4 * (tk % BS));
                    ks0 = ks.x; ks1 = ks.y; kz0 = kz.x + 1024.f; kz1 = kz.y + 1024.f;
                }
#pragma unroll
                for (int r = 0; r < 2; ++r) {
                    if (r == 1 && rows - 16 * rt <= 8) break;   // rows 8..15 of the tile are padding (warp-uniform)
                    float s0 = acc4[2 * r], s1 = acc4[2 * r + 1];
                    if constexpr (U8) {
                        s0 = (s0 - kz0 * qsum[r]) * (ks0 * qsc[r]);
                        s1 = (s1 - kz1 * qsum[r]) * (ks1 * qsc[r]);
                    } else {
                        s0 *= qsc[r]; s1 *= qsc[r];
                    }
                    // selects, not products: stale key bytes past the context may decode to NaN
                    csum[j][0] += (tile_base + tk < vis[r]) ? exp2_fast(s0 - lse2[r]) : 0.f;
                    csum[j][1] += (tile_base + tk + 1 < vis[r]) ? exp2_fast(s1 - lse2[r]) : 0.f;
                }
            }
        }
        // column sums over the 8 row groups held by lanes with equal c
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = csum[j][e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                csum[j][e] = v;
            }
        if (g == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tk = U8 ? 8 * c + 2 * j : 8 * j + 2 * c;
                if (tk < valid && tile_base + tk < out_room) out[tile_base + tk] = csum[j][0];
                if (tk + 1 < valid && tile_base + tk + 1 < out_room) out[tile_base + tk + 1] = csum[j][1];
            }
        }
    }
    if constexpr (!U8) cp_async_wait<0>();
}

// scores[pos] = sum over kv heads of the per-head partials, in head order; zeros for sequences
// whose window is 0 (their slots still count toward the offsets,
// src/cpp/src/continuous_batching/model_runner.hpp:1536-1537).
__global__ void __launch_bounds__(256) score_reduce_kernel(KernelArgs a) {
    const int s = blockIdx.y;
    SeqView sv;
    const bool valid = seq_view(a, s, sv);
    const long long off = a.score_offsets[s], len = a.score_offsets[s + 1] - off;
    // a sequence whose slot does not fit into `scores` gets zeros where the slot is in range (the kernels
    // that would have produced its numbers skipped it and raised PA_DEV_BAD_BEGINS)
    const bool fits = off + len <= a.scores_len;
    const bool live = fits && a.stile_prefix[s + 1] > a.stile_prefix[s];
    const bool from_decode = a.score_raw != nullptr && valid && fits && sv.n == 1 && a.score_aggregation_window[s] > 0;
    if (from_decode) {
        // probabilities from the decode kernel's scaled logits (base 2) and the row's log-sum-exp, added
        // over the q heads in head order
        const int G = a.g.Hq / a.g.Hkv, gtiles = (G + 15) / 16, HK = a.g.Hkv * gtiles;
        const int SL = a.rows_per_tile <= 8 ? 8 : 16;
        const float* lse = a.lse + (long long)sv.t0 * a.g.Hq;
        constexpr float kLog2e = 1.4426950408889634f;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (long long)gridDim.x * blockDim.x) {
            if (off + i >= a.scores_len) break;
            float v = 0.f;
            for (int hkp = 0; hkp < HK; ++hkp) {
                const int hk = hkp / gtiles;
                const int hbase = hk * G + (hkp % gtiles) * 16;
                const int hcount = min(16, hk * G + G - hbase);
                const float4* raw = reinterpret_cast<const float4*>(a.score_raw + ((long long)hkp * a.scores_len + off + i) * SL);
                for (int q = 0; q < SL / 4; ++q) {
                    const float4 x = __ldcs(raw + q);
                    const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (4 * q + e < hcount) v += exp2_fast(xs[e] - __ldg(lse + hbase + 4 * q + e) * kLog2e);
                }
            }
            a.scores[off + i] = v;
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        if (live)
            for (int hk = 0; hk < a.g.Hkv; ++hk) v += a.score_part[(long long)hk * a.scores_len + off + i];
        if (off + i < a.scores_len) a.scores[off + i] = v;
    }
}

template <int D, int BS, int CACHE>
cudaError_t launch_score_t(const KernelArgs& a, cudaStream_t stream, int sm_count) {
    using Cfg = ScoreCfg<D, BS, CACHE>;
    auto kern = score_kernel<D, BS, CACHE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) return e;
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kScoreWarps * 32, Cfg::SMEM);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const long long max_tiles = (a.scores_len / kTileS + a.num_sequences) * a.g.Hkv;
    long long ctas = (long long)std::min(per_sm, 4) * sm_count;
    ctas = std::max(1LL, std::min(ctas, (max_tiles / 4 + kScoreWarps) / kScoreWarps));
    kern<<<(unsigned)ctas, kScoreWarps * 32, Cfg::SMEM, stream>>>(a);
    return cudaGetLastError();
}

template <int D, int BS>
cudaError_t launch_score_c(const KernelArgs& a, cudaStream_t stream, int sm_count) {
    switch (a.g.cache) {
        case PA_DTYPE_U8: return launch_score_t<D, BS, PA_DTYPE_U8>(a, stream, sm_count);
        case PA_DTYPE_F16: return launch_score_t<D, BS, PA_DTYPE_F16>(a, stream, sm_count);
        case PA_DTYPE_BF16: return launch_score_t<D, BS, PA_DTYPE_BF16>(a, stream, sm_count);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_scores(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches) {
    if (!a.scores || !a.score_aggregation_window || a.num_sequences <= 0) return cudaSuccess;
    cudaError_t e = cudaErrorInvalidValue;
    if (a.g.D == 128 && a.g.bs == 32) e = launch_score_c<128, 32>(a, stream, sm_count);
    else if (a.g.D == 128 && a.g.bs == 16) e = launch_score_c<128, 16>(a, stream, sm_count);
    else if (a.g.D == 64 && a.g.bs == 32) e = launch_score_c<64, 32>(a, stream, sm_count);
    else if (a.g.D == 64 && a.g.bs == 16) e = launch_score_c<64, 16>(a, stream, sm_count);
    if (e != cudaSuccess) return e;
    ++*launches;
    const int gx = (int)std::max<long long>(1, std::min<long long>((a.max_context_len + 255) / 256, 64));
    score_reduce_kernel<<<dim3(gx, a.num_sequences), 256, 0, stream>>>(a);
    ++*launches;
    return cudaGetLastError();
}

}  // namespace pa
