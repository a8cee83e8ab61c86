// Paged decode attention for sm_100a: rows with exactly one new token.
//
// Persistent kernel: the grid is (resident CTAs per SM) x (SM count) and every WARP is an
// independent worker.  The 32-token tiles of all (decode row, head tile) "streams" form one
// global sequence (row-major, then head tile, then position); the plan step of the cache-write
// launch publishes its per-row prefix sum, and worker w takes the w-th equal slice of that
// sequence.  A slice crosses at most a few stream boundaries, so a warp reduces one to three
// "runs", each into one partial result; no queue, no atomics on the load path.
// A warp owns a private shared-memory ring whose loads run ahead of the math across run
// boundaries:
//   * u8 cache   - lane 0 issues one TMA-engine bulk copy per (block, head) record (data +
//                  per-token scale / zero-point, contiguous and 16-byte aligned), completion on
//                  an mbarrier; bytes become exact f16 in registers (byte | 0x6400 = 1024 + byte)
//                  and both offsets are folded algebraically:
//                     q.k  = ks * (q.(1024 + k_u8) - (kz + 1024) * sum(q))
//                     p.v  = sum_t (p*vs)_t * (1024 + v_u8) - sum_t (p*vs)_t * (vz_t + 1024)
//   * f16 / bf16 - all lanes issue 16-byte cp.async into an XOR-swizzled tile read by ldmatrix.
// Q.K^T and P.V run on mma.sync m16n8k16 with the GQA group as the M dimension, so a KV byte is
// read from HBM once for all q heads that share it.  Softmax is online with a lazily updated
// reference maximum.  A stream cut by slice boundaries is merged by the warp whose partial
// completes it (one atomic counter per stream, no waiting).
// HBM-bound: 2*Hkv*(D+8) bytes per context token for the u8 cache.
#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>

#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kTile = 32;  // context tokens per pipeline stage
constexpr int kDecodeWarps = 4;
constexpr int kDecodeMaxCtasPerSm = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLazyMax = 8.f;  // the running reference may lag the true row maximum by 2^8
constexpr int kFoldEvery = 4;     // u8: tiles between two removals of the zero-point term from the accumulators

enum : int { kFirst = 1, kLast = 2, kEnd = 4 };

// What the loader records for each ring stage; read by the whole warp when the tile is consumed.
struct __align__(16) StageDesc {
    int flags;  // kFirst (run starts: load Q, clear state) | kLast (run ends: publish) | kEnd
    int valid;  // live tokens in the tile (1..32)
    int run;    // index of the run's record in the warp's run ring
    int tok0;   // context position of the tile's first token
};

// One run (consecutive tiles of one stream inside a worker's slice), kept in shared memory so that
// it costs no registers while its tiles are in flight.
struct __align__(16) RunRec {
    int t0;          // row of the stream's token in query / output
    int hkp;         // head tile: kv head * gtiles + tile of the GQA group
    int stream;      // s * HK + hkp
    int nparts;      // workers whose slices touch the stream (1 => write the output directly)
    int first_slot;  // partial slot of the stream's first worker (slots are consecutive)
    int slot;        // this worker's partial slot
    long long score_off;  // index into score_raw of position 0 of the stream, -1: the row's logits are not kept
};
constexpr int kRunRing = 4;

template <int D, int BS, int CACHE>
struct DecodeCfg {
    static constexpr bool U8 = CACHE == PA_DTYPE_U8;
    static constexpr bool BF16 = CACHE == PA_DTYPE_BF16;
    static constexpr int REC = U8 ? BS * (D + 8) : BS * D * 2;  // bytes of one (block, head) record
    static constexpr int NREC = kTile / BS;                     // records per tile
    static constexpr int HALF_STAGE = NREC * REC;               // K part (V part has the same size)
    static constexpr int STAGE = 2 * HALF_STAGE;
#ifndef PA_DECODE_STAGES
#define PA_DECODE_STAGES 2
#endif
    static constexpr int NSTAGE = PA_DECODE_STAGES;
    static constexpr int RING = NSTAGE * STAGE;                 // per warp
    // rounded to 128 bytes: every warp's ring must start 16-byte aligned for bulk copies and 16-byte loads
    static constexpr int WARP_SMEM = (RING + NSTAGE * (int)sizeof(StageDesc) + kRunRing * (int)sizeof(RunRec) + NSTAGE * 8 + 127) / 128 * 128;
    static constexpr int SMEM = kDecodeWarps * WARP_SMEM;
    static_assert(WARP_SMEM % 16 == 0 && STAGE % 16 == 0 && REC % 16 == 0, "bulk copies and 16-byte loads need 16-byte aligned stages");
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void store_pair(void* out, long long idx, int act, float v0, float v1) {
    if (act == PA_DTYPE_F32) *reinterpret_cast<float2*>((float*)out + idx) = make_float2(v0, v1);
    else if (act == PA_DTYPE_F16) *reinterpret_cast<__half2*>((__half*)out + idx) = __floats2half2_rn(v0, v1);
    else *reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)out + idx) = __floats2bfloat162_rn(v0, v1);
}

#ifdef PA_DECODE_PROF
__device__ unsigned long long g_decode_prof[8192 * 8];   // per worker: start, first tile ready, end (ns), tiles, cycles waiting for tiles, cycles in all, cycles in produce
#endif

// SC: the launch keeps the scaled logits of rows whose scores are wanted (a.score_raw is set); a
// separate instantiation so that steps without a score output run the same code as before.
template <int D, int BS, int CACHE, bool HI, bool SC>
__global__ void __launch_bounds__(kDecodeWarps * 32, (HI || PA_DECODE_STAGES > 2) ? 2 : 3) decode_kernel(KernelArgs a) {
    using Cfg = DecodeCfg<D, BS, CACHE>;
    constexpr bool U8 = Cfg::U8;
    constexpr bool BF16 = Cfg::BF16;
    constexpr int NKK = D / 16;   // k-steps of Q.K^T
    constexpr int NDT = D / 8;    // n-tiles of P.V
    constexpr int ROWS = HI ? 2 : 1;
    constexpr int NS = Cfg::NSTAGE;

    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;
    uint8_t* ring = smem + warp * Cfg::WARP_SMEM;
    StageDesc* descs = reinterpret_cast<StageDesc*>(ring + Cfg::RING);
    RunRec* runs = reinterpret_cast<RunRec*>(ring + Cfg::RING + NS * sizeof(StageDesc));
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + Cfg::RING + NS * sizeof(StageDesc) + kRunRing * sizeof(RunRec));
    if constexpr (U8) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < NS; ++i) mbar_init(&bars[i], 1);
            mbar_fence_init();
        }
        __syncwarp();
    }

    const int G = a.g.Hq / a.g.Hkv;
    const int gtiles = (G + 15) / 16;
    const int HK = a.g.Hkv * gtiles;
    const int RT = a.rows_per_tile;
    const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)D);
    bool bad_index = false;
    // everything below reads what the launch before this one wrote (plan, start records, cache)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- this worker's slice of the global tile sequence -----------------------------------------
    const int all_workers = gridDim.x * kDecodeWarps;
    const int wid = blockIdx.x * kDecodeWarps + warp;
    WorkerStart ws0;
    ws0.s = -1;
    if (a.worker_start && a.decode_all_workers == all_workers) {   // one start record per worker
        const int4 lo4 = __ldcg(reinterpret_cast<const int4*>(a.worker_start + wid));
        const int4 hi4 = __ldcg(reinterpret_cast<const int4*>(a.worker_start + wid) + 1);
        ws0 = WorkerStart{lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
    }
    const int total_tiles = ws0.s != -1 ? ws0.total_tiles : a.plan->total_tiles;   // all streams
    const DecodeSlices sl = decode_slices(total_tiles, all_workers);
    int g_tile = 0, g_end = 0;       // next global tile to load, end of the slice

    // ---- loader state (warp-uniform registers) -------------------------------------------------------
    int r_s = -1, r_hkp = 0, r_tiles = 0;   // current stream: row, head tile, tiles of the row per head tile
    int r_tok = 0, r_end = 0;                // token cursor and end of the current run
    int r_tb = 0, r_nb = 0, r_seq = 0;       // block table of the row, run counter
    int w_blk0 = 0, tbl = 0;                 // block window: lane j holds block_indices[r_tb + w_blk0 + j]
    bool r_first = false;
    bool dropped_once = false;

    auto load_window = [&](int first_block) {
        w_blk0 = first_block;
        const int bi = first_block + lane;
        int blk = 0;
        if (bi < r_nb) {
            blk = a.block_indices[r_tb + bi];
            if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
        }
        tbl = blk;
    };

    // Common part of starting a run at tile `tile0` of stream (r_s, r_hkp).
    auto start_run = [&](int tile0, int p0, int ctx, int t0row) {
        const int ntile = min(r_tiles - tile0, g_end - g_tile);
        r_tok = tile0 * kTile;
        r_end = min(ctx, (tile0 + ntile) * kTile);
        const int s_begin = p0 * HK + r_hkp * r_tiles;             // global tile range of the stream
        const int first_w = sl.worker_of(s_begin), last_w = sl.worker_of(s_begin + r_tiles - 1);
        const int stream = r_s * HK + r_hkp;
        ++r_seq;
        if (lane == 0) {
            // rows whose attention scores are wanted (window > 0) leave their scaled logits behind
            long long score_off = -1;
            if constexpr (SC) {
                if (a.score_aggregation_window[r_s] > 0) {
                    // the row's slot must lie inside `scores` (and so inside score_raw, which is sized from
                    // the same scores_len): a caller's scores_len shorter than the metadata implies is
                    // reported, and the row leaves no logits behind
                    const long long off = a.score_offsets[r_s];
                    if (off >= 0 && off + ctx <= a.scores_len) score_off = ((long long)r_hkp * a.scores_len + off) * (RT <= 8 ? 8 : 16);
                    else atomicOr(a.status, PA_DEV_BAD_BEGINS);
                }
            }
            runs[r_seq % kRunRing] = RunRec{t0row, r_hkp, stream, last_w - first_w + 1, stream + first_w, stream + wid, score_off};
        }
        g_tile += ntile;
        r_first = true;
        load_window(r_tok / BS);
    };
    // Moves the loader to its next run: the first tile of the next stream of the slice.  False when the slice is done.
    auto advance = [&]() -> bool {
        if (g_tile >= g_end) return false;
        if (++r_hkp == HK) {
            r_hkp = 0;
            do {
                ++r_s;
                r_tiles = __ldcg(a.tile_prefix + r_s + 1) - __ldcg(a.tile_prefix + r_s);
            } while (r_tiles == 0);
        }
        r_tb = a.block_indices_begins[r_s];
        r_nb = a.block_indices_begins[r_s + 1] - r_tb;
        start_run(0, __ldcg(a.tile_prefix + r_s), a.past_lens[r_s] + 1, a.subsequence_begins[r_s]);
        return true;
    };
    // The worker's own slice: from the record the plan step prepared, else by binary search in the prefix sums.
    g_tile = (int)sl.begin(wid);
    g_end = (int)sl.end(wid);
    if (g_tile < g_end) {
        int p0, ctx, t0row;
        if (ws0.s >= 0) {
            r_s = ws0.s;
            p0 = ws0.p0;
            r_tiles = ws0.r_tiles;
            ctx = ws0.ctx; r_tb = ws0.tb; r_nb = ws0.nb; t0row = ws0.t0;
        } else {
            const int key = g_tile / HK;
            int lo = 0, hi = a.num_sequences;  // tile_prefix[lo] <= key < tile_prefix[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (__ldcg(a.tile_prefix + mid) <= key) lo = mid; else hi = mid;
            }
            r_s = lo;
            p0 = __ldcg(a.tile_prefix + r_s);
            r_tiles = __ldcg(a.tile_prefix + r_s + 1) - p0;
            ctx = a.past_lens[r_s] + 1;
            r_tb = a.block_indices_begins[r_s];
            r_nb = a.block_indices_begins[r_s + 1] - r_tb;
            t0row = a.subsequence_begins[r_s];
        }
        const int off = g_tile - p0 * HK;
        r_hkp = off / r_tiles;
        start_run(off % r_tiles, p0, ctx, t0row);
    }

    // Issues the next tile of the load stream into ring stage `slot` and records its descriptor.
#ifdef PA_DECODE_PROF
    long long prof_adv = 0, prof_tma = 0;
#endif
    auto produce = [&](int slot) {
#ifdef PA_DECODE_PROF
        const long long prof_a0 = clock64();
#endif
        if (r_tok >= r_end && !advance()) {
            if (lane == 0) descs[slot] = StageDesc{kEnd, 0, 0, 0};
            if constexpr (!U8) cp_async_commit();
            return;
        }
        uint8_t* st = ring + slot * Cfg::STAGE;
        const int hk = r_hkp / gtiles;
        const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)hk * a.g.head_bytes;
        const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)hk * a.g.head_bytes;
        const int bi0 = r_tok / BS;
        if (bi0 + Cfg::NREC - 1 - w_blk0 >= 32) load_window(bi0);
#ifdef PA_DECODE_PROF
        prof_adv += clock64() - prof_a0;
#endif
        int blocks[Cfg::NREC];
        bool live[Cfg::NREC];
#pragma unroll
        for (int r = 0; r < Cfg::NREC; ++r) {
            live[r] = (bi0 + r) * BS < r_end;
            blocks[r] = __shfl_sync(0xffffffffu, tbl, (bi0 + r - w_blk0) & 31);
        }
        if constexpr (U8) {
            // Test hook (PA_B200_TEST_DROP_FIRST_COPY): worker 0 arms the barrier of its first tile and issues no copy,
            // so that the bounded wait below runs out; nothing is in flight for that stage when it does.
            const bool drop = a.test_drop_copy && wid == 0 && !dropped_once;
            dropped_once = true;
#ifdef PA_DECODE_PROF
            const long long prof_b0 = clock64();
#endif
            if (lane == 0) {
                uint32_t bytes = 0;
#pragma unroll
                for (int r = 0; r < Cfg::NREC; ++r) bytes += live[r] ? 2 * Cfg::REC : 0;
                mbar_expect_tx(&bars[slot], bytes);
            }
            // one copy per lane (key / value record of each block of the tile): the copies of a tile leave as one
            // warp instruction instead of one after the other
            if (lane < 2 * Cfg::NREC) {
                const int r = lane >> 1;
                const bool is_v = lane & 1;
                int blk = blocks[0];
                bool lv = live[0];
                if constexpr (Cfg::NREC > 1) {
                    if (r == 1) { blk = blocks[1]; lv = live[1]; }
                }
                if (lv && !drop)
                    bulk_g2s(st + (is_v ? Cfg::HALF_STAGE : 0) + r * Cfg::REC, (is_v ? vc : kc) + (long long)blk * a.g.block_bytes, Cfg::REC, &bars[slot]);
            }
#ifdef PA_DECODE_PROF
            prof_tma += clock64() - prof_b0;
#endif
        } else {
            constexpr int CPR = D / 8;  // 16-byte chunks per token row
#pragma unroll
            for (int r = 0; r < Cfg::NREC; ++r)
                if (live[r]) {
                    const uint8_t* ksrc = kc + (long long)blocks[r] * a.g.block_bytes;
                    const uint8_t* vsrc = vc + (long long)blocks[r] * a.g.block_bytes;
#pragma unroll
                    for (int i = lane; i < BS * CPR; i += 32) {
                        const int row = r * BS + i / CPR, ch = i % CPR;
                        const int dst = row * (2 * D) + ((ch ^ (row & 7)) << 4);
                        cp_async16(st + dst, ksrc + (long long)i * 16);
                        cp_async16(st + Cfg::HALF_STAGE + dst, vsrc + (long long)i * 16);
                    }
                }
            cp_async_commit();
        }
        const int valid = min(kTile, r_end - r_tok);
        const bool last = r_tok + kTile >= r_end;
        if (lane == 0)
            descs[slot] = StageDesc{(r_first ? kFirst : 0) | (last ? kLast : 0), valid, r_seq % kRunRing, r_tok};
        r_first = false;
        r_tok += kTile;
    };

    // ---- consumer state --------------------------------------------------------------------------
    uint32_t qa[NKK][4];
    float qsum[ROWS], qscale[ROWS];
    float oacc[NDT][2 * ROWS];
    float m_run[ROWS], l_run[ROWS], z_run[ROWS];
    int hbase = 0, hcount = 0, t0 = 0;

#ifdef PA_DECODE_PROF
    unsigned long long prof_t[4] = {0, 0, 0, 0};
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_t[0]));
    long long prof_wait = 0, prof_prod = 0;
    const long long prof_c0 = clock64();
#endif
#pragma unroll
    for (int p = 0; p < NS - 1; ++p) produce(p);

    for (int it = 0;; ++it) {
        __syncwarp();  // every lane is done with the stage that is refilled next
#ifdef PA_DECODE_PROF
        const long long prof_p0 = clock64();
#endif
        produce((it + NS - 1) % NS);
        __syncwarp();
#ifdef PA_DECODE_PROF
        const long long prof_w0 = clock64();
        prof_prod += prof_w0 - prof_p0;
#endif
        const int slot = it % NS;
        const StageDesc d = descs[slot];
        if (d.flags & kEnd) break;
        if constexpr (U8) {
            if (!mbar_wait_bounded(&bars[slot], (it / NS) & 1, a.test_drop_copy ? (1u << 10) : (1u << 22))) {
                // the copy never arrived: flag it, let the copies of the other stages land (bounded), and leave
                if (lane == 0) atomicOr(a.status, PA_DEV_WAIT_TIMEOUT_DECODE);
#pragma unroll
                for (int o = 1; o < NS; ++o) {
                    const int other = (it + o) % NS;
                    if (!(descs[other].flags & kEnd)) mbar_wait_bounded(&bars[other], ((it + o) / NS) & 1, 1u << 16);
                }
                break;
            }
        } else {
            cp_async_wait<NS - 1>();
            __syncwarp();
        }
#ifdef PA_DECODE_PROF
        if (it == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_t[1]));
        prof_wait += clock64() - prof_w0;
#endif
        const uint8_t* st = ring + slot * Cfg::STAGE;
        const int valid = d.valid;

        if (d.flags & kFirst) {
            // ---- Q fragments of the run -------------------------------------------------------------
            // u8: the contraction index is permuted so that one 16-byte shared load of a key row
            // feeds four k-steps: k-step 4*half + i covers dims 64*half + 16*c + 4*i + {0..3}.
            t0 = runs[d.run].t0;
            const int hkp = runs[d.run].hkp;
            const int hk = hkp / gtiles;
            hbase = hk * G + (hkp % gtiles) * 16;
            hcount = min(16, hk * G + G - hbase);
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const int hrow = g + 8 * r;
                const bool live = hrow < hcount;
                const long long qoff = ((long long)t0 * a.g.Hq + hbase + hrow) * D;
                float q[D / 4];
                float amax = 0.f;
#pragma unroll
                for (int e = 0; e < D / 4; ++e) {
                    int dd;
                    if constexpr (U8) dd = 64 * (e / 16) + 16 * c + (e % 16);
                    else dd = 16 * (e / 4) + 2 * c + (e & 1) + 8 * ((e >> 1) & 1);
                    q[e] = live ? load_act(a.query, qoff + dd, a.g.act) : 0.f;
                    amax = fmaxf(amax, fabsf(q[e]));
                }
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                float qmul = 1.f;  // exact power-of-two prescale that keeps |q| inside the f16 range
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
                        __half2 h = *reinterpret_cast<__half2*>(&packed);
                        sum += __low2float(h) + __high2float(h);
                    }
                    qa[e / 4][r + 2 * ((e >> 1) & 1)] = packed;
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                qsum[r] = sum;
                qscale[r] = sm_scale * kLog2e / qmul;
                m_run[r] = -INFINITY; l_run[r] = 0.f; z_run[r] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < NDT; ++i)
#pragma unroll
                for (int r = 0; r < 2 * ROWS; ++r) oacc[i][r] = 0.f;
        }

        if constexpr (!U8) {
            if (valid < kTile) {  // stale rows of a partly filled block may hold NaN bit patterns
                constexpr int CPR = D / 8;
                for (int i = lane; i < (kTile - valid) * CPR; i += 32) {
                    const int row = valid + i / CPR, ch = i % CPR;
                    *reinterpret_cast<uint4*>(const_cast<uint8_t*>(st) + Cfg::HALF_STAGE + row * 2 * D + (ch << 4)) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
        }

        // ---- S = Q.K^T over four 8-token n-tiles ------------------------------------------------
        float sacc[4][2 * ROWS];
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
                    for (int i = 0; i < 4; ++i)  // bytes stay offset by 1024; removed with the zero-point
                        mma16816<false, HI>(acc4, qa[4 * h + i], __byte_perm(ww[i], 0x64646464u, 0x4140),
                                            __byte_perm(ww[i], 0x64646464u, 0x4342));
                }
            } else {
#pragma unroll
                for (int p = 0; p < NKK / 2; ++p) {
                    const int row = 8 * j + (lane & 7), ch = 4 * p + (lane >> 3);
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(st + row * 2 * D + ((ch ^ (row & 7)) << 4)));
                    mma16816<BF16, HI>(acc4, qa[2 * p], b[0], b[1]);
                    mma16816<BF16, HI>(acc4, qa[2 * p + 1], b[2], b[3]);
                }
            }
            sacc[j][0] = acc4[0]; sacc[j][1] = acc4[1];
            if constexpr (HI) { sacc[j][2] = acc4[2]; sacc[j][3] = acc4[3]; }
        }

        // ---- scale, mask, online softmax -----------------------------------------------------------
        float vsc[4][2], vzp[4][2];
        float tmax[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) tmax[r] = -INFINITY;
        // Score output of decode rows: the scaled logits (base 2) of every (position, q head) are left in
        // score_raw[head tile][position][8 or 16 head rows]; the score step turns them into probabilities
        // once the row's log-sum-exp is known, instead of reading the keys and multiplying a second time.
        // All 8 lanes of a token write, dead head rows too, so that every store fills whole 32-byte sectors.
        constexpr int SL = 8 * ROWS;
        float* score_dst = nullptr;
        if constexpr (SC) {
            const long long so = runs[d.run].score_off;
            if (so >= 0) score_dst = a.score_raw + so + (long long)d.tok0 * SL + g;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tk = U8 ? 8 * c + 2 * j : 8 * j + 2 * c;  // tile token of accumulator column 0
            float ks0 = 1.f, ks1 = 1.f, kz0 = 0.f, kz1 = 0.f;
            if constexpr (U8) {
                const uint8_t* kp = st + (tk / BS) * Cfg::REC + BS * D;
                const float2 ks = *reinterpret_cast<const float2*>(kp + 4 * (tk % BS));
                const float2 kz = *reinterpret_cast<const float2*>(kp + 4 * BS + 4 * (tk % BS));
                ks0 = ks.x; ks1 = ks.y; kz0 = kz.x + 1024.f; kz1 = kz.y + 1024.f;
                const uint8_t* vp = st + Cfg::HALF_STAGE + (tk / BS) * Cfg::REC + BS * D;
                const float2 vs = *reinterpret_cast<const float2*>(vp + 4 * (tk % BS));
                const float2 vz = *reinterpret_cast<const float2*>(vp + 4 * BS + 4 * (tk % BS));
                vsc[j][0] = vs.x; vsc[j][1] = vs.y; vzp[j][0] = vz.x + 1024.f; vzp[j][1] = vz.y + 1024.f;
            }
            const bool ok0 = tk < valid, ok1 = tk + 1 < valid;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float s0 = sacc[j][2 * r], s1 = sacc[j][2 * r + 1];
                if constexpr (U8) {
                    s0 = (s0 - kz0 * qsum[r]) * (ks0 * qscale[r]);
                    s1 = (s1 - kz1 * qsum[r]) * (ks1 * qscale[r]);
                } else {
                    s0 *= qscale[r]; s1 *= qscale[r];
                }
                s0 = ok0 ? s0 : -INFINITY;
                s1 = ok1 ? s1 : -INFINITY;
                if constexpr (SC) {
                    if (score_dst) {
                        if (ok0) __stcs(score_dst + tk * SL + 8 * r, s0);
                        if (ok1) __stcs(score_dst + (tk + 1) * SL + 8 * r, s1);
                    }
                }
                sacc[j][2 * r] = s0; sacc[j][2 * r + 1] = s1;
                tmax[r] = fmaxf(tmax[r], fmaxf(s0, s1));
            }
        }
        // The reference maximum is raised only when the tile maximum exceeds it by more than
        // kLazyMax (warp-uniform decision), so most tiles skip the rescale of the accumulators.
        bool grow = false;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float mx = tmax[r];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            tmax[r] = mx;
            grow |= mx > m_run[r] + kLazyMax;
        }
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const float m_new = fmaxf(m_run[r], tmax[r]);
                const float alpha = fast_exp2(m_run[r] - m_new);  // 0 on the first tile
                m_run[r] = m_new;
                l_run[r] *= alpha;
                z_run[r] *= alpha;
#pragma unroll
                for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] *= alpha; oacc[i][2 * r + 1] *= alpha; }
            }
        }
        uint32_t pa_frag[2][4];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float lsum = 0.f, zsum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float p0 = fast_exp2(sacc[j][2 * r] - m_run[r]), p1 = fast_exp2(sacc[j][2 * r + 1] - m_run[r]);
                lsum += p0 + p1;
                uint32_t packed;
                if constexpr (U8) {
                    const int tk = 8 * c + 2 * j;
                    // masked tokens have p == 0; the select keeps garbage scale bits (NaN) out
                    packed = pack_h2(tk < valid ? p0 * vsc[j][0] : 0.f, tk + 1 < valid ? p1 * vsc[j][1] : 0.f);
                    const __half2 h = *reinterpret_cast<__half2*>(&packed);
                    zsum += (tk < valid ? __low2float(h) * vzp[j][0] : 0.f) + (tk + 1 < valid ? __high2float(h) * vzp[j][1] : 0.f);
                } else if constexpr (BF16) {
                    packed = pack_bf2(p0, p1);
                } else {
                    packed = pack_h2(p0, p1);
                }
                pa_frag[j >> 1][r + 2 * (j & 1)] = packed;
            }
            l_run[r] += lsum;
            z_run[r] += zsum;
        }
        if constexpr (!HI) { pa_frag[0][1] = pa_frag[0][3] = pa_frag[1][1] = pa_frag[1][3] = 0u; }

        // ---- O += P.V -----------------------------------------------------------------------------
        if constexpr (U8) {
#pragma unroll
            for (int i = 0; i < NDT; ++i) {
                const int dd = 8 * i + g;
                const uint8_t* vp = st + Cfg::HALF_STAGE + ((8 * c) / BS) * Cfg::REC + dd * BS + ((8 * c) % BS);
                const uint2 w = *reinterpret_cast<const uint2*>(vp);
                float acc4[4];
                acc4[0] = oacc[i][0]; acc4[1] = oacc[i][1];
                if constexpr (HI) { acc4[2] = oacc[i][2]; acc4[3] = oacc[i][3]; }
                mma16816<false, HI>(acc4, pa_frag[0], __byte_perm(w.x, 0x64646464u, 0x4140), __byte_perm(w.x, 0x64646464u, 0x4342));
                mma16816<false, HI>(acc4, pa_frag[1], __byte_perm(w.y, 0x64646464u, 0x4140), __byte_perm(w.y, 0x64646464u, 0x4342));
                oacc[i][0] = acc4[0]; oacc[i][1] = acc4[1];
                if constexpr (HI) { oacc[i][2] = acc4[2]; oacc[i][3] = acc4[3]; }
            }
        } else {
#pragma unroll
            for (int kt = 0; kt < 2; ++kt)
#pragma unroll
                for (int q = 0; q < NDT / 2; ++q) {
                    const int row = 16 * kt + 8 * ((lane >> 3) & 1) + (lane & 7), ch = 2 * q + (lane >> 4);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(st + Cfg::HALF_STAGE + row * 2 * D + ((ch ^ (row & 7)) << 4)));
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int i = 2 * q + e;
                        float acc4[4];
                        acc4[0] = oacc[i][0]; acc4[1] = oacc[i][1];
                        if constexpr (HI) { acc4[2] = oacc[i][2]; acc4[3] = oacc[i][3]; }
                        mma16816<BF16, HI>(acc4, pa_frag[kt], b[2 * e], b[2 * e + 1]);
                        oacc[i][0] = acc4[0]; oacc[i][1] = acc4[1];
                        if constexpr (HI) { oacc[i][2] = acc4[2]; oacc[i][3] = acc4[3]; }
                    }
                }
        }

        if (!(d.flags & kLast)) {
            if constexpr (U8) {
                // The value bytes enter the MMA as 1024 + byte, so the accumulators carry about a
                // thousand times the magnitude of the result until the zero-point term is taken out,
                // and the tensor core truncates every accumulation at that magnitude: over thousands
                // of tiles the lost bits add up to a visible bias. Taking the term out every few
                // tiles keeps the accumulators near the size of the result.
                if ((it & (kFoldEvery - 1)) == kFoldEvery - 1) {
#pragma unroll
                    for (int r = 0; r < ROWS; ++r) {
                        float z = z_run[r];
                        z += __shfl_xor_sync(0xffffffffu, z, 1); z += __shfl_xor_sync(0xffffffffu, z, 2);
                        z_run[r] = 0.f;
#pragma unroll
                        for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] -= z; oacc[i][2 * r + 1] -= z; }
                    }
                }
            }
            continue;
        }

        // ---- end of the run: fold the zero-point term, publish ---------------------------------------
        float lrow[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float l = l_run[r], z = z_run[r];
            l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
            z += __shfl_xor_sync(0xffffffffu, z, 1); z += __shfl_xor_sync(0xffffffffu, z, 2);
            lrow[r] = l;
#pragma unroll
            for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] -= z; oacc[i][2 * r + 1] -= z; }
        }
        const RunRec fin = runs[d.run];
        if (fin.nparts == 1) {  // the run is the whole stream
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                const int hrow = g + 8 * r;
                if (hrow >= hcount) continue;
                const long long row = (long long)t0 * a.g.Hq + hbase + hrow;
                const float inv = 1.f / lrow[r];
#pragma unroll
                for (int i = 0; i < NDT; ++i) store_pair(a.output, row * D + 8 * i + 2 * c, a.g.act, oacc[i][2 * r] * inv, oacc[i][2 * r + 1] * inv);
                if (c == 0 && a.lse) a.lse[row] = (m_run[r] + log2f(lrow[r])) * kLn2;
            }
            continue;
        }
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int hrow = g + 8 * r;
            if (hrow >= hcount) continue;
            const long long prow = (long long)fin.slot * RT + hrow;
#pragma unroll
            for (int i = 0; i < NDT; ++i)
                __stcg(reinterpret_cast<float2*>(a.part_o + prow * D + 8 * i + 2 * c), make_float2(oacc[i][2 * r], oacc[i][2 * r + 1]));
            if (c == 0) __stcg(reinterpret_cast<float2*>(a.part_ml + prow * 2), make_float2(m_run[r], lrow[r]));
        }
        __threadfence();
        __syncwarp();
        int done = 0;
        if (lane == 0) done = atomicAdd(&a.stream_done[fin.stream], 1) + 1;
        done = __shfl_sync(0xffffffffu, done, 0);
        if (done != fin.nparts) continue;
        // ---- this partial completed the stream: merge all of its partials ---------------------------
        __threadfence();
        const int nparts = fin.nparts;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int hrow = g + 8 * r;
            if (hrow >= hcount) continue;
            float m = -INFINITY;
            float l = 0.f;
            float o[NDT][2];
#pragma unroll
            for (int i = 0; i < NDT; ++i) { o[i][0] = 0.f; o[i][1] = 0.f; }
            // the partials are read in groups of four with all loads of a group in flight together
            for (int j0 = 0; j0 < nparts; j0 += 4) m = fmaxf(m, [&] {
                float mm = -INFINITY;
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (j0 + u < nparts) mm = fmaxf(mm, __ldcg(a.part_ml + ((long long)(fin.first_slot + j0 + u) * RT + hrow) * 2));
                return mm;
            }());
            for (int j0 = 0; j0 < nparts; j0 += 4) {
                float f[4];
                long long prow[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const bool on = j0 + u < nparts;
                    prow[u] = (long long)(fin.first_slot + (on ? j0 + u : 0)) * RT + hrow;
                    const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.part_ml + prow[u] * 2));
                    f[u] = on ? fast_exp2(ml.x - m) : 0.f;
                    l += f[u] * ml.y;
                }
#pragma unroll
                for (int i = 0; i < NDT; ++i) {
                    float2 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float2*>(a.part_o + prow[u] * D + 8 * i + 2 * c));
#pragma unroll
                    for (int u = 0; u < 4; ++u) { o[i][0] += f[u] * v[u].x; o[i][1] += f[u] * v[u].y; }
                }
            }
            const long long row = (long long)t0 * a.g.Hq + hbase + hrow;
            const float inv = 1.f / l;
#pragma unroll
            for (int i = 0; i < NDT; ++i) store_pair(a.output, row * D + 8 * i + 2 * c, a.g.act, o[i][0] * inv, o[i][1] * inv);
            if (c == 0 && a.lse) a.lse[row] = (m + log2f(l)) * kLn2;
        }
    }
    if constexpr (!U8) cp_async_wait<0>();
    if (__any_sync(0xffffffffu, bad_index) && lane == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
#ifdef PA_DECODE_PROF
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_t[3]));
    if (lane == 0 && wid < 8192) {
        g_decode_prof[wid * 8 + 0] = prof_t[0];
        g_decode_prof[wid * 8 + 1] = prof_t[1] - prof_t[0];
        g_decode_prof[wid * 8 + 2] = prof_t[3] - prof_t[0];
        g_decode_prof[wid * 8 + 3] = (unsigned long long)(sl.end(wid) - sl.begin(wid));
        g_decode_prof[wid * 8 + 4] = (unsigned long long)prof_wait;
        g_decode_prof[wid * 8 + 5] = (unsigned long long)(clock64() - prof_c0);
        g_decode_prof[wid * 8 + 6] = (unsigned long long)prof_prod;
        g_decode_prof[wid * 8 + 7] = ((unsigned long long)prof_adv << 32) | (unsigned long long)(prof_tma & 0xffffffffll);
    }
#endif
}

// CTAs of the launch: the resident ones; never more workers than slices could exist (upper bound known on the host).
long long decode_ctas(const KernelArgs& a, int per_sm, int sm_count) {
    const long long max_slices = (a.max_tiles + kDecodeMinSlice - 1) / kDecodeMinSlice;
    const long long cap = std::max(1LL, (max_slices + kDecodeWarps - 1) / kDecodeWarps);
    return std::max(1LL, std::min((long long)std::min(per_sm, kDecodeMaxCtasPerSm) * sm_count, cap));
}

// Resident CTAs per SM of one instantiation on the current device; the shared-memory opt-in and the
// occupancy query are made once per (instantiation, device), not on every step.
template <int D, int BS, int CACHE>
int occupancy_t(const KernelArgs& a) {
    using Cfg = DecodeCfg<D, BS, CACHE>;
    constexpr int kMaxDevices = 64;
    static std::atomic<int> cache[4][kMaxDevices];   // 0 = unknown, else per_sm + 1
    const bool hi = a.g.Hq / a.g.Hkv > 8;
    const bool sc = a.score_raw != nullptr && a.score_aggregation_window != nullptr;
    const int slot = (hi ? 2 : 0) + (sc ? 1 : 0);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    const bool cached = dev >= 0 && dev < kMaxDevices;
    if (cached) {
        const int v = cache[slot][dev].load(std::memory_order_acquire);
        if (v > 0) return v - 1;
    }
    auto kern = hi ? (sc ? decode_kernel<D, BS, CACHE, true, true> : decode_kernel<D, BS, CACHE, true, false>)
                   : (sc ? decode_kernel<D, BS, CACHE, false, true> : decode_kernel<D, BS, CACHE, false, false>);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) return 0;
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDecodeWarps * 32, Cfg::SMEM) != cudaSuccess) return 0;
    if (cached) cache[slot][dev].store(per_sm + 1, std::memory_order_release);
    return per_sm;
}

template <int D, int BS, int CACHE>
cudaError_t launch_decode_t(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0, cudaEvent_t ev1) {
    using Cfg = DecodeCfg<D, BS, CACHE>;
    const int G = a.g.Hq / a.g.Hkv;
    const bool hi = G > 8;
    const bool sc = a.score_raw != nullptr && a.score_aggregation_window != nullptr;
    auto kern = hi ? (sc ? decode_kernel<D, BS, CACHE, true, true> : decode_kernel<D, BS, CACHE, true, false>)
                   : (sc ? decode_kernel<D, BS, CACHE, false, true> : decode_kernel<D, BS, CACHE, false, false>);
    const int per_sm = occupancy_t<D, BS, CACHE>(a);
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    const long long ctas = decode_ctas(a, per_sm, sm_count);
    if (ev0) cudaEventRecord(ev0, stream);
    // Programmatic dependent launch: the launch is queued behind the cache-write kernel without a full
    // stream serialisation; that kernel never triggers early, so the CTAs start when it has finished, and
    // they still wait (griddepcontrol.wait) before the first read of anything it writes.  An event record
    // in between (kernel timing) serialises as usual.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kDecodeWarps * 32);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) return e;
    if (ev1) cudaEventRecord(ev1, stream);
    ++*launches;
    return cudaGetLastError();
}

template <int D, int BS>
cudaError_t launch_decode_c(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0, cudaEvent_t ev1) {
    switch (a.g.cache) {
        case PA_DTYPE_U8: return launch_decode_t<D, BS, PA_DTYPE_U8>(a, stream, sm_count, launches, ev0, ev1);
        case PA_DTYPE_F16: return launch_decode_t<D, BS, PA_DTYPE_F16>(a, stream, sm_count, launches, ev0, ev1);
        case PA_DTYPE_BF16: return launch_decode_t<D, BS, PA_DTYPE_BF16>(a, stream, sm_count, launches, ev0, ev1);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

int decode_max_workers(int sm_count) { return sm_count * kDecodeMaxCtasPerSm * kDecodeWarps; }

int decode_launch_workers(const KernelArgs& a, int sm_count) {
    if (a.num_sequences <= 0) return 0;
    int per_sm = 0;
#define PA_OCC(D_, BS_)                                                                           \
    switch (a.g.cache) {                                                                          \
        case PA_DTYPE_U8: per_sm = occupancy_t<D_, BS_, PA_DTYPE_U8>(a); break;                   \
        case PA_DTYPE_F16: per_sm = occupancy_t<D_, BS_, PA_DTYPE_F16>(a); break;                 \
        case PA_DTYPE_BF16: per_sm = occupancy_t<D_, BS_, PA_DTYPE_BF16>(a); break;               \
    }
    if (a.g.D == 128 && a.g.bs == 32) { PA_OCC(128, 32) }
    else if (a.g.D == 128 && a.g.bs == 16) { PA_OCC(128, 16) }
    else if (a.g.D == 64 && a.g.bs == 32) { PA_OCC(64, 32) }
    else if (a.g.D == 64 && a.g.bs == 16) { PA_OCC(64, 16) }
#undef PA_OCC
    if (per_sm < 1) return 0;
    return (int)decode_ctas(a, per_sm, sm_count) * kDecodeWarps;
}

cudaError_t launch_decode(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0, cudaEvent_t ev1) {
    if (a.num_sequences <= 0) return cudaSuccess;
    if (a.g.D == 128 && a.g.bs == 32) return launch_decode_c<128, 32>(a, stream, sm_count, launches, ev0, ev1);
    if (a.g.D == 128 && a.g.bs == 16) return launch_decode_c<128, 16>(a, stream, sm_count, launches, ev0, ev1);
    if (a.g.D == 64 && a.g.bs == 32) return launch_decode_c<64, 32>(a, stream, sm_count, launches, ev0, ev1);
    if (a.g.D == 64 && a.g.bs == 16) return launch_decode_c<64, 16>(a, stream, sm_count, launches, ev0, ev1);
    return cudaErrorInvalidValue;
}

}  // namespace pa

#ifdef PA_DECODE_PROF
extern "C" int pa_b200_debug_read_decode_prof(void* dst, size_t bytes) {
    return (int)cudaMemcpyFromSymbol(dst, pa::g_decode_prof, bytes);
}
#endif
