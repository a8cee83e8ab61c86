// Paged decode attention for sm_100a, SM-shared variant: u8 cache, head size 128, up to 8 query heads per KV head.
//
// Same arithmetic as decode_kernel (pa_decode.cu) - mma.sync m16n8k16 with the GQA group on M, bytes as exact f16
// (1024 + byte), online softmax with a lazy reference maximum - but the work is handed out differently.  There, every
// warp owns a fixed slice of the tile sequence; warps of one launch run up to a factor two apart in speed and every
// stream boundary inside a slice costs a chain of dependent global loads, so the slowest warp decides the kernel time.
// Here one CTA per SM owns a slice and its warps take 32-token tiles from counters in shared memory:
//   * per "chapter" (up to kShRuns runs and ShCfg::TILES tiles) thread 0 walks the slice and lists its runs (consecutive
//     tiles of one stream); all threads then stage the block ids of every tile in shared memory and the query rows of
//     every run - f16, prescaled, in the register order of the fragments, with their sums - in a global scratch of the
//     CTA: the global metadata reads of the chapter are made once per CTA instead of once per warp;
//   * the warps spread over a window of kShAcc runs in proportion to the runs' tiles; every run hands its tiles out from
//     its own counter (atomicAdd in shared memory), a warp stays with a run until the run has no tile left and then moves
//     on inside the window, which slides as its first runs are used up; the loader of a warp looks run and block up in
//     the tables and issues the bulk copies into the warp's private two-stage ring;
//   * a warp that leaves a run adds its partial (m, l, O) to the run's accumulator in shared memory (a ring of kShAcc
//     accumulators, each behind a lock); the warp whose tiles complete the run takes the result out and either writes the
//     output (the stream lies in this CTA alone) or publishes the CTA's partial exactly as a worker of decode_kernel does
//     (slot = stream + CTA), the CTA that completes the stream merging the partials;
//   * the slices are cut in a sequence in which every stream is followed by a few tiles that do not exist
//     (KernelArgs::decode_phantom), so that a CTA whose slice holds many streams gets fewer tiles.
// The order in which partials are added depends on timing, so the last bits of the output differ between launches.
// No warp waits for another one except at chapter boundaries (__syncthreads) and at an accumulator's lock; every wait
// on an mbarrier or a lock is bounded, and one that runs out sets a status bit and makes the CTA stop taking tiles.
// HBM-bound: 2*Hkv*(D+8) bytes per context token.
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kTile = 32;
constexpr int kShMaxWarps = 12;
constexpr int kShRuns = 24;     // runs per chapter (ring of run records)
constexpr int kShAcc = 6;       // runs the warps spread over at a time = runs whose reduction can be open (ring of accumulators)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kLazyMax = 8.f;
constexpr int kFoldEvery = 4;
constexpr int kShQEntry = 2048 + 64;   // bytes of one staged query entry: 16 registers x 32 lanes in fragment order, then (sum, scale) of 8 rows
constexpr int kEndRun = -2;     // descriptor of a stage without a tile: the chapter has no more tiles

struct __align__(16) ShDesc {
    int run;    // run sequence number inside the CTA, kEndRun: no tile
    int valid;  // live tokens in the tile (1..32)
    int tok0;   // context position of the tile's first token
    int pad;
};

// One run of the CTA: consecutive tiles of one stream inside the CTA's slice.  Lives in a ring indexed by
// the run's sequence number; a run that is cut by a chapter boundary keeps its record.
struct __align__(16) ShRun {
    int t0;          // row of the stream's token in query / output
    int hk;          // kv head
    int stream;      // s * Hkv + hk
    int nparts;      // CTAs whose slices touch the stream (1 => write the output directly)
    int first_slot;  // partial slot of the stream's first CTA (slots are consecutive)
    int slot;        // this CTA's partial slot
    int total;       // tiles of the run (all chapters)
    int upto;        // tiles of the run handed out up to the end of this chapter
    int ctx;         // context length of the row
    int g_first;     // this chapter: index of the run's first tile in the chapter
    int n_ch;        // this chapter: tiles of the run
    int tok_base;    // this chapter: context position of that first tile
    int blk_base;    // this chapter: index of its first block id in the block table
    int next;        // this chapter: tiles of the run handed out so far (the run's own counter)
    long long score_off;  // index into score_raw of position 0 of the stream, -1: logits are not kept
    int tb, nb;      // block table of the row: begin and length
    int vtail;       // phantom tiles of the slicing sequence that follow the run
    int pad[3];
};
static_assert(sizeof(ShRun) % 16 == 0, "run records are copied as a whole");

// Header of one accumulator of the ring: the reduction of the warps' partials of one run.
struct __align__(16) ShAcc {
    int lock;    // 0 free, 1 held
    int turn;    // sequence number of the run this accumulator serves now: entry e serves the runs e, e + kShAcc, ... in order
    int tiles;   // tiles of that run reduced so far
    int pad;
};

// Walk state of thread 0 across chapters, and what it tells the CTA about the chapter.
struct ShCtl {
    int win_lo;      // first run of the chapter (index in the chapter) that still has tiles to hand out
    int abort;       // a wait ran out: nobody takes tiles any more
    int ntiles;      // tiles of the chapter
    int first_seq;   // sequence number of the chapter's first run
    int nruns;       // runs of the chapter
    int new_first;   // first run of the chapter whose query rows are not staged yet (sequence number)
    int more;        // the slice has tiles beyond this chapter
    int cont;        // the chapter's last run goes on in the next chapter
    int bad;         // a block id was out of range
    // walk
    int r_s, hk, r_tiles, p0, pos, ctx, tb, nb, t0row, g_tile, seq;
};

template <int D, int BS>
struct ShCfg {
    static constexpr int REC = BS * (D + 8);
    static constexpr int NREC = kTile / BS;
    static constexpr int HALF_STAGE = NREC * REC;
    static constexpr int STAGE = 2 * HALF_STAGE;
    static constexpr int NS = 2;
    static constexpr int WARP_SMEM = (NS * STAGE + NS * (int)sizeof(ShDesc) + NS * 8 + 127) / 128 * 128;
    static constexpr int TILES = BS == 32 ? 640 : 320;   // tiles per chapter (sizes the block table)
    static constexpr int AROW = D + 8;                   // floats per accumulator row (padding spreads the rows over the banks)
    static constexpr size_t tables(int rt) {
        return (sizeof(ShCtl) + 15) / 16 * 16 + kShRuns * sizeof(ShRun) + kShAcc * sizeof(ShAcc) + (size_t)TILES * NREC * sizeof(int) +
               (size_t)kShAcc * rt * (AROW * 4 + 8);
    }
    // 12 warps when the tables leave room for their rings, else 11 (more than 4 query heads per kv head)
    static constexpr int warps(int rt) { return (size_t)kShMaxWarps * WARP_SMEM + tables(rt) <= 232448 ? kShMaxWarps : kShMaxWarps - 1; }
    static constexpr size_t smem(int rt) { return (size_t)warps(rt) * WARP_SMEM + tables(rt); }
};

__device__ __forceinline__ float fast_exp2s(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void store_pair_s(void* out, long long idx, int act, float v0, float v1) {
    if (act == PA_DTYPE_F32) *reinterpret_cast<float2*>((float*)out + idx) = make_float2(v0, v1);
    else if (act == PA_DTYPE_F16) *reinterpret_cast<__half2*>((__half*)out + idx) = __floats2half2_rn(v0, v1);
    else *reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)out + idx) = __floats2bfloat162_rn(v0, v1);
}

// m16n8k16 with rows 8..15 of A zero: a0 / a2 are the two live A registers, c0 / c1 the live accumulators.
__device__ __forceinline__ void mma_lo(float& c0, float& c1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float t2, t3;
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
        : "+f"(c0), "+f"(c1), "=f"(t2), "=f"(t3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
    (void)t2; (void)t3;
}

// Reduces `n` partials (m, l, O) of `rt` rows each, laid out [partial][row][D] / [partial][row][2], with a whole
// warp: lane j owns the columns 4j..4j+3 of every row (D == 128), so a row of a partial is one coalesced 512-byte
// read, and the per-partial factors 2^(m - max) are computed by lane = partial and handed round by shuffles.
// `mask` selects partials (bit w, for n <= 32); pass all ones otherwise.  Results: acc[row] (unnormalised), m, l.
template <int D>
__device__ __forceinline__ void merge_partials(const float* po, const float* pml, int n, unsigned mask, int rt, int lane, float4 (&acc)[8],
                                               float (&mrow)[8], float (&lrow)[8]) {
    static_assert(D == 128, "one float4 per lane and row");
#pragma unroll
    for (int k = 0; k < 8; ++k) { acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); mrow[k] = -INFINITY; lrow[k] = 0.f; }
    for (int c0 = 0; c0 < n; c0 += 32) {
        const int w = c0 + lane;
        const bool on = w < n && ((mask >> (w & 31)) & 1u);
        const int cnt = min(32, n - c0);
        float fk[8];   // factor of partial w for each row
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            fk[k] = 0.f;
            if (k < rt) {
                float2 ml = make_float2(-INFINITY, 0.f);
                if (on) ml = __ldcg(reinterpret_cast<const float2*>(pml + ((long long)w * rt + k) * 2));
                float mx = ml.x;
#pragma unroll
                for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                const float m_new = fmaxf(mrow[k], mx);
                const float alpha = mrow[k] == -INFINITY ? 0.f : fast_exp2s(mrow[k] - m_new);
                const float f = on && ml.x != -INFINITY ? fast_exp2s(ml.x - m_new) : 0.f;
                float ls = f * ml.y;
#pragma unroll
                for (int o = 16; o; o >>= 1) ls += __shfl_xor_sync(0xffffffffu, ls, o);
                lrow[k] = lrow[k] * alpha + ls;
                acc[k].x *= alpha; acc[k].y *= alpha; acc[k].z *= alpha; acc[k].w *= alpha;
                mrow[k] = m_new;
                fk[k] = f;
            }
        }
        // O: four partials' rows in flight at a time
        for (int j0 = 0; j0 < cnt; j0 += 4) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (k < rt) {
                    float4 v[4];
                    float fw[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int j = j0 + u < cnt ? j0 + u : j0;
                        fw[u] = j0 + u < cnt ? __shfl_sync(0xffffffffu, fk[k], j) : 0.f;
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (fw[u] != 0.f) v[u] = __ldcg(reinterpret_cast<const float4*>(po + ((long long)(c0 + j) * rt + k) * D + 4 * lane));
                    }
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        acc[k].x += fw[u] * v[u].x; acc[k].y += fw[u] * v[u].y; acc[k].z += fw[u] * v[u].z; acc[k].w += fw[u] * v[u].w;
                    }
                }
            }
        }
    }
}

#ifdef PA_DECODE_PROF
__device__ unsigned long long g_shared_prof[8192 * 12];   // per warp: start, first tile ready, end (ns), tiles, cycles: wait, all, produce, flush
#define SPROF(...) __VA_ARGS__
#else
#define SPROF(...)
#endif

template <int D, int BS, bool SC>
__global__ void __launch_bounds__(kShMaxWarps * 32, 1) decode_shared_kernel(KernelArgs a) {
    SPROF(unsigned long long pt0, pt1 = 0, pt3; long long pw = 0, pp = 0, pf = 0, pfl = 0, pff = 0; int ptiles = 0, pflush = 0, pfinal = 0; const long long pc0 = clock64();)
    SPROF(asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(pt0));)
    using Cfg = ShCfg<D, BS>;
    constexpr int NKK = D / 16;   // k-steps of Q.K^T
    constexpr int NDT = D / 8;    // n-tiles of P.V
    constexpr int NS = Cfg::NS;
    constexpr int NREC = Cfg::NREC;

    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, c = lane & 3;
    const int RT = a.rows_per_tile;    // q heads per kv head (<= 8)
    const int nwarps = blockDim.x >> 5;
    const int Hkv = a.g.Hkv;
    uint8_t* ring = smem + warp * Cfg::WARP_SMEM;
    ShDesc* descs = reinterpret_cast<ShDesc*>(ring + NS * Cfg::STAGE);
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring + NS * Cfg::STAGE + NS * sizeof(ShDesc));
    uint8_t* tab = smem + nwarps * Cfg::WARP_SMEM;
    ShCtl* ctl = reinterpret_cast<ShCtl*>(tab);                 tab += (sizeof(ShCtl) + 15) / 16 * 16;
    ShRun* runs = reinterpret_cast<ShRun*>(tab);                tab += kShRuns * sizeof(ShRun);
    ShAcc* accs = reinterpret_cast<ShAcc*>(tab);                tab += kShAcc * sizeof(ShAcc);
    int* blk = reinterpret_cast<int*>(tab);                     tab += Cfg::TILES * NREC * sizeof(int);
    float2* acc_ml = reinterpret_cast<float2*>(tab);            tab += (size_t)kShAcc * RT * sizeof(float2);   // [kShAcc][RT] (max, sum)
    float* acc_o = reinterpret_cast<float*>(tab);               // [kShAcc][RT][AROW]

    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < NS; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)D);
    // everything below reads what the launch before this one wrote (plan, start records, cache)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int cta = blockIdx.x, nctas = gridDim.x;
    // ---- the CTA's slice; thread 0 keeps the walk state in shared memory --------------------------------
    if (tid == 0) {
        WorkerStart ws;
        ws.s = -1;
        const bool planned = a.worker_start && a.decode_all_workers == nctas;
        if (planned) {
            const int4 lo4 = __ldcg(reinterpret_cast<const int4*>(a.worker_start + cta));
            const int4 hi4 = __ldcg(reinterpret_cast<const int4*>(a.worker_start + cta) + 1);
            ws = WorkerStart{lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
        }
        const int total_tiles = ws.s != -1 ? ws.total_tiles : a.plan->total_tiles;
        const DecodeSlices sl = decode_slices(total_tiles, nctas);
        const int g_tile = (int)sl.begin(cta), g_end = (int)sl.end(cta);
        ctl->abort = 0;
        for (int i = 0; i < kShAcc; ++i) accs[i] = ShAcc{0, i, 0, 0};
        ctl->bad = 0;
        ctl->seq = 0;
        ctl->cont = 0;
        ctl->g_tile = g_tile;
        ctl->more = g_tile < g_end;
        if (g_tile < g_end) {
            int r_s, p0, r_tiles;
            if (ws.s >= 0) {
                r_s = ws.s; p0 = ws.p0; r_tiles = ws.r_tiles;
                ctl->ctx = ws.ctx; ctl->tb = ws.tb; ctl->nb = ws.nb; ctl->t0row = ws.t0;
            } else {
                const int key = g_tile / Hkv;
                int lo = 0, hi = a.num_sequences;  // tile_prefix[lo] <= key < tile_prefix[hi]
                while (hi - lo > 1) {
                    const int mid = (lo + hi) >> 1;
                    if (__ldcg(a.tile_prefix + mid) <= key) lo = mid; else hi = mid;
                }
                r_s = lo;
                p0 = __ldcg(a.tile_prefix + r_s);
                r_tiles = __ldcg(a.tile_prefix + r_s + 1) - p0;
                ctl->ctx = a.past_lens[r_s] + 1;
                ctl->tb = a.block_indices_begins[r_s];
                ctl->nb = a.block_indices_begins[r_s + 1] - ctl->tb;
                ctl->t0row = a.subsequence_begins[r_s];
            }
            const int off = g_tile - p0 * Hkv;
            ctl->r_s = r_s; ctl->p0 = p0; ctl->r_tiles = r_tiles;
            ctl->hk = off / r_tiles;
            ctl->pos = off % r_tiles;
        }
    }

    // ---- consumer state (per warp) -------------------------------------------------------------------
    uint32_t qa[NKK][2];            // live A registers of the query fragments
    float qsum = 0.f, qscale = 0.f;
    float oacc[NDT][2];
    float m_run = -INFINITY, l_run = 0.f, z_run = 0.f;
    int my_run = -1, my_tiles = 0;  // run in work (sequence number) and tiles of it this warp has reduced
    uint32_t phases = 0;            // parity of the next completion of each ring stage
    bool dead = false;              // this warp met a wait that ran out

    const long long part_stride = (long long)RT * D;   // floats of one partial
    uint8_t* cta_q = a.cta_q + (size_t)cta * kShRuns * kShQEntry;

    // Adds this warp's partial of run `seq` to the run's accumulator in shared memory (under the accumulator's lock) and,
    // if that completes the run inside the CTA, publishes (or writes) the result.
    auto flush = [&](int seq) {
        const int ae = seq % kShAcc;
        ShAcc* hd = &accs[ae];
        float l = l_run, z = z_run;
        l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
        z += __shfl_xor_sync(0xffffffffu, z, 1); z += __shfl_xor_sync(0xffffffffu, z, 2);
        const ShRun fin = runs[seq % kShRuns];
        // ---- take the lock of the accumulator once it is this run's turn.  The runs of an entry are served strictly in
        // order, so a wait here is always for an older run; a warp holds the partial of one run at a time and needs nothing
        // from a newer run to add it, so the oldest unfinished run of an entry can always finish and the waits end (they are
        // bounded all the same).  Serving whichever run comes first instead would deadlock: a warp may already have taken a
        // tile of the newer run when it comes here with the partial of the older one.
        int state = 0;   // 1: first partial of the run, 2: a later one, 0: not acquired
        for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
            if (lane == 0) {
                if (atomicCAS(&hd->lock, 0, 1) == 0) {
                    if (*reinterpret_cast<volatile int*>(&hd->turn) == seq) state = *reinterpret_cast<volatile int*>(&hd->tiles) == 0 ? 1 : 2;
                    else atomicExch(&hd->lock, 0);
                }
            }
            state = __shfl_sync(0xffffffffu, state, 0);
            if (state) break;
            __nanosleep(64);
        }
        if (!state) {
            if (lane == 0) { atomicOr(a.status, PA_DEV_WAIT_TIMEOUT_DECODE); atomicExch(&ctl->abort, 1); }
            my_tiles = 0;
            return;
        }
        SPROF(pfl += clock64() - pl0;)
        __threadfence_block();
        float* ao = acc_o + (long long)ae * RT * Cfg::AROW;
        float2* aml = acc_ml + ae * RT;
        if (g < RT) {
            float fa = 0.f, fb = 1.f, m_n = m_run;
            float2 old = make_float2(-INFINITY, 0.f);
            if (state == 2) {
                old = aml[g];
                m_n = fmaxf(old.x, m_run);
                fa = fast_exp2s(old.x - m_n);
                fb = fast_exp2s(m_run - m_n);
            }
            float* row = ao + g * Cfg::AROW + 2 * c;
#pragma unroll
            for (int i = 0; i < NDT; ++i) {
                float2 v = make_float2(0.f, 0.f);
                if (state == 2) v = *reinterpret_cast<const float2*>(row + 8 * i);
                v.x = v.x * fa + (oacc[i][0] - z) * fb;
                v.y = v.y * fa + (oacc[i][1] - z) * fb;
                *reinterpret_cast<float2*>(row + 8 * i) = v;
            }
            __syncwarp(RT >= 8 ? 0xffffffffu : ((1u << (4 * RT)) - 1u));   // the four lanes of a row have read (max, sum) before lane c == 0 replaces it
            if (c == 0) aml[g] = make_float2(m_n, old.y * fa + l * fb);
        }
        __threadfence_block();
        __syncwarp();
        int done = 0;
        if (lane == 0) { done = hd->tiles + my_tiles; hd->tiles = done; }
        done = __shfl_sync(0xffffffffu, done, 0);
        my_tiles = 0;
        if (done != fin.total) {
            if (lane == 0) atomicExch(&hd->lock, 0);
            return;
        }
        // ---- this partial completed the run inside the CTA: take the result out and free the accumulator --------
        SPROF(const long long pq0 = clock64(); ++pfinal;)
        float4 acc[8];
        float mrow[8], lrow[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); mrow[k] = -INFINITY; lrow[k] = 0.f;
            if (k < RT) {
                acc[k] = *reinterpret_cast<const float4*>(ao + k * Cfg::AROW + 4 * lane);
                const float2 ml = aml[k];
                mrow[k] = ml.x; lrow[k] = ml.y;
            }
        }
        __syncwarp();
        if (lane == 0) { hd->turn = seq + kShAcc; hd->tiles = 0; __threadfence_block(); atomicExch(&hd->lock, 0); }
        if (fin.nparts > 1) {
            // the stream has tiles in other CTAs: publish the CTA's partial; the CTA that completes the stream merges
            float* po = a.part_o + (long long)fin.slot * part_stride;
            float* pml = a.part_ml + (long long)fin.slot * RT * 2;
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < RT) {
                    __stcg(reinterpret_cast<float4*>(po + k * D + 4 * lane), acc[k]);
                    if (lane == 0) __stcg(reinterpret_cast<float2*>(pml + k * 2), make_float2(mrow[k], lrow[k]));
                }
            __threadfence();
            __syncwarp();
            int sdone = 0;
            if (lane == 0) sdone = atomicAdd(&a.stream_done[fin.stream], 1) + 1;
            sdone = __shfl_sync(0xffffffffu, sdone, 0);
            if (sdone != fin.nparts) return;
            __threadfence();
            merge_partials<D>(a.part_o + (long long)fin.first_slot * part_stride, a.part_ml + (long long)fin.first_slot * RT * 2, fin.nparts, 0xffffffffu,
                              RT, lane, acc, mrow, lrow);
        }
        // ---- the stream is complete: normalise and write ------------------------------------------------
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (k < RT) {
                const long long row = (long long)fin.t0 * a.g.Hq + fin.hk * RT + k;
                const float inv = 1.f / lrow[k];
                const long long idx = row * D + 4 * lane;
                store_pair_s(a.output, idx, a.g.act, acc[k].x * inv, acc[k].y * inv);
                store_pair_s(a.output, idx + 2, a.g.act, acc[k].z * inv, acc[k].w * inv);
                if (lane == 0 && a.lse) a.lse[row] = (mrow[k] + log2f(lrow[k])) * kLn2;
            }
        SPROF(pff += clock64() - pq0;)
    };

    bool ch_started_before = false;
    for (;;) {   // chapters
        // ---- thread 0 lists the runs of the chapter (walk state in registers while it does) --------------------
        if (tid == 0) {
            const int total_tiles = a.plan->total_tiles;
            const DecodeSlices sl = decode_slices(total_tiles, nctas);
            const int g_end = (int)sl.end(cta);
            int g_tile = ctl->g_tile, seq = ctl->seq;
            int nruns = 0, ntiles = 0, nblk = 0;
            int r_s = ctl->r_s, hk = ctl->hk, r_tiles = ctl->r_tiles, p0 = ctl->p0, pos = ctl->pos;
            int w_ctx = ctl->ctx, w_tb = ctl->tb, w_nb = ctl->nb, w_t0 = ctl->t0row;
            bool cont = ctl->cont != 0;
            // a run cut by the previous chapter goes on with its record (and its staged query rows)
            if (cont) --seq;
            const int first_seq = seq, new_first = cont ? seq + 1 : seq;
            // The slices are cut in a sequence in which every stream is followed by a.decode_phantom tiles that do not
            // exist: a CTA whose slice holds many streams (each costs it time beyond its tiles) gets fewer tiles.
            const int ph = a.decode_phantom;
            const unsigned per1 = (unsigned)sl.per1;   // one class of slices: worker of a tile = tile / per1
            while (g_tile < g_end && nruns < kShRuns && ntiles < Cfg::TILES) {
                ShRun& r = runs[seq % kShRuns];
                const bool fresh = seq >= new_first;
                bool have = true;
                int total = 0, upto = 0, vtail = 0;
                if (fresh) {
                    const int v_all = min(r_tiles - pos, g_end - g_tile);              // tiles of the stream in the slice, phantoms included
                    const int n_all = max(0, min(pos + v_all, r_tiles - ph) - pos);   // real ones
                    if (n_all == 0) {   // only phantoms: nothing to do for this stream
                        g_tile += v_all; pos += v_all;
                        have = false;
                    } else {
                        const unsigned s_begin = (unsigned)(p0 * Hkv + hk * r_tiles);   // global tile range of the stream
                        const int first_w = (int)(s_begin / per1), last_w = (int)((s_begin + (unsigned)(r_tiles - ph - 1)) / per1);
                        const int stream = r_s * Hkv + hk;
                        long long score_off = -1;
                        if constexpr (SC) {
                            if (a.score_aggregation_window[r_s] > 0) {
                                const long long off = a.score_offsets[r_s];
                                if (off >= 0 && off + w_ctx <= a.scores_len) score_off = ((long long)hk * a.scores_len + off) * 8;
                                else atomicOr(a.status, PA_DEV_BAD_BEGINS);
                            }
                        }
                        r.t0 = w_t0; r.hk = hk; r.stream = stream; r.nparts = last_w - first_w + 1;
                        r.first_slot = stream + first_w; r.slot = stream + cta; r.total = n_all; r.ctx = w_ctx;
                        r.score_off = score_off; r.tb = w_tb; r.nb = w_nb; r.vtail = v_all - n_all;
                        total = n_all; vtail = v_all - n_all;
                    }
                } else {
                    total = r.total; upto = r.upto; vtail = r.vtail;
                }
                if (have) {
                    const int n = min(total - upto, Cfg::TILES - ntiles);
                    r.g_first = ntiles; r.n_ch = n; r.tok_base = pos * kTile; r.blk_base = nblk; r.next = 0;
                    upto += n;
                    r.upto = upto;
                    cont = upto < total;
                    ntiles += n; nblk += n * NREC; g_tile += n; pos += n;
                    if (!cont) { g_tile += vtail; pos += vtail; }   // past the stream's phantoms
                    ++seq; ++nruns;
                }
                if (pos == r_tiles && g_tile < g_end) {   // next stream
                    pos = 0;
                    if (++hk == Hkv) {
                        hk = 0;
                        do {
                            ++r_s;
                            p0 = __ldcg(a.tile_prefix + r_s);
                            r_tiles = __ldcg(a.tile_prefix + r_s + 1) - p0;
                        } while (r_tiles == 0);
                        w_ctx = a.past_lens[r_s] + 1;
                        w_tb = a.block_indices_begins[r_s];
                        w_nb = a.block_indices_begins[r_s + 1] - w_tb;
                        w_t0 = a.subsequence_begins[r_s];
                    }
                }
            }
            ctl->r_s = r_s; ctl->hk = hk; ctl->r_tiles = r_tiles; ctl->p0 = p0; ctl->pos = pos;
            ctl->ctx = w_ctx; ctl->tb = w_tb; ctl->nb = w_nb; ctl->t0row = w_t0;
            ctl->g_tile = g_tile; ctl->seq = seq; ctl->cont = cont ? 1 : 0;
            ctl->first_seq = first_seq; ctl->new_first = new_first;
            ctl->nruns = nruns; ctl->ntiles = ntiles; ctl->win_lo = 0;
            ctl->more = g_tile < g_end;
        }
        __syncthreads();
        const int ch_ntiles = ctl->ntiles, ch_first = ctl->first_seq, ch_nruns = ctl->nruns, ch_new = ctl->new_first;
        const bool ch_more = ctl->more != 0;
        if (ch_ntiles == 0) break;

        // ---- all threads stage the block ids of the chapter's tiles ---------------------------------------------
        for (int k = 0; k < ch_nruns; ++k) {
            const ShRun& r = runs[(ch_first + k) % kShRuns];
            const int bi0 = r.tok_base / BS;
            for (int j = tid; j < r.n_ch * NREC; j += nwarps * 32) {
                const int bi = bi0 + j;
                int b = 0;
                if (bi < r.nb) {
                    b = a.block_indices[r.tb + bi];
                    if (b < 0 || b >= a.num_blocks) { b = 0; ctl->bad = 1; }
                }
                blk[r.blk_base + j] = b;
            }
        }
        __syncthreads();

        // ---- this warp's loader: next tile of the chapter into ring stage `slot` ---------------------------
        // The warps spread over a window of kShAcc runs, in proportion to the runs' tiles, and every run hands its tiles
        // out from its own counter: a warp stays with one run until the run has no tile left and then moves on inside the
        // window, which slides as its first runs are used up.  So a warp meets few runs (each costs it a query load and a
        // locked update of the run's accumulator) and the warps of a run do not leave it all at the same moment.
        int pr;   // index (in the chapter) of the run this warp takes tiles from
        {
            const int wn = min(kShAcc, ch_nruns);
            const int wt = runs[(ch_first + wn - 1) % kShRuns].g_first + runs[(ch_first + wn - 1) % kShRuns].n_ch;   // tiles of the first window
            const int target = (int)(((long long)(2 * warp + 1) * wt) / (2 * nwarps));
            pr = 0;
            while (pr + 1 < wn && target >= runs[(ch_first + pr) % kShRuns].g_first + runs[(ch_first + pr) % kShRuns].n_ch) ++pr;
        }
        int ahead = 0;            // lane 0: index already taken from the counter of run `pr` for the next call
        bool have_ahead = false;  // (the atomic's latency then falls into the tile's arithmetic, not into the loader)
        auto produce = [&](int slot) {
            int k = -1;
            if (!*reinterpret_cast<volatile int*>(&ctl->abort)) {
                for (int tries = 0; tries <= ch_nruns; ++tries) {
                    ShRun& rr = runs[(ch_first + pr) % kShRuns];
                    int kk = rr.n_ch;
                    if (have_ahead) kk = ahead;
                    else if (lane == 0 && *reinterpret_cast<volatile int*>(&rr.next) < rr.n_ch) kk = atomicAdd(&rr.next, 1);
                    have_ahead = false;
                    kk = __shfl_sync(0xffffffffu, kk, 0);
                    if (kk < rr.n_ch) {
                        k = kk;
                        if (lane == 0) ahead = *reinterpret_cast<volatile int*>(&rr.next) < rr.n_ch ? atomicAdd(&rr.next, 1) : rr.n_ch;
                        have_ahead = true;
                        break;
                    }
                    // the run is used up: slide the window past used-up runs, go to the next run inside it
                    int lo = 0;
                    if (lane == 0) {
                        lo = *reinterpret_cast<volatile int*>(&ctl->win_lo);
                        while (lo < ch_nruns && *reinterpret_cast<volatile int*>(&runs[(ch_first + lo) % kShRuns].next) >= runs[(ch_first + lo) % kShRuns].n_ch) ++lo;
                        atomicMax(&ctl->win_lo, lo);
                    }
                    lo = __shfl_sync(0xffffffffu, lo, 0);
                    if (lo >= ch_nruns) break;
                    ++pr;
                    if (pr < lo || pr >= min(lo + kShAcc, ch_nruns)) pr = lo;
                }
            }
            if (k < 0) {
                if (lane == 0) descs[slot] = ShDesc{kEndRun, 0, 0, 0};
                return;
            }
            const ShRun& r = runs[(ch_first + pr) % kShRuns];
            const int t = r.g_first + k;
            const int tok0 = r.tok_base + k * kTile;
            uint8_t* st = ring + slot * Cfg::STAGE;
            // Test hook (PA_B200_TEST_DROP_FIRST_COPY): the warp of CTA 0 that takes the first tile arms its barrier and issues no
            // copy, so that the bounded wait below runs out; nothing is in flight for that stage when it does.
            const bool drop = a.test_drop_copy && cta == 0 && t == 0 && ch_first == 0 && !ch_started_before;
            if (lane == 0) {
                uint32_t bytes = 0;
#pragma unroll
                for (int rr = 0; rr < NREC; ++rr) bytes += (tok0 + rr * BS < r.ctx) ? 2 * Cfg::REC : 0;
                mbar_expect_tx(&bars[slot], bytes);
                descs[slot] = ShDesc{ch_first + pr, min(kTile, r.ctx - tok0), tok0, 0};
            }
            // one copy per lane: key / value record of each block of the tile
            if (lane < 2 * NREC) {
                const int rr = lane >> 1;
                const bool is_v = lane & 1;
                if (tok0 + rr * BS < r.ctx && !drop) {
                    const int b = blk[r.blk_base + k * NREC + rr];
                    const uint8_t* src = (const uint8_t*)(is_v ? a.value_cache : a.key_cache) + (long long)r.hk * a.g.head_bytes +
                                         (long long)b * a.g.block_bytes;
                    bulk_g2s(st + (is_v ? Cfg::HALF_STAGE : 0) + rr * Cfg::REC, src, Cfg::REC, &bars[slot]);
                }
            }
        };

#pragma unroll
        for (int p = 0; p < NS - 1; ++p) produce(p);

        // (staged while the first tiles are on their way)
        // Query rows of the chapter's new runs: f16, prescaled, in the register order of the fragments (lane (g, c) of a
        // consumer reads its 16 registers of row g as four 16-byte loads), with the row's sum and softmax scale.  Staged in
        // global scratch of the CTA: it is read once per (warp, run) and comes from the L2.
        {
            const int npairs = (ch_first + ch_nruns - ch_new) * RT;
            for (int p = warp; p < npairs; p += nwarps) {
                const int seq = ch_new + p / RT, hrow = p % RT;
                const ShRun& r = runs[seq % kShRuns];
                uint8_t* entry = cta_q + (size_t)(seq % kShRuns) * kShQEntry;
                const long long qoff = ((long long)r.t0 * a.g.Hq + r.hk * RT + hrow) * D + lane * 4;
                float q[4];
                load_act_vec<4>(a.query, qoff, a.g.act, q);
                float amax = fmaxf(fmaxf(fabsf(q[0]), fabsf(q[1])), fmaxf(fabsf(q[2]), fabsf(q[3])));
#pragma unroll
                for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                float qmul = 1.f;  // exact power-of-two prescale that keeps |q| inside the f16 range
                if (amax > 32768.f && amax < INFINITY) {
                    int ex;
                    frexpf(amax, &ex);
                    qmul = ldexpf(1.f, 15 - ex);
                }
                const uint32_t lo = pack_h2(q[0] * qmul, q[1] * qmul), hi = pack_h2(q[2] * qmul, q[3] * qmul);
                const __half2 hl = *reinterpret_cast<const __half2*>(&lo), hh = *reinterpret_cast<const __half2*>(&hi);
                float sum = __low2float(hl) + __high2float(hl) + __low2float(hh) + __high2float(hh);
#pragma unroll
                for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                // dims 4*lane .. 4*lane+3 are k-step 4*h + i of consumer lane (hrow, cc): h = lane / 16, cc = (lane % 16) / 4, i = lane % 4
                const int ks = 4 * (lane >> 4) + (lane & 3), cc = (lane & 15) >> 2;
                const int reg = 2 * ks;   // registers reg, reg + 1 of that lane
                uint32_t* dst = reinterpret_cast<uint32_t*>(entry) + ((reg >> 2) * 32 + 4 * hrow + cc) * 4 + (reg & 3);
                __stcg(reinterpret_cast<uint2*>(dst), make_uint2(lo, hi));
                if (lane == 0) __stcg(reinterpret_cast<float2*>(entry + 2048) + hrow, make_float2(sum, sm_scale * kLog2e / qmul));
            }
        }
        __syncthreads();

        for (int it = 0; !dead; ++it) {
            __syncwarp();  // every lane is done with the stage that is refilled next
            SPROF(const long long pp0 = clock64();)
            produce((it + NS - 1) % NS);
            __syncwarp();
            SPROF(pp += clock64() - pp0;)
            const int slot = it % NS;
            const ShDesc d = descs[slot];
            if (d.run != my_run) {
                // a run cut by the chapter boundary stays in the registers across it
                const bool keep = d.run == kEndRun && my_run == ch_first + ch_nruns - 1 && my_run >= 0 &&
                                  runs[my_run % kShRuns].upto < runs[my_run % kShRuns].total;
                SPROF(const long long pf0 = clock64();)
                if (my_run >= 0 && !keep) { flush(my_run); my_run = -1; }
                SPROF(pf += clock64() - pf0;)
                if (d.run == kEndRun) break;
                // ---- Q fragments of the run: the contraction index is permuted so that one 16-byte shared load of
                // a key row feeds four k-steps: k-step 4*half + i covers dims 64*half + 16*c + 4*i + {0..3}
                my_run = d.run;
                {
                    const uint8_t* entry = cta_q + (size_t)(my_run % kShRuns) * kShQEntry;
                    const int gl = g < RT ? g : 0;
#pragma unroll
                    for (int u4 = 0; u4 < NKK / 2; ++u4) {
                        const uint4 w = __ldcg(reinterpret_cast<const uint4*>(entry) + u4 * 32 + 4 * gl + c);
                        qa[2 * u4][0] = w.x; qa[2 * u4][1] = w.y; qa[2 * u4 + 1][0] = w.z; qa[2 * u4 + 1][1] = w.w;
                    }
                    const float2 qm = __ldcg(reinterpret_cast<const float2*>(entry + 2048) + gl);
                    qsum = qm.x; qscale = qm.y;
                    if (g >= RT) {
#pragma unroll
                        for (int kk = 0; kk < NKK; ++kk) { qa[kk][0] = 0u; qa[kk][1] = 0u; }
                        qsum = 0.f;
                    }
                }
                m_run = -INFINITY; l_run = 0.f; z_run = 0.f;
#pragma unroll
                for (int i = 0; i < NDT; ++i) { oacc[i][0] = 0.f; oacc[i][1] = 0.f; }
            }
            SPROF(const long long pw0 = clock64();)
            if (!mbar_wait_bounded(&bars[slot], (phases >> slot) & 1, a.test_drop_copy ? (1u << 10) : (1u << 22))) {
                // the copy never arrived: flag it, stop the CTA's hand-out, let the copy of the other stage land (bounded)
                if (lane == 0) { atomicOr(a.status, PA_DEV_WAIT_TIMEOUT_DECODE); atomicExch(&ctl->abort, 1); }
                const int other = (it + 1) % NS;
                if (descs[other].run != kEndRun) mbar_wait_bounded(&bars[other], (phases >> other) & 1, 1u << 16);
                dead = true;
                break;
            }
            phases ^= 1u << slot;
            SPROF(pw += clock64() - pw0; if (!pt1) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(pt1)); ++ptiles;)
            const uint8_t* st = ring + slot * Cfg::STAGE;
            const int valid = d.valid;

            // ---- S = Q.K^T over four 8-token n-tiles: the four accumulator chains advance together -------------------
            float sacc[4][2];
            {
                uint4 kw[4][D / 64];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int row = 8 * (g >> 1) + 2 * j + (g & 1);
                    const uint8_t* kp = st + (row / BS) * Cfg::REC + (row % BS) * D + 16 * c;
#pragma unroll
                    for (int h = 0; h < D / 64; ++h) kw[j][h] = *reinterpret_cast<const uint4*>(kp + 64 * h);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) { sacc[j][0] = 0.f; sacc[j][1] = 0.f; }
#pragma unroll
                for (int h = 0; h < D / 64; ++h)
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {   // bytes stay offset by 1024; removed with the zero-point
                            const uint32_t w = i == 0 ? kw[j][h].x : i == 1 ? kw[j][h].y : i == 2 ? kw[j][h].z : kw[j][h].w;
                            mma_lo(sacc[j][0], sacc[j][1], qa[4 * h + i][0], qa[4 * h + i][1], __byte_perm(w, 0x64646464u, 0x4140), __byte_perm(w, 0x64646464u, 0x4342));
                        }
            }

            // ---- scale, mask, online softmax -----------------------------------------------------------
            float vsc[4][2], vzp[4][2];
            float tmax = -INFINITY;
            float* score_dst = nullptr;
            if constexpr (SC) {
                const long long so = runs[my_run % kShRuns].score_off;
                if (so >= 0) score_dst = a.score_raw + so + (long long)d.tok0 * 8 + g;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tk = 8 * c + 2 * j;  // tile token of accumulator column 0
                const uint8_t* kp = st + (tk / BS) * Cfg::REC + BS * D;
                const float2 ks = *reinterpret_cast<const float2*>(kp + 4 * (tk % BS));
                const float2 kz = *reinterpret_cast<const float2*>(kp + 4 * BS + 4 * (tk % BS));
                const uint8_t* vp = st + Cfg::HALF_STAGE + (tk / BS) * Cfg::REC + BS * D;
                const float2 vs = *reinterpret_cast<const float2*>(vp + 4 * (tk % BS));
                const float2 vz = *reinterpret_cast<const float2*>(vp + 4 * BS + 4 * (tk % BS));
                vsc[j][0] = vs.x; vsc[j][1] = vs.y; vzp[j][0] = vz.x + 1024.f; vzp[j][1] = vz.y + 1024.f;
                const bool ok0 = tk < valid, ok1 = tk + 1 < valid;
                float s0 = (sacc[j][0] - (kz.x + 1024.f) * qsum) * (ks.x * qscale);
                float s1 = (sacc[j][1] - (kz.y + 1024.f) * qsum) * (ks.y * qscale);
                s0 = ok0 ? s0 : -INFINITY;
                s1 = ok1 ? s1 : -INFINITY;
                if constexpr (SC) {
                    if (score_dst) {
                        if (ok0) __stcs(score_dst + tk * 8, s0);
                        if (ok1) __stcs(score_dst + (tk + 1) * 8, s1);
                    }
                }
                sacc[j][0] = s0; sacc[j][1] = s1;
                tmax = fmaxf(tmax, fmaxf(s0, s1));
            }
            // The reference maximum is raised only when the tile maximum exceeds it by more than kLazyMax
            // (warp-uniform decision), so most tiles skip the rescale of the accumulators.
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
            tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
            if (__any_sync(0xffffffffu, tmax > m_run + kLazyMax)) {
                const float m_new = fmaxf(m_run, tmax);
                const float alpha = fast_exp2s(m_run - m_new);  // 0 on the first tile
                m_run = m_new;
                l_run *= alpha;
                z_run *= alpha;
#pragma unroll
                for (int i = 0; i < NDT; ++i) { oacc[i][0] *= alpha; oacc[i][1] *= alpha; }
            }
            uint32_t pa_frag[2][2];   // live A registers of P for the two 16-token k-steps
            {
                float lsum = 0.f, zsum = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float p0 = fast_exp2s(sacc[j][0] - m_run), p1 = fast_exp2s(sacc[j][1] - m_run);
                    lsum += p0 + p1;
                    const int tk = 8 * c + 2 * j;
                    // masked tokens have p == 0; the select keeps garbage scale bits (NaN) out
                    const uint32_t packed = pack_h2(tk < valid ? p0 * vsc[j][0] : 0.f, tk + 1 < valid ? p1 * vsc[j][1] : 0.f);
                    const __half2 h = *reinterpret_cast<const __half2*>(&packed);
                    zsum += (tk < valid ? __low2float(h) * vzp[j][0] : 0.f) + (tk + 1 < valid ? __high2float(h) * vzp[j][1] : 0.f);
                    pa_frag[j >> 1][j & 1] = packed;
                }
                l_run += lsum;
                z_run += zsum;
            }

            // ---- O += P.V -----------------------------------------------------------------------------
#pragma unroll
            for (int i = 0; i < NDT; ++i) {
                const int dd = 8 * i + g;
                const uint8_t* vp = st + Cfg::HALF_STAGE + ((8 * c) / BS) * Cfg::REC + dd * BS + ((8 * c) % BS);
                const uint2 w = *reinterpret_cast<const uint2*>(vp);
                mma_lo(oacc[i][0], oacc[i][1], pa_frag[0][0], pa_frag[0][1], __byte_perm(w.x, 0x64646464u, 0x4140), __byte_perm(w.x, 0x64646464u, 0x4342));
                mma_lo(oacc[i][0], oacc[i][1], pa_frag[1][0], pa_frag[1][1], __byte_perm(w.y, 0x64646464u, 0x4140), __byte_perm(w.y, 0x64646464u, 0x4342));
            }
            ++my_tiles;
            // The value bytes enter the MMA as 1024 + byte, so the accumulators carry about a thousand times the
            // magnitude of the result until the zero-point term is taken out, and the tensor core truncates every
            // accumulation at that magnitude; taking the term out every few tiles keeps the lost bits small.
            if ((my_tiles & (kFoldEvery - 1)) == 0) {
                float z = z_run;
                z += __shfl_xor_sync(0xffffffffu, z, 1); z += __shfl_xor_sync(0xffffffffu, z, 2);
                z_run = 0.f;
#pragma unroll
                for (int i = 0; i < NDT; ++i) { oacc[i][0] -= z; oacc[i][1] -= z; }
            }
        }
        __syncthreads();   // everyone is done with the chapter's tables
        if (!ch_more || *reinterpret_cast<volatile int*>(&ctl->abort)) break;
        dead = false;
        ch_started_before = true;
    }
    if (tid == 0 && ctl->bad) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
#ifdef PA_DECODE_PROF
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(pt3));
    const int pwid = cta * nwarps + warp;
    if (lane == 0 && pwid < 8192) {
        g_shared_prof[pwid * 12 + 0] = pt0;
        g_shared_prof[pwid * 12 + 1] = pt1 ? pt1 - pt0 : 0;
        g_shared_prof[pwid * 12 + 2] = pt3 - pt0;
        g_shared_prof[pwid * 12 + 3] = (unsigned long long)ptiles;
        g_shared_prof[pwid * 12 + 4] = (unsigned long long)pw;
        g_shared_prof[pwid * 12 + 5] = (unsigned long long)(clock64() - pc0);
        g_shared_prof[pwid * 12 + 6] = (unsigned long long)pp;
        g_shared_prof[pwid * 12 + 7] = (unsigned long long)pf;
        g_shared_prof[pwid * 12 + 8] = (unsigned long long)pfl;
        g_shared_prof[pwid * 12 + 9] = (unsigned long long)pff;
        g_shared_prof[pwid * 12 + 10] = (unsigned long long)pflush;
        g_shared_prof[pwid * 12 + 11] = (unsigned long long)pfinal;
    }
#endif
}

template <int D, int BS>
cudaError_t launch_shared_t(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0, cudaEvent_t ev1) {
    using Cfg = ShCfg<D, BS>;
    const bool sc = a.score_raw != nullptr && a.score_aggregation_window != nullptr;
    auto kern = sc ? decode_shared_kernel<D, BS, true> : decode_shared_kernel<D, BS, false>;
    const size_t smem = Cfg::smem(a.rows_per_tile);
    static std::atomic<size_t> set[2];   // largest opt-in made per instantiation
    if (set[sc ? 1 : 0].load(std::memory_order_acquire) < smem) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set[sc ? 1 : 0].store(smem, std::memory_order_release);
    }
    if (ev0) cudaEventRecord(ev0, stream);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)decode_shared_ctas(a, sm_count));
    cfg.blockDim = dim3(Cfg::warps(a.rows_per_tile) * 32);
    cfg.dynamicSmemBytes = smem;
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

}  // namespace


int decode_shared_chapter_tiles(const CacheGeom& g) { return g.bs == 32 ? ShCfg<128, 32>::TILES : ShCfg<128, 16>::TILES; }

int decode_shared_max_chapters() {
    static const int v = [] {
        const char* e = std::getenv("PA_B200_DECODE_SHARED_CHAPTERS");
        const int n = e ? std::atoi(e) : 4;
        return n < 1 ? 1 : n;
    }();
    return v;
}

int decode_shared_phantom() {
    static const int v = [] {
        const char* e = std::getenv("PA_B200_DECODE_PHANTOM");
        const int n = e ? std::atoi(e) : kDecodeSharedPhantom;
        return n < 0 ? 0 : n;
    }();
    return v;
}

size_t decode_shared_scratch_bytes(int sm_count) { return (size_t)sm_count * kShRuns * kShQEntry; }

bool decode_shared_supported(const CacheGeom& g) {
    static const bool on = [] {
        const char* e = std::getenv("PA_B200_DECODE_SHARED");
        return e ? std::atoi(e) != 0 : true;
    }();
    return on && g.cache == PA_DTYPE_U8 && g.Hq / g.Hkv <= 8 && g.D == 128 && (g.bs == 16 || g.bs == 32);
}

// One CTA per SM; fewer when the step is small (at least kDecodeMinSlice tiles each, as decode_slices cuts them).
int decode_shared_ctas(const KernelArgs& a, int sm_count) {
    const long long want = (a.max_tiles + kDecodeMinSlice - 1) / kDecodeMinSlice;
    return (int)std::max(1LL, std::min((long long)sm_count, want));
}

cudaError_t launch_decode_shared(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0, cudaEvent_t ev1) {
    if (a.num_sequences <= 0) return cudaSuccess;
    if (a.g.D == 128 && a.g.bs == 32) return launch_shared_t<128, 32>(a, stream, sm_count, launches, ev0, ev1);
    if (a.g.D == 128 && a.g.bs == 16) return launch_shared_t<128, 16>(a, stream, sm_count, launches, ev0, ev1);
    return cudaErrorInvalidValue;
}

}  // namespace pa

#ifdef PA_DECODE_PROF
extern "C" int pa_b200_debug_read_shared_prof(void* dst, size_t bytes) {
    return (int)cudaMemcpyFromSymbol(dst, pa::g_shared_prof, bytes);
}
#endif
