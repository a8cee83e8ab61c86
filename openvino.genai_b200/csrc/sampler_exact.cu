// Multinomial rows over the full vocabulary (no active top-k), bit for bit as the reference computes
// them on the host:
//   TemperatureLogitTransform   src/cpp/src/sampling/logit_transformers.hpp:299-362
//       p_i = expf((x_i - max) * (1 / T)), sum in index order in single precision, p_i /= sum
//   MinPFilter                  logit_transformers.hpp:157-190   (keep p_i >= float(min_p) * p_max)
//   TopPFilter                  logit_transformers.hpp:94-139    (sort descending, add until the float sum > top_p)
//   Sampler::_multinomial_sample  src/cpp/src/sampling/sampler.cpp:1036-1089
//       total = sum of the kept probabilities in their order, r = total * u, first running sum > r
// Every float the reference produces on the way is reproduced: expf with the host libm's bits and
// the sequential sums through the step algebra of fsum_exact.cuh, so token ids agree with the
// reference except where several kept elements have exactly the same probability and the draw falls
// among them (their relative order after std::sort is not defined; the lowest index is taken here).
//
// One CTA works on one row at a time (persistent grid, rows dealt round robin).  Passes over a row:
//   1. maximum;  2. expf and the index-order sum (tile by tile, a block scan of steps per tile), the
//   exponentials parked in a per-CTA scratch row;  3. division by the sum, probabilities back to the
//   scratch row, and either the index-order total (no top-p) or the first level's bin counts;
//   then, without top-p, one more partial pass that stops at the drawn element; with top-p the
//   walk of fsum_exact.cuh: a few passes that sum whole bins as translations and list the rest.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/sampler_b200.h"
#include "fsum_exact.cuh"
#include "sampler_kernels.h"

namespace sampler {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kListCap = 4096;
constexpr uint32_t kTopCount = 96;
constexpr double kMargin = 1.0 / 4096;
constexpr double kDrawMargin = 1.0 / 512;
constexpr int kBinsPerThread = fsx::kBins / kThreads;
static_assert(fsx::kBins % kThreads == 0, "bins are dealt evenly to the threads");

struct RunSum {
    uint32_t pa, pc;
    uint32_t reset;
};

struct ExactShared {
    uint32_t A[fsx::kBins];
    uint32_t C[fsx::kBins];
    float R[fsx::kBins];
    uint32_t PA[fsx::kBins];
    uint32_t PC[fsx::kBins];
    uint16_t next[fsx::kBins + 2];
    uint8_t E[fsx::kBins];
    uint8_t flag[fsx::kBins];
    uint32_t tie_bits[fsx::kBins / 32];
    unsigned long long list[kListCap];
    int list_n;
    // block scan / reduce scratch
    fsx::Step scan_step[kWarps];
    unsigned long long tile_sum[2][kWarps];
    unsigned long long exp_tab[32];
    RunSum scan_run[kWarps];
    double scan_d[kWarps];
    unsigned long long scan_u[kWarps];
    float red_f[kWarps];
    int red_i[kWarps];
    // chain broadcast
    uint32_t bc_E, bc_S;
    int bc_idx;
    // walk control (written by thread 0)
    fsx::Walk walk;
    fsx::Level level;
    uint32_t rest_cnt;
    int ctl;
    int cleared;
    int prof_passes;
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ float block_max(float v, ExactShared& sh) {
    v = warp_max(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh.red_f[w] = v;
    __syncthreads();
    v = lane < kWarps ? sh.red_f[lane] : -CUDART_INF_F;
    return warp_max(v);
}

__device__ int block_min_int(int v, ExactShared& sh) {
    v = __reduce_min_sync(0xffffffffu, v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh.red_i[w] = v;
    __syncthreads();
    v = lane < kWarps ? sh.red_i[lane] : 0x7fffffff;
    return __reduce_min_sync(0xffffffffu, v);
}

__device__ unsigned long long block_sum_u64(unsigned long long v, ExactShared& sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh.scan_u[w] = v;
    __syncthreads();
    v = lane < kWarps ? sh.scan_u[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Exclusive scan over the block of one value per thread with an associative, not necessarily
// commutative operation (left operand = earlier threads).  Returns the combination of all earlier
// threads' values; *total receives the combination of all.
template <class T, class Op>
__device__ T block_scan_exclusive(T v, T identity, Op op, T* warp_buf, T* total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    T incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        union { T t; uint32_t u[sizeof(T) / 4]; } a, r;
        a.t = incl;
#pragma unroll
        for (int i = 0; i < (int)(sizeof(T) / 4); ++i) r.u[i] = __shfl_up_sync(0xffffffffu, a.u[i], o);
        if (lane >= o) incl = op(r.t, incl);
    }
    __syncthreads();
    if (lane == 31) warp_buf[w] = incl;
    __syncthreads();
    T before = identity;
    T all = identity;
    for (int i = 0; i < kWarps; ++i) {
        const T wi = warp_buf[i];
        if (i < w) before = op(before, wi);
        all = op(all, wi);
    }
    if (total) *total = all;
    // exclusive within the warp
    T excl_lane;
    {
        union { T t; uint32_t u[sizeof(T) / 4]; } a, r;
        a.t = incl;
#pragma unroll
        for (int i = 0; i < (int)(sizeof(T) / 4); ++i) r.u[i] = __shfl_up_sync(0xffffffffu, a.u[i], 1);
        excl_lane = lane ? r.t : identity;
    }
    return op(before, excl_lane);
}

struct StepOp {
    __device__ fsx::Step operator()(fsx::Step f, fsx::Step g) const { return fsx::then(f, g); }
};

// ---- index-order sums ---------------------------------------------------------------------------------
// Adds the kept values of a row in index order to the float sum s, exactly as the host loop
// `s += v[i]` does.  A tile is kTile consecutive elements, kPer per thread.  While the sum stays in
// its binade and no element of the tile is a tie, the tile's amounts are plain integers whose order
// does not matter: one block reduction per tile.  A tile with a tie, a change of binade or (with
// `use_thr`) the first running sum above `thr` is redone as a block scan of two-state steps.
//   load(i, raw, keep)   fetches elements i .. i + kPer - 1 (keep = false beyond the row)
//   xform(i, raw, keep)  turns them into the values to add (and may drop elements or park results)
// Returns the index of the first element whose running sum exceeds thr (-1: none, or !use_thr).
// All threads call this with the same arguments; s is returned to all.
constexpr int kPer = 8;
constexpr int kTile = kThreads * kPer;

template <class LoadFn, class XformFn>
__device__ long long chain_sum(float& s, long long V, LoadFn&& load, XformFn&& xform, float thr, bool use_thr, ExactShared& sh) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t E = fsx::state_exp(s), S = fsx::state_sig(s);
    float raw[kPer], nxt[kPer];
    bool keep[kPer], nkeep[kPer];
    load((long long)kPer * tid, raw, keep);
    int parity = 0;
    for (long long base = 0; base < V; base += kTile, parity ^= 1) {
        if (base + kTile < V) load(base + kTile + (long long)kPer * tid, nxt, nkeep);   // in flight while this tile is added
        float x[kPer];
#pragma unroll
        for (int e = 0; e < kPer; ++e) x[e] = raw[e];
        xform(base + (long long)kPer * tid, x, keep);
        // fast path: the tile as one integer
        {
            uint32_t mine = 0;
            bool tie = false;
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                if (!keep[e]) continue;
                bool t;
                const fsx::Step st = fsx::step_of(x[e], E, &t);
                tie |= t;
                mine = fsx::sat_add(mine, st.a);
            }
            const uint32_t wsum = __reduce_add_sync(0xffffffffu, mine);   // a thread's amounts saturate at 2^26: 32 of them fit
            if (lane == 0) sh.tile_sum[parity][warp] = wsum;
            const int any_tie = __syncthreads_or(tie ? 1 : 0);
            unsigned long long tot = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) tot += sh.tile_sum[parity][w];
            if (!any_tie && tot < fsx::kOne24 && S + (uint32_t)tot < fsx::kOne24 &&
                !(use_thr && fsx::state_float(E, S + (uint32_t)tot) > thr)) {
                S += (uint32_t)tot;
#pragma unroll
                for (int e = 0; e < kPer; ++e) { raw[e] = nxt[e]; keep[e] = nkeep[e]; }
                continue;
            }
        }
        // slow path: scan of steps, one real addition where the binade changes
        int from = 0;   // elements of the tile below `from` are already in the sum
        for (;;) {
            fsx::Step loc[kPer];
            fsx::Step acc = fsx::step_identity();
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                if (keep[e] && kPer * tid + e >= from) acc = fsx::then(acc, fsx::step_of(x[e], E));
                loc[e] = acc;
            }
            fsx::Step total;
            const fsx::Step excl = block_scan_exclusive(acc, fsx::step_identity(), StepOp(), sh.scan_step, &total);
            const uint32_t S_end = fsx::apply(total, S);
            const bool crossed = S_end >= fsx::kOne24;
            const bool over = use_thr && !crossed && fsx::state_float(E, S_end) > thr;
            if (!crossed && !over) { S = S_end; break; }
            // first element at which the sum leaves the binade or exceeds the threshold
            int mine = 0x7fffffff;
#pragma unroll
            for (int e = kPer - 1; e >= 0; --e) {
                if (!(keep[e] && kPer * tid + e >= from)) continue;
                const uint32_t Se = fsx::apply(fsx::then(excl, loc[e]), S);
                if (Se >= fsx::kOne24 || (use_thr && fsx::state_float(E, Se) > thr)) mine = kPer * tid + e;
            }
            const int first = block_min_int(mine, sh);
            if (first / kPer == tid) {
                const int e = first % kPer;
                fsx::Step pre = excl;   // steps of this thread's elements before e (skipped ones are identities)
#pragma unroll
                for (int q = 0; q < kPer; ++q) if (q + 1 == e) pre = fsx::then(excl, loc[q]);
                float xe = 0.f;
#pragma unroll
                for (int q = 0; q < kPer; ++q) if (q == e) xe = x[q];
                const float before = fsx::state_float(E, fsx::apply(pre, S));
                const float after = __fadd_rn(before, xe);
                sh.bc_E = fsx::state_exp(after);
                sh.bc_S = fsx::state_sig(after);
            }
            __syncthreads();
            E = sh.bc_E; S = sh.bc_S;
            __syncthreads();
            if (use_thr && fsx::state_float(E, S) > thr) { s = fsx::state_float(E, S); return base + first; }
            from = first + 1;
        }
#pragma unroll
        for (int e = 0; e < kPer; ++e) { raw[e] = nxt[e]; keep[e] = nkeep[e]; }
    }
    s = fsx::state_float(E, S);
    return -1;
}

// ---- bins: classification, prefix tables -----------------------------------------------------------------
struct RunSumOp {
    __device__ RunSum operator()(RunSum a, RunSum b) const {
        if (b.reset) return b;
        const unsigned long long pc = (unsigned long long)a.pc + b.pc;
        return RunSum{fsx::sat_add(a.pa, b.pa), pc > 0x7fffffffull ? 0x7fffffffu : (uint32_t)pc, a.reset};
    }
};

__device__ fsx::Bins bins_of(ExactShared& sh) { return fsx::Bins{sh.A, sh.C, sh.R, sh.PA, sh.PC, sh.next, sh.E, sh.flag}; }

// PA / PC per run of plain bins and the next-stop table (fsum_exact.cuh: walk_level)
__device__ void prepare_walk(ExactShared& sh) {
    const int tid = threadIdx.x, j0 = tid * kBinsPerThread;
    const fsx::Bins b = bins_of(sh);
    // code of the nearest non-empty bin: 0 none, 1 not plain, 2 + E plain
    int last = 0;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        if (sh.C[j] != 0) last = fsx::bin_plain(b, j) ? 2 + (int)sh.E[j] : 1;
    }
    int* ibuf = sh.red_i;
    const int before = block_scan_exclusive(last, 0, [](int a, int c) { return c ? c : a; }, ibuf, (int*)nullptr);
    bool stop[kBinsPerThread];
    int prev = before;
    RunSum acc{0u, 0u, 0u};
    RunSum loc[kBinsPerThread];
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        stop[k] = false;
        if (sh.C[j] != 0) {
            const bool plain = fsx::bin_plain(b, j);
            stop[k] = fsx::bin_is_stop(b, j, prev >= 2 ? prev - 2 : -1);
            prev = plain ? 2 + (int)sh.E[j] : 1;
            RunSum el{plain ? sh.A[j] : 0u, plain ? sh.C[j] : 0u, stop[k] ? 1u : 0u};
            acc = RunSumOp()(acc, el);
        }
        loc[k] = acc;
    }
    __syncthreads();
    const RunSum excl = block_scan_exclusive(acc, RunSum{0u, 0u, 0u}, RunSumOp(), sh.scan_run, (RunSum*)nullptr);
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const RunSum r = RunSumOp()(excl, loc[k]);
        sh.PA[j0 + k] = r.pa;
        sh.PC[j0 + k] = r.pc;
    }
    // next stop at or after j: reverse scan of the minimum
    int nearest = fsx::kBins;
    int locn[kBinsPerThread];
#pragma unroll
    for (int k = kBinsPerThread - 1; k >= 0; --k) {
        if (stop[k]) nearest = j0 + k;
        locn[k] = nearest;
    }
    // threads after this one: scan over reversed thread order
    __syncthreads();
    int* rev = sh.red_i;
    // reversed exclusive scan: combine values of threads with a higher index
    {
        int v = nearest;
        const int lane = tid & 31, w = tid >> 5;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int dn = __shfl_down_sync(0xffffffffu, incl, o);
            if (lane + o < 32) incl = min(incl, dn);
        }
        if (lane == 0) rev[w] = incl;
        __syncthreads();
        int after = fsx::kBins;
        for (int i = w + 1; i < kWarps; ++i) after = min(after, rev[i]);
        const int dn1 = __shfl_down_sync(0xffffffffu, incl, 1);
        const int excl_after = min(after, lane < 31 ? dn1 : fsx::kBins);
#pragma unroll
        for (int k = 0; k < kBinsPerThread; ++k) sh.next[j0 + k] = (uint16_t)min(locn[k], excl_after);
    }
    if (tid == 0) { sh.next[fsx::kBins] = (uint16_t)fsx::kBins; sh.next[fsx::kBins + 1] = (uint16_t)fsx::kBins; }
    __syncthreads();
}

// Hypotheses and list marks for the bins from j_from on, given the exact sum and count before that
// bin (tests/cpp/topp_model.hpp::classify is the sequential statement of the same rules).
__device__ void classify_bins(ExactShared& sh, int j_from, float s, uint32_t cnt, float thr, uint32_t limit, double thr2) {
    const int tid = threadIdx.x, j0 = tid * kBinsPerThread;
    __syncthreads();
    if (tid == 0) {
        sh.cleared = 0;
        if ((int)sh.C[j_from] > kListCap - sh.list_n) { sh.cleared = 1; sh.list_n = 0; }
    }
    __syncthreads();
    if (sh.cleared) {
#pragma unroll
        for (int k = 0; k < kBinsPerThread; ++k)
            if (sh.flag[j0 + k] & fsx::kBinListed) sh.flag[j0 + k] = 0;
    }
    const int room = kListCap - sh.list_n;
    double mass = 0.0;
    unsigned long long count = 0;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        if (j >= j_from && sh.C[j] != 0) { mass += (double)sh.R[j]; count += sh.C[j]; }
    }
    const double mass_before = block_scan_exclusive(mass, 0.0, [](double a, double c) { return a + c; }, sh.scan_d, (double*)nullptr);
    const unsigned long long count_before =
        block_scan_exclusive(count, 0ull, [](unsigned long long a, unsigned long long c) { return a + c; }, sh.scan_u, (unsigned long long*)nullptr);
    double cum = (double)s + mass_before;
    unsigned long long cc = (unsigned long long)cnt + count_before;
    bool want[kBinsPerThread];
    uint32_t Eh[kBinsPerThread];
    bool reach[kBinsPerThread];
    unsigned long long wanted = 0;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        want[k] = false; reach[k] = false; Eh[k] = 0;
        if (j < j_from || sh.C[j] == 0) continue;
        const double lo = cum, hi = cum + (double)sh.R[j];
        const unsigned long long cbefore = cc;
        cum = hi; cc += sh.C[j];
        if (lo * (1.0 - kMargin) > (double)thr || (limit && cbefore >= limit)) continue;   // beyond what the walk can reach
        reach[k] = true;
        if (sh.flag[j] & fsx::kBinListed) continue;
        const bool certain = fsx::hyp_exponent(lo, hi, kMargin, &Eh[k]);
        bool w = j == j_from || !certain || cbefore < kTopCount;
        if (lo * (1.0 - kMargin) <= (double)thr && (double)thr <= hi * (1.0 + kMargin)) w = true;
        if (thr2 > 0.0 && lo * (1.0 - kDrawMargin) <= thr2 && thr2 <= hi * (1.0 + kDrawMargin)) w = true;
        if (limit && cbefore + sh.C[j] >= limit) w = true;
        const bool same_hyp = (sh.flag[j] & fsx::kBinValid) && sh.E[j] == Eh[k];
        if (same_hyp && (sh.flag[j] & fsx::kBinTie)) w = true;
        want[k] = w;
        if (w) wanted += sh.C[j];
    }
    unsigned long long wanted_before =
        block_scan_exclusive(wanted, 0ull, [](unsigned long long a, unsigned long long c) { return a + c; }, sh.scan_u, (unsigned long long*)nullptr);
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        if (!reach[k] || (sh.flag[j] & fsx::kBinListed)) continue;
        if (want[k]) {
            wanted_before += sh.C[j];
            if (wanted_before <= (unsigned long long)room) { sh.flag[j] = fsx::kBinCollect; continue; }
        }
        const bool same_hyp = (sh.flag[j] & fsx::kBinValid) && sh.E[j] == Eh[k];
        if (!same_hyp) { sh.E[j] = (uint8_t)Eh[k]; sh.flag[j] = fsx::kBinDirty; sh.A[j] = 0; }
    }
    for (int i = tid; i < fsx::kBins / 32; i += kThreads) sh.tie_bits[i] = 0;
    __syncthreads();
}

// Descending bitonic sort of the list (padded with zeros, which sort last).
__device__ void sort_list(ExactShared& sh) {
    const int n = sh.list_n;
    int m = 1;
    while (m < n) m <<= 1;
    for (int i = n + threadIdx.x; i < m; i += kThreads) sh.list[i] = 0ull;
    __syncthreads();
    for (int k = 2; k <= m; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < m; i += kThreads) {
                const int l = i ^ j;
                if (l > i) {
                    const unsigned long long a = sh.list[i], c = sh.list[l];
                    const bool desc = (i & k) == 0;
                    if (desc ? a < c : a > c) { sh.list[i] = c; sh.list[l] = a; }
                }
            }
            __syncthreads();
        }
    }
}

struct RowCtx {
    const float* prob;   // the row's probabilities (scratch)
    long long V;
    float min_thr;
    bool vec_ok;
};

// Calls fn(p, index) for every kept candidate of the current level.
template <class F>
__device__ __forceinline__ void for_candidates(const RowCtx& c, uint32_t F_level, F&& fn) {
    const int tid = threadIdx.x;
    auto one = [&](float p, long long i) {
        if (!(p >= c.min_thr)) return;
        const uint32_t key = __float_as_uint(p);
        if (key < F_level) fn(p, key, i);
    };
    if (c.vec_ok) {
        const float4* r4 = reinterpret_cast<const float4*>(c.prob);
        const long long n4 = c.V >> 2;
        long long i = tid;
        for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = r4[i + u * kThreads];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long e = 4 * (i + u * kThreads);
                one(v[u].x, e); one(v[u].y, e + 1); one(v[u].z, e + 2); one(v[u].w, e + 3);
            }
        }
        for (; i < n4; i += kThreads) {
            const float4 v = r4[i];
            one(v.x, 4 * i); one(v.y, 4 * i + 1); one(v.z, 4 * i + 2); one(v.w, 4 * i + 3);
        }
        for (long long j = 4 * n4 + tid; j < c.V; j += kThreads) one(c.prob[j], j);
    } else {
        for (long long i = tid; i < c.V; i += kThreads) one(c.prob[i], i);
    }
}

// counts and approximate masses of the level's bins
__device__ void pass_counts(ExactShared& sh, const RowCtx& c) {
    const int tid = threadIdx.x;
    for (int j = tid; j < fsx::kBins; j += kThreads) {
        sh.A[j] = 0; sh.C[j] = 0; sh.R[j] = 0.f; sh.E[j] = 0; sh.flag[j] = 0;
    }
    if (tid == 0) sh.list_n = 0;
    __syncthreads();
    const fsx::Level L = sh.level;
    unsigned long long rest = 0;
    for_candidates(c, L.F, [&](float p, uint32_t key, long long) {
        const uint32_t j = fsx::bin_of(L, key);
        if (j >= (uint32_t)fsx::kBins) { ++rest; return; }
        atomicAdd(&sh.C[j], 1u);
        atomicAdd(&sh.R[j], p);
    });
    rest = block_sum_u64(rest, sh);
    if (tid == 0) sh.rest_cnt = rest > 0xffffffffull ? 0xffffffffu : (uint32_t)rest;
    __syncthreads();
}

// amounts of the dirty bins, elements of the bins to collect
__device__ void pass_amounts(ExactShared& sh, const RowCtx& c) {
    const fsx::Level L = sh.level;
    if (threadIdx.x == 0) ++sh.prof_passes;
    for_candidates(c, L.F, [&](float p, uint32_t key, long long i) {
        const uint32_t j = fsx::bin_of(L, key);
        if (j >= (uint32_t)fsx::kBins) return;
        const uint8_t f = sh.flag[j];
        if (f & fsx::kBinCollect) {
            const int pos = atomicAdd(&sh.list_n, 1);
            if (pos < kListCap) sh.list[pos] = fsx::make_entry(key, (uint32_t)i);
        } else if (f & fsx::kBinDirty) {
            bool tie;
            const fsx::Step st = fsx::step_of(p, sh.E[j], &tie);
            if (!tie) {
                const uint32_t old = atomicAdd(&sh.A[j], st.a);
                tie = old + st.a >= 0x80000000u;   // too much for one binade: never taken as a whole
            }
            if (tie) atomicOr(&sh.tie_bits[j >> 5], 1u << (j & 31));
        }
    });
    __syncthreads();
    for (int j = threadIdx.x; j < fsx::kBins; j += kThreads) {
        const uint8_t f = sh.flag[j];
        if (f & fsx::kBinCollect) sh.flag[j] = fsx::kBinListed;
        else if (f & fsx::kBinDirty) {
            const bool tie = (sh.tie_bits[j >> 5] >> (j & 31)) & 1u;
            sh.flag[j] = (uint8_t)(fsx::kBinValid | (tie ? fsx::kBinTie : 0));
        }
    }
    if (threadIdx.x == 0 && sh.list_n > kListCap) sh.list_n = kListCap;   // cannot happen: marks are granted within the room
    __syncthreads();
    sort_list(sh);
}

enum { kCtlDone = 0, kCtlNewLevel = 1, kCtlClassify = 2, kCtlRepeat = 3 };

// One run of the sorted walk from the top of the row: until the running sum exceeds thr or `limit`
// elements are in (tests/cpp/topp_model.hpp::run is the sequential statement).  Returns with
// sh.walk filled; sh.walk.status == kWalkFound or kWalkEnd (every candidate added).
__device__ void sorted_run(ExactShared& sh, const RowCtx& c, uint32_t F_top, float thr, uint32_t limit, double thr2, bool& have_level) {
    const int tid = threadIdx.x;
    __syncthreads();
    if (tid == 0) {
        sh.walk.s = 0.0f; sh.walk.cnt = 0; sh.walk.j = 0; sh.walk.li = 0;
    }
    if (!have_level || sh.level.F != F_top || sh.level.sh != fsx::kTopSh) {
        __syncthreads();
        if (tid == 0) sh.level = fsx::Level{F_top, fsx::kTopSh};
        have_level = false;
    }
    __syncthreads();
    for (;;) {
        if (!have_level) { pass_counts(sh, c); have_level = true; }
        prepare_walk(sh);
        if (tid == 0) {
            fsx::Walk w = sh.walk;
            const fsx::Bins b = bins_of(sh);
            const fsx::Level L = sh.level;
            fsx::walk_level(w, L, b, reinterpret_cast<const uint64_t*>(sh.list), sh.list_n, thr, limit);
            int ctl = kCtlDone;
            if (w.status == fsx::kWalkEnd) {
                const unsigned long long span = (unsigned long long)fsx::kBins << L.sh;
                if (sh.rest_cnt != 0 && span < L.F) {
                    sh.level = fsx::Level{(uint32_t)(L.F - span), fsx::kTopSh};
                    w.j = 0; w.li = 0;
                    ctl = kCtlNewLevel;
                }
            } else if (w.status == fsx::kWalkUnresolved) {
                const int j = w.j;
                if ((int)sh.C[j] > kListCap) {
                    if (L.sh == 0) {   // one key, too many copies to list
                        const uint32_t key = L.F - 1u - (uint32_t)j;
                        bool found, by_limit = false;
                        fsx::add_repeated(w.s, w.cnt, __uint_as_float(key), sh.C[j], thr, limit, &found, &by_limit);
                        if (found) {
                            w.status = fsx::kWalkFound; w.hit_key = key; w.hit_idx = 0xffffffffu; w.by_limit = by_limit;
                            ctl = kCtlDone;
                        } else {
                            w.j = j + 1;
                            sh.C[j] = 0;   // the bin is in the sum: the walk passes over it from now on
                            ctl = kCtlRepeat;
                        }
                    } else {
                        sh.level = fsx::Level{L.F - ((uint32_t)j << L.sh), L.sh >= fsx::kSubBits ? L.sh - fsx::kSubBits : 0};
                        w.j = 0; w.li = 0;
                        ctl = kCtlNewLevel;
                    }
                } else {
                    ctl = kCtlClassify;
                }
            }
            sh.walk = w;
            sh.ctl = ctl;
        }
        __syncthreads();
        const int ctl = sh.ctl;
        if (ctl == kCtlDone) break;
        if (ctl == kCtlNewLevel) { have_level = false; continue; }
        if (ctl == kCtlRepeat) continue;
        classify_bins(sh, sh.walk.j, sh.walk.s, sh.walk.cnt, thr, limit, thr2);
        if (tid == 0 && sh.cleared) sh.walk.li = 0;
        pass_amounts(sh, c);
    }
    // an element found by repetition of one key: its index is the lowest one holding the key
    if (sh.walk.status == fsx::kWalkFound && sh.walk.hit_idx == 0xffffffffu) {
        const uint32_t key = sh.walk.hit_key;
        int mine = 0x7fffffff;
        for (long long i = tid; i < c.V; i += kThreads)
            if (__float_as_uint(c.prob[i]) == key && c.prob[i] >= c.min_thr) { mine = (int)i; break; }
        const int idx = block_min_int(mine, sh);
        if (tid == 0) sh.walk.hit_idx = (uint32_t)idx;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kThreads, 2) sampler_exact_kernel(StepArgs a, float* scratch) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    ExactShared& sh = *reinterpret_cast<ExactShared*>(smem_raw);
    const int tid = threadIdx.x;
    const long long V = a.vocab;
    float* prob = scratch + (size_t)blockIdx.x * (size_t)((V + 3) & ~3LL);
    if (tid < 32) sh.exp_tab[tid] = fsx::kExp2TabDev[tid];
    __syncthreads();
#ifdef SAMPLER_EXACT_PROF
    long long prof_t[8];
#define PROF_MARK(i) prof_t[i] = clock64()
#else
#define PROF_MARK(i)
#endif
    for (int r = blockIdx.x; r < a.num_rows; r += gridDim.x) {
        const sampler_row_params p = a.rows[r];
        if (!(p.do_sample & SAMPLER_ROW_MULTINOMIAL)) continue;
        if (p.logits_row < 0 || p.logits_row >= a.num_logit_rows) continue;   // reported by the first kernel
        const bool top_k_active = p.top_k > 0 && p.top_k < 0x7fffffffffffffffLL;
        if (top_k_active && p.top_k < V) continue;                            // the top-k path of the first kernel
        const float* row = a.logits + p.logits_row * V;
        const bool raw_lp = (p.do_sample & SAMPLER_ROW_RAW_LOG_PROB) != 0;
        const float raw_lse = raw_lp ? a.out_log_prob[r] : 0.f;   // left there by the first kernel (NaN: no scratch for the raw logits)
        const bool vec_ok = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        __syncthreads();

        // 1. maximum
        PROF_MARK(0);
        if (tid == 0) sh.prof_passes = 0;
        float mx = -CUDART_INF_F;
        if (vec_ok) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            const long long n4 = V >> 2;
            for (long long i = tid; i < n4; i += kThreads) {
                const float4 q = r4[i];
                mx = fmaxf(mx, fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)));
            }
            for (long long j = 4 * n4 + tid; j < V; j += kThreads) mx = fmaxf(mx, row[j]);
        } else {
            for (long long i = tid; i < V; i += kThreads) mx = fmaxf(mx, row[i]);
        }
        mx = block_max(mx, sh);

        // 2. exponentials (parked in the scratch row) and their index-order sum
        const float T = p.temperature;
        const float inv_T = __fdiv_rn(1.0f, T);
        auto load_from = [&](const float* src) {
            return [src, V, vec_ok](long long i, float (&x)[kPer], bool (&keep)[kPer]) {
                if (vec_ok && i + kPer <= V) {
                    const float4 q0 = *reinterpret_cast<const float4*>(src + i), q1 = *reinterpret_cast<const float4*>(src + i + 4);
                    x[0] = q0.x; x[1] = q0.y; x[2] = q0.z; x[3] = q0.w; x[4] = q1.x; x[5] = q1.y; x[6] = q1.z; x[7] = q1.w;
#pragma unroll
                    for (int e = 0; e < kPer; ++e) keep[e] = true;
                } else {
#pragma unroll
                    for (int e = 0; e < kPer; ++e) {
                        keep[e] = i + e < V;
                        x[e] = keep[e] ? src[i + e] : 0.f;
                    }
                }
            };
        };
        // stores of kPer results: 16-byte pieces where the row allows (the scratch row is 16-byte aligned)
        auto store8 = [&](long long i, const float (&x)[kPer], const bool (&keep)[kPer]) {
            if (i + kPer <= V) {
                *reinterpret_cast<float4*>(prob + i) = make_float4(x[0], x[1], x[2], x[3]);
                *reinterpret_cast<float4*>(prob + i + 4) = make_float4(x[4], x[5], x[6], x[7]);
            } else {
#pragma unroll
                for (int e = 0; e < kPer; ++e) if (keep[e]) prob[i + e] = x[e];
            }
        };
        PROF_MARK(1);
        float norm = 0.0f;
        chain_sum(norm, V, load_from(row), [&](long long i, float (&x)[kPer], bool (&keep)[kPer]) {
#pragma unroll
            for (int e = 0; e < kPer; ++e) {
                const float d = __fsub_rn(x[e], mx);
                x[e] = keep[e] ? fsx::expf_libm(T == 1.0f ? d : __fmul_rn(d, inv_T), reinterpret_cast<const uint64_t*>(sh.exp_tab)) : 0.f;
            }
            store8(i, x, keep);
        }, 0.f, false, sh);
        __syncthreads();
        PROF_MARK(2);

        // 3. probabilities; the largest one is that of the maximum logit
        const float pmax = __fdiv_rn(1.0f, norm);
        const bool min_p_active = p.min_p > 0.0f;
        const float min_thr = min_p_active ? __fmul_rn((float)(double)p.min_p, pmax) : 0.0f;
        const bool top_p_active = p.top_p != 1.0f;
        RowCtx ctx{prob, V, min_thr, true};
        float total = 0.0f;
        long long kept_count = 0, last_kept = -1;
        if (!top_p_active) {
            // index-order total of the kept probabilities
            long long my_last = -1;
            unsigned long long my_cnt = 0;
            chain_sum(total, V, load_from(prob), [&](long long i, float (&x)[kPer], bool (&keep)[kPer]) {
#pragma unroll
                for (int e = 0; e < kPer; ++e) x[e] = keep[e] ? __fdiv_rn(x[e], norm) : 0.f;
                store8(i, x, keep);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    keep[e] = keep[e] && x[e] >= min_thr;
                    if (keep[e]) { my_last = i + e; ++my_cnt; }
                }
            }, 0.f, false, sh);
            kept_count = (long long)block_sum_u64(my_cnt, sh);
            const int m = block_min_int(my_last < 0 ? 0x7fffffff : -(int)my_last, sh);   // minimum of the negated = the highest index
            last_kept = m == 0x7fffffff ? -1 : -(long long)m;
        } else {
            // division, and the counts / approximate masses of the first level's bins in the same pass
            const uint32_t F_top = __float_as_uint(pmax) + 1u;
            if (tid == 0) sh.level = fsx::Level{F_top, fsx::kTopSh};
            for (int j = tid; j < fsx::kBins; j += kThreads) { sh.A[j] = 0; sh.C[j] = 0; sh.R[j] = 0.f; sh.E[j] = 0; sh.flag[j] = 0; }
            if (tid == 0) sh.list_n = 0;
            __syncthreads();
            const fsx::Level L = sh.level;
            unsigned long long rest = 0;
            const auto ld = load_from(prob);
            for (long long base = (long long)kPer * tid; base < V; base += kTile) {
                float x[kPer];
                bool keep[kPer];
                ld(base, x, keep);
#pragma unroll
                for (int e = 0; e < kPer; ++e) x[e] = keep[e] ? __fdiv_rn(x[e], norm) : 0.f;
                store8(base, x, keep);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    if (!keep[e] || !(x[e] >= min_thr)) continue;
                    const uint32_t key = __float_as_uint(x[e]);
                    if (key >= L.F) continue;
                    const uint32_t j = fsx::bin_of(L, key);
                    if (j >= (uint32_t)fsx::kBins) { ++rest; continue; }
                    atomicAdd(&sh.C[j], 1u);
                    atomicAdd(&sh.R[j], x[e]);
                }
            }
            rest = block_sum_u64(rest, sh);
            if (tid == 0) sh.rest_cnt = rest > 0xffffffffull ? 0xffffffffu : (uint32_t)rest;
        }
        __syncthreads();
        PROF_MARK(3);

        long long pick = -1;
        float pick_p = 0.f;
        bool uniform_fallback = false;
        if (!top_p_active) {
            if (!(total > 0.0f && isfinite(total))) {
                uniform_fallback = true;
            } else {
                const float rr = __fmul_rn(total, p.rand_u);
                float run = 0.0f;
                pick = chain_sum(run, V, load_from(prob), [&](long long, float (&x)[kPer], bool (&keep)[kPer]) {
#pragma unroll
                    for (int e = 0; e < kPer; ++e) keep[e] = keep[e] && x[e] >= min_thr;
                }, rr, true, sh);
                if (pick < 0) pick = last_kept;   // rounding left r at or beyond the total: the last kept element
            }
            if (pick >= 0) pick_p = prob[pick];
        } else {
            // 4. the sorted walk: the kept set, its total, then the draw over the same running sums
            const uint32_t F_top = __float_as_uint(pmax) + 1u;
            bool have_level = true;   // the division pass counted the first level's bins
            sorted_run(sh, ctx, F_top, p.top_p, 0u, (double)p.rand_u * (double)p.top_p, have_level);
            PROF_MARK(4);
            const uint32_t n_keep = sh.walk.cnt;
            total = sh.walk.s;
            kept_count = n_keep;
            __syncthreads();
            if (!(total > 0.0f && isfinite(total)) || n_keep == 0) {
                uniform_fallback = true;
            } else {
                const float rr = __fmul_rn(total, p.rand_u);
                sorted_run(sh, ctx, F_top, rr, n_keep, 0.0, have_level);
                if (sh.walk.status == fsx::kWalkFound) {
                    pick = sh.walk.hit_idx;
                    pick_p = __uint_as_float(sh.walk.hit_key);
                } else {   // cannot happen: the element limit ends the second run
                    if (tid == 0) atomicOr(a.status, 16u);
                    pick = 0; pick_p = prob[0];
                }
            }
            __syncthreads();
        }
        PROF_MARK(5);
#ifdef SAMPLER_EXACT_PROF
        if (tid == 0 && blockIdx.x == 0)
            printf("exact row %d: max %lld  exp+norm %lld  div(+total|+counts) %lld  run1|draw %lld  run2 %lld  (cycles) passes %d\n", r, prof_t[1] - prof_t[0],
                   prof_t[2] - prof_t[1], prof_t[3] - prof_t[2], (top_p_active ? prof_t[4] : prof_t[5]) - prof_t[3], top_p_active ? prof_t[5] - prof_t[4] : 0LL, sh.prof_passes);
#endif
        if (tid == 0) {
            float lp;
            if (uniform_fallback) {
                // non-finite or empty mass: the reference draws an index uniformly (sampler.cpp:1047-1059)
                const long long n = kept_count > 0 ? kept_count : V;
                long long k = (long long)(p.rand_u * (float)n);
                if (k > n - 1) k = n - 1;
                pick = k < V ? k : V - 1;
                lp = logf(1.0f / (float)n);
            } else {
                lp = logf(pick_p) - logf(total);
                if (raw_lp) {
                    float raw = row[pick];
                    const long long h0 = a.hist_offsets ? a.hist_offsets[r] : 0, h1 = a.hist_offsets ? a.hist_offsets[r + 1] : 0;
                    if (a.hist_raw)
                        for (long long i = h0; i < h1; ++i)
                            if (a.hist_ids[i] == pick) { raw = a.hist_raw[i]; break; }
                    lp = raw_lse != raw_lse ? CUDART_NAN_F : raw - raw_lse;
                }
            }
            a.out_token[r] = pick;
            a.out_log_prob[r] = lp;
        }
        __syncthreads();
    }
}

__global__ void expf_selftest_kernel(const float* in, float* out, long long n) {
    __shared__ uint64_t tab[32];
    if (threadIdx.x < 32) tab[threadIdx.x] = fsx::kExp2TabDev[threadIdx.x];
    __syncthreads();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) out[i] = fsx::expf_libm(in[i], tab);
}

}  // namespace

cudaError_t launch_expf_selftest(const float* in, float* out, long long n, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    expf_selftest_kernel<<<592, 256, 0, stream>>>(in, out, n);
    return cudaGetLastError();
}

size_t sampler_exact_smem_bytes() { return sizeof(ExactShared); }

size_t sampler_exact_scratch_bytes(int ctas, long long vocab) { return (size_t)ctas * (size_t)((vocab + 3) & ~3LL) * sizeof(float); }

cudaError_t launch_sampler_exact(const StepArgs& a, float* scratch, int ctas, cudaStream_t stream) {
    if (a.num_rows <= 0 || ctas <= 0) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(sampler_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ExactShared));
    if (e != cudaSuccess) return e;
    const int grid = a.num_rows < ctas ? a.num_rows : ctas;
    sampler_exact_kernel<<<grid, kThreads, sizeof(ExactShared), stream>>>(a, scratch);
    return cudaGetLastError();
}

}  // namespace sampler
