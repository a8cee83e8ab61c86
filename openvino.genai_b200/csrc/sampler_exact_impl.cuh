// Body of the exact full-vocabulary sampler (sampler_exact.cu includes this file once per CTA size, inside a namespace of
// its own: SX_THREADS threads per CTA, SX_CTAS_PER_SM resident CTAs).  No include guard on purpose.

constexpr int kThreads = SX_THREADS;
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
    // checkpoints of the top-p run's walk over the first level's bins (fsx::Checkpoints), for the draws of the same row
    float ck_s[fsx::kBins / fsx::kCkGroup];
    uint32_t ck_cnt[fsx::kBins / fsx::kCkGroup];   // 0xffffffff: the walk never stood at a bin of this group
    uint16_t ck_j[fsx::kBins / fsx::kCkGroup];
    uint16_t ck_li[fsx::kBins / fsx::kCkGroup];
    int ck_on;         // the checkpoints belong to this row
    int ck_li_stale;   // the list was emptied after some were taken: their list positions are void
    // block scan / reduce scratch
    fsx::Step scan_step[kWarps];
    uint32_t scan_u32[kWarps];
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
    int prof_slow_spans;
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
    // every warp scans the warp totals itself (lane i holds warp i's): four shuffle rounds instead of a walk over all of them
    T wt = lane < kWarps ? warp_buf[lane] : identity;
#pragma unroll
    for (int o = 1; o < kWarps; o <<= 1) {
        union { T t; uint32_t u[sizeof(T) / 4]; } a, r;
        a.t = wt;
#pragma unroll
        for (int i = 0; i < (int)(sizeof(T) / 4); ++i) r.u[i] = __shfl_up_sync(0xffffffffu, a.u[i], o);
        if (lane >= o && lane < kWarps) wt = op(r.t, wt);
    }
    auto pick = [&](int src) {
        union { T t; uint32_t u[sizeof(T) / 4]; } a, r;
        a.t = wt;
#pragma unroll
        for (int i = 0; i < (int)(sizeof(T) / 4); ++i) r.u[i] = __shfl_sync(0xffffffffu, a.u[i], src);
        return r.t;
    };
    const T all = pick(kWarps - 1);
    const T before_incl = pick(w > 0 ? w - 1 : 0);
    const T before = w > 0 ? before_incl : identity;
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
// `s += v[i]` over a whole row, exactly as the host loop does it, without a barrier per tile.
// The row is cut into spans of consecutive elements; every warp owns whole spans.  A first pass leaves
// an approximate mass per span, from which the exponent of the running sum at each span is
// hypothesised; the exact pass then adds a span's amounts under that hypothesis into one integer
// A[j] (their order does not matter while no element is a tie and the sum stays in its binade).
// One thread walks the spans and checks each hypothesis against the exact sum so far; a span that
// fails (tie, change of binade, wrong guess, or the draw's threshold inside it) is added element by
// element with a block scan of two-state steps.  Spans share the bin arrays of the sorted walk, which
// runs later.
constexpr int kSpanBase = 2048;
constexpr int kHead = 256;          // elements at the start of a row that one thread adds with real additions

struct SpanGeom {
    long long len;   // elements per span
    int count;       // spans of the row (<= fsx::kBins)
};
__device__ __forceinline__ SpanGeom span_geom(long long V) {
    const long long mult = (V + (long long)kSpanBase * fsx::kBins - 1) / ((long long)kSpanBase * fsx::kBins);
    const long long len = kSpanBase * (mult < 1 ? 1 : mult);
    return SpanGeom{len, (int)((V + len - 1) / len)};
}

// Calls fn(values[4], keep[4], index of values[0]) for every group of four consecutive elements of span j,
// dealt to the lanes of the calling warp; four 16-byte loads in flight per lane.
template <class F>
__device__ __forceinline__ void for_span(const float* src, long long V, bool vec_ok, const SpanGeom& g, int j, F&& fn) {
    const int lane = threadIdx.x & 31;
    const long long lo = (long long)j * g.len, hi = min(V, lo + g.len);
    for (long long base = lo + 4 * lane; base < hi; base += 4 * 32 * 4) {
        float x[4][4];
        bool keep[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long i = base + (long long)u * 128;
            if (vec_ok && i + 4 <= hi) {
                const float4 q = *reinterpret_cast<const float4*>(src + i);
                x[u][0] = q.x; x[u][1] = q.y; x[u][2] = q.z; x[u][3] = q.w;
                keep[u][0] = keep[u][1] = keep[u][2] = keep[u][3] = true;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    keep[u][e] = i + e < hi;
                    x[u][e] = keep[u][e] ? src[i + e] : 0.f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) fn(x[u], keep[u], base + (long long)u * 128);
    }
}

// Hypothesised exponent of the running sum at every span, from the approximate masses R[] scaled by
// `scale` and a sum that starts at zero.  A span whose range (widened by the margin) is not inside one
// binade gets exponent 0, which no sum has: the walk then adds it element by element.
__device__ void hypothesise_spans(ExactShared& sh, int spans, float scale) {
    const int tid = threadIdx.x, j0 = tid * kBinsPerThread;
    double mass = 0.0;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k)
        if (j0 + k < spans) mass += (double)sh.R[j0 + k] * (double)scale;
    double cum = block_scan_exclusive(mass, 0.0, [](double a, double c) { return a + c; }, sh.scan_d, (double*)nullptr);
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        if (j >= spans) break;
        const double lo = cum, hi = cum + (double)sh.R[j] * (double)scale;
        cum = hi;
        uint32_t E;
        const bool certain = fsx::hyp_exponent(lo, hi, kMargin, &E);
        sh.E[j] = certain ? (uint8_t)E : (uint8_t)0;
        sh.A[j] = 0;
    }
    for (int i = tid; i < fsx::kBins / 32; i += kThreads) sh.tie_bits[i] = 0;
    __syncthreads();
}

// Adds span j element by element (block scan of steps, real additions where the binade changes) to the
// state (E, S).  Values come from `src` and are kept when >= min_thr.  With use_thr the scan stops at the
// first running sum above thr and returns that element's index (else -1).
__device__ long long span_exact(ExactShared& sh, const float* src, long long V, bool vec_ok, const SpanGeom& g, int j, float min_thr, uint32_t& E,
                                uint32_t& S, float thr, bool use_thr) {
    const int tid = threadIdx.x;
    const long long lo = (long long)j * g.len, hi = min(V, lo + g.len);
    for (long long base = lo; base < hi; base += kThreads * 4) {
        float x[4];
        bool keep[4];
        const long long i0 = base + 4 * tid;
        if (vec_ok && i0 + 4 <= hi) {
            const float4 q = *reinterpret_cast<const float4*>(src + i0);
            x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
#pragma unroll
            for (int e = 0; e < 4; ++e) keep[e] = x[e] >= min_thr;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                x[e] = i0 + e < hi ? src[i0 + e] : 0.f;
                keep[e] = i0 + e < hi && x[e] >= min_thr;
            }
        }
        int from = 0;   // elements of the tile below `from` are already in the sum
        if (base == 0) {
            // The sum starts at zero and changes binade at almost every one of the first additions: one thread
            // adds the head of the row with real additions (every scan below costs a few barriers per change).
            float* head = reinterpret_cast<float*>(sh.list);
            if (tid < kHead / 4) {
#pragma unroll
                for (int e = 0; e < 4; ++e) head[4 * tid + e] = keep[e] ? x[e] : -1.0f;   // -1: not in the sum
            }
            __syncthreads();
            if (tid == 0) {
                float s = fsx::state_float(E, S);
                int hit = -1;
                const int n = (int)min((long long)kHead, hi - base);
                for (int i = 0; i < n; ++i) {
                    const float v = head[i];
                    if (v < 0.0f) continue;
                    s = __fadd_rn(s, v);
                    if (use_thr && s > thr) { hit = i; break; }
                }
                sh.bc_E = fsx::state_exp(s); sh.bc_S = fsx::state_sig(s); sh.bc_idx = hit;
            }
            __syncthreads();
            E = sh.bc_E; S = sh.bc_S;
            const int hit = sh.bc_idx;
            __syncthreads();
            if (hit >= 0) return base + hit;
            from = kHead;
        }
        for (;;) {
            // Without a tie among the remaining elements their amounts are plain integers: an integer scan finds where
            // the sum leaves the binade or exceeds the threshold.  With one, the scan composes two-state steps.
            {
                const float scale = fsx::amount_scale(E);
                uint32_t amt[4], mine_sum = 0;
                bool defer = scale == 0.0f;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    amt[e] = 0;
                    if (keep[e] && 4 * tid + e >= from) {
                        bool d;
                        amt[e] = fsx::plain_amount(x[e], scale, &d);
                        defer |= d;
                    }
                    mine_sum = fsx::sat_add(mine_sum, amt[e] > fsx::kSat ? fsx::kSat : amt[e]);
                }
                if (!__syncthreads_or(defer ? 1 : 0)) {
                    uint32_t total_amt;
                    const uint32_t before = block_scan_exclusive(mine_sum, 0u, [](uint32_t p, uint32_t q) { return fsx::sat_add(p, q); }, sh.scan_u32, &total_amt);
                    const bool crossed_i = S + total_amt >= fsx::kOne24;
                    const bool over_i = use_thr && !crossed_i && fsx::state_float(E, S + total_amt) > thr;
                    if (!crossed_i && !over_i) { S += total_amt; break; }
                    int mine_first = 0x7fffffff;
                    uint32_t run = before, run_before_first = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t prev = run;
                        run = fsx::sat_add(run, amt[e]);
                        if (!(keep[e] && 4 * tid + e >= from) || mine_first != 0x7fffffff) continue;
                        if (S + run >= fsx::kOne24 || (use_thr && fsx::state_float(E, S + run) > thr)) { mine_first = 4 * tid + e; run_before_first = prev; }
                    }
                    const int first = block_min_int(mine_first, sh);
                    if (first >> 2 == tid) {
                        const int e = first & 3;
                        const float xe = e == 0 ? x[0] : e == 1 ? x[1] : e == 2 ? x[2] : x[3];
                        const float after = __fadd_rn(fsx::state_float(E, S + run_before_first), xe);
                        sh.bc_E = fsx::state_exp(after);
                        sh.bc_S = fsx::state_sig(after);
                    }
                    __syncthreads();
                    E = sh.bc_E; S = sh.bc_S;
                    __syncthreads();
                    if (use_thr && fsx::state_float(E, S) > thr) return base + first;
                    from = first + 1;
                    continue;
                }
            }
            fsx::Step loc[4];
            fsx::Step acc = fsx::step_identity();
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (keep[e] && 4 * tid + e >= from) acc = fsx::then(acc, fsx::step_of(x[e], E));
                loc[e] = acc;
            }
            fsx::Step total;
            const fsx::Step excl = block_scan_exclusive(acc, fsx::step_identity(), StepOp(), sh.scan_step, &total);
            const uint32_t S_end = fsx::apply(total, S);
            const bool crossed = S_end >= fsx::kOne24;
            const bool over = use_thr && !crossed && fsx::state_float(E, S_end) > thr;
            if (!crossed && !over) { S = S_end; break; }
            int mine = 0x7fffffff;   // first element at which the sum leaves the binade or exceeds the threshold
#pragma unroll
            for (int e = 3; e >= 0; --e) {
                if (!(keep[e] && 4 * tid + e >= from)) continue;
                const uint32_t Se = fsx::apply(fsx::then(excl, loc[e]), S);
                if (Se >= fsx::kOne24 || (use_thr && fsx::state_float(E, Se) > thr)) mine = 4 * tid + e;
            }
            const int first = block_min_int(mine, sh);
            if (first >> 2 == tid) {
                const int e = first & 3;
                const fsx::Step pre = e == 0 ? excl : fsx::then(excl, e == 1 ? loc[0] : e == 2 ? loc[1] : loc[2]);   // skipped elements are identities
                const float xe = e == 0 ? x[0] : e == 1 ? x[1] : e == 2 ? x[2] : x[3];
                const float after = __fadd_rn(fsx::state_float(E, fsx::apply(pre, S)), xe);
                sh.bc_E = fsx::state_exp(after);
                sh.bc_S = fsx::state_sig(after);
            }
            __syncthreads();
            E = sh.bc_E; S = sh.bc_S;
            __syncthreads();
            if (use_thr && fsx::state_float(E, S) > thr) return base + first;
            from = first + 1;
        }
    }
    return -1;
}

// Walks the spans from the start of the row: whole spans where the hypothesis holds, span_exact
// elsewhere.  Returns the final sum in s; with use_thr, the index of the first element whose running
// sum exceeds thr (-1: none).
__device__ long long walk_spans(ExactShared& sh, const float* src, long long V, bool vec_ok, const SpanGeom& g, float min_thr, float& s, float thr,
                                bool use_thr) {
    uint32_t E = 1u, S = 0u;
    int j = 0;
    __syncthreads();
    for (;;) {
        if (threadIdx.x == 0) {
            while (j < g.count) {
                const uint32_t add = sh.A[j];
                const bool tie = (sh.tie_bits[j >> 5] >> (j & 31)) & 1u;
                if (tie || (uint32_t)sh.E[j] != E) break;
                if (S == 0u || add >= fsx::kOne24 || S + add >= fsx::kOne24) break;
                if (use_thr && fsx::state_float(E, S + add) > thr) break;
                S += add;
                ++j;
            }
            sh.bc_E = E; sh.bc_S = S; sh.bc_idx = j;
        }
        __syncthreads();
        E = sh.bc_E; S = sh.bc_S; j = sh.bc_idx;
        __syncthreads();
        if (j >= g.count) break;
#ifdef SAMPLER_EXACT_PROF
        if (threadIdx.x == 0) ++sh.prof_slow_spans;
#endif
        const long long hit = span_exact(sh, src, V, vec_ok, g, j, min_thr, E, S, thr, use_thr);
        if (hit >= 0) { s = fsx::state_float(E, S); return hit; }
        ++j;
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
        if ((int)sh.C[j_from] > kListCap - sh.list_n) { sh.cleared = 1; sh.list_n = 0; sh.ck_li_stale = 1; }
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
    bool cert[kBinsPerThread];
    unsigned long long wanted = 0;
#pragma unroll
    for (int k = 0; k < kBinsPerThread; ++k) {
        const int j = j0 + k;
        want[k] = false; reach[k] = false; Eh[k] = 0; cert[k] = false;
        if (j < j_from || sh.C[j] == 0) continue;
        const double lo = cum, hi = cum + (double)sh.R[j];
        const unsigned long long cbefore = cc;
        cum = hi; cc += sh.C[j];
        if (lo * (1.0 - kMargin) > (double)thr || (limit && cbefore >= limit)) continue;   // beyond what the walk can reach
        reach[k] = true;
        if (sh.flag[j] & fsx::kBinListed) continue;
        const bool certain = fsx::hyp_exponent(lo, hi, kMargin, &Eh[k]);
        cert[k] = certain;
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
            if (wanted_before <= (unsigned long long)room) {
                sh.E[j] = (uint8_t)(cert[k] ? Eh[k] : 0u);   // the exponent under which its elements may later be taken as one step, or none
                sh.flag[j] = fsx::kBinCollect;
                continue;
            }
        }
        const bool same_hyp = (sh.flag[j] & fsx::kBinValid) && sh.E[j] == Eh[k];
        if (!same_hyp) { sh.E[j] = (uint8_t)Eh[k]; sh.flag[j] = fsx::kBinDirty; sh.A[j] = 0; sh.PA[j] = 0; }
    }
    for (int i = tid; i < fsx::kBins / 32; i += kThreads) sh.tie_bits[i] = 0;
    __syncthreads();
}

// Descending bitonic sort of the list (padded with zeros, which sort last).
__device__ void sort_list(ExactShared& sh) {
    const int n = sh.list_n;
    int m = 64;   // at least one warp's block of 64 entries
    while (m < n) m <<= 1;
    for (int i = n + threadIdx.x; i < m; i += kThreads) sh.list[i] = 0ull;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // compare-exchange steps whose partners lie inside one block of 64 entries (j <= 32) are done by the block's warp with
    // warp-level synchronisation only; the whole CTA meets only around the steps that reach across blocks
    auto local_steps = [&](int k, int j_first) {   // the steps j_first, j_first / 2, ..., 1 of merge size k
        for (int b0 = warp * 64; b0 < m; b0 += kWarps * 64) {
            for (int j = j_first; j > 0; j >>= 1) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int i = b0 + lane + 32 * h;
                    const int l = i ^ j;
                    if (l > i) {
                        const unsigned long long a = sh.list[i], c = sh.list[l];
                        const bool desc = (i & k) == 0;
                        if (desc ? a < c : a > c) { sh.list[i] = c; sh.list[l] = a; }
                    }
                }
                __syncwarp();
            }
        }
    };
    for (int k = 2; k <= 64 && k <= m; k <<= 1) local_steps(k, k >> 1);
    __syncthreads();
    for (int k = 128; k <= m; k <<= 1) {
        for (int j = k >> 1; j >= 64; j >>= 1) {
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
        local_steps(k, 32);
        __syncthreads();
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
            // the amount (below 2^24) goes in as two 16-bit pieces (A: low, PA: high; PA is rebuilt by prepare_walk afterwards):
            // neither piece can overflow while the bin has fewer than 2^16 elements, so no result of an atomic is needed and
            // the additions do not wait for one another
            bool tie;
            const uint32_t amount = fsx::plain_amount(p, fsx::amount_scale(sh.E[j]), &tie);
            if (!tie) {
                atomicAdd(&sh.A[j], amount & 0xffffu);
                atomicAdd(&sh.PA[j], amount >> 16);
            } else {
                atomicOr(&sh.tie_bits[j >> 5], 1u << (j & 31));
            }
        }
    });
    __syncthreads();
    for (int j = threadIdx.x; j < fsx::kBins; j += kThreads) {
        const uint8_t f = sh.flag[j];
        if (f & fsx::kBinCollect) sh.flag[j] = fsx::kBinListed;
        else if (f & fsx::kBinDirty) {
            bool tie = (sh.tie_bits[j >> 5] >> (j & 31)) & 1u;
            const unsigned long long whole = ((unsigned long long)sh.PA[j] << 16) + sh.A[j];
            if (whole >= 0x80000000ull || sh.C[j] >= 65536u) tie = true;   // too much for one binade: never taken as a whole
            sh.A[j] = tie ? 0u : (uint32_t)whole;
            sh.flag[j] = (uint8_t)(fsx::kBinValid | (tie ? fsx::kBinTie : 0));
        }
    }
    if (threadIdx.x == 0 && sh.list_n > kListCap) sh.list_n = kListCap;   // cannot happen: marks are granted within the room
    __syncthreads();
    sort_list(sh);
    // Every listed bin with a hypothesis: the composition of its elements' steps in list order (one thread per bin: a bin holds
    // a handful of elements; its entries are the run of keys of the bin's range in the sorted list).
    if (sh.list_n > kTopCount + 64) {   // (a list of little more than the row's first elements has no bin worth a step)
        const int n = sh.list_n;
        const unsigned long long* list = sh.list;
        for (int j = threadIdx.x; j < fsx::kBins; j += kThreads) {
            const uint8_t f = sh.flag[j];
            if (!(f & fsx::kBinListed)) continue;
            sh.flag[j] = (uint8_t)(f & ~fsx::kBinStep);
            const uint32_t E = sh.E[j];
            if (E < 24u || E > 254u) continue;
            const uint32_t hi_key = L.F - 1u - ((uint32_t)j << L.sh);
            const long long lo_ll = (long long)L.F - ((long long)(j + 1) << L.sh);
            const uint32_t lo_key = lo_ll > 0 ? (uint32_t)lo_ll : 0u;
            int a = 0, z = n;   // first entry with key <= hi_key
            while (a < z) {
                const int mid = (a + z) >> 1;
                if (fsx::entry_key(list[mid]) > hi_key) a = mid + 1; else z = mid;
            }
            fsx::Step st = fsx::step_identity();
            uint32_t cnt = 0;
            for (int i = a; i < n; ++i) {
                const uint32_t key = fsx::entry_key(list[i]);
                if (key < lo_key) break;
                st = fsx::then(st, fsx::step_of(__uint_as_float(key), E));
                ++cnt;
            }
            if (cnt == sh.C[j] && fsx::step_packs(st)) {
                sh.A[j] = fsx::pack_step(st);
                sh.flag[j] = (uint8_t)(f | fsx::kBinStep);
            }
        }
        __syncthreads();
    }
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
    const bool record = limit == 0 && sh.ck_on != 0;   // the top-p run of a row leaves checkpoints, its draws use them
    if (limit != 0 && have_level && sh.ck_on != 0) {
        // the last bin at which the top-p run stood with a sum and a count that this run has not passed either
        int best = -1;
        for (int g = tid; g < fsx::kBins / fsx::kCkGroup; g += kThreads) {
            const uint32_t cn = sh.ck_cnt[g];
            if (cn != 0xffffffffu && cn < limit && sh.ck_s[g] <= thr) best = g;
        }
        best = -block_min_int(-best, sh);
        if (tid == 0 && best >= 0 && sh.ck_j[best] > 0) {
            sh.walk.s = sh.ck_s[best]; sh.walk.cnt = sh.ck_cnt[best]; sh.walk.j = (int)sh.ck_j[best];
            sh.walk.li = sh.ck_li_stale ? 0 : (int)sh.ck_li[best];
        }
        __syncthreads();
    }
    for (;;) {
        if (!have_level) { pass_counts(sh, c); have_level = true; }
        prepare_walk(sh);
        if (tid == 0) {
            fsx::Walk w = sh.walk;
            const fsx::Bins b = bins_of(sh);
            const fsx::Level L = sh.level;
            const fsx::Checkpoints ck{sh.ck_s, sh.ck_cnt, sh.ck_j, sh.ck_li};
            const bool top_level = L.F == F_top && L.sh == fsx::kTopSh;
            fsx::walk_level(w, L, b, reinterpret_cast<const uint64_t*>(sh.list), sh.list_n, thr, limit, record && top_level ? &ck : nullptr);
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

__global__ void __launch_bounds__(kThreads, SX_CTAS_PER_SM) sampler_exact_kernel(StepArgs a, float* scratch) {
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
#ifdef SAMPLER_EXACT_PROF
        unsigned long long prof_g0;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(prof_g0));
#endif
        if (tid == 0) { sh.prof_passes = 0; sh.prof_slow_spans = 0; }
        const SpanGeom sg = span_geom(V);
        const float T = p.temperature;
        const float inv_T = __fdiv_rn(1.0f, T);
        const int lane = tid & 31, warp = tid >> 5;
        float mx = -CUDART_INF_F;
        if (vec_ok) {
            const float4* r4 = reinterpret_cast<const float4*>(row);
            const long long n4 = V >> 2;
            long long i = tid;
            for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
                float4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) q[u] = r4[i + u * kThreads];
#pragma unroll
                for (int u = 0; u < 4; ++u) mx = fmaxf(mx, fmaxf(fmaxf(q[u].x, q[u].y), fmaxf(q[u].z, q[u].w)));
            }
            for (; i < n4; i += kThreads) {
                const float4 q = r4[i];
                mx = fmaxf(mx, fmaxf(fmaxf(q.x, q.y), fmaxf(q.z, q.w)));
            }
            for (long long j = 4 * n4 + tid; j < V; j += kThreads) mx = fmaxf(mx, row[j]);
        } else {
            for (long long i = tid; i < V; i += kThreads) mx = fmaxf(mx, row[i]);
        }
        mx = block_max(mx, sh);
        PROF_MARK(1);

        // 2. exponentials (parked in the scratch row) with a float sum per span for the hypotheses, the
        //    spans' amounts under those, and the index-order sum
        for (int j = warp; j < sg.count; j += kWarps) {
            float mass = 0.f;
            for_span(row, V, vec_ok, sg, j, [&](const float (&x)[4], const bool (&keep)[4], long long i) {
                float y[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float d = __fsub_rn(x[e], mx);
                    y[e] = keep[e] ? fsx::expf_libm(T == 1.0f ? d : __fmul_rn(d, inv_T), reinterpret_cast<const uint64_t*>(sh.exp_tab)) : 0.f;
                    mass += y[e];
                }
                if (keep[3]) *reinterpret_cast<float4*>(prob + i) = make_float4(y[0], y[1], y[2], y[3]);
                else {
#pragma unroll
                    for (int e = 0; e < 3; ++e) if (keep[e]) prob[i + e] = y[e];
                }
            });
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mass += __shfl_xor_sync(0xffffffffu, mass, o);
            if (lane == 0) sh.R[j] = mass;
        }
        __syncthreads();
        PROF_MARK(6);
        hypothesise_spans(sh, sg.count, 1.0f);
        // every lane re-reads the elements it wrote itself
        auto span_amounts = [&](float min_keep, long long* last, unsigned long long* count) {
            for (int j = warp; j < sg.count; j += kWarps) {
                const float scale = fsx::amount_scale(sh.E[j]);
                uint32_t amount = 0;
                bool tie = false;
                for_span(prob, V, true, sg, j, [&](const float (&x)[4], const bool (&keep)[4], long long i) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (!(keep[e] && x[e] >= min_keep)) continue;
                        bool t;
                        amount += fsx::plain_amount(x[e], scale, &t);   // below 2^24 each unless deferred: a lane's 64 or so cannot overflow
                        tie |= t;
                        if (last) { *last = i + e; ++*count; }
                    }
                });
                const unsigned long long whole = (unsigned long long)__reduce_add_sync(0xffffffffu, amount >> 16) * 65536ull + __reduce_add_sync(0xffffffffu, amount & 0xffffu);
                const bool any_tie = __any_sync(0xffffffffu, tie) || scale == 0.0f;
                if (lane == 0) {
                    sh.A[j] = whole >= fsx::kOne24 ? fsx::kOne24 : (uint32_t)whole;
                    if (any_tie) atomicOr(&sh.tie_bits[j >> 5], 1u << (j & 31));
                }
            }
        };
        span_amounts(0.0f, nullptr, nullptr);
        PROF_MARK(7);
        float norm = 0.0f;
        walk_spans(sh, prob, V, true, sg, 0.0f, norm, 0.f, false);
        PROF_MARK(2);

        // 3. probabilities; the largest one is that of the maximum logit
        const float pmax = __fdiv_rn(1.0f, norm);
        const float inv_norm = pmax;   // RN(1 / norm), the shared reciprocal of the row's divisions
        const bool min_p_active = p.min_p > 0.0f;
        const float min_thr = min_p_active ? __fmul_rn((float)(double)p.min_p, pmax) : 0.0f;
        const bool top_p_active = p.top_p != 1.0f;
        RowCtx ctx{prob, V, min_thr, true};
        float total = 0.0f;
        long long kept_count = 0, last_kept = -1;
        const uint32_t F_level = __float_as_uint(pmax) + 1u;
        if (top_p_active) {
            __syncthreads();
            if (tid == 0) sh.level = fsx::Level{F_level, fsx::kTopSh};
            for (int j = tid; j < fsx::kBins; j += kThreads) { sh.A[j] = 0; sh.C[j] = 0; sh.R[j] = 0.f; sh.E[j] = 0; sh.flag[j] = 0; }
            if (tid == 0) sh.list_n = 0;
            __syncthreads();
        }
        {
            // division; with top-p also the counts / approximate masses of the first level's bins
            const fsx::Level L = fsx::Level{F_level, fsx::kTopSh};
            unsigned long long rest = 0;
            for (int j = warp; j < sg.count; j += kWarps) {
                for_span(prob, V, true, sg, j, [&](const float (&x)[4], const bool (&keep)[4], long long i) {
                    float y[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) y[e] = keep[e] ? fsx::div_shared(x[e], norm, inv_norm) : 0.f;
                    if (keep[3]) *reinterpret_cast<float4*>(prob + i) = make_float4(y[0], y[1], y[2], y[3]);
                    else {
#pragma unroll
                        for (int e = 0; e < 3; ++e) if (keep[e]) prob[i + e] = y[e];
                    }
                    if (!top_p_active) return;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (!keep[e] || !(y[e] >= min_thr)) continue;
                        const uint32_t key = __float_as_uint(y[e]);
                        if (key >= L.F) continue;
                        const uint32_t b = fsx::bin_of(L, key);
                        if (b >= (uint32_t)fsx::kBins) { ++rest; continue; }
                        atomicAdd(&sh.C[b], 1u);
                        atomicAdd(&sh.R[b], y[e]);
                    }
                });
            }
            if (top_p_active) {
                rest = block_sum_u64(rest, sh);
                if (tid == 0) sh.rest_cnt = rest > 0xffffffffull ? 0xffffffffu : (uint32_t)rest;
            }
        }
        if (!top_p_active) {
            // index-order total of the kept probabilities: the spans' masses are those of the exponentials over the sum
            // (min-p drops mass: a guess that no longer holds only costs a scan of the span)
            __syncthreads();
            hypothesise_spans(sh, sg.count, inv_norm);
            long long my_last = -1;
            unsigned long long my_cnt = 0;
            span_amounts(min_thr, &my_last, &my_cnt);
            kept_count = (long long)block_sum_u64(my_cnt, sh);
            const int m = block_min_int(my_last < 0 ? 0x7fffffff : -(int)my_last, sh);   // minimum of the negated = the highest index
            last_kept = m == 0x7fffffff ? -1 : -(long long)m;
            walk_spans(sh, prob, V, true, sg, min_thr, total, 0.f, false);
        }
        __syncthreads();
        PROF_MARK(3);

        // 4. the kept set and its total (top-p: the sorted walk), then the draws over the same running sums
        const uint32_t F_top = F_level;
        bool have_level = true;   // top-p: the division pass counted the first level's bins
        uint32_t n_keep = 0;
        if (top_p_active) {
            for (int j = tid; j < fsx::kBins / fsx::kCkGroup; j += kThreads) sh.ck_cnt[j] = 0xffffffffu;
            if (tid == 0) { sh.ck_on = 1; sh.ck_li_stale = 0; }
            __syncthreads();
            sorted_run(sh, ctx, F_top, p.top_p, 0u, (double)p.rand_u * (double)p.top_p, have_level);
            n_keep = sh.walk.cnt;
            total = sh.walk.s;
            kept_count = n_keep;
            __syncthreads();
        }
        PROF_MARK(4);
        const bool uniform_fallback = !(total > 0.0f && isfinite(total)) || (top_p_active && n_keep == 0);
        const long long x0 = a.extra_offsets ? a.extra_offsets[r] : 0, x1 = a.extra_offsets ? a.extra_offsets[r + 1] : 0;
        for (long long k = -1; k < x1 - x0; ++k) {   // the row's own draw, then the further ones (sampler.cpp:1065)
            const float u = k < 0 ? p.rand_u : a.extra_rand_u[x0 + k];
            long long pick = -1;
            float pick_p = 0.f;
            if (!uniform_fallback) {
                const float rr = __fmul_rn(total, u);
                if (!top_p_active) {
                    float run = 0.0f;
                    pick = walk_spans(sh, prob, V, true, sg, min_thr, run, rr, true);   // the same sums again, up to the draw
                    if (pick < 0) pick = last_kept;   // rounding left r at or beyond the total: the last kept element
                    if (pick >= 0) pick_p = prob[pick];
                } else {
                    sorted_run(sh, ctx, F_top, rr, n_keep, 0.0, have_level);
                    if (sh.walk.status == fsx::kWalkFound) {
                        pick = sh.walk.hit_idx;
                        pick_p = __uint_as_float(sh.walk.hit_key);
                    } else {   // cannot happen: the element limit ends the run
                        if (tid == 0) atomicOr(a.status, 16u);
                        pick = 0; pick_p = prob[0];
                    }
                    __syncthreads();
                }
            }
            if (tid == 0) {
                float lp;
                if (uniform_fallback) {
                    // non-finite or empty mass: the reference draws an index uniformly (sampler.cpp:1047-1059)
                    const long long n = kept_count > 0 ? kept_count : V;
                    long long q = (long long)(u * (float)n);
                    if (q > n - 1) q = n - 1;
                    pick = q < V ? q : V - 1;
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
                if (k < 0) { a.out_token[r] = pick; a.out_log_prob[r] = lp; }
                else { a.extra_out_token[x0 + k] = pick; a.extra_out_log_prob[x0 + k] = lp; }
            }
        }
        PROF_MARK(5);
#ifdef SAMPLER_EXACT_PROF
        if (tid == 0) {
            unsigned long long g1;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g1));
            const unsigned long long dur = (g1 - prof_g0) / 1000;
            if (blockIdx.x % 64 == 0 || dur > 450)
                printf("block %d row %d start %llu us dur %llu us: max %lld  exp %lld  hyp+amounts %lld  walk %lld  div(+total|+counts) %lld  keep %lld  draws %lld  (cycles) passes %d slow spans %d of %d\n",
                       blockIdx.x, r, (prof_g0 / 1000) % 100000, dur, prof_t[1] - prof_t[0], prof_t[6] - prof_t[1], prof_t[7] - prof_t[6], prof_t[2] - prof_t[7], prof_t[3] - prof_t[2],
                       prof_t[4] - prof_t[3], prof_t[5] - prof_t[4], sh.prof_passes, sh.prof_slow_spans, sg.count);
        }
#endif
        __syncthreads();
    }
}

