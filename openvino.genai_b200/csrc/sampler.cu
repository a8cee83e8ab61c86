// Sampler step for sm_100a: one kernel launch for the whole batch, one CTA per sampled row.
//
// Phases of a row (src/cpp/src/sampling/logit_processor.hpp:28-112 fixes the order):
//   1. penalties, in place on the logits row, one thread per distinct history id, in the
//      reference's float (+) double -> float arithmetic with every step individually rounded;
//   2. greedy rows: strict-> argmax with lowest-index ties over the row (one HBM pass);
//   3. multinomial rows with an active top-k: the reference keeps a K-element min-heap whose final
//      ARRAY ORDER feeds every later float sum and the draw itself, so the order is reproduced
//      exactly: 15 producer warps stream the row with 16-byte loads, keep only elements above a
//      (stale, hence conservative) copy of the heap minimum, and compact them in index order into
//      a double buffer; warp 0 re-checks them 32 at a time and one lane replays libstdc++'s
//      pop_heap / push_heap on the few hundred that really enter, while the producers filter the
//      next chunk.  Softmax, min-p, top-p and the draw then run over <= K elements in one thread,
//      in the reference's order of operations;
//   4. multinomial rows over the full vocabulary get their penalties here and are finished by
//      sampler_exact_kernel (sampler_exact.cu), which reproduces the reference's index-order and
//      sorted-order float sums exactly.
// HBM-bound: the row is read once.
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "../../include/sampler_b200.h"
#include "sampler_kernels.h"

namespace sampler {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kProducerThreads = kThreads - 32;       // warps 1..15 filter, warp 0 replays the heap
constexpr int kPerThread = 8;                         // elements a producer thread filters per round
constexpr int kChunk = kProducerThreads * kPerThread; // elements per filter round
constexpr int kMaxTopK = 1024;                        // heap capacity in shared memory

struct __align__(8) Cand {
    float v;
    int idx;
};

__device__ __forceinline__ void named_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ __forceinline__ void named_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// expf as "exp in double, rounded once to float": within an ulp of glibc's expf and equal to it
// except where glibc's own result is not the correctly rounded one.
__device__ __forceinline__ float exp_as_float(float x) { return (float)exp((double)x); }

// ---- libstdc++ heap primitives on (value, index) pairs with comp(a, b) = a.v > b.v (min-heap) ----
__device__ void push_heap_from(Cand* h, int hole, int top, Cand value) {
    int parent = (hole - 1) / 2;
    while (hole > top && h[parent].v > value.v) {
        h[hole] = h[parent];
        hole = parent;
        parent = (hole - 1) / 2;
    }
    h[hole] = value;
}

__device__ void adjust_heap(Cand* h, int hole, int len, Cand value) {
    const int top = hole;
    int child = hole;
    while (child < (len - 1) / 2) {
        child = 2 * (child + 1);
        const Cand right = h[child], left = h[child - 1];   // both children in flight together
        const bool take_left = right.v > left.v;
        if (take_left) --child;
        h[hole] = take_left ? left : right;
        hole = child;
    }
    if ((len & 1) == 0 && child == (len - 2) / 2) {
        child = 2 * (child + 1);
        h[hole] = h[child - 1];
        hole = child - 1;
    }
    push_heap_from(h, hole, top, value);
}

__device__ void make_heap(Cand* h, int len) {
    if (len < 2) return;
    for (int parent = (len - 2) / 2;; --parent) {
        adjust_heap(h, parent, len, h[parent]);
        if (parent == 0) return;
    }
}

// pop_heap(first, last) followed by back() = x and push_heap(first, last), as TopKFilter does
// (src/cpp/src/sampling/logit_transformers.hpp:240-246).
__device__ __forceinline__ void replace_min(Cand* h, int k, Cand x) {
    if (k > 1) {
        const Cand last = h[k - 1];
        h[k - 1] = h[0];
        adjust_heap(h, 0, k - 1, last);
    }
    h[k - 1] = x;
    push_heap_from(h, k - 1, 0, x);
}

// replace_min for the replay lane of the top-k path: the same comparisons and moves, written with
// 32-bit shared-memory addresses and paired 8-byte accesses so that one level of the heap costs
// one shared-memory round trip.  The writes of the popped minimum and of x into slot k - 1 that
// libstdc++ performs in between are dead (the slot is not read before it is overwritten).
__device__ __forceinline__ void lds_cand(uint32_t addr, float& v, int& i) {
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=f"(v), "=r"(i) : "r"(addr));
}
__device__ __forceinline__ void sts_cand(uint32_t addr, float v, int i) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(addr), "f"(v), "r"(i) : "memory");
}
__device__ __forceinline__ void replace_min_shared(uint32_t base, int k, float xv, int xi) {
    if (k > 1) {
        const int len = k - 1;
        float lastv;
        int lasti;
        lds_cand(base + 8u * len, lastv, lasti);
        // __adjust_heap(first, 0, len, last)
        int hole = 0, child = 0;
        const int half = (len - 1) / 2;
        while (child < half) {
            child = 2 * (child + 1);
            float rv, lv;
            int ri, li;
            lds_cand(base + 8u * child, rv, ri);
            lds_cand(base + 8u * (child - 1), lv, li);
            const bool take_left = rv > lv;
            if (take_left) --child;
            sts_cand(base + 8u * hole, take_left ? lv : rv, take_left ? li : ri);
            hole = child;
        }
        if ((len & 1) == 0 && child == (len - 2) / 2) {
            child = 2 * (child + 1);
            float v;
            int i;
            lds_cand(base + 8u * (child - 1), v, i);
            sts_cand(base + 8u * hole, v, i);
            hole = child - 1;
        }
        // __push_heap(first, hole, 0, last)
        while (hole > 0) {
            const int parent = (hole - 1) / 2;
            float pv;
            int pi;
            lds_cand(base + 8u * parent, pv, pi);
            if (!(pv > lastv)) break;
            sts_cand(base + 8u * hole, pv, pi);
            hole = parent;
        }
        sts_cand(base + 8u * hole, lastv, lasti);
    }
    // push_heap(first, first + k) with x in the last slot
    int hole = k - 1;
    while (hole > 0) {
        const int parent = (hole - 1) / 2;
        float pv;
        int pi;
        lds_cand(base + 8u * parent, pv, pi);
        if (!(pv > xv)) break;
        sts_cand(base + 8u * hole, pv, pi);
        hole = parent;
    }
    sts_cand(base + 8u * hole, xv, xi);
}

// ---- libstdc++ partial_sort / sort on (value, index) pairs with comp(a, b) = a.v > b.v --------------
// TopPFilter sorts candidates with std::partial_sort and std::sort; neither is stable, so to scan
// equal probabilities in the reference's order the algorithms themselves are restated:
// heap-select + sort-heap, and introsort (median-of-three, threshold 16, depth 2*floor(log2 n))
// with the final guarded / unguarded insertion pass.
__device__ __forceinline__ bool desc(const Cand& a, const Cand& b) { return a.v > b.v; }
__device__ __forceinline__ void swap_cand(Cand& a, Cand& b) { const Cand t = a; a = b; b = t; }

__device__ void pop_heap_into(Cand* first, int len, Cand* result) {  // __pop_heap(first, first + len, result)
    const Cand value = *result;
    *result = first[0];
    adjust_heap(first, 0, len, value);
}

__device__ void std_partial_sort(Cand* v, int middle, int n) {
    make_heap(v, middle);
    for (int i = middle; i < n; ++i)
        if (desc(v[i], v[0])) pop_heap_into(v, middle, &v[i]);
    for (int last = middle; last > 1;) {
        --last;
        pop_heap_into(v, last, &v[last]);
    }
}

__device__ void unguarded_linear_insert(Cand* v, int last) {
    const Cand val = v[last];
    int next = last - 1;
    while (desc(val, v[next])) {
        v[last] = v[next];
        last = next;
        --next;
    }
    v[last] = val;
}

__device__ void insertion_sort(Cand* v, int first, int last) {
    if (first == last) return;
    for (int i = first + 1; i != last; ++i) {
        if (desc(v[i], v[first])) {
            const Cand val = v[i];
            for (int j = i; j > first; --j) v[j] = v[j - 1];
            v[first] = val;
        } else {
            unguarded_linear_insert(v, i);
        }
    }
}

__device__ void move_median_to_first(Cand* v, int result, int a, int b, int c) {
    if (desc(v[a], v[b])) {
        if (desc(v[b], v[c])) swap_cand(v[result], v[b]);
        else if (desc(v[a], v[c])) swap_cand(v[result], v[c]);
        else swap_cand(v[result], v[a]);
    } else if (desc(v[a], v[c])) swap_cand(v[result], v[a]);
    else if (desc(v[b], v[c])) swap_cand(v[result], v[c]);
    else swap_cand(v[result], v[b]);
}

__device__ int unguarded_partition(Cand* v, int first, int last, int pivot) {
    for (;;) {
        while (desc(v[first], v[pivot])) ++first;
        --last;
        while (desc(v[pivot], v[last])) --last;
        if (!(first < last)) return first;
        swap_cand(v[first], v[last]);
        ++first;
    }
}

__device__ void std_sort(Cand* v, int n) {
    if (n == 0) return;
    int lg = 0;
    for (int t = n; t > 1; t >>= 1) ++lg;
    // explicit stack instead of the recursive call on [cut, last): the two halves are independent
    int stack_first[48], stack_last[48], stack_depth[48];
    int sp = 0;
    stack_first[sp] = 0; stack_last[sp] = n; stack_depth[sp] = 2 * lg; ++sp;
    while (sp > 0) {
        --sp;
        int first = stack_first[sp], last = stack_last[sp], depth = stack_depth[sp];
        while (last - first > 16) {
            if (depth == 0) {
                std_partial_sort(v + first, last - first, last - first);
                break;
            }
            --depth;
            const int mid = first + (last - first) / 2;
            move_median_to_first(v, first, first + 1, mid, last - 1);
            const int cut = unguarded_partition(v, first + 1, last, first);
            stack_first[sp] = cut; stack_last[sp] = last; stack_depth[sp] = depth; ++sp;
            last = cut;
        }
    }
    if (n > 16) {
        insertion_sort(v, 0, 16);
        for (int i = 16; i < n; ++i) unguarded_linear_insert(v, i);
    } else {
        insertion_sort(v, 0, n);
    }
}

// ---- block reductions -------------------------------------------------------------------------------
template <class T>
__device__ __forceinline__ T shfl_xor_any(T v, int o) {
    static_assert(sizeof(T) % 4 == 0, "word-sized types only");
    union { T t; uint32_t w[sizeof(T) / 4]; } in, out;
    in.t = v;
#pragma unroll
    for (int i = 0; i < (int)(sizeof(T) / 4); ++i) out.w[i] = __shfl_xor_sync(0xffffffffu, in.w[i], o);
    return out.t;
}

template <class T, class Op>
__device__ T block_reduce(T v, T identity, Op op, T* sh) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, shfl_xor_any(v, o));
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sh[w] = v;
    __syncthreads();
    v = lane < kWarps ? sh[lane] : identity;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = op(v, shfl_xor_any(v, o));
    return v;
}

struct ArgMax {
    float v;
    int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // strict '>' with the lowest index among equals; NaN never wins (sampler.cpp:952-961)
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

// Order-preserving 32-bit key of a float: larger float <=> larger unsigned key.
__device__ __forceinline__ uint32_t float_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Calls fn(value, index) once for every element of a row, in no particular order. 16-byte loads,
// four of them in flight per thread: with one 4-byte load per iteration a pass over the row is bound
// by the latency of that load, not by bandwidth.
template <class F>
__device__ __forceinline__ void for_row(const float* row, long long V, int tid, F&& fn) {
    if ((reinterpret_cast<uintptr_t>(row) & 15) != 0) {
        for (long long i = tid; i < V; i += kThreads) fn(row[i], i);
        return;
    }
    const float4* r4 = reinterpret_cast<const float4*>(row);
    const long long n4 = V >> 2;
    long long i = tid;
    for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = r4[i + u * kThreads];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long e = 4 * (i + u * kThreads);
            fn(v[u].x, e); fn(v[u].y, e + 1); fn(v[u].z, e + 2); fn(v[u].w, e + 3);
        }
    }
    for (; i < n4; i += kThreads) {
        const float4 v = r4[i];
        fn(v.x, 4 * i); fn(v.y, 4 * i + 1); fn(v.z, 4 * i + 2); fn(v.w, 4 * i + 3);
    }
    for (long long j = 4 * n4 + tid; j < V; j += kThreads) fn(row[j], j);
}

struct Shared {
    Cand heap[kMaxTopK];
    Cand cand[2][kChunk];          // survivors of two filter rounds
    int cand_count[2];
    float tau;                 // producers' copy of the heap minimum (may lag, never leads)
    int warp_off[kWarps];
    float red_f[kWarps];
    double red_d[kWarps];
    int red_i[kWarps];
    unsigned long long red_u[kWarps];
    ArgMax red_a[kWarps];
};

// ---- phase 1: penalties ---------------------------------------------------------------------------------
__device__ void apply_history(float* row, long long V, const sampler_row_params& p, const int32_t* ids, const uint32_t* meta,
                              long long n, uint32_t* status, float* raw_out) {
    const double rep = (double)p.repetition_penalty, pres = (double)p.presence_penalty, freq = (double)p.frequency_penalty;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        const int id = ids[i];
        const uint32_t m = meta[i];
        if (id < 0 || id >= V) {
            atomicOr(status, 1u);
            continue;
        }
        float v = row[id];
        if (raw_out) raw_out[i] = v;   // the raw logit, for rows that report raw log-probabilities
        if (m & SAMPLER_HIST_STOP_MASK) v = -CUDART_INF_F;
        if (p.repetition_penalty != 1.0f && (m & (SAMPLER_HIST_IN_PROMPT | SAMPLER_HIST_GENERATED)))
            v = v >= 0 ? (float)__ddiv_rn((double)v, rep) : (float)__dmul_rn((double)v, rep);
        if (m & SAMPLER_HIST_GENERATED) {
            if (p.presence_penalty != 0.0f) v = v >= 0 ? (float)__dsub_rn((double)v, pres) : (float)__dadd_rn((double)v, pres);
            if (p.frequency_penalty != 0.0f) {
                const double t = __dmul_rn(freq, (double)(m >> 3));
                v = v >= 0 ? (float)__dsub_rn((double)v, t) : (float)__dadd_rn((double)v, t);
            }
        }
        row[id] = v;
    }
}

// ---- phase 3 tail: softmax / min-p / top-p over the K heap entries, then the draws, one thread -------
// Mirrors TemperatureLogitTransform, MinPFilter, TopPFilter (logit_transformers.hpp:90-362) and
// Sampler::_multinomial_sample (sampler.cpp:979-1095) statement by statement.  The distribution is
// built once; a request with num_return_sequences > 1 draws from it several times (sampler.cpp:1065).
struct TopKDist {
    int n;          // kept candidates, v[0 .. n)
    bool defer;     // expf deferred into the draw (top-k without top-p / min-p): v holds scaled logits
    bool uniform;   // non-finite or empty mass: uniform draws
    float mx, sum;  // deferred form: maximum and float sum of the exponentials
    float total;    // normal form: float sum of the kept probabilities
};

__device__ TopKDist build_top_k_dist(Cand* v, int n, const sampler_row_params& p) {
    TopKDist d{n, false, false, 0.f, 0.f, 0.f};
    const bool min_p_active = p.min_p > 0.0f;
    d.defer = p.top_p == 1.0f && !min_p_active;
    const float T = p.temperature;
    if (d.defer) {
        if (T != 1.0f) {
            const float f = 1.0f / T;
            for (int i = 0; i < n; ++i) v[i].v *= f;
        }
        float mx = v[0].v;
        for (int i = 1; i < n; ++i) if (v[i].v > mx) mx = v[i].v;
        float sum = 0.0f;
        for (int i = 0; i < n; ++i) sum += exp_as_float(v[i].v - mx);
        d.uniform = !(sum > 0.0f && isfinite(sum));
        if (d.uniform) sum = (float)n;
        d.mx = mx; d.sum = sum;
        return d;
    }
    {   // softmax(logits / T) over the heap array, in array order
        float mx = v[0].v;
        for (int i = 1; i < n; ++i) if (v[i].v > mx) mx = v[i].v;
        float sum = 0.0f;
        if (T == 1.0f) {
            for (int i = 0; i < n; ++i) { v[i].v = exp_as_float(v[i].v - mx); sum += v[i].v; }
        } else {
            const float f = 1.0f / T;
            for (int i = 0; i < n; ++i) { v[i].v = exp_as_float((v[i].v - mx) * f); sum += v[i].v; }
        }
        for (int i = 0; i < n; ++i) v[i].v = __fdiv_rn(v[i].v, sum);
    }
    if (min_p_active) {
        float mx = 0.0f;
        int arg = 0;
        for (int i = 0; i < n; ++i) if (v[i].v > mx) { mx = v[i].v; arg = i; }
        const float thr = (float)(double)p.min_p * mx;
        int m = 0;
        for (int i = 0; i < n; ++i) if (v[i].v >= thr) v[m++] = v[i];
        if (m == 0) { v[0] = v[arg]; m = 1; }
        n = m;
    }
    if (p.top_p != 1.0f) {
        // TopPFilter::apply: partial sorts of the top 16, 32, ... 1024 until the running float sum
        // exceeds top_p, else a full sort (logit_transformers.hpp:94-139)
        const double tp = (double)p.top_p;
        bool done = false;
        for (int step = 16; step <= 1024 && !done; step *= 2) {
            if (n <= step) break;
            std_partial_sort(v, step, n);
            float sum = 0.0f;
            for (int i = 0; i < step; ++i) {
                sum += v[i].v;
                if ((double)sum > tp) { n = i + 1; done = true; break; }
            }
        }
        if (!done) {
            std_sort(v, n);
            float sum = 0.0f;
            int keep = 0;
            for (int i = 0; i < n; ++i) {
                sum += v[i].v;
                ++keep;
                if ((double)sum > tp) break;
            }
            n = keep;
        }
    }
    float total = 0.0f;
    for (int i = 0; i < n; ++i) total += v[i].v;
    d.n = n;
    d.total = total;
    d.uniform = !(total > 0.0f && isfinite(total));
    return d;
}

// One draw with the uniform number u: the candidate's vocabulary index and its log-probability.
__device__ void draw_top_k(const Cand* v, const TopKDist& d, float u, float* out_p, long long* out_idx) {
    const int n = d.n;
    if (d.defer) {
        const float log_sum = logf(d.sum) + (d.uniform ? 0.0f : d.mx);
        const float r = d.sum * u;
        float run = 0.0f;
        int pick = n - 1;
        for (int i = 0; i < n; ++i) {
            run += d.uniform ? 1.0f : exp_as_float(v[i].v - d.mx);
            if (run > r) { pick = i; break; }
        }
        *out_p = d.uniform ? logf(1.0f / (float)n) : v[pick].v - log_sum;
        *out_idx = v[pick].idx;
        return;
    }
    if (d.uniform) {
        int pick = (int)(u * (float)n);
        if (pick > n - 1) pick = n - 1;
        *out_p = logf(1.0f / (float)n);
        *out_idx = v[pick].idx;
        return;
    }
    const float log_total = logf(d.total);
    const float r = d.total * u;
    float run = 0.0f;
    int pick = n - 1;
    for (int i = 0; i < n; ++i) {
        run += v[i].v;
        if (run > r) { pick = i; break; }
    }
    *out_p = logf(v[pick].v) - log_total;
    *out_idx = v[pick].idx;
}

__global__ void __launch_bounds__(kThreads, 2) sampler_kernel(StepArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Shared& sh = *reinterpret_cast<Shared*>(smem_raw);
    const int r = blockIdx.x;
    const sampler_row_params p = a.rows[r];
    const long long V = a.vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (p.logits_row < 0 || p.logits_row >= a.num_logit_rows) {
        if (tid == 0) { atomicOr(a.status, 2u); a.out_token[r] = -1; a.out_log_prob[r] = 0.f; }
        return;
    }
    float* row = a.logits + p.logits_row * V;

    const bool multinomial = (p.do_sample & SAMPLER_ROW_MULTINOMIAL) != 0;
    const bool raw_lp = (p.do_sample & SAMPLER_ROW_RAW_LOG_PROB) != 0;
    const long long h0 = a.hist_offsets ? a.hist_offsets[r] : 0, h1 = a.hist_offsets ? a.hist_offsets[r + 1] : 0;

    // ---- 0. log-partition of the raw row (FullVocabLogSumExpTransform, logit_transformers.hpp:264-277) ----
    // The reference adds the exponentials in single precision in index order; here they are added in
    // double precision in parallel and rounded once, which is within an ulp or two of any float order.
    float raw_lse = 0.f;
    bool raw_ok = true;
    if (raw_lp) {
        float mx0 = -CUDART_INF_F;
        for_row(row, V, tid, [&](float x, long long) { mx0 = fmaxf(mx0, x); });
        mx0 = block_reduce(mx0, -CUDART_INF_F, [](float x, float y) { return fmaxf(x, y); }, sh.red_f);
        double s0 = 0.0;
        for_row(row, V, tid, [&](float x, long long) { s0 += (double)expf(x - mx0); });
        s0 = block_reduce(s0, 0.0, [](double x, double y) { return x + y; }, sh.red_d);
        raw_lse = logf((float)s0) + mx0;
        if (h1 > h0 && !a.hist_raw) {
            raw_ok = false;
            if (tid == 0) atomicOr(a.status, 4u);
        }
    }
    // the raw log-probability of the selected token: its logit before the penalties minus the log-partition
    auto raw_log_prob = [&](long long idx) {
        if (!raw_ok) return CUDART_NAN_F;
        float raw = row[idx];
        for (long long i = h0; i < h1; ++i)
            if (a.hist_ids[i] == idx) { raw = a.hist_raw[i]; break; }
        return raw - raw_lse;
    };

    // ---- grammar bitmask (logit_processor.hpp:52-57: after the stop-token mask, before the penalties; both only
    //      write -inf, so their order does not show) ------------------------------------------------
    if (a.bitmask_index) {
        const int mi = a.bitmask_index[r];
        if (mi >= 0) {
            const uint32_t* mask = reinterpret_cast<const uint32_t*>(a.token_bitmasks) + (long long)mi * a.bitmask_words;
            for (long long w = tid; w < a.bitmask_words; w += kThreads) {
                uint32_t denied = ~mask[w];
                if (w == a.bitmask_words - 1 && (V & 31)) denied &= (1u << (V & 31)) - 1u;   // bits beyond the vocabulary
                while (denied) {
                    const int b = __ffs(denied) - 1;
                    denied &= denied - 1;
                    row[32 * w + b] = -CUDART_INF_F;
                }
            }
            __syncthreads();
        }
    }

    // ---- 1. penalties ------------------------------------------------------------------------------
    if (h1 > h0) apply_history(row, V, p, a.hist_ids + h0, a.hist_meta + h0, h1 - h0, a.status, raw_lp && raw_ok ? a.hist_raw + h0 : nullptr);
    __syncthreads();

    // ---- 2. greedy ----------------------------------------------------------------------------------
    if (!multinomial) {
        ArgMax best{-CUDART_INF_F, 0x7fffffff};
        long long done = 0;
        if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
            // 16-byte loads, four in flight per thread; indices ascend per thread so the first maximum is kept
            const float4* row4 = reinterpret_cast<const float4*>(row);
            const long long n4 = V >> 2;
            long long i = tid;
            for (; i + 3 * kThreads < n4; i += 4 * kThreads) {
                float4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) q[u] = __ldcs(row4 + i + u * kThreads);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int b = (int)((i + u * kThreads) << 2);
                    if (q[u].x > best.v) { best.v = q[u].x; best.i = b; }
                    if (q[u].y > best.v) { best.v = q[u].y; best.i = b + 1; }
                    if (q[u].z > best.v) { best.v = q[u].z; best.i = b + 2; }
                    if (q[u].w > best.v) { best.v = q[u].w; best.i = b + 3; }
                }
            }
            for (; i < n4; i += kThreads) {
                const float4 q = __ldcs(row4 + i);
                const int b = (int)(i << 2);
                if (q.x > best.v) { best.v = q.x; best.i = b; }
                if (q.y > best.v) { best.v = q.y; best.i = b + 1; }
                if (q.z > best.v) { best.v = q.z; best.i = b + 2; }
                if (q.w > best.v) { best.v = q.w; best.i = b + 3; }
            }
            done = V;
        }
        for (long long i = done + tid; i < V; i += kThreads) {
            const float x = row[i];
            if (x > best.v) { best.v = x; best.i = (int)i; }
        }
        best = block_reduce(best, ArgMax{-CUDART_INF_F, 0x7fffffff}, better, sh.red_a);
        if (tid == 0) {
            const int chosen = best.i == 0x7fffffff ? 0 : best.i;  // all -inf / NaN: the reference returns index 0
            a.out_token[r] = chosen;
            a.out_log_prob[r] = raw_lp ? raw_log_prob(chosen) : 0.f;   // sampler.cpp:965-974
        }
        return;
    }

    const bool top_k_active = p.top_k > 0 && p.top_k < 0x7fffffffffffffffLL;
    if (top_k_active && p.top_k < V && p.top_k <= kMaxTopK) {
        // ---- 3. exact top-k heap replay --------------------------------------------------------------
        const int K = (int)p.top_k;
        // the producers start at the first 16-byte boundary at or after K; warp 0 feeds the (at
        // most 3) elements in between to the heap itself
        const bool vec_ok = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        const long long start = vec_ok ? min(V, ((long long)K + 3) & ~3LL) : K;
        if (warp == 0) {
            for (int i = lane; i < K; i += 32) sh.heap[i] = Cand{row[i], i};
            __syncwarp();
            if (lane == 0) {
                make_heap(sh.heap, K);
                for (long long i = K; i < start; ++i) {
                    const float x = row[i];
                    if (x > sh.heap[0].v) replace_min(sh.heap, K, Cand{x, (int)i});
                }
                sh.tau = sh.heap[0].v;
            }
        }
        __syncthreads();
        const long long n_rest = V - start;
        const int rounds = (int)((n_rest + kChunk - 1) / kChunk);
        if (warp == 0) {
            // consumer: re-checks the survivors of round c, 32 at a time, while the producers filter
            // round c + 1; lane 0 owns the heap
            float heap_min = sh.heap[0].v;
            const uint32_t heap_addr = (uint32_t)__cvta_generic_to_shared(sh.heap);
            for (int c = 0; c < rounds; ++c) {
                const int b = c & 1;
                named_sync(1 + b, kThreads);           // full[b]
                const int n = sh.cand_count[b];
                for (int base = 0; base < n; base += 32) {
                    const int i = base + lane;
                    Cand x = i < n ? sh.cand[b][i] : Cand{-CUDART_INF_F, 0};
                    unsigned mask = __ballot_sync(0xffffffffu, i < n && x.v > heap_min);
                    while (mask) {
                        const int src = __ffs(mask) - 1;
                        mask &= mask - 1;
                        const float xv = __shfl_sync(0xffffffffu, x.v, src);
                        const int xi = __shfl_sync(0xffffffffu, x.idx, src);
                        if (xv > heap_min) {           // the minimum may have risen since the ballot
                            if (lane == 0) replace_min_shared(heap_addr, K, xv, xi);
                            __syncwarp();
                            heap_min = sh.heap[0].v;
                            // the minimum rose: drop the survivors it has overtaken in one vote
                            mask &= __ballot_sync(0xffffffffu, i < n && x.v > heap_min);
                        }
                    }
                }
                if (lane == 0) *reinterpret_cast<volatile float*>(&sh.tau) = heap_min;
                __syncwarp();
                __threadfence_block();
                if (c == 0 && rounds > 1) named_arrive(7, kThreads);   // round 1 is filtered with the minimum reached after round 0
                named_arrive(3 + b, kThreads);         // empty[b]
            }
        } else {
            const int ptid = tid - 32, pwarp = warp - 1;
            float x[kPerThread], xn[kPerThread];
            auto load_round = [&](int c, float (&dst)[kPerThread]) {
                const long long base = start + (long long)c * kChunk + (long long)ptid * kPerThread;
                if (vec_ok && base + kPerThread <= V) {
                    const float4 q0 = __ldcs(reinterpret_cast<const float4*>(row + base));
                    const float4 q1 = __ldcs(reinterpret_cast<const float4*>(row + base + 4));
                    dst[0] = q0.x; dst[1] = q0.y; dst[2] = q0.z; dst[3] = q0.w;
                    dst[4] = q1.x; dst[5] = q1.y; dst[6] = q1.z; dst[7] = q1.w;
                } else {
#pragma unroll
                    for (int e = 0; e < kPerThread; ++e) dst[e] = base + e < V ? row[base + e] : CUDART_NAN_F;  // NaN never passes '>'
                }
            };
            load_round(0, x);
            for (int c = 0; c < rounds; ++c) {
                const int b = c & 1;
                if (c + 1 < rounds) load_round(c + 1, xn);  // in flight while this round is compacted
                if (c >= 2) named_sync(3 + b, kThreads);    // wait until the consumer drained buffer b
                // The first elements raise the heap minimum quickly; filtering round 1 with the stale
                // minimum of the first K elements would let nearly all of it through.
                if (c == 1) named_sync(7, kThreads);
                const float tau = *reinterpret_cast<volatile float*>(&sh.tau);
                const long long base = start + (long long)c * kChunk + (long long)ptid * kPerThread;
                int mine = 0;
#pragma unroll
                for (int e = 0; e < kPerThread; ++e) mine += x[e] > tau ? 1 : 0;
                // ordered compaction: exclusive prefix of `mine` over the producer threads
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int u = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += u;
                }
                if (lane == 31) sh.warp_off[pwarp] = incl;
                named_sync(5, kProducerThreads);
                int off = 0;
                for (int w = 0; w < pwarp; ++w) off += sh.warp_off[w];
                if (ptid == kProducerThreads - 1) sh.cand_count[b] = off + incl;
                int pos = off + incl - mine;
#pragma unroll
                for (int e = 0; e < kPerThread; ++e)
                    if (x[e] > tau) sh.cand[b][pos++] = Cand{x[e], (int)(base + e)};
                named_sync(6, kProducerThreads);       // warp_off is reused next round
                __threadfence_block();
                named_arrive(1 + b, kThreads);         // full[b]
#pragma unroll
                for (int e = 0; e < kPerThread; ++e) x[e] = xn[e];
            }
        }
        __syncthreads();
        if (tid == 0) {
            const TopKDist dist = build_top_k_dist(sh.heap, K, p);
            const long long x0 = a.extra_offsets ? a.extra_offsets[r] : 0, x1 = a.extra_offsets ? a.extra_offsets[r + 1] : 0;
            for (long long k = -1; k < x1 - x0; ++k) {   // the row's own draw, then the further ones
                float lp;
                long long idx;
                draw_top_k(sh.heap, dist, k < 0 ? p.rand_u : a.extra_rand_u[x0 + k], &lp, &idx);
                if (raw_lp && !dist.uniform) lp = raw_log_prob(idx);   // sampler.cpp:1022-1029, 1076-1081
                if (k < 0) { a.out_token[r] = idx; a.out_log_prob[r] = lp; }
                else { a.extra_out_token[x0 + k] = idx; a.extra_out_log_prob[x0 + k] = lp; }
            }
        }
        return;
    }

    // ---- 4. full vocabulary ---------------------------------------------------------------------------
    if (top_k_active && p.top_k < V) {
        // a heap larger than the shared-memory capacity: not supported, and said so (status bit 3, token -1)
        if (tid == 0) {
            atomicOr(a.status, 8u); a.out_token[r] = -1; a.out_log_prob[r] = 0.f;
            if (a.extra_offsets)
                for (long long k = a.extra_offsets[r]; k < a.extra_offsets[r + 1]; ++k) { a.extra_out_token[k] = -1; a.extra_out_log_prob[k] = 0.f; }
        }
        return;
    }
    // The row is finished by sampler_exact_kernel (sampler_exact.cu), launched right after this one: it
    // needs the penalised row, which is in place now, and for raw log-probabilities the log-partition
    // of the raw row, parked in the row's output slot (NaN: no scratch for the raw logits).
    if (tid == 0) a.out_log_prob[r] = raw_lp ? (raw_ok ? raw_lse : CUDART_NAN_F) : 0.f;
}

}  // namespace

size_t sampler_smem_bytes() { return sizeof(Shared); }

cudaError_t launch_sampler(const StepArgs& a, cudaStream_t stream) {
    if (a.num_rows <= 0) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(sampler_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Shared));
    if (e != cudaSuccess) return e;
    sampler_kernel<<<a.num_rows, kThreads, sizeof(Shared), stream>>>(a);
    return cudaGetLastError();
}

}  // namespace sampler
