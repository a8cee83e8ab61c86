// Exact emulation of two pieces of host arithmetic the reference Sampler relies on, in a form that
// can run in parallel:
//
//  1. glibc's single-precision expf as x86-64 machines with FMA run it (the result every
//     TemperatureLogitTransform element goes through, src/cpp/src/sampling/logit_transformers.hpp:327-356).
//     The published algorithm: k = round(x * 32 / ln 2), r = x * 32 / ln 2 - k taken with one fused
//     multiply-add, exp(x) = 2^(k / 32) * (1 + r * C2 + r^2 * (C1 + r * C0)) in double precision with a
//     32-entry table of 2^(i / 32), rounded once to float.  The restatement below returns the same
//     bits as that libm for every finite input in [-103.9, 88.7] (checked exhaustively on the host by
//     tests/cpp/fsum_exact_test.cpp over a stride of the range and by the GPU test on the device).
//
//  2. A running float sum `s += x[i]` over non-negative terms in a fixed order
//     (logit_transformers.hpp:343-359, 105-125; sampling/sampler.cpp:1036-1074).  While s stays inside
//     one binade its ulp u is constant and fl(s + x) = s + u * round_half_even(x / u) is an integer
//     addition on S = s / u whose amount depends on S only through its parity (a tie x / u = q + 1/2
//     rounds to the even neighbour).  A term therefore acts as a two-state function
//         S -> S + a   (S even),   S -> S + b   (S odd),
//     and such functions compose associatively, so a block scan reproduces the sequential sum bit
//     for bit.  For a term that is not a tie a == b: those are plain translations and commute, which
//     is what lets a sum over sorted probabilities be taken from histograms.  A step that leaves the
//     binade (S reaches 2^24) is redone with one real float addition.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define FSX_HD __host__ __device__ __forceinline__
#else
#define FSX_HD inline
#include <cmath>
#endif

namespace fsx {

// ---- expf -------------------------------------------------------------------------------------
// 2^(i / 32), i = 0..31, correctly rounded to double, with i << 47 subtracted from the bit pattern so
// that adding k << 47 puts floor(k / 32) into the exponent field.
#define FSX_EXP2_TABLE                                                                                  \
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,         \
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,         \
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,         \
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,         \
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,         \
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,         \
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,         \
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
static const uint64_t kExp2TabHost[32] = {FSX_EXP2_TABLE};
#if defined(__CUDACC__)
// Device copy.  Lanes of a warp index it with different values: kernels copy it to shared memory first
// (a constant-bank read with divergent addresses is replayed once per address).
static __device__ const uint64_t kExp2TabDev[32] = {FSX_EXP2_TABLE};
#endif

FSX_HD double u64_as_double(uint64_t u) {
#if defined(__CUDA_ARCH__)
    return __longlong_as_double((long long)u);
#else
    double d; memcpy(&d, &u, 8); return d;
#endif
}
FSX_HD uint64_t double_as_u64(double d) {
#if defined(__CUDA_ARCH__)
    return (uint64_t)__double_as_longlong(d);
#else
    uint64_t u; memcpy(&u, &d, 8); return u;
#endif
}
FSX_HD uint32_t float_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
FSX_HD float bits_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
FSX_HD double fma_rn(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
    return __fma_rn(a, b, c);
#else
    return std::fma(a, b, c);
#endif
}
FSX_HD double mul_rn(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dmul_rn(a, b);
#else
    return a * b;   // build with -ffp-contract=off
#endif
}
FSX_HD double add_rn(double a, double b) {
#if defined(__CUDA_ARCH__)
    return __dadd_rn(a, b);
#else
    return a + b;
#endif
}
FSX_HD float fadd_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}

// expf(x) with the host libm's bits.  Inputs at or below -103.972 give 0, -inf gives 0, NaN stays NaN;
// arguments above 88.7 do not occur here (the callers pass x - max <= 0) and saturate to +inf.
FSX_HD float expf_libm(float x, const uint64_t* tab) {
    if (!(x >= -103.972076f)) return x != x ? x : 0.0f;       // underflow to zero (and NaN passthrough)
    if (x > 88.72283f) return bits_float(0x7f800000u);
    const double kInvLn2N = 0x1.71547652b82fep+0 * 32.0;
    const double kShift = 0x1.8p+52;
    const double kC0 = 0x1.c6af84b912394p-5 / 32768.0, kC1 = 0x1.ebfce50fac4f3p-3 / 1024.0, kC2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double xd = (double)x;
    double kd = fma_rn(kInvLn2N, xd, kShift);
    const uint64_t ki = double_as_u64(kd);
    kd = add_rn(kd, -kShift);
    const double r = fma_rn(kInvLn2N, xd, -kd);
    const double s = u64_as_double(tab[ki & 31] + (ki << 47));
    const double z = fma_rn(kC0, r, kC1);
    const double r2 = mul_rn(r, r);
    double y = fma_rn(kC2, r, 1.0);
    y = fma_rn(z, r2, y);
    y = mul_rn(y, s);
    return (float)y;
}

#if !defined(__CUDA_ARCH__)
inline float expf_libm(float x) { return expf_libm(x, kExp2TabHost); }
#endif

// a / b correctly rounded (what the host's `/=` gives, logit_transformers.hpp:357-359) for a whole row
// that shares the divisor: with y = RN(1 / b), q0 = RN(a y), the remainder a - b q0 is exact in one fused
// multiply-add and RN(q0 + rem y) is the rounded quotient.  Small numerators, whose remainder would
// be a denormal, take the plain division.
FSX_HD float div_shared(float a, float b, float y) {
    if (!(a >= 0x1p-90f)) {
#if defined(__CUDA_ARCH__)
        return __fdiv_rn(a, b);
#else
        return a / b;
#endif
    }
#if defined(__CUDA_ARCH__)
    const float q0 = __fmul_rn(a, y);
    const float rem = __fmaf_rn(-q0, b, a);
    return __fmaf_rn(rem, y, q0);
#else
    const float q0 = a * y;
    const float rem = std::fma(-q0, b, a);
    return std::fma(rem, y, q0);
#endif
}

// ---- running float sums -------------------------------------------------------------------------
constexpr uint32_t kOne24 = 1u << 24;
constexpr uint32_t kSat = 1u << 26;   // amounts saturate here: any state that meets one has left its binade

// A float s >= 0 as (E, S): s = S * 2^(E - 150) with E the biased exponent (1 for zero and denormals,
// where S < 2^23) and S the significand with its hidden bit.
FSX_HD uint32_t state_exp(float s) { const uint32_t e = float_bits(s) >> 23; return e ? e : 1u; }
FSX_HD uint32_t state_sig(float s) {
    const uint32_t b = float_bits(s);
    return (b >> 23) ? ((b & 0x7fffffu) | 0x800000u) : b;
}
FSX_HD float state_float(uint32_t E, uint32_t S) {   // S < 2^24; S < 2^23 only when E == 1
    return bits_float(S >= 0x800000u ? ((E << 23) | (S & 0x7fffffu)) : S);
}

struct Step {
    uint32_t a, b;   // amount added to an even / odd state
};
FSX_HD Step step_identity() { return Step{0u, 0u}; }
FSX_HD uint32_t sat_add(uint32_t x, uint32_t y) { const uint32_t z = x + y; return z > kSat ? kSat : z; }

// The step of adding x (finite, >= 0) to a sum whose biased exponent is E.  `tie` is set when the
// amount depends on the parity of the sum.
FSX_HD Step step_of(float x, uint32_t E, bool* tie) {
    const uint32_t bx = float_bits(x);
    uint32_t ex = bx >> 23, m = bx & 0x7fffffu;
    if (ex) m |= 0x800000u; else ex = 1u;
    *tie = false;
    const int d = (int)E - (int)ex;
    if (d <= 0) {
        const uint32_t k = d < -2 ? kSat : (m << (-d));
        const uint32_t c = k > kSat ? kSat : k;
        return Step{c, c};
    }
    if (d >= 25) return Step{0u, 0u};
    const uint32_t q = m >> d, rem = m & ((1u << d) - 1u), half = 1u << (d - 1);
    if (rem == half) {
        *tie = true;
        return Step{q + (q & 1u), q + 1u - (q & 1u)};
    }
    const uint32_t c = q + (rem > half ? 1u : 0u);
    return Step{c, c};
}
FSX_HD Step step_of(float x, uint32_t E) { bool t; return step_of(x, E, &t); }

// The amount of a term that is not a tie, in five float operations, for the passes that add whole spans
// or bins.  scale = 2^(150 - E) turns x into units of the sum's ulp exactly (a power of two); rintf
// rounds to nearest, and the distance to the rounded value tells a tie (exactly one half).  `defer` is
// set for a tie and for a term of 2^24 ulps or more, which the callers add element by element.
FSX_HD float amount_scale(uint32_t E) {   // 0 where the scale is not a normal float: such sums go element by element
    return (E >= 24u && E <= 254u) ? bits_float((277u - E) << 23) : 0.0f;
}
FSX_HD uint32_t plain_amount(float x, float scale, bool* defer) {
    const float t = x * scale;
#if defined(__CUDA_ARCH__)
    const float r = rintf(t);
    *defer = fabsf(t - r) == 0.5f || !(t < 16777216.0f);
    return __float2uint_rz(r);
#else
    const float r = std::nearbyint(t);   // round half to even in the default rounding mode
    *defer = std::fabs(t - r) == 0.5f || !(t < 16777216.0f);
    return t < 4294967040.0f ? (uint32_t)r : 0xffffffffu;
#endif
}

// g after f
FSX_HD Step then(Step f, Step g) {
    return Step{sat_add(f.a, (f.a & 1u) ? g.b : g.a), sat_add(f.b, ((f.b + 1u) & 1u) ? g.b : g.a)};
}
FSX_HD uint32_t apply(Step f, uint32_t S) { return S + ((S & 1u) ? f.b : f.a); }


// ---- sums over probabilities sorted in descending order --------------------------------------------
// TopPFilter adds the sorted probabilities one by one until the running float sum exceeds top_p
// (logit_transformers.hpp:105-125) and the draw walks the same running sums (sampler.cpp:1065-1074).
// Keys are the bit patterns of the probabilities (non-negative floats: larger key <=> larger value).
// A level cuts the keys below `F` into kBins bins of 2^sh consecutive keys, highest keys first; what
// lies below the last bin is the level's rest.  A bin whose elements cannot meet a tie, a change of
// binade, the threshold or the element limit is added as one translation: the sum of its elements'
// amounts under the hypothesised exponent E[j] of the running sum, which does not depend on their
// order.  Every other bin is listed element by element, sorted, and added with real float additions.
// Hypotheses come from approximate masses and are checked by the walk itself: a bin whose hypothesis
// does not hold is never taken as a whole, so a wrong guess costs another pass, not a wrong sum.

constexpr int kBins = 2048;
constexpr int kTopSh = 16;          // first level: 128 bins per binade of the probabilities, 16 binades
constexpr int kSubBits = 11;        // a bin that has to be cut further becomes a level of its own

enum : uint8_t {
    kBinListed = 1,    // the bin's elements are in the list
    kBinTie = 2,       // an element of the bin is a tie under E[j]
    kBinValid = 4,     // A[j] holds the sum of amounts under E[j]
    kBinDirty = 8,     // A[j] is to be accumulated by the next pass
    kBinCollect = 16,  // the next pass appends the bin's elements to the list
    kBinStep = 32,     // listed bin: A[j] holds the composition of its elements' steps under E[j], in list order (pack_step)
};

struct Level {
    uint32_t F;   // keys < F belong to this level
    int sh;
};
FSX_HD uint32_t bin_of(Level L, uint32_t key) {   // key < L.F; kBins and above = the level's rest
    return (L.F - 1u - key) >> L.sh;
}

struct Bins {
    uint32_t* A;      // [kBins] sum of amounts (valid bins)
    uint32_t* C;      // [kBins] element counts
    float* R;         // [kBins] approximate masses, for the hypotheses only
    uint32_t* PA;     // [kBins] sum of A over the plain bins from the last stop up to and including j (saturating)
    uint32_t* PC;     // [kBins] the same for C
    uint16_t* next;   // [kBins + 1] next[j] = first stop bin at or after j (kBins if none)
    uint8_t* E;       // [kBins] hypothesised exponent
    uint8_t* flag;    // [kBins]
};

// A step whose even-state amount is below 2^24 and whose two amounts differ by less than 128, in one word.
FSX_HD bool step_packs(Step st) {
    const long long d = (long long)st.b - (long long)st.a;
    return st.a < kOne24 && st.b < kSat && d >= -128 && d <= 127;
}
FSX_HD uint32_t pack_step(Step st) { return st.a | ((uint32_t)(uint8_t)(int8_t)((int)st.b - (int)st.a) << 24); }
FSX_HD Step unpack_step(uint32_t w) {
    const uint32_t a = w & 0xffffffu;
    return Step{a, (uint32_t)((int)a + (int)(int8_t)(uint8_t)(w >> 24))};
}

// plain: non-empty, summed as a whole
FSX_HD bool bin_plain(const Bins& b, int j) {
    return b.C[j] != 0 && (b.flag[j] & (kBinListed | kBinTie | kBinValid)) == kBinValid;
}
// A stop is a non-empty bin at which the walk has to look: listed, unresolved, or the first bin of a
// run of plain bins (after a bin that is not plain, or where the hypothesis changes).
// prev_plain_E: E of the nearest non-empty bin before j if that bin is plain, else -1.
FSX_HD bool bin_is_stop(const Bins& b, int j, int prev_plain_E) {
    if (b.C[j] == 0) return false;
    if (!bin_plain(b, j)) return true;
    return (int)b.E[j] != prev_plain_E;
}

struct Walk {
    float s;          // running sum so far
    uint32_t cnt;     // elements added so far
    int j;            // next bin
    int li;           // next list entry
    int status;       // kWalk*
    uint32_t hit_key; // found: the element at which the sum exceeded the threshold or the limit was reached
    uint32_t hit_idx;
    bool by_limit;    // found by the element limit, not by the threshold
};
enum { kWalkFound = 0, kWalkUnresolved = 1, kWalkEnd = 2 };

FSX_HD uint32_t entry_key(uint64_t e) { return (uint32_t)(e >> 32); }
FSX_HD uint32_t entry_idx(uint64_t e) { return 0xffffffffu - (uint32_t)e; }
FSX_HD uint64_t make_entry(uint32_t key, uint32_t idx) { return ((uint64_t)key << 32) | (0xffffffffu - idx); }

// Where a walk stood when it came to a bin: the exact sum and count of everything before the bin, and its place in the list.
// A later walk of the same row with a lower threshold may start from the last such record that is still below its threshold
// instead of from the top (the sums are the same additions in the same order).
// One record per group of kCkGroup bins (the last bin of the group the walk came to).
constexpr int kCkGroup = 4;
struct Checkpoints {
    float* s;
    uint32_t* cnt;
    uint16_t* j;
    uint16_t* li;
};

// Continues the walk from (w.s, w.cnt, w.j, w.li) until the running sum exceeds `thr`, `limit`
// elements have been added (limit 0: no limit), a bin cannot be taken, or the level ends.
// `list` is sorted in descending order (key, then ascending index).  One thread runs this.
FSX_HD void walk_level(Walk& w, Level L, const Bins& b, const uint64_t* list, int list_n, float thr, uint32_t limit, const Checkpoints* ck = nullptr) {
    for (;;) {
        if (w.j >= kBins) { w.status = kWalkEnd; return; }
        const int j = w.j;
        if (ck) { const int g = j / kCkGroup; ck->s[g] = w.s; ck->cnt[g] = w.cnt; ck->j[g] = (uint16_t)j; ck->li[g] = (uint16_t)w.li; }
        if (b.C[j] == 0) { w.j = (int)b.next[j]; continue; }     // only empty bins up to the next stop
        const uint8_t f = b.flag[j];
        if (f & kBinListed) {
            if ((f & kBinStep) && w.s != 0.0f && (uint32_t)b.E[j] == state_exp(w.s)) {
                // The bin's elements as one step: while the sum stays in the binade of the hypothesis (it only grows, so the end
                // tells), below the threshold and short of the element limit, the composition of the elements' two-state steps
                // in list order is what adding them one by one gives.
                const uint32_t E = state_exp(w.s), S = state_sig(w.s);
                const Step st = unpack_step(b.A[j]);
                const uint32_t S2 = apply(st, S), n = b.C[j];
                if (S2 < kOne24 && !(state_float(E, S2) > thr) && !(limit && w.cnt + n >= limit)) {
                    while (w.li < list_n) {   // entries added earlier
                        const uint32_t key = entry_key(list[w.li]);
                        if (key >= L.F || bin_of(L, key) < (uint32_t)j) ++w.li; else break;
                    }
                    w.li += (int)n;
                    w.s = state_float(E, S2);
                    w.cnt += n;
                    ++w.j;
                    continue;
                }
            }
            while (w.li < list_n) {   // entries of this bin, one real addition each
                const uint64_t e = list[w.li];
                const uint32_t key = entry_key(e);
                const uint32_t bj = key < L.F ? bin_of(L, key) : 0u;
                if (key >= L.F || bj < (uint32_t)j) { ++w.li; continue; }   // added earlier
                if (bj != (uint32_t)j) break;
                w.s = fadd_rn(w.s, bits_float(key));
                ++w.cnt;
                ++w.li;
                const bool over = w.s > thr;
                if (over || (limit && w.cnt >= limit)) {
                    w.status = kWalkFound; w.hit_key = key; w.hit_idx = entry_idx(e); w.by_limit = !over;
                    return;
                }
            }
            ++w.j;
            continue;
        }
        if ((f & kBinTie) || !(f & kBinValid)) { w.status = kWalkUnresolved; return; }
        // a run of plain (and empty) bins: from the stop j up to the next stop
        const uint32_t E = state_exp(w.s), S = state_sig(w.s);
        if (w.s == 0.0f || (uint32_t)b.E[j] != E || (int)b.next[j] != j) { w.status = kWalkUnresolved; return; }
        const int k = (int)b.next[j + 1];
        int lo = j, hi = k;      // bins j .. lo - 1 can be taken as a whole
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            const uint32_t add = b.PA[mid - 1], n = b.PC[mid - 1];
            const bool ok = add < kOne24 && S + add < kOne24 && !(state_float(E, S + add) > thr) && !(limit && w.cnt + n >= limit);
            if (ok) lo = mid; else hi = mid - 1;
        }
        if (lo > j) {
            w.s = state_float(E, S + b.PA[lo - 1]);
            w.cnt += b.PC[lo - 1];
        }
        w.j = lo;
        if (lo < k) { w.status = kWalkUnresolved; return; }
    }
}

// The exponent hypothesised for a float sum whose real-valued counterpart runs from lo to hi, and
// whether the range widened by the relative margin stays inside one binade.
FSX_HD bool hyp_exponent(double lo, double hi, double margin, uint32_t* E) {
    const float flo = (float)(lo * (1.0 - margin)), fhi = (float)(hi * (1.0 + margin));
    *E = state_exp(flo);
    return lo > 0.0 && state_exp(flo) == state_exp(fhi);
}

// Adds `c` copies of x to the sum s (real additions where the binade changes, powers of the step
// otherwise) until the sum exceeds thr or `limit` elements have been added.  Returns the number of
// copies added; *found tells whether it stopped for the threshold or the limit.
FSX_HD uint32_t add_repeated(float& s, uint32_t& cnt, float x, uint32_t c, float thr, uint32_t limit, bool* found, bool* by_limit) {
    uint32_t done = 0;
    *found = false;
    while (done < c) {
        const uint32_t E = state_exp(s);
        uint32_t S = state_sig(s);
        if (s != 0.0f) {
            Step pw[32];
            pw[0] = step_of(x, E);
            int top = 0;
            while ((1u << (top + 1)) <= c - done && top < 30) { pw[top + 1] = then(pw[top], pw[top]); ++top; }
            uint32_t n = 0;
            for (int k = top; k >= 0; --k) {
                const uint32_t m = 1u << k;
                if (n + m > c - done) continue;
                const uint32_t S2 = apply(pw[k], S);
                if (S2 >= kOne24 || state_float(E, S2) > thr || (limit && cnt + n + m >= limit)) continue;
                S = S2; n += m;
            }
            s = state_float(E, S);
            cnt += n; done += n;
            if (done == c) break;
        }
        s = fadd_rn(s, x);   // the copy that changes the binade, meets the threshold or the limit
        ++cnt; ++done;
        const bool over = s > thr;
        if (over || (limit && cnt >= limit)) { *found = true; *by_limit = !over; return done; }
    }
    return done;
}

}  // namespace fsx
