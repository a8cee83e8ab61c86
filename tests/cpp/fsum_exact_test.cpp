// CPU checks of openvino.genai_b200/csrc/fsum_exact.cuh, the arithmetic the exact full-vocabulary
// sampler kernel is built from:
//   1. expf_libm against this machine's libm expf (strided sweep of every binade + random inputs);
//   2. the two-state steps: a scan of composed steps against the plain sequential float sum, with
//      binade changes, ties, denormals and zeros in the data;
//   3. the sorted walk (levels, bins, lists, hypotheses) as the kernel runs it, pass by pass, against
//      std::sort + sequential sums: number of kept elements, kept total and the drawn element.
// Build: g++ -O2 -std=c++17 -ffp-contract=off -I openvino.genai_b200/csrc tests/cpp/fsum_exact_test.cpp
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "fsum_exact.cuh"
#include "topp_model.hpp"

static int g_fail = 0;
#define CHECK(cond, ...)                                  \
    do {                                                  \
        if (!(cond)) {                                    \
            if (++g_fail < 20) { std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } \
        }                                                 \
    } while (0)

static void test_table() {
    for (int i = 0; i < 32; ++i) {
        const long double v = exp2l((long double)i / 32);
        const double d = (double)v;
        uint64_t u;
        std::memcpy(&u, &d, 8);
        CHECK(fsx::kExp2TabHost[i] == u - ((uint64_t)i << 47), "table entry %d", i);
    }
}

static void test_expf(long long stride) {
    long long n = 0;
    for (uint64_t b = 0x80000000u; b <= 0xc2d00000u; b += stride) {   // -0 .. -104
        const float x = fsx::bits_float((uint32_t)b);
        const float want = expf(x), got = fsx::expf_libm(x);
        CHECK(std::memcmp(&want, &got, 4) == 0, "expf(%a): libm %a restated %a", x, want, got);
        ++n;
    }
    for (uint64_t b = 0; b <= 0x42b00000u; b += stride) {             // +0 .. 88
        const float x = fsx::bits_float((uint32_t)b);
        const float want = expf(x), got = fsx::expf_libm(x);
        CHECK(std::memcmp(&want, &got, 4) == 0, "expf(%a): libm %a restated %a", x, want, got);
        ++n;
    }
    const float specials[] = {-INFINITY, -200.0f, -103.98f, -103.97f, -103.9f, -87.4f, -0.0f, 0.0f};
    for (float x : specials) {
        const float want = expf(x), got = fsx::expf_libm(x);
        CHECK(std::memcmp(&want, &got, 4) == 0, "expf(%a): libm %a restated %a", x, want, got);
    }
    std::printf("expf: %lld inputs compared\n", n);
}

// sequential reference and a tiled scan that uses only steps (and one real addition per binade change)
static float seq_sum(const std::vector<float>& x) {
    float s = 0.0f;
    for (float v : x) s += v;
    return s;
}
static float scan_sum(const std::vector<float>& x, size_t tile) {
    float s = 0.0f;
    for (size_t base = 0; base < x.size(); base += tile) {
        const size_t n = std::min(tile, x.size() - base);
        size_t from = 0;
        while (from < n) {
            const uint32_t E = fsx::state_exp(s), S = fsx::state_sig(s);
            // inclusive scan of the steps of elements from..n-1 under E
            std::vector<fsx::Step> pre(n - from);
            fsx::Step acc = fsx::step_identity();
            for (size_t i = from; i < n; ++i) { acc = fsx::then(acc, fsx::step_of(x[base + i], E)); pre[i - from] = acc; }
            size_t cross = n;
            for (size_t i = from; i < n; ++i)
                if (fsx::apply(pre[i - from], S) >= fsx::kOne24) { cross = i; break; }
            if (cross == n) { s = fsx::state_float(E, fsx::apply(pre.back(), S)); break; }
            const float before = cross == from ? s : fsx::state_float(E, fsx::apply(pre[cross - 1 - from], S));
            s = before + x[base + cross];
            from = cross + 1;
        }
    }
    return s;
}

static void test_scan(std::mt19937_64& rng) {
    std::uniform_real_distribution<double> U(0.0, 1.0);
    for (int trial = 0; trial < 400; ++trial) {
        const size_t n = 1 + (size_t)(U(rng) * 5000);
        std::vector<float> x(n);
        const int kind = trial % 8;
        for (auto& v : x) {
            switch (kind) {
                case 0: v = (float)U(rng); break;
                case 1: v = (float)std::exp(-20.0 * U(rng)); break;
                case 2: v = std::ldexp((float)(rng() % 64), -(int)(rng() % 30)); break;   // many ties and zeros
                case 3: v = std::ldexp(1.0f, -(int)(rng() % 40)); break;                    // powers of two
                case 4: v = fsx::bits_float((uint32_t)(rng() % 0x01000000u)); break;        // denormals and tiny normals
                case 5: v = (rng() & 1) ? 0.0f : (float)U(rng) * 1e-3f; break;
                case 6: v = std::ldexp((float)(1 + rng() % 7), (int)(rng() % 20) - 10); break;
                default: v = (float)std::exp(8.0 * U(rng) - 10.0); break;
            }
        }
        const float want = seq_sum(x);
        for (size_t tile : {size_t(1), size_t(7), size_t(64), size_t(2048)}) {
            const float got = scan_sum(x, tile);
            CHECK(std::memcmp(&want, &got, 4) == 0, "scan kind %d n %zu tile %zu: %a vs %a", kind, n, tile, want, got);
        }
    }
}

// plain_amount against step_of, div_shared against the division
static void test_amount_and_division(std::mt19937_64& rng) {
    for (int i = 0; i < 4000000; ++i) {
        const uint32_t E = 24 + (uint32_t)(rng() % 200);
        const int ex = (int)E - (int)(rng() % 40) + 3;
        if (ex < 1 || ex > 254) continue;
        uint32_t m = (uint32_t)(rng() & 0x7fffffu);
        if (i % 3 == 0) m &= ~((1u << (rng() % 23)) - 1u);   // many ties and exact multiples
        const float x = fsx::bits_float(((uint32_t)ex << 23) | m);
        bool tie, defer;
        const fsx::Step st = fsx::step_of(x, E, &tie);
        const uint32_t a = fsx::plain_amount(x, fsx::amount_scale(E), &defer);
        if (st.a >= fsx::kOne24) { CHECK(defer, "amount of %a under E %u: not deferred", x, E); continue; }
        CHECK(defer == tie, "amount of %a under E %u: tie %d defer %d", x, E, (int)tie, (int)defer);
        if (!tie) CHECK(a == st.a, "amount of %a under E %u: %u vs %u", x, E, a, st.a);
    }
    for (int i = 0; i < 4000000; ++i) {
        const float b = fsx::bits_float(0x3e000000u + (uint32_t)(rng() % (12u << 23)));
        const float a = fsx::bits_float((uint32_t)(rng() % 0x40000000u));
        const float got = fsx::div_shared(a, b, 1.0f / b), want = a / b;
        CHECK(std::memcmp(&got, &want, 4) == 0, "%a / %a: %a vs %a", a, b, got, want);
    }
}

// add_repeated against a loop
static void test_repeated(std::mt19937_64& rng) {
    std::uniform_real_distribution<double> U(0.0, 1.0);
    for (int trial = 0; trial < 2000; ++trial) {
        const float x = trial % 3 == 0 ? std::ldexp(1.0f, -(int)(rng() % 24)) : (float)std::exp(-16.0 * U(rng));
        const uint32_t c = 1 + (uint32_t)(rng() % 200000);
        float s0 = trial % 4 == 0 ? 0.0f : (float)U(rng);
        const float thr = trial % 2 ? (float)(U(rng) * 2.0) : INFINITY;
        const uint32_t cnt0 = (uint32_t)(rng() % 10), limit = trial % 5 == 0 ? cnt0 + 1 + (uint32_t)(rng() % c) : 0;
        float s = s0; uint32_t cnt = cnt0; uint32_t want_done = 0; bool want_found = false, want_by_limit = false;
        for (uint32_t i = 0; i < c; ++i) {
            s += x; ++cnt; ++want_done;
            const bool over = s > thr;
            if (over || (limit && cnt >= limit)) { want_found = true; want_by_limit = !over; break; }
        }
        float s2 = s0; uint32_t cnt2 = cnt0; bool found = false, by_limit = false;
        const uint32_t done = fsx::add_repeated(s2, cnt2, x, c, thr, limit, &found, &by_limit);
        CHECK(done == want_done && found == want_found && (!found || by_limit == want_by_limit) && std::memcmp(&s, &s2, 4) == 0 && cnt == cnt2,
              "repeat x %a c %u s0 %a thr %a limit %u: done %u/%u found %d/%d sum %a/%a", x, c, s0, thr, limit, done, want_done, found, want_found, s2, s);
    }
}

// ---- the sorted walk, as the kernel runs it --------------------------------------------------------
struct Ref { uint32_t n_keep; float total; uint32_t pick_key; bool fallback; };
static Ref reference_top_p(const std::vector<float>& p, float top_p, float u, float min_thr) {
    std::vector<float> v;
    for (float x : p) if (x >= min_thr) v.push_back(x);
    std::sort(v.begin(), v.end(), std::greater<float>());
    float sum = 0.0f;
    size_t n = 0;
    for (float x : v) { sum += x; ++n; if (sum > top_p) break; }
    Ref r;
    r.n_keep = (uint32_t)n; r.total = sum;
    const float rr = sum * u;
    float run = 0.0f;
    size_t pick = n - 1;
    r.fallback = true;
    for (size_t i = 0; i < n; ++i) { run += v[i]; if (run > rr) { pick = i; r.fallback = false; break; } }
    r.pick_key = fsx::float_bits(v[pick]);
    return r;
}

static std::vector<float> softmax_row(std::mt19937_64& rng, int V, int kind) {
    std::normal_distribution<float> N(0.0f, 1.0f);
    std::vector<float> x(V);
    switch (kind) {
        case 0: for (auto& v : x) v = 2.0f * N(rng); break;                                   // N(0, 4)
        case 1: for (auto& v : x) v = 2.0f * N(rng); for (int i = 0; i < 8; ++i) x[rng() % V] += 15.0f; break;
        case 2: for (auto& v : x) v = 0.0f; break;                                            // all equal
        case 3: for (auto& v : x) v = (float)(int)(4.0f * N(rng)) * 0.25f; break;             // heavily quantised
        case 4: for (auto& v : x) v = 0.3f * N(rng); break;                                   // flat
        case 5: for (auto& v : x) v = 6.0f * N(rng); break;                                   // peaked
        case 6: { for (auto& v : x) v = 2.0f * N(rng); for (auto& v : x) { uint32_t b = fsx::float_bits(v) & 0xffff0000u; v = fsx::bits_float(b); } break; }  // bf16 logits
        default: for (auto& v : x) v = (rng() % 3 == 0) ? -INFINITY : N(rng); break;          // masked entries
    }
    float mx = -INFINITY;
    for (float v : x) mx = std::max(mx, v);
    float sum = 0.0f;
    for (auto& v : x) { v = expf(v - mx); sum += v; }
    for (auto& v : x) v /= sum;
    return x;
}

static void test_walk(std::mt19937_64& rng, int rows) {
    std::uniform_real_distribution<float> U(0.0f, 1.0f);
    long long passes = 0, steps = 0, resumed = 0;
    int runs = 0;
    for (int t = 0; t < rows; ++t) {
        const int kind = t % 8;
        const int V = kind == 2 ? (t % 16 == 2 ? 128256 : 5000) : (t % 3 == 0 ? 128256 : 2000 + (int)(rng() % 60000));
        const std::vector<float> p = softmax_row(rng, V, kind);
        const float top_ps[] = {0.95f, 0.9f, 0.5f, 0.999f, 0.1f, 0.9999999f};
        const float top_p = top_ps[(t / 8) % 6];
        const float u = U(rng);
        float pmax = 0.0f;
        for (float x : p) pmax = std::max(pmax, x);
        const float min_thr = (t % 5 == 4) ? 0.01f * pmax : 0.0f;
        const Ref want = reference_top_p(p, top_p, u, min_thr);
        topp_model::Model m(p.data(), V, min_thr);
        const topp_model::Result got = m.solve(top_p, u);
        passes += m.passes; steps += m.steps_made; resumed += m.resumed; ++runs;
        CHECK(got.n_keep == want.n_keep && std::memcmp(&got.total, &want.total, 4) == 0 && got.pick_key == want.pick_key,
              "row %d kind %d V %d top_p %g u %g: n %u/%u total %a/%a pick key %08x/%08x", t, kind, V, top_p, u, got.n_keep, want.n_keep,
              got.total, want.total, got.pick_key, want.pick_key);
        if (got.pick_key == want.pick_key) CHECK(fsx::float_bits(p[got.pick_idx]) == got.pick_key, "row %d: picked index does not hold the picked key", t);
    }
    std::printf("walk: %d rows, %.2f passes over the row on average, %lld listed bins composed into steps, %lld draws started from a checkpoint\n", runs,
                (double)passes / runs, steps, resumed);
    CHECK(resumed > 0, "no draw ever started from a checkpoint: that path went untested");
    CHECK(steps > 0, "no listed bin was ever composed into a step: that path of walk_level went untested");
}

int main(int argc, char** argv) {
    const long long stride = argc > 1 ? std::atoll(argv[1]) : 997;
    const int rows = argc > 2 ? std::atoi(argv[2]) : 96;
    std::mt19937_64 rng(12345);
    test_table();
    test_expf(stride);
    test_scan(rng);
    test_repeated(rng);
    test_amount_and_division(rng);
    test_walk(rng, rows);
    if (g_fail) { std::printf("%d check(s) failed\n", g_fail); return 1; }
    std::printf("fsum_exact: all checks passed\n");
    return 0;
}
