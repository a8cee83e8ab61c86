// TEST INFRASTRUCTURE - CPU restatement of the Sampler's per-row numeric path.
//
// Follows, in this order, the reference's
//   LogitProcessor chain           src/cpp/src/sampling/logit_processor.hpp:28-124
//   penalty / filter arithmetic    src/cpp/src/sampling/logit_transformers.hpp:90-525
//   greedy and multinomial choice  src/cpp/src/sampling/sampler.cpp:939-1095
// and is compiled with the same libstdc++ the reference would use on Linux, so std::make_heap /
// pop_heap / push_heap / partial_sort / sort and glibc expf / logf behave identically.
// Pinned by the reference's golden vectors (tests/cpp/logit_filtering.cpp) through
// tests/golden/logit_filtering.json, and cross-checked against the reference's own
// logit_transformers.hpp compiled unmodified (oracle/ref_sampler_bridge.cpp) where that is built.
// Multinomial draws have no known-answer test in the reference: for them parity is pinned only by
// this cross-check of every transform plus the line-by-line restatement of _multinomial_sample.
//
// Difference from the reference that tests rely on: the softmax of the full-vocabulary path is
// computed on a scratch copy, so after the call `logits` holds the penalised logits (the
// reference overwrites the row with probabilities, logit_transformers.hpp:343-359).
//
// Only tests, the smoke check and the benchmark's CPU-baseline leg may call this file.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstddef>
#include <cstring>
#include <limits>
#include <random>
#include <thread>
#include <vector>

#include "../include/sampler_b200.h"

namespace {

struct Tok {
    float p;
    int64_t idx;
};

struct RowState {
    float* data;       // working row (scratch copy once a filter needs to overwrite it)
    size_t size;       // live element count (vocab, or the filtered count)
    std::vector<Tok> vec;  // late-initialised candidate list
    bool defer_expf = false;
    bool has_vec() const { return !vec.empty(); }
    void init_vec() {
        vec.reserve(size);
        for (size_t i = 0; i < size; ++i) vec.push_back(Tok{data[i], (int64_t)i});
    }
    void resize(size_t n) { size = n; vec.resize(n); }
};

// logit_transformers.hpp:200-249 - K-element min-heap over the row, strict '>' replacement.
void top_k_filter(RowState& st, size_t k) {
    if (k >= st.size) return;
    auto min_first = [](const Tok& a, const Tok& b) { return a.p > b.p; };
    st.vec.resize(k);
    for (size_t i = 0; i < k; ++i) st.vec[i] = Tok{st.data[i], (int64_t)i};
    std::make_heap(st.vec.begin(), st.vec.end(), min_first);
    for (size_t i = k; i < st.size; ++i) {
        if (st.data[i] > st.vec[0].p) {
            std::pop_heap(st.vec.begin(), st.vec.end(), min_first);
            st.vec.back() = Tok{st.data[i], (int64_t)i};
            std::push_heap(st.vec.begin(), st.vec.end(), min_first);
        }
    }
    st.size = k;
}

// logit_transformers.hpp:299-362
void temperature(RowState& st, float T, bool defer) {
    if (defer && st.has_vec()) {
        if (T != 1.0f) {
            const float f = 1.0f / T;
            for (size_t i = 0; i < st.size; ++i) st.vec[i].p *= f;
        }
        st.defer_expf = true;
        return;
    }
    if (st.has_vec()) {
        float mx = st.vec[0].p;
        for (size_t i = 1; i < st.size; ++i) if (st.vec[i].p > mx) mx = st.vec[i].p;
        float sum = 0.0f;
        if (T == 1.0f) {
            for (size_t i = 0; i < st.size; ++i) { st.vec[i].p = expf(st.vec[i].p - mx); sum += st.vec[i].p; }
        } else {
            const float f = 1.0f / T;
            for (size_t i = 0; i < st.size; ++i) { st.vec[i].p = expf((st.vec[i].p - mx) * f); sum += st.vec[i].p; }
        }
        for (size_t i = 0; i < st.size; ++i) st.vec[i].p /= sum;
    } else {
        const float mx = *std::max_element(st.data, st.data + st.size);
        float sum = 0.0f;
        if (T == 1.0f) {
            for (size_t i = 0; i < st.size; ++i) { st.data[i] = expf(st.data[i] - mx); sum += st.data[i]; }
        } else {
            const float f = 1.0f / T;
            for (size_t i = 0; i < st.size; ++i) { st.data[i] = expf((st.data[i] - mx) * f); sum += st.data[i]; }
        }
        for (size_t i = 0; i < st.size; ++i) st.data[i] /= sum;
    }
}

// logit_transformers.hpp:157-190
void min_p_filter(RowState& st, double min_p) {
    if (!st.has_vec()) st.init_vec();
    float mx = 0.0f;
    size_t arg = 0;
    for (size_t i = 0; i < st.size; ++i)
        if (st.vec[i].p > mx) { mx = st.vec[i].p; arg = i; }
    const float thr = static_cast<float>(min_p) * mx;
    size_t n = 0;
    for (size_t i = 0; i < st.size; ++i)
        if (st.vec[i].p >= thr) st.vec[n++] = st.vec[i];
    if (n == 0) { st.vec[0] = st.vec[arg]; n = 1; }
    st.resize(n);
}

// logit_transformers.hpp:94-139
void top_p_filter(RowState& st, double top_p) {
    if (!st.has_vec()) st.init_vec();
    auto desc = [](const Tok& a, const Tok& b) { return a.p > b.p; };
    for (size_t step = 16; step <= 1024; step *= 2) {
        if (st.vec.size() <= step) break;
        std::partial_sort(st.vec.begin(), st.vec.begin() + step, st.vec.end(), desc);
        float sum = 0.0f;
        for (size_t i = 0; i < step; ++i) {
            sum += st.vec[i].p;
            if (sum > top_p) { st.resize(i + 1); return; }
        }
    }
    std::sort(st.vec.begin(), st.vec.end(), desc);
    float sum = 0.0f;
    size_t n = 0;
    for (const Tok& t : st.vec) {
        sum += t.p;
        ++n;
        if (sum > top_p) break;
    }
    st.resize(n);
}

// sampler.cpp:939-977 with top_logprobs == 0
Tok greedy(const RowState& st) {
    float best = -std::numeric_limits<float>::infinity();
    size_t arg = 0;
    for (size_t i = 0; i < st.size; ++i) {
        const float v = st.has_vec() ? st.vec[i].p : st.data[i];
        if (v > best) { best = v; arg = st.has_vec() ? (size_t)st.vec[i].idx : i; }
    }
    return Tok{0.0f, (int64_t)arg};
}

// sampler.cpp:979-1095 for one draw with the uniform number already drawn
Tok multinomial(const RowState& st, float u, bool* uniform_fallback) {
    *uniform_fallback = false;
    if (st.defer_expf) {
        float mx = st.vec[0].p;
        for (size_t i = 1; i < st.size; ++i) if (st.vec[i].p > mx) mx = st.vec[i].p;
        std::vector<float> w(st.size);
        float sum = 0.0f;
        for (size_t i = 0; i < st.size; ++i) { w[i] = expf(st.vec[i].p - mx); sum += w[i]; }
        const bool uniform = !(sum > 0.0f && std::isfinite(sum));
        if (uniform) { std::fill(w.begin(), w.end(), 1.0f); sum = static_cast<float>(st.size); }
        const float log_sum = logf(sum) + (uniform ? 0.0f : mx);
        const float r = sum * u;
        float run = 0.0f;
        size_t pick = st.size - 1;
        for (size_t i = 0; i < st.size; ++i) { run += w[i]; if (run > r) { pick = i; break; } }
        const float lp = uniform ? std::log(1.0f / static_cast<float>(st.size)) : st.vec[pick].p - log_sum;
        *uniform_fallback = uniform;
        return Tok{lp, st.vec[pick].idx};
    }
    float total = 0.0f;
    if (st.has_vec()) for (size_t i = 0; i < st.size; ++i) total += st.vec[i].p;
    else for (size_t i = 0; i < st.size; ++i) total += st.data[i];
    if (!(total > 0.0f && std::isfinite(total))) {
        // the reference draws an index with uniform_int_distribution here; with a pre-drawn u the
        // restatement maps u to an index the same way the kernel does
        const size_t pick = std::min(st.size - 1, (size_t)(u * (float)st.size));
        *uniform_fallback = true;
        return Tok{std::log(1.0f / st.size), st.has_vec() ? st.vec[pick].idx : (int64_t)pick};
    }
    const float log_total = std::log(total);
    const float r = total * u;
    float run = 0.0f;
    size_t pick = st.size - 1;
    if (st.has_vec()) {
        for (size_t i = 0; i < st.size; ++i) { run += st.vec[i].p; if (run > r) { pick = i; break; } }
        return Tok{std::log(st.vec[pick].p) - log_total, st.vec[pick].idx};
    }
    for (size_t i = 0; i < st.size; ++i) { run += st.data[i]; if (run > r) { pick = i; break; } }
    return Tok{std::log(st.data[pick]) - log_total, (int64_t)pick};
}

int process_row(const sampler_step_args* a, int r, std::vector<float>& scratch) {
    const sampler_row_params& p = a->rows[r];
    if (p.logits_row < 0 || p.logits_row >= a->num_logit_rows) return SAMPLER_ERR_INVALID_ARG;
    float* row = a->logits + p.logits_row * a->vocab;
    const size_t V = (size_t)a->vocab;
    const int64_t h0 = a->hist_offsets ? a->hist_offsets[r] : 0, h1 = a->hist_offsets ? a->hist_offsets[r + 1] : 0;
    for (int64_t i = h0; i < h1; ++i)
        if (a->hist_ids[i] < 0 || (size_t)a->hist_ids[i] >= V) return SAMPLER_ERR_BAD_TOKEN_ID;

    // logprobs > 0: log-partition of the raw row first (logit_transformers.hpp:264-277), and the raw
    // logits kept aside: the reference's penalties then work on a copy and the reported
    // log-probability is raw_logit[token] - log-partition (sampler.cpp:967-974, 1022-1029, 1076-1081).
    // This restatement keeps the penalties in place, as the entry point it checks does.
    const bool raw_lp = (p.do_sample & SAMPLER_ROW_RAW_LOG_PROB) != 0;
    float raw_lse = 0.0f;
    std::vector<float> raw;
    if (raw_lp) {
        const float max_logit = *std::max_element(row, row + V);
        float sum = 0.0f;
        for (size_t i = 0; i < V; ++i) sum += expf(row[i] - max_logit);
        raw_lse = logf(sum) + max_logit;
        raw.assign(row, row + V);
    }

    // stop-token mask while generated_len < min_new_tokens (logit_transformers.hpp:452-463)
    for (int64_t i = h0; i < h1; ++i)
        if (a->hist_meta[i] & SAMPLER_HIST_STOP_MASK) row[a->hist_ids[i]] = -std::numeric_limits<float>::infinity();
    // grammar bitmask (structured_output/xgrammar_backend.cpp:187-207): a cleared bit makes the logit -inf
    if (a->struct_size == sizeof(sampler_step_args) && a->token_bitmasks && a->bitmask_index && a->bitmask_index[r] >= 0) {
        const int32_t* mask = a->token_bitmasks + (int64_t)a->bitmask_index[r] * a->bitmask_words;
        for (size_t i = 0; i < V; ++i)
            if (!((uint32_t)mask[i / 32] >> (i % 32) & 1u)) row[i] = -std::numeric_limits<float>::infinity();
    }
    // repetition: unique prompt ids, then generated ids not in the prompt (403-427)
    if (p.repetition_penalty != 1.0f) {
        const double pen = p.repetition_penalty;
        for (int64_t i = h0; i < h1; ++i)
            if (a->hist_meta[i] & (SAMPLER_HIST_IN_PROMPT | SAMPLER_HIST_GENERATED)) {
                float& v = row[a->hist_ids[i]];
                if (v >= 0) v /= pen; else v *= pen;
            }
    }
    // presence: generated ids only (507-519)
    if (p.presence_penalty != 0.0f) {
        const double pen = p.presence_penalty;
        for (int64_t i = h0; i < h1; ++i)
            if (a->hist_meta[i] & SAMPLER_HIST_GENERATED) {
                float& v = row[a->hist_ids[i]];
                if (v >= 0) v -= pen; else v += pen;
            }
    }
    // frequency: generated ids only, scaled by the occurrence count (481-493)
    if (p.frequency_penalty != 0.0f) {
        const double pen = p.frequency_penalty;
        for (int64_t i = h0; i < h1; ++i)
            if (a->hist_meta[i] & SAMPLER_HIST_GENERATED) {
                float& v = row[a->hist_ids[i]];
                const size_t count = a->hist_meta[i] >> 3;
                if (v >= 0) v -= pen * count; else v += pen * count;
            }
    }

    RowState st;
    st.data = row;
    st.size = V;
    Tok out;
    bool uniform_fallback = false;
    if (!(p.do_sample & SAMPLER_ROW_MULTINOMIAL)) {
        out = greedy(st);
    } else {
        const bool top_k_active = p.top_k > 0 && p.top_k < std::numeric_limits<int64_t>::max();
        if (top_k_active) top_k_filter(st, (size_t)p.top_k);
        const bool min_p_active = p.min_p > 0.0f;
        const bool defer = top_k_active && p.top_p == 1.0f && !min_p_active;
        if (!st.has_vec()) {  // the full-vocabulary softmax overwrites its input: work on a copy
            scratch.assign(row, row + V);
            st.data = scratch.data();
        }
        temperature(st, p.temperature, defer);
        if (min_p_active) min_p_filter(st, p.min_p);
        if (p.top_p != 1.0f) top_p_filter(st, p.top_p);
        out = multinomial(st, p.rand_u, &uniform_fallback);
        // num_return_sequences > 1: further draws from the same distribution, one uniform number each (sampler.cpp:1065-1089)
        const bool extras = a->struct_size == sizeof(sampler_step_args) && a->extra_offsets;
        if (extras)
            for (int64_t k = a->extra_offsets[r]; k < a->extra_offsets[r + 1]; ++k) {
                bool uf = false;
                Tok more = multinomial(st, a->extra_rand_u[k], &uf);
                if (raw_lp && !uf) more.p = raw[(size_t)more.idx] - raw_lse;
                a->extra_out_token[k] = more.idx;
                a->extra_out_log_prob[k] = more.p;
            }
    }
    if (raw_lp && !uniform_fallback) out.p = raw[(size_t)out.idx] - raw_lse;
    a->out_token[r] = out.idx;
    a->out_log_prob[r] = out.p;
    return SAMPLER_OK;
}

}  // namespace

extern "C" {

// One task per row over `threads` workers, as the reference's ThreadPool does per request
// (sampler.cpp:1751-1754).
int sampler_oracle_step(const sampler_step_args* a, int threads) {
    if (!a || (a->struct_size != sizeof(sampler_step_args) && a->struct_size != SAMPLER_STEP_ARGS_SIZE_V1)) return SAMPLER_ERR_INVALID_ARG;
    std::atomic<int> next{0};
    std::atomic<int> status{SAMPLER_OK};
    auto work = [&] {
        std::vector<float> scratch;
        for (int r; (r = next.fetch_add(1)) < a->num_rows;) {
            const int rc = process_row(a, r, scratch);
            if (rc != SAMPLER_OK) status.store(rc);
        }
    };
    const int nt = std::max(1, std::min(threads, a->num_rows));
    if (nt == 1) {
        work();
    } else {
        std::vector<std::thread> pool;
        for (int t = 0; t < nt; ++t) pool.emplace_back(work);
        for (auto& th : pool) th.join();
    }
    return status.load();
}

// Exposes single transforms on a caller-provided row for the golden-vector tests.
// which: 0 temperature(T = param), 1 top-p, 2 top-k(k = param), 3 min-p.  Returns the number of
// surviving candidates written to out_p / out_idx (or `n` probabilities in place for temperature).
int sampler_oracle_transform(int which, float* data, int n, double param, float* out_p, int64_t* out_idx) {
    RowState st;
    st.data = data;
    st.size = (size_t)n;
    switch (which) {
        case 0: temperature(st, (float)param, false); break;
        case 1: top_p_filter(st, param); break;
        case 2: top_k_filter(st, (size_t)param); break;
        case 3: min_p_filter(st, param); break;
        default: return -1;
    }
    if (!st.has_vec()) {
        for (int i = 0; i < n; ++i) { out_p[i] = data[i]; out_idx[i] = i; }
        return n;
    }
    for (size_t i = 0; i < st.size; ++i) { out_p[i] = st.vec[i].p; out_idx[i] = st.vec[i].idx; }
    return (int)st.size;
}

// n uniform numbers from std::mt19937(seed) through std::uniform_real_distribution<float>(0, 1),
// the stream a request's RequestSamplerContext produces (sampler.hpp:130-138, sampler.cpp:980).
void sampler_oracle_uniform_stream(uint32_t seed, int n, float* out) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> u(0.0f, 1.0f);
    for (int i = 0; i < n; ++i) out[i] = u(rng);
}

int sampler_oracle_hardware_threads() { return (int)std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"
