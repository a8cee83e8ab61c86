// TEST INFRASTRUCTURE - C entry points around the reference's own logit transformers.
//
// Compiles src/cpp/src/sampling/logit_transformers.hpp from the reference tree UNMODIFIED (behind
// the include shim in oracle/ref_shim/sampler) and exposes each transformer so that tests can run
// the reference's golden vectors through the reference's own code and compare the oracle's
// restatement (oracle/sampler_oracle.cpp) with it on random inputs.  The output library lives in
// oracle/_ref/ and is never linked into the product.
#include <cstdint>
#include <cstring>
#include <memory>

#include "sampling/logit_transformers.hpp"

using namespace ov::genai;
using namespace ov::genai::LogitTransformers;

namespace {

int export_logits(const Logits& logits, float* out_p, int64_t* out_idx) {
    if (!logits.is_vector_initialized()) {
        for (size_t i = 0; i < logits.m_size; ++i) { out_p[i] = logits.m_data[i]; out_idx[i] = (int64_t)i; }
        return (int)logits.m_size;
    }
    for (size_t i = 0; i < logits.m_size; ++i) { out_p[i] = logits.m_vector[i].m_log_prob; out_idx[i] = logits.m_vector[i].m_index; }
    return (int)logits.m_size;
}

}  // namespace

extern "C" {

// which: 0 temperature(param), 1 top-p, 2 top-k, 3 min-p.  Same contract as
// sampler_oracle_transform.  Returns -2 if the reference threw.
int ref_transform(int which, float* data, int n, double param, float* out_p, int64_t* out_idx) {
    try {
        Logits logits(data, (size_t)n);
        switch (which) {
            case 0: TemperatureLogitTransform(param).apply(logits); break;
            case 1: TopPFilter(param).apply(logits); break;
            case 2: TopKFilter((size_t)param).apply(logits); break;
            case 3: MinPFilter(param).apply(logits); break;
            default: return -1;
        }
        return export_logits(logits, out_p, out_idx);
    } catch (const ov::Exception&) {
        return -2;
    }
}

// Penalties, in place on `data`.  which: 0 repetition, 1 frequency, 2 presence.
// `prompt_ids` feed the unique-prompt set (repetition only), `generated_ids` the occurrence map.
// Returns 0, or -2 if the reference threw (out-of-range id).
int ref_penalty(int which, float* data, int n, double penalty, const int64_t* prompt_ids, int n_prompt,
                const int64_t* generated_ids, int n_generated) {
    try {
        Logits logits(data, (size_t)n);
        TokenIds gen(generated_ids, generated_ids + n_generated);
        if (which == 0) {
            RepetitionPenaltyTransform t(penalty);
            auto prompt = std::make_shared<std::set<int64_t>>(prompt_ids, prompt_ids + n_prompt);
            t.set_unique_prompt_token_ids(prompt);
            t.extract_generated_tokens(gen);
            t.apply(logits);
        } else if (which == 1) {
            FrequencyPenaltyTransform t(penalty);
            t.apply(logits, gen);
        } else if (which == 2) {
            PresencePenaltyTransform t(penalty);
            t.apply(logits, gen);
        } else {
            return -1;
        }
        return 0;
    } catch (const ov::Exception&) {
        return -2;
    }
}

// EOS mask in place (EOSPenaltyTransform with min_generated_tokens = max).
int ref_eos_mask(float* data, int n, const int64_t* stop_ids, int n_stop) {
    Logits logits(data, (size_t)n);
    std::set<int64_t> stops(stop_ids, stop_ids + n_stop);
    EOSPenaltyTransform(stops, std::numeric_limits<size_t>::max()).apply(logits);
    return 0;
}

// The multinomial filter chain in LogitProcessor order: top-k -> temperature -> min-p -> top-p
// (logit_processor.hpp:80-104) on one row; returns the surviving candidates in the order the
// sampler would scan them and reports whether expf was deferred.
int ref_filter_chain(float* data, int n, int64_t top_k, float temperature, float top_p, float min_p, float* out_p,
                     int64_t* out_idx, int* deferred) {
    Logits logits(data, (size_t)n);
    const bool top_k_active = top_k > 0 && top_k < std::numeric_limits<int64_t>::max();
    if (top_k_active) TopKFilter((size_t)top_k).apply(logits);
    const bool min_p_active = min_p > 0.0f;
    const bool defer = top_k_active && top_p == 1.0f && !min_p_active;
    TemperatureLogitTransform(temperature, defer).apply(logits);
    if (min_p_active) MinPFilter(min_p).apply(logits);
    if (top_p != 1.0f) TopPFilter(top_p).apply(logits);
    *deferred = logits.m_defer_expf ? 1 : 0;
    return export_logits(logits, out_p, out_idx);
}

}  // extern "C"
