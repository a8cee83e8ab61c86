// The sampling-relevant subset of ov::genai::GenerationConfig
// (src/cpp/include/openvino/genai/generation_config.hpp:649-709 for the defaults,
// src/cpp/src/generation_config.cpp:264-290 for the mode predicates, 292-401 for validate()).
// Beam search, tree search, assisted generation and structured output are not part of the
// accelerated path; validate() rejects them so that a caller cannot reach the CUDA step with a
// configuration it does not implement.
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>
#include <set>
#include <stdexcept>
#include <string>

namespace genai_b200 {

struct GenerationConfig {
    // generic
    size_t max_new_tokens = std::numeric_limits<size_t>::max();
    size_t min_new_tokens = 0;
    bool ignore_eos = false;
    int64_t eos_token_id = -1;
    std::set<int64_t> stop_token_ids;
    size_t logprobs = 0;
    size_t num_return_sequences = 1;
    // beam search (only checked, never run here)
    size_t num_beams = 1;
    size_t tree_depth = 0;
    // penalties
    float repetition_penalty = 1.0f;
    float presence_penalty = 0.0f;
    float frequency_penalty = 0.0f;
    // multinomial
    bool do_sample = false;
    float temperature = 1.0f;
    float top_p = 1.0f;
    size_t top_k = std::numeric_limits<size_t>::max();   // 0 and SIZE_MAX both mean "off" (logit_processor.hpp:85-86)
    float min_p = 0.0f;
    size_t rng_seed = 0;

    bool is_beam_search() const { return num_beams > 1; }
    bool is_tree_search() const { return tree_depth > 0; }
    bool is_greedy_decoding() const { return !do_sample && !is_beam_search() && !is_tree_search(); }
    bool is_multinomial() const { return do_sample; }

    void set_eos_token_id(int64_t id) {
        eos_token_id = id;
        stop_token_ids.insert(id);
    }

    // Throws std::invalid_argument where the reference's OPENVINO_ASSERT would throw ov::Exception.
    void validate() const {
        auto fail = [](const std::string& what) { throw std::invalid_argument(what); };
        if (num_return_sequences == 0) fail("num_return_sequences must be greater than 0");
        if (eos_token_id != -1 && stop_token_ids.count(eos_token_id) == 0) fail("'stop_token_ids' must contain 'eos_token_id'");
        for (int64_t id : stop_token_ids)
            if (id < 0) fail("'stop_token_ids' must be non-negative");
        const bool bounded = max_new_tokens != std::numeric_limits<size_t>::max();
        if (ignore_eos && !bounded) fail("ignore_eos is true: 'max_new_tokens' should be defined");
        if (eos_token_id == -1 && stop_token_ids.empty() && !bounded) fail("either 'eos_token_id', 'stop_token_ids' or 'max_new_tokens' should be defined");
        if (max_new_tokens == 0) fail("'max_new_tokens' must be greater than 0");
        if (min_new_tokens > max_new_tokens) fail("'min_new_tokens' must be less or equal to 'max_new_tokens'");
        if (!(repetition_penalty > 0.0f)) fail("'repetition_penalty' must be a strictly positive float");
        if (frequency_penalty < -2.0f || frequency_penalty > 2.0f) fail("'frequency_penalty' must be in [-2.0, 2.0]");
        if (presence_penalty < -2.0f || presence_penalty > 2.0f) fail("'presence_penalty' must be in [-2.0, 2.0]");
        if (do_sample) {
            if (!(top_p > 0.0f && top_p <= 1.0f)) fail("When 'do_sample' is true, top_p must be in (0.0, 1.0]");
            if (!(temperature > 0.0f)) fail("When 'do_sample' is true, temperature must be a strictly positive float");
            if (!(min_p >= 0.0f && min_p < 1.0f)) fail("When 'do_sample' is true, min_p must be in [0.0, 1.0)");
        }
        if (is_beam_search() || is_tree_search()) fail("beam search and tree search are outside the accelerated Sampler step");
        if (num_return_sequences > 1 && !do_sample) fail("num_return_sequences > 1 needs multinomial sampling (beam search is outside the accelerated Sampler step)");
    }
};

}  // namespace genai_b200
