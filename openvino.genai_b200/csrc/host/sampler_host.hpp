// Host half of the Sampler, mirroring ov::genai::Sampler for the greedy and multinomial modes
// (src/cpp/src/sampling/sampler.hpp:104-180, sampler.cpp:1475-1810): per-request state (the
// std::mt19937 engine, the unique prompt ids, the generated-token count map), the packing of one
// step's rows for the CUDA kernel, token registration and the stop checks.  The numeric work of
// the step runs in sampler_b200_step / sampler_b200_step_host; there is no CPU fallback.
#pragma once

#include <cstdint>
#include <map>
#include <memory>
#include <random>
#include <set>
#include <unordered_map>
#include <vector>

#include "../../../include/sampler_b200.h"
#include "generation_config.hpp"

namespace genai_b200 {

// A sequence a request forked when it drew num_return_sequences tokens from its first distribution
// (sampler.cpp:1163-1182, 1539-1549): it shares the request's engine, token-count map and penalties.
struct ForkedSequence {
    std::vector<int64_t> generated_ids;
    std::vector<float> generated_log_probs;
    bool finished = false;
    int64_t logits_row = 0;   // set by the scheduler for every later step
};

// One request as the Sampler sees it: the reference's SequenceGroup, whose first Sequence is held
// inline and whose further sequences (num_return_sequences > 1) appear in `forks` after the first step.
struct SequenceGroup {
    uint64_t request_id = 0;
    std::vector<int64_t> prompt_ids;
    GenerationConfig sampling_params;
    // filled by the Sampler
    std::vector<int64_t> generated_ids;
    std::vector<float> generated_log_probs;
    bool finished = false;
    enum class FinishReason { NONE, STOP, LENGTH } finish_reason = FinishReason::NONE;
    // set by the scheduler for each step: does this group sample a token in this step, and from
    // which row of the logits tensor (the row of its last scheduled token)
    bool requires_sampling = true;
    int64_t logits_row = 0;
    std::vector<ForkedSequence> forks;
    // structured output: the grammar matcher's next-token bitmask for this step, ceil(vocab / 32) int32 words with bit
    // (t & 31) of word t / 32 set iff token t is allowed (xgrammar_backend.cpp:148-165); null: no grammar, or terminated
    const int32_t* token_bitmask = nullptr;
    bool all_finished() const {
        if (!finished) return false;
        for (const ForkedSequence& f : forks) if (!f.finished) return false;
        return true;
    }
};

struct SamplerOutput {
    std::vector<uint64_t> m_dropped_sequences;   // requests that finished in this step
    size_t num_generated_tokens = 0;
    std::unordered_map<uint64_t, size_t> num_generated_tokens_per_request;   // zero for chunked-prefill rows
};

class Sampler {
public:
    // The step function has the signature of sampler_b200_step_host; tests substitute the CPU
    // restatement to obtain the expected token streams from the same host logic.
    using StepHostFn = int (*)(sampler_handle*, const sampler_step_args*, int);

    explicit Sampler(int device = 0);
    ~Sampler();
    Sampler(const Sampler&) = delete;
    Sampler& operator=(const Sampler&) = delete;

    // One sampling step over HOST logits [num_logit_rows, vocab] (mutated in place like the
    // reference's, sampler.cpp:927-937).  Throws std::runtime_error with the library's message on
    // a failing status, std::invalid_argument on a configuration validate() rejects.
    SamplerOutput sample(const std::vector<SequenceGroup*>& sequence_groups, float* logits, int64_t num_logit_rows, int64_t vocab);

    // The same over DEVICE logits; row parameters and history are staged through the handle's
    // own device buffers on `stream` (a cudaStream_t).
    SamplerOutput sample_device(const std::vector<SequenceGroup*>& sequence_groups, float* logits_dev, int64_t num_logit_rows, int64_t vocab,
                                void* stream);

    void clear_request_info(uint64_t request_id);          // sampler.cpp: drops the request's context
    void set_step_function(StepHostFn fn) { m_step_host = fn; }

    // ---- pieces exposed for tests ---------------------------------------------------------------
    struct PackedStep {
        std::vector<sampler_row_params> rows;
        std::vector<int64_t> hist_offsets;
        std::vector<int32_t> hist_ids;
        std::vector<uint32_t> hist_meta;
        std::vector<SequenceGroup*> groups;   // group of each row
        std::vector<int> sequence;            // -1: the group's first sequence, k: forks[k]
        std::vector<int64_t> extra_offsets;   // further draws of each row (a request's first sampled token with num_return_sequences > 1)
        std::vector<float> extra_rand_u;
        std::vector<int32_t> bitmask_index;   // mask of each row, -1: none
        std::vector<const int32_t*> bitmasks; // distinct masks of the step
    };
    PackedStep pack(const std::vector<SequenceGroup*>& sequence_groups);
    SamplerOutput commit(const PackedStep& step, const std::vector<int64_t>& tokens, const std::vector<float>& log_probs,
                         const std::vector<int64_t>& extra_tokens = {}, const std::vector<float>& extra_log_probs = {});
    // the reference's LogitProcessor::decrease_generated_token_occurance (logit_processor.hpp:148-151):
    // the entry stays in the map at zero and still receives the repetition penalty
    void decrease_generated_token_occurance(uint64_t request_id, int64_t token_id);

private:
    struct RequestSamplerContext {
        std::mt19937 rng_engine;
        std::set<int64_t> unique_prompt_token_ids;
        std::map<int64_t, size_t> unique_generated_token_ids;
        size_t generated_len = 0;
        explicit RequestSamplerContext(size_t seed) : rng_engine(seed) {}
    };
    RequestSamplerContext& context_of(SequenceGroup& group);
    void register_new_token(RequestSamplerContext& ctx, std::vector<int64_t>& ids, std::vector<float>& log_probs, int64_t token, float log_prob);
    bool should_stop(const GenerationConfig& cfg, const std::vector<int64_t>& ids) const;

    int m_device;
    sampler_handle* m_handle = nullptr;
    StepHostFn m_step_host = nullptr;
    std::map<uint64_t, std::unique_ptr<RequestSamplerContext>> m_contexts;
    // device staging of sample_device
    void* m_dev_buf = nullptr;
    size_t m_dev_bytes = 0;
    void* m_pinned = nullptr;
    size_t m_pinned_bytes = 0;
};

}  // namespace genai_b200
