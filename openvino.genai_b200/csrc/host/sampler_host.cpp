// Host half of the Sampler: see sampler_host.hpp.
#include "sampler_host.hpp"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <limits>
#include <stdexcept>
#include <string>

namespace genai_b200 {

namespace {

void check(int rc, const char* what) {
    if (rc != SAMPLER_OK) throw std::runtime_error(std::string(what) + ": " + sampler_b200_last_error());
}
void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

Sampler::Sampler(int device) : m_device(device) {
    check(sampler_b200_create(device, 0, 0, &m_handle), "sampler_b200_create");
    m_step_host = &sampler_b200_step_host;
}

Sampler::~Sampler() {
    if (m_dev_buf) cudaFree(m_dev_buf);
    if (m_pinned) cudaFreeHost(m_pinned);
    if (m_handle) sampler_b200_destroy(m_handle);
}

Sampler::RequestSamplerContext& Sampler::context_of(SequenceGroup& group) {
    auto it = m_contexts.find(group.request_id);
    if (it == m_contexts.end()) {
        // sampler.cpp:1734-1737: the engine is seeded once per request with rng_seed; the unique
        // prompt ids are collected by the LogitProcessor constructor (logit_processor.hpp:33-35)
        group.sampling_params.validate();
        auto ctx = std::make_unique<RequestSamplerContext>(group.sampling_params.rng_seed);
        ctx->unique_prompt_token_ids.insert(group.prompt_ids.begin(), group.prompt_ids.end());
        it = m_contexts.emplace(group.request_id, std::move(ctx)).first;
    }
    return *it->second;
}

void Sampler::clear_request_info(uint64_t request_id) { m_contexts.erase(request_id); }

void Sampler::decrease_generated_token_occurance(uint64_t request_id, int64_t token_id) {
    auto it = m_contexts.find(request_id);
    if (it == m_contexts.end()) throw std::invalid_argument("unknown request");
    auto e = it->second->unique_generated_token_ids.find(token_id);
    if (e == it->second->unique_generated_token_ids.end()) throw std::invalid_argument("token was never generated");
    if (e->second > 0) --e->second;
}

Sampler::PackedStep Sampler::pack(const std::vector<SequenceGroup*>& sequence_groups) {
    PackedStep st;
    st.hist_offsets.push_back(0);
    for (SequenceGroup* g : sequence_groups) {
        if (!g->requires_sampling || g->finished) continue;   // chunked-prefill rows produce no token
        RequestSamplerContext& ctx = context_of(*g);
        const GenerationConfig& cfg = g->sampling_params;
        sampler_row_params row{};
        row.logits_row = g->logits_row;
        row.do_sample = cfg.is_multinomial() ? SAMPLER_ROW_MULTINOMIAL : 0;
        if (cfg.logprobs > 0) row.do_sample |= SAMPLER_ROW_RAW_LOG_PROB;   // logit_processor.hpp:36-47
        // top_k: SIZE_MAX (and anything that does not fit) means "off" on both sides of the boundary
        row.top_k = cfg.top_k >= (size_t)std::numeric_limits<int64_t>::max() ? std::numeric_limits<int64_t>::max() : (int64_t)cfg.top_k;
        row.temperature = cfg.temperature;
        row.top_p = cfg.top_p;
        row.min_p = cfg.min_p;
        row.repetition_penalty = cfg.repetition_penalty;
        row.presence_penalty = cfg.presence_penalty;
        row.frequency_penalty = cfg.frequency_penalty;
        // one draw per sampled token from the request's own engine (sampler.cpp:979-1095); greedy
        // rows leave the engine untouched
        row.rand_u = 0.f;
        if (row.do_sample & SAMPLER_ROW_MULTINOMIAL) {
            std::uniform_real_distribution<float> dist(0.0f, 1.0f);
            row.rand_u = dist(ctx.rng_engine);
        }
        st.rows.push_back(row);
        st.groups.push_back(g);

        // history: one entry per distinct id, flags say which maps hold it
        const bool mask_stops = cfg.min_new_tokens > 0 && ctx.generated_len < cfg.min_new_tokens;   // logit_transformers.hpp:447-473
        std::map<int64_t, uint32_t> entries;   // id -> (count << 3) | flags
        for (int64_t id : ctx.unique_prompt_token_ids) entries[id] |= SAMPLER_HIST_IN_PROMPT;
        for (const auto& kv : ctx.unique_generated_token_ids) {
            uint32_t& e = entries[kv.first];
            e |= SAMPLER_HIST_GENERATED;
            e |= (uint32_t)std::min<size_t>(kv.second, (1u << 29) - 1) << 3;
        }
        if (mask_stops)
            for (int64_t id : cfg.stop_token_ids) entries[id] |= SAMPLER_HIST_STOP_MASK;
        for (const auto& kv : entries) {
            if (kv.first < std::numeric_limits<int32_t>::min() || kv.first > std::numeric_limits<int32_t>::max())
                throw std::invalid_argument("token id " + std::to_string(kv.first) + " does not fit 32 bits");
            st.hist_ids.push_back((int32_t)kv.first);
            st.hist_meta.push_back(kv.second);
        }
        st.hist_offsets.push_back((int64_t)st.hist_ids.size());
    }
    return st;
}

void Sampler::register_new_token(SequenceGroup& group, RequestSamplerContext& ctx, int64_t token, float log_prob) {
    // logit_processor.hpp:134-146 and sampler.cpp:1133-1148
    ++ctx.unique_generated_token_ids[token];
    group.generated_ids.push_back(token);
    group.generated_log_probs.push_back(log_prob);
    ctx.generated_len = group.generated_ids.size();
}

void Sampler::try_finish_generation(SequenceGroup& group, SamplerOutput& out) {
    // sampler.cpp:1097-1131 without stop strings
    const GenerationConfig& cfg = group.sampling_params;
    const size_t generated_len = group.generated_ids.size();
    const bool stop_hit = !cfg.ignore_eos && cfg.stop_token_ids.count(group.generated_ids.back()) > 0;
    if (cfg.max_new_tokens <= generated_len || stop_hit) {
        group.finished = true;
        if (stop_hit) group.finish_reason = SequenceGroup::FinishReason::STOP;
        else if (cfg.max_new_tokens == generated_len) group.finish_reason = SequenceGroup::FinishReason::LENGTH;
        out.m_dropped_sequences.push_back(group.request_id);
    }
}

SamplerOutput Sampler::commit(const PackedStep& step, const std::vector<int64_t>& tokens, const std::vector<float>& log_probs) {
    SamplerOutput out;
    for (size_t r = 0; r < step.groups.size(); ++r) {
        SequenceGroup& g = *step.groups[r];
        if (tokens[r] < 0) throw std::runtime_error("the Sampler step produced no token for a row");
        register_new_token(g, context_of(g), tokens[r], log_probs[r]);
        ++out.num_generated_tokens;
        out.num_generated_tokens_per_request[g.request_id] = 1;
        try_finish_generation(g, out);
    }
    return out;
}

SamplerOutput Sampler::sample(const std::vector<SequenceGroup*>& sequence_groups, float* logits, int64_t num_logit_rows, int64_t vocab) {
    PackedStep st = pack(sequence_groups);
    SamplerOutput zero;
    for (SequenceGroup* g : sequence_groups) zero.num_generated_tokens_per_request[g->request_id] = 0;
    if (st.rows.empty()) return zero;
    std::vector<int64_t> tokens(st.rows.size(), -1);
    std::vector<float> log_probs(st.rows.size(), 0.f);
    sampler_step_args a{};
    a.struct_size = sizeof(a);
    a.logits = logits;
    a.num_logit_rows = num_logit_rows;
    a.vocab = vocab;
    a.num_rows = (int32_t)st.rows.size();
    a.rows = st.rows.data();
    a.hist_offsets = st.hist_offsets.data();
    a.hist_ids = st.hist_ids.data();
    a.hist_meta = st.hist_meta.data();
    a.out_token = tokens.data();
    a.out_log_prob = log_probs.data();
    check(m_step_host(m_handle, &a, 1), "sampler step");
    SamplerOutput out = commit(st, tokens, log_probs);
    for (const auto& kv : zero.num_generated_tokens_per_request) out.num_generated_tokens_per_request.emplace(kv.first, 0);
    return out;
}

SamplerOutput Sampler::sample_device(const std::vector<SequenceGroup*>& sequence_groups, float* logits_dev, int64_t num_logit_rows, int64_t vocab,
                                     void* stream) {
    PackedStep st = pack(sequence_groups);
    SamplerOutput zero;
    for (SequenceGroup* g : sequence_groups) zero.num_generated_tokens_per_request[g->request_id] = 0;
    if (st.rows.empty()) return zero;
    check_cuda(cudaSetDevice(m_device), "cudaSetDevice");
    // a null stream means the legacy default stream here; the C ABI reads null as "the handle's own
    // stream", so name the legacy stream explicitly to keep the copies and the kernel in one queue
    cudaStream_t s = stream ? (cudaStream_t)stream : cudaStreamLegacy;
    const size_t n = st.rows.size();
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    const size_t o_rows = 0, o_off = o_rows + up(n * sizeof(sampler_row_params)), o_ids = o_off + up((n + 1) * 8);
    const size_t o_meta = o_ids + up(st.hist_ids.size() * 4), o_tok = o_meta + up(st.hist_meta.size() * 4), o_lp = o_tok + up(n * 8);
    const size_t o_raw = o_lp + up(n * 4);   // device only: raw logits of the history entries
    const size_t total = o_raw + up(st.hist_ids.size() * 4);
    if (total > m_dev_bytes) {   // grow-only staging
        if (m_dev_buf) check_cuda(cudaFree(m_dev_buf), "cudaFree");
        if (m_pinned) check_cuda(cudaFreeHost(m_pinned), "cudaFreeHost");
        m_dev_bytes = m_pinned_bytes = std::max(total, 2 * m_dev_bytes);
        check_cuda(cudaMalloc(&m_dev_buf, m_dev_bytes), "cudaMalloc");
        check_cuda(cudaMallocHost(&m_pinned, m_pinned_bytes), "cudaMallocHost");
    }
    uint8_t* hp = (uint8_t*)m_pinned;
    uint8_t* dp = (uint8_t*)m_dev_buf;
    std::memcpy(hp + o_rows, st.rows.data(), n * sizeof(sampler_row_params));
    std::memcpy(hp + o_off, st.hist_offsets.data(), (n + 1) * 8);
    if (!st.hist_ids.empty()) {
        std::memcpy(hp + o_ids, st.hist_ids.data(), st.hist_ids.size() * 4);
        std::memcpy(hp + o_meta, st.hist_meta.data(), st.hist_meta.size() * 4);
    }
    check_cuda(cudaMemcpyAsync(dp, hp, o_tok, cudaMemcpyHostToDevice, s), "copy of the row parameters");
    sampler_step_args a{};
    a.struct_size = sizeof(a);
    a.logits = logits_dev;
    a.num_logit_rows = num_logit_rows;
    a.vocab = vocab;
    a.num_rows = (int32_t)n;
    a.rows = (const sampler_row_params*)(dp + o_rows);
    a.hist_offsets = (const int64_t*)(dp + o_off);
    a.hist_ids = (const int32_t*)(dp + o_ids);
    a.hist_meta = (const uint32_t*)(dp + o_meta);
    a.out_token = (int64_t*)(dp + o_tok);
    a.out_log_prob = (float*)(dp + o_lp);
    a.hist_raw = (float*)(dp + o_raw);
    a.stream = (void*)s;
    check(sampler_b200_step(m_handle, &a), "sampler_b200_step");
    check_cuda(cudaMemcpyAsync(hp + o_tok, dp + o_tok, o_raw - o_tok, cudaMemcpyDeviceToHost, s), "copy of the sampled ids");
    check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    uint32_t bits = 0;
    check(sampler_b200_last_device_status(m_handle, &bits), "sampler_b200_last_device_status");
    if (bits & 1u) throw std::runtime_error("input_ids token out of bounds");
    std::vector<int64_t> tokens(n);
    std::vector<float> log_probs(n);
    std::memcpy(tokens.data(), hp + o_tok, n * 8);
    std::memcpy(log_probs.data(), hp + o_lp, n * 4);
    SamplerOutput out = commit(st, tokens, log_probs);
    for (const auto& kv : zero.num_generated_tokens_per_request) out.num_generated_tokens_per_request.emplace(kv.first, 0);
    return out;
}

}  // namespace genai_b200
