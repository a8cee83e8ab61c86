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
    st.extra_offsets.push_back(0);
    for (SequenceGroup* g : sequence_groups) {
        if (!g->requires_sampling || g->all_finished()) continue;   // chunked-prefill rows produce no token
        RequestSamplerContext& ctx = context_of(*g);
        const GenerationConfig& cfg = g->sampling_params;
        sampler_row_params base{};
        base.do_sample = cfg.is_multinomial() ? SAMPLER_ROW_MULTINOMIAL : 0;
        if (cfg.logprobs > 0) base.do_sample |= SAMPLER_ROW_RAW_LOG_PROB;   // logit_processor.hpp:36-47
        // top_k: 0, SIZE_MAX (and anything that does not fit) mean "off" on both sides of the boundary (logit_processor.hpp:85-86)
        base.top_k = (cfg.top_k == 0 || cfg.top_k >= (size_t)std::numeric_limits<int64_t>::max()) ? std::numeric_limits<int64_t>::max() : (int64_t)cfg.top_k;
        base.temperature = cfg.temperature;
        base.top_p = cfg.top_p;
        base.min_p = cfg.min_p;
        base.repetition_penalty = cfg.repetition_penalty;
        base.presence_penalty = cfg.presence_penalty;
        base.frequency_penalty = cfg.frequency_penalty;

        // history: one entry per distinct id, flags say which maps hold it; shared by every sequence of the request
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
        for (const auto& kv : entries)
            if (kv.first < std::numeric_limits<int32_t>::min() || kv.first > std::numeric_limits<int32_t>::max())
                throw std::invalid_argument("token id " + std::to_string(kv.first) + " does not fit 32 bits");

        int mask_index = -1;
        if (g->token_bitmask) {
            for (size_t i = 0; i < st.bitmasks.size(); ++i) if (st.bitmasks[i] == g->token_bitmask) mask_index = (int)i;
            if (mask_index < 0) { mask_index = (int)st.bitmasks.size(); st.bitmasks.push_back(g->token_bitmask); }
        }

        // the request's sequences in order: the first one, then the running forks; each takes its draw(s) from the request's
        // own engine, in this order (sampler.cpp:979-1095, 1539-1549); greedy rows leave the engine untouched
        const bool first_token = g->generated_ids.empty() && g->forks.empty();
        const size_t n_total = g->forks.size() + 1;
        for (size_t q = 0; q < n_total; ++q) {
            const bool done = q == 0 ? g->finished : g->forks[q - 1].finished;
            if (done) continue;
            sampler_row_params row = base;
            row.logits_row = q == 0 ? g->logits_row : g->forks[q - 1].logits_row;
            row.rand_u = 0.f;
            size_t extras = 0;
            if (row.do_sample & SAMPLER_ROW_MULTINOMIAL) {
                std::uniform_real_distribution<float> dist(0.0f, 1.0f);
                row.rand_u = dist(ctx.rng_engine);
                if (first_token && cfg.num_return_sequences > 1) {
                    extras = cfg.num_return_sequences - 1;
                    for (size_t k = 0; k < extras; ++k) st.extra_rand_u.push_back(dist(ctx.rng_engine));
                }
            }
            st.rows.push_back(row);
            st.groups.push_back(g);
            st.sequence.push_back(q == 0 ? -1 : (int)q - 1);
            st.extra_offsets.push_back(st.extra_offsets.back() + (int64_t)extras);
            st.bitmask_index.push_back(mask_index);
            for (const auto& kv : entries) {
                st.hist_ids.push_back((int32_t)kv.first);
                st.hist_meta.push_back(kv.second);
            }
            st.hist_offsets.push_back((int64_t)st.hist_ids.size());
        }
    }
    return st;
}

void Sampler::register_new_token(RequestSamplerContext& ctx, std::vector<int64_t>& ids, std::vector<float>& log_probs, int64_t token, float log_prob) {
    // logit_processor.hpp:134-146 and sampler.cpp:1133-1148: the count map belongs to the request
    ++ctx.unique_generated_token_ids[token];
    ids.push_back(token);
    log_probs.push_back(log_prob);
    ctx.generated_len = ids.size();
}

bool Sampler::should_stop(const GenerationConfig& cfg, const std::vector<int64_t>& ids) const {
    // sampler.cpp:1097-1131 without stop strings
    const bool stop_hit = !cfg.ignore_eos && cfg.stop_token_ids.count(ids.back()) > 0;
    return cfg.max_new_tokens <= ids.size() || stop_hit;
}

SamplerOutput Sampler::commit(const PackedStep& step, const std::vector<int64_t>& tokens, const std::vector<float>& log_probs,
                              const std::vector<int64_t>& extra_tokens, const std::vector<float>& extra_log_probs) {
    SamplerOutput out;
    for (size_t r = 0; r < step.groups.size(); ++r) {
        SequenceGroup& g = *step.groups[r];
        const GenerationConfig& cfg = g.sampling_params;
        RequestSamplerContext& ctx = context_of(g);
        if (tokens[r] < 0) throw std::runtime_error("the Sampler step produced no token for a row");
        const int q = step.sequence[r];
        std::vector<int64_t>& ids = q < 0 ? g.generated_ids : g.forks[q].generated_ids;
        std::vector<float>& lps = q < 0 ? g.generated_log_probs : g.forks[q].generated_log_probs;
        register_new_token(ctx, ids, lps, tokens[r], log_probs[r]);
        ++out.num_generated_tokens;
        out.num_generated_tokens_per_request[g.request_id] += 1;
        const bool stop = should_stop(cfg, ids);
        if (q < 0) {
            if (stop) {
                g.finished = true;
                const bool stop_hit = !cfg.ignore_eos && cfg.stop_token_ids.count(ids.back()) > 0;
                g.finish_reason = stop_hit ? SequenceGroup::FinishReason::STOP : SequenceGroup::FinishReason::LENGTH;
            }
        } else if (stop) {
            g.forks[q].finished = true;
        }
        // the further draws of a request's first token become its forked sequences (sampler.cpp:1163-1182)
        const int64_t x0 = step.extra_offsets.empty() ? 0 : step.extra_offsets[r], x1 = step.extra_offsets.empty() ? 0 : step.extra_offsets[r + 1];
        for (int64_t k = x0; k < x1; ++k) {
            if (extra_tokens.at((size_t)k) < 0) throw std::runtime_error("the Sampler step produced no token for a further draw");
            g.forks.emplace_back();
            ForkedSequence& f = g.forks.back();
            register_new_token(ctx, f.generated_ids, f.generated_log_probs, extra_tokens[(size_t)k], extra_log_probs[(size_t)k]);
            ++out.num_generated_tokens;
            out.num_generated_tokens_per_request[g.request_id] += 1;
            f.finished = should_stop(cfg, f.generated_ids);
        }
        if (g.all_finished()) out.m_dropped_sequences.push_back(g.request_id);
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
    std::vector<int64_t> extra_tokens((size_t)st.extra_offsets.back(), -1);
    std::vector<float> extra_log_probs((size_t)st.extra_offsets.back(), 0.f);
    if (!extra_tokens.empty()) {
        a.extra_offsets = st.extra_offsets.data();
        a.extra_rand_u = st.extra_rand_u.data();
        a.extra_out_token = extra_tokens.data();
        a.extra_out_log_prob = extra_log_probs.data();
    }
    std::vector<int32_t> masks;
    if (!st.bitmasks.empty()) {
        const size_t words = (size_t)(vocab + 31) / 32;
        masks.resize(st.bitmasks.size() * words);
        for (size_t i = 0; i < st.bitmasks.size(); ++i) std::memcpy(masks.data() + i * words, st.bitmasks[i], words * sizeof(int32_t));
        a.token_bitmasks = masks.data();
        a.bitmask_index = st.bitmask_index.data();
        a.bitmask_words = (int64_t)words;
    }
    check(m_step_host(m_handle, &a, 1), "sampler step");
    SamplerOutput out = commit(st, tokens, log_probs, extra_tokens, extra_log_probs);
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
    const size_t nx = (size_t)st.extra_offsets.back();
    const size_t words = st.bitmasks.empty() ? 0 : (size_t)(vocab + 31) / 32;
    auto up = [](size_t x) { return (x + 255) / 256 * 256; };
    // inputs first (one host->device copy), then the outputs (one device->host copy), then device-only scratch
    size_t off = 0;
    auto take = [&](size_t bytes) { const size_t o = off; off += up(bytes); return o; };
    const size_t o_rows = take(n * sizeof(sampler_row_params)), o_off = take((n + 1) * 8), o_ids = take(st.hist_ids.size() * 4);
    const size_t o_meta = take(st.hist_meta.size() * 4), o_xoff = take(nx ? (n + 1) * 8 : 0), o_xu = take(nx * 4);
    const size_t o_midx = take(words ? n * 4 : 0), o_mask = take(st.bitmasks.size() * words * 4);
    const size_t in_bytes = off;
    const size_t o_tok = take(n * 8), o_lp = take(n * 4), o_xtok = take(nx * 8), o_xlp = take(nx * 4);
    const size_t out_end = off;
    const size_t o_raw = take(st.hist_ids.size() * 4);   // device only: raw logits of the history entries
    const size_t total = off;
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
    if (nx) {
        std::memcpy(hp + o_xoff, st.extra_offsets.data(), (n + 1) * 8);
        std::memcpy(hp + o_xu, st.extra_rand_u.data(), nx * 4);
    }
    if (words) {
        std::memcpy(hp + o_midx, st.bitmask_index.data(), n * 4);
        for (size_t i = 0; i < st.bitmasks.size(); ++i) std::memcpy(hp + o_mask + i * words * 4, st.bitmasks[i], words * 4);
    }
    check_cuda(cudaMemcpyAsync(dp, hp, in_bytes, cudaMemcpyHostToDevice, s), "copy of the row parameters");
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
    if (nx) {
        a.extra_offsets = (const int64_t*)(dp + o_xoff);
        a.extra_rand_u = (const float*)(dp + o_xu);
        a.extra_out_token = (int64_t*)(dp + o_xtok);
        a.extra_out_log_prob = (float*)(dp + o_xlp);
    }
    if (words) {
        a.token_bitmasks = (const int32_t*)(dp + o_mask);
        a.bitmask_index = (const int32_t*)(dp + o_midx);
        a.bitmask_words = (int64_t)words;
    }
    a.stream = (void*)s;
    check(sampler_b200_step(m_handle, &a), "sampler_b200_step");
    check_cuda(cudaMemcpyAsync(hp + o_tok, dp + o_tok, out_end - o_tok, cudaMemcpyDeviceToHost, s), "copy of the sampled ids");
    check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    uint32_t bits = 0;
    check(sampler_b200_last_device_status(m_handle, &bits), "sampler_b200_last_device_status");
    if (bits & 1u) throw std::runtime_error("input_ids token out of bounds");
    if (bits & 8u) throw std::runtime_error("top_k above the sampler's heap capacity of 1024 (and below the vocabulary) is not supported");
    std::vector<int64_t> tokens(n), extra_tokens(nx);
    std::vector<float> log_probs(n), extra_log_probs(nx);
    std::memcpy(tokens.data(), hp + o_tok, n * 8);
    std::memcpy(log_probs.data(), hp + o_lp, n * 4);
    if (nx) {
        std::memcpy(extra_tokens.data(), hp + o_xtok, nx * 8);
        std::memcpy(extra_log_probs.data(), hp + o_xlp, nx * 4);
    }
    SamplerOutput out = commit(st, tokens, log_probs, extra_tokens, extra_log_probs);
    for (const auto& kv : zero.num_generated_tokens_per_request) out.num_generated_tokens_per_request.emplace(kv.first, 0);
    return out;
}

}  // namespace genai_b200
