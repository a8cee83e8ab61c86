// Tests of the C++ host layer (csrc/host): GenerationConfig, the ModelRunner marshalling mirror and
// the host half of the Sampler.  Built and run by tests/test_host_layer.py.
//   host_layer_test cpu <rotation fixture file>
//   host_layer_test gpu <path of the CPU restatement's shared library>
// The GPU mode drives the same host logic twice, once over the CUDA step and once over the CPU
// restatement of the reference's sampler, and compares the token streams.
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <random>
#include <string>
#include <vector>

#include "generation_config.hpp"
#include "model_runner_host.hpp"
#include "sampler_host.hpp"

using namespace genai_b200;

static int g_checks = 0, g_failed = 0;
#define CHECK(cond)                                                                  \
    do {                                                                             \
        ++g_checks;                                                                  \
        if (!(cond)) { ++g_failed; std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); } \
    } while (0)

template <class F> static bool throws(F f) {
    try { f(); } catch (const std::exception&) { return true; }
    return false;
}

static void test_generation_config() {
    GenerationConfig c;
    // generation_config.hpp:649-709
    CHECK(c.temperature == 1.0f && c.top_p == 1.0f && c.top_k == std::numeric_limits<size_t>::max() && c.min_p == 0.0f);
    CHECK(c.repetition_penalty == 1.0f && c.presence_penalty == 0.0f && c.frequency_penalty == 0.0f && c.rng_seed == 0 && !c.do_sample);
    CHECK(c.is_greedy_decoding() && !c.is_multinomial());
    c.max_new_tokens = 10;
    c.validate();
    c.do_sample = true;
    CHECK(!c.is_greedy_decoding() && c.is_multinomial());
    c.validate();
    auto bad = [&](auto mutate) { GenerationConfig x = c; mutate(x); return throws([&] { x.validate(); }); };
    CHECK(bad([](GenerationConfig& x) { x.top_p = 0.f; }));
    CHECK(bad([](GenerationConfig& x) { x.top_p = 1.5f; }));
    CHECK(bad([](GenerationConfig& x) { x.temperature = 0.f; }));
    CHECK(!bad([](GenerationConfig& x) { x.top_k = 0; }));                         // 0 = top-k off (logit_processor.hpp:85-86)
    CHECK(!bad([](GenerationConfig& x) { x.num_return_sequences = 3; }));
    CHECK(bad([](GenerationConfig& x) { x.num_return_sequences = 3; x.do_sample = false; }));
    CHECK(bad([](GenerationConfig& x) { x.min_p = 1.f; }));
    CHECK(bad([](GenerationConfig& x) { x.repetition_penalty = 0.f; }));
    CHECK(bad([](GenerationConfig& x) { x.frequency_penalty = 2.5f; }));
    CHECK(bad([](GenerationConfig& x) { x.presence_penalty = -2.5f; }));
    CHECK(bad([](GenerationConfig& x) { x.eos_token_id = 7; }));                  // not in stop_token_ids
    CHECK(!bad([](GenerationConfig& x) { x.set_eos_token_id(7); }));
    CHECK(bad([](GenerationConfig& x) { x.stop_token_ids.insert(-3); }));
    CHECK(bad([](GenerationConfig& x) { x.min_new_tokens = 11; }));
    CHECK(bad([](GenerationConfig& x) { x.max_new_tokens = std::numeric_limits<size_t>::max(); }));   // no stop condition
    CHECK(bad([](GenerationConfig& x) { x.num_beams = 4; }));
    CHECK(!bad([](GenerationConfig& x) { x.logprobs = 1; }));   // raw log-probabilities are reported by the step
}

static void test_attention_inputs() {
    const size_t bs = 4;
    std::vector<ScheduledSequence> seqs(3);
    // a prefill chunk of 6 tokens on an empty cache
    seqs[0].seq_id = 5; seqs[0].num_scheduled_tokens = 6; seqs[0].block_table = {10, 11};
    // a decode row: 9 tokens processed, block 1 hidden by a sparse mask
    seqs[1].seq_id = 2; seqs[1].num_processed_tokens = 9; seqs[1].num_scheduled_tokens = 1; seqs[1].block_table = {20, 21, 22};
    seqs[1].skipped_logical_blocks = {1}; seqs[1].can_generate_tokens = true;
    // a decode row after eviction of 4 tokens, SnapKV window still open
    seqs[2].seq_id = 9; seqs[2].num_processed_tokens = 12; seqs[2].num_evicted_tokens = 4; seqs[2].num_scheduled_tokens = 1;
    seqs[2].block_table = {30, 31, 32}; seqs[2].score_aggregation_window = 3; seqs[2].can_generate_tokens = true;
    AttentionInputs in = build_attention_inputs(seqs, bs, true);
    CHECK((in.past_lens == std::vector<int32_t>{0, 5, 8}));
    CHECK((in.subsequence_begins == std::vector<int32_t>{0, 6, 7, 8}));
    CHECK((in.block_indices_begins == std::vector<int32_t>{0, 2, 4, 7}));
    CHECK((in.block_indices == std::vector<int32_t>{10, 11, 20, 22, 30, 31, 32}));
    CHECK((in.score_aggregation_window == std::vector<int32_t>{1, 1, 3}));
    CHECK(in.max_context_len == 13 && in.num_tokens == 8);
    CHECK(build_attention_inputs(seqs, bs, false).score_aggregation_window.empty());

    // rotation inputs: ascending seq_id whatever the scheduled order
    std::map<uint64_t, std::vector<std::pair<size_t, int32_t>>> rot;
    rot[9] = {{1, 2}, {2, 2}};
    rot[2] = {{2, 1}};
    RotationInputs r = build_rotation_inputs(rot, seqs);
    CHECK((r.rotated_block_indices == std::vector<int32_t>{22, 31, 32}));
    CHECK((r.rotation_deltas == std::vector<int32_t>{1, 2, 2}));
    rot[77] = {{0, 1}};
    CHECK(throws([&] { build_rotation_inputs(rot, seqs); }));

    // score spans: every sequence owns a slot; the unfinished prompt without a window hands nothing on
    auto spans = collect_attention_scores(seqs, bs);
    CHECK(spans.size() == 2 && spans.count(5) == 0);
    CHECK(spans[2].begin == 6 && spans[2].end == 6 + 10 - 4);      // 10 context tokens, one block skipped
    CHECK(spans[9].begin == 12 && spans[9].end == 12 + 13 - 4);    // 13 context tokens, 4 evicted
}

// The reference's proof-of-concept dumps (block size, head size, blocks before eviction, evicted
// logical indices, then per rotated block its index after eviction, head/2 sines, head/2 cosines).
static void test_rotation_lut(const char* fixture) {
    std::ifstream f(fixture);
    CHECK(f.good());
    int files = 0;
    f >> files;
    for (int k = 0; k < files; ++k) {
        size_t bs = 0, head = 0, before = 0, nev = 0, nrot = 0;
        f >> bs >> head >> before >> nev;
        std::set<size_t> evicted;
        for (size_t i = 0; i < nev; ++i) { size_t e; f >> e; evicted.insert(e); }
        std::vector<size_t> kept;
        for (size_t b = 0; b < before; ++b) if (!evicted.count(b)) kept.push_back(b);
        const std::vector<float> lut = make_rotation_trig_lut(1024 / bs + 1, bs, head);
        f >> nrot;
        for (size_t i = 0; i < nrot; ++i) {
            size_t after = 0;
            f >> after;
            CHECK(after < kept.size());
            const size_t delta = kept[after] - after;   // blocks the block moves toward the start
            for (size_t j = 0; j < head / 2; ++j) { float s; f >> s; CHECK(std::fabs(s - lut[delta * head + head / 2 + j]) <= 1e-2f); }
            for (size_t j = 0; j < head / 2; ++j) { float c; f >> c; CHECK(std::fabs(c - lut[delta * head + j]) <= 1e-2f); }
        }
    }
    // closed form on one entry: row 3, block size 32, head 128, theta 1e6, j = 5
    const std::vector<float> lut = make_rotation_trig_lut(8, 32, 128, 1e6);
    const double ang = 3.0 * 32.0 * std::pow(1e6, -10.0 / 128.0);
    CHECK(std::fabs(lut[3 * 128 + 5] - (float)std::cos(ang)) == 0.f && std::fabs(lut[3 * 128 + 64 + 5] + (float)std::sin(ang)) == 0.f);
}

static SequenceGroup make_group(uint64_t id, const GenerationConfig& cfg, std::vector<int64_t> prompt, int64_t row) {
    SequenceGroup g;
    g.request_id = id;
    g.sampling_params = cfg;
    g.prompt_ids = std::move(prompt);
    g.logits_row = row;
    return g;
}

// pack(): history entries, the stop mask window, the RNG stream, without any device work.
static void test_sampler_pack() {
    Sampler sampler(0);
    GenerationConfig cfg;
    cfg.max_new_tokens = 8;
    cfg.do_sample = true;
    cfg.top_k = 5;
    cfg.repetition_penalty = 1.2f;
    cfg.min_new_tokens = 2;
    cfg.set_eos_token_id(3);
    cfg.rng_seed = 0;
    SequenceGroup g = make_group(1, cfg, {7, 7, 9}, 4);
    GenerationConfig greedy;
    greedy.max_new_tokens = 8;
    SequenceGroup h = make_group(2, greedy, {1}, 0);
    std::vector<SequenceGroup*> groups{&g, &h};

    Sampler::PackedStep st = sampler.pack(groups);
    CHECK(st.rows.size() == 2 && st.rows[0].logits_row == 4 && st.rows[0].do_sample == 1 && st.rows[0].top_k == 5);
    CHECK(st.rows[1].do_sample == 0 && st.rows[1].top_k == std::numeric_limits<int64_t>::max() && st.rows[1].rand_u == 0.f);
    // first two outputs of uniform_real_distribution<float>(0, 1) over std::mt19937(0)
    CHECK(std::fabs(st.rows[0].rand_u - 0.548813522f) < 1e-7f);
    // prompt ids once each, stop id masked while generated_len < min_new_tokens
    CHECK((st.hist_offsets == std::vector<int64_t>{0, 3, 4}));
    CHECK((st.hist_ids == std::vector<int32_t>{3, 7, 9, 1}));
    CHECK(st.hist_meta[0] == SAMPLER_HIST_STOP_MASK && st.hist_meta[1] == SAMPLER_HIST_IN_PROMPT && st.hist_meta[2] == SAMPLER_HIST_IN_PROMPT);

    // two generated tokens: 9 (also a prompt id) twice
    SamplerOutput out = sampler.commit(st, {9, 5}, {-0.5f, 0.f});
    CHECK(out.num_generated_tokens == 2 && out.m_dropped_sequences.empty());
    st = sampler.pack(groups);
    CHECK(std::fabs(st.rows[0].rand_u - 0.592844605f) < 1e-7f);
    sampler.commit(st, {9, 6}, {-0.25f, 0.f});
    st = sampler.pack(groups);
    // min_new_tokens reached: no stop mask any more; 9 is in both maps with count 2
    CHECK((st.hist_ids == std::vector<int32_t>{7, 9, 1, 5, 6}));
    CHECK(st.hist_meta[1] == ((2u << 3) | SAMPLER_HIST_IN_PROMPT | SAMPLER_HIST_GENERATED));
    CHECK(st.hist_meta[3] == ((1u << 3) | SAMPLER_HIST_GENERATED));
    // an entry decremented to zero stays in the map (and keeps its repetition penalty)
    sampler.decrease_generated_token_occurance(2, 5);
    st = sampler.pack(groups);
    CHECK(st.hist_meta[3] == SAMPLER_HIST_GENERATED);
    // stop token ends the request with reason STOP, the length limit with LENGTH
    out = sampler.commit(st, {3, 6}, {0.f, 0.f});
    CHECK(g.finished && g.finish_reason == SequenceGroup::FinishReason::STOP && out.m_dropped_sequences == std::vector<uint64_t>{1});
    CHECK(g.generated_ids == (std::vector<int64_t>{9, 9, 3}) && g.generated_log_probs[0] == -0.5f);
    for (int i = 0; i < 5; ++i) {
        st = sampler.pack(groups);
        CHECK(st.rows.size() == 1);   // the finished request is not sampled again
        out = sampler.commit(st, {6}, {0.f});
    }
    CHECK(h.finished && h.finish_reason == SequenceGroup::FinishReason::LENGTH && h.generated_ids.size() == 8);
    // a request that does not sample in this step (chunked prefill) is skipped and draws nothing
    SequenceGroup p = make_group(3, cfg, {4}, 0);
    p.requires_sampling = false;
    std::vector<SequenceGroup*> only{&p};
    CHECK(sampler.pack(only).rows.empty());
    // invalid configurations never reach the device
    GenerationConfig broken = cfg;
    broken.temperature = -1.f;
    SequenceGroup b = make_group(4, broken, {4}, 0);
    std::vector<SequenceGroup*> bad{&b};
    CHECK(throws([&] { sampler.pack(bad); }));
}

// ---- GPU: whole generations through the CUDA step against the CPU restatement ---------------------
typedef int (*oracle_step_fn)(const sampler_step_args*, int);
static oracle_step_fn g_oracle_step = nullptr;
static int oracle_step_adapter(sampler_handle*, const sampler_step_args* a, int) { return g_oracle_step(a, 4); }

static std::vector<GenerationConfig> request_configs() {
    std::vector<GenerationConfig> v;
    GenerationConfig greedy;
    greedy.max_new_tokens = 12;
    greedy.repetition_penalty = 1.3f;
    v.push_back(greedy);
    GenerationConfig a;   // top-k with deferred exponentials
    a.max_new_tokens = 12; a.do_sample = true; a.top_k = 20; a.temperature = 0.8f; a.rng_seed = 11;
    v.push_back(a);
    GenerationConfig b = a;   // top-k, top-p, all penalties
    b.top_p = 0.9f; b.repetition_penalty = 1.1f; b.presence_penalty = 0.2f; b.frequency_penalty = 0.1f; b.rng_seed = 12;
    v.push_back(b);
    GenerationConfig c = a;   // full vocabulary, min-p
    c.top_k = std::numeric_limits<size_t>::max(); c.min_p = 0.05f; c.temperature = 1.3f; c.rng_seed = 13;
    v.push_back(c);
    GenerationConfig d = a;   // stop tokens masked for the first steps, short length limit
    d.min_new_tokens = 3; d.max_new_tokens = 7; d.set_eos_token_id(17); d.stop_token_ids.insert(23); d.rng_seed = 14;
    v.push_back(d);
    GenerationConfig e = greedy;   // greedy with a stop token that the spikes make likely
    e.set_eos_token_id(5); e.repetition_penalty = 1.0f;
    v.push_back(e);
    GenerationConfig f = b;   // three sequences from one request: three draws from the first distribution, then one row each
    f.num_return_sequences = 3; f.rng_seed = 15; f.top_k = 0; f.top_p = 0.8f;   // top_k 0 = off: the full-vocabulary path
    v.push_back(f);
    GenerationConfig h = a;   // a grammar that only allows multiples of three
    h.rng_seed = 16;
    v.push_back(h);
    return v;
}

static void fill_logits(std::vector<float>& logits, int64_t rows, int64_t vocab, int step) {
    std::mt19937 gen(1234 + step);
    std::normal_distribution<float> nd(0.f, 2.f);
    for (auto& x : logits) x = nd(gen);
    for (int64_t r = 0; r < rows; ++r)
        for (int s = 0; s < 4; ++s) logits[r * vocab + (gen() % 64)] += 6.f;   // a few likely ids in [0, 64): repeats and stop hits
}

struct Generation { std::vector<std::vector<int64_t>> ids; std::vector<std::vector<float>> lps; std::vector<int> reasons; std::vector<std::vector<int64_t>> fork_ids; };

static Generation generate(Sampler& sampler, bool device_logits) {
    const int64_t vocab = 4096;
    std::vector<GenerationConfig> cfgs = request_configs();
    std::vector<SequenceGroup> groups;
    for (size_t i = 0; i < cfgs.size(); ++i) groups.push_back(make_group(100 + i, cfgs[i], {(int64_t)i, 40, 41, 40}, (int64_t)i));
    std::vector<SequenceGroup*> ptrs;
    for (auto& g : groups) ptrs.push_back(&g);
    std::vector<int32_t> grammar((size_t)(vocab + 31) / 32, 0);
    for (int64_t tkn = 0; tkn < vocab; tkn += 3) grammar[(size_t)tkn / 32] |= (int32_t)(1u << (tkn % 32));
    groups[7].token_bitmask = grammar.data();
    const int64_t rows = (int64_t)groups.size() + 2;   // two more rows once the three-sequence request has forked
    std::vector<float> logits(rows * vocab);
    float* dev = nullptr;
    if (device_logits && cudaMalloc(&dev, logits.size() * 4) != cudaSuccess) { CHECK(false); return {}; }
    for (int step = 0; step < 14; ++step) {
        fill_logits(logits, rows, vocab, step);
        // the scheduler's part: a row of the logits tensor for every running sequence
        int64_t next_row = (int64_t)groups.size();
        for (auto& g : groups)
            for (auto& fk : g.forks) fk.logits_row = next_row++;
        if (device_logits) {
            cudaMemcpy(dev, logits.data(), logits.size() * 4, cudaMemcpyHostToDevice);
            sampler.sample_device(ptrs, dev, rows, vocab, nullptr);
        } else {
            sampler.sample(ptrs, logits.data(), rows, vocab);
        }
        if (std::getenv("HOST_LAYER_TEST_VERBOSE")) {
            std::printf("step %d:", step);
            for (auto& g : groups) std::printf(" %lld", g.generated_ids.empty() ? -1LL : (long long)g.generated_ids.back());
            std::printf("\n");
        }
    }
    if (dev) cudaFree(dev);
    Generation out;
    for (auto& g : groups) {
        out.ids.push_back(g.generated_ids); out.lps.push_back(g.generated_log_probs); out.reasons.push_back((int)g.finish_reason);
        for (auto& fk : g.forks) out.fork_ids.push_back(fk.generated_ids);
    }
    return out;
}

static void test_sampler_gpu(const char* oracle_lib) {
    void* so = dlopen(oracle_lib, RTLD_NOW);
    CHECK(so != nullptr);
    if (!so) return;
    g_oracle_step = (oracle_step_fn)dlsym(so, "sampler_oracle_step");
    CHECK(g_oracle_step != nullptr);
    Sampler expected_sampler(0), host_sampler(0), device_sampler(0);
    expected_sampler.set_step_function(&oracle_step_adapter);
    const Generation want = generate(expected_sampler, false);
    const Generation got_host = generate(host_sampler, false);
    const Generation got_dev = generate(device_sampler, true);
    CHECK(want.ids.size() == 8);
    // the three-sequence request forked twice; its sequences differ and every one of them equals the expected stream
    CHECK(want.fork_ids.size() == 2 && got_host.fork_ids == want.fork_ids && got_dev.fork_ids == want.fork_ids);
    CHECK(want.fork_ids.size() == 2 && (want.fork_ids[0] != want.ids[6] || want.fork_ids[1] != want.ids[6]));
    // the grammar's request only produced allowed ids
    for (int64_t id : got_dev.ids[7]) CHECK(id % 3 == 0);
    for (size_t i = 0; i < want.ids.size(); ++i) {
        CHECK(!want.ids[i].empty());
        CHECK(want.ids[i] == got_host.ids[i]);
        CHECK(want.ids[i] == got_dev.ids[i]);
        CHECK(want.reasons[i] == got_host.reasons[i] && want.reasons[i] == got_dev.reasons[i]);
        for (size_t k = 0; k < want.lps[i].size() && k < got_host.lps[i].size() && k < got_dev.lps[i].size(); ++k) {
            CHECK(std::fabs(want.lps[i][k] - got_host.lps[i][k]) <= 1e-5f * std::max(1.f, std::fabs(want.lps[i][k])));
            CHECK(got_host.lps[i][k] == got_dev.lps[i][k]);
        }
        std::printf("request %zu: %zu tokens, reason %d, first ids %lld %lld\n", i, want.ids[i].size(), want.reasons[i],
                    (long long)want.ids[i][0], (long long)(want.ids[i].size() > 1 ? want.ids[i][1] : -1));
    }
    // the length-limited request stops at 7 tokens or earlier on a stop token after the masked steps
    CHECK(want.ids[4].size() <= 7 && want.ids[4].size() >= 3);
}

int main(int argc, char** argv) {
    if (argc < 3) { std::printf("usage: host_layer_test cpu <rotation fixture> | gpu <oracle library>\n"); return 2; }
    const std::string mode = argv[1];
    try {
        if (mode == "cpu") {
            test_generation_config();
            test_attention_inputs();
            test_rotation_lut(argv[2]);
        } else if (mode == "gpu") {
            test_sampler_pack();
            std::printf("pack: %d checks, %d failed\n", g_checks, g_failed);
            test_sampler_gpu(argv[2]);
        } else {
            return 2;
        }
    } catch (const std::exception& e) {
        std::printf("EXCEPTION %s\n", e.what());
        return 1;
    }
    std::printf("%s: %d checks, %d failed\n", mode.c_str(), g_checks, g_failed);
    return g_failed ? 1 : 0;
}
