// TEST INFRASTRUCTURE.  C entry points over the reference's own CacheEvictionAlgorithm,
// SnapKVScoreAggregationCalculator and CacheRotationCalculator, compiled unmodified from
//   src/cpp/src/continuous_batching/cache/cache_eviction.cpp
//   src/cpp/src/continuous_batching/cache/kvcrush.cpp
// behind oracle/ref_shim/eviction.  The tests feed it the score vectors the CUDA operator and the
// CPU restatement produce and compare the sets of logical blocks the reference would evict.
#include <cstdint>
#include <cstring>
#include <set>
#include <vector>

#include "continuous_batching/cache/cache_eviction.hpp"

using namespace ov::genai;

extern "C" {

// One sequence, one decoder layer: registers `num_steps` score vectors (step i has lens[i] floats,
// concatenated in `scores`, with snapkv[i] aggregated SnapKV rows) and returns the logical blocks
// evict_logical_blocks() selects after the last one.  aggregation: 0 = SUM, 1 = NORM_SUM.
// Returns the number of evicted blocks written to `out_blocks` (at most `cap`), or -1 on an
// exception (message in `err`).
int ref_eviction_select(int start_size, int recent_size, int max_cache_size, int aggregation, int snapkv_window, int block_size,
                        int max_pool_window, const float* scores, const int64_t* lens, const int32_t* snapkv, int num_steps,
                        int32_t* out_blocks, int cap, char* err, int err_cap) {
    try {
        CacheEvictionConfig cfg(start_size, recent_size, max_cache_size, aggregation == 0 ? AggregationMode::SUM : AggregationMode::NORM_SUM,
                                /*apply_rotation=*/false, snapkv_window);
        CacheEvictionAlgorithm algo(cfg, block_size, /*num_decoder_layers=*/1, max_pool_window);
        size_t off = 0;
        std::vector<std::set<size_t>> evicted;
        for (int i = 0; i < num_steps; ++i) {
            ov::Tensor t(ov::element::f32, ov::Shape{(size_t)lens[i]});
            std::memcpy(t.data<float>(), scores + off, (size_t)lens[i] * sizeof(float));
            off += (size_t)lens[i];
            AttentionScoresForEachDecoderLayer layers{t};
            algo.register_new_token_scores(layers, (size_t)snapkv[i]);
        }
        evicted = algo.evict_logical_blocks();
        int n = 0;
        for (size_t b : evicted.at(0)) {
            if (n < cap) out_blocks[n] = (int32_t)b;
            ++n;
        }
        return n;
    } catch (const std::exception& e) {
        if (err && err_cap > 0) { std::strncpy(err, e.what(), err_cap - 1); err[err_cap - 1] = 0; }
        return -1;
    }
}

// The same algorithm kept alive over several steps (one sequence, one layer): register a step's scores,
// evict, register more ... as the pipeline does (pipeline_impl.cpp:884-959).
void* ref_eviction_new(int start_size, int recent_size, int max_cache_size, int aggregation, int snapkv_window, int block_size, int max_pool_window) {
    try {
        CacheEvictionConfig cfg(start_size, recent_size, max_cache_size, aggregation == 0 ? AggregationMode::SUM : AggregationMode::NORM_SUM,
                                /*apply_rotation=*/false, snapkv_window);
        return new CacheEvictionAlgorithm(cfg, block_size, /*num_decoder_layers=*/1, max_pool_window);
    } catch (const std::exception&) {
        return nullptr;
    }
}
void ref_eviction_free(void* h) { delete static_cast<CacheEvictionAlgorithm*>(h); }
int ref_eviction_register(void* h, const float* scores, int64_t len, int snapkv, char* err, int err_cap) {
    try {
        ov::Tensor t(ov::element::f32, ov::Shape{(size_t)len});
        std::memcpy(t.data<float>(), scores, (size_t)len * sizeof(float));
        AttentionScoresForEachDecoderLayer layers{t};
        static_cast<CacheEvictionAlgorithm*>(h)->register_new_token_scores(layers, (size_t)snapkv);
        return 0;
    } catch (const std::exception& e) {
        if (err && err_cap > 0) { std::strncpy(err, e.what(), err_cap - 1); err[err_cap - 1] = 0; }
        return -1;
    }
}
int ref_eviction_evict(void* h, int32_t* out_blocks, int cap, char* err, int err_cap) {
    try {
        auto evicted = static_cast<CacheEvictionAlgorithm*>(h)->evict_logical_blocks();
        int n = 0;
        for (size_t b : evicted.at(0)) {
            if (n < cap) out_blocks[n] = (int32_t)b;
            ++n;
        }
        return n;
    } catch (const std::exception& e) {
        if (err && err_cap > 0) { std::strncpy(err, e.what(), err_cap - 1); err[err_cap - 1] = 0; }
        return -1;
    }
}

// SnapKVScoreAggregationCalculator::get_num_token_scores_to_aggregate
int ref_snapkv_window(int snapkv_window_size, int prompt_len, int num_processed, int num_scheduled) {
    SnapKVScoreAggregationCalculator calc(snapkv_window_size);
    return (int)calc.get_num_token_scores_to_aggregate(prompt_len, num_scheduled, num_processed);
}

// CacheRotationCalculator LUT rows: out_cos / out_sin are [rows][head / 2]
int ref_rotation_lut(int block_size, int rows, int head_size, double theta, float* out_cos, float* out_sin) {
    CacheRotationCalculator calc(block_size, rows, head_size, theta);
    const auto& c = calc.get_cos_lut();
    const auto& s = calc.get_sin_lut();
    for (int i = 0; i < rows; ++i)
        for (int j = 0; j < head_size / 2; ++j) {
            out_cos[i * (head_size / 2) + j] = c[i][j];
            out_sin[i * (head_size / 2) + j] = s[i][j];
        }
    return 0;
}

}  // extern "C"
