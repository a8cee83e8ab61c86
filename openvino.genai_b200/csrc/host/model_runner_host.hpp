// Host marshalling around the PagedAttention operator, mirroring what
// ov::genai::ModelRunner::forward hands to the operator each step
// (src/cpp/src/continuous_batching/model_runner.hpp:462-1012): the per-sequence tensors
// (past_lens, subsequence_begins, block_indices, block_indices_begins, max_context_len,
// score_aggregation_window), the rotation inputs in ascending seq_id order (1483-1509), the slicing
// of the score output back into per-sequence spans (1518-1568) and the rotation LUT
// (pipeline_impl.cpp:256-287 over cache/cache_eviction.cpp:543-573).  Header-only, no device code.
#pragma once

#include <cmath>
#include <cstdint>
#include <map>
#include <optional>
#include <set>
#include <stdexcept>
#include <utility>
#include <vector>

namespace genai_b200 {

// One running sequence of the scheduler's output for this step.
struct ScheduledSequence {
    uint64_t seq_id = 0;
    size_t num_processed_tokens = 0;     // tokens of the sequence already in the cache before this step
    size_t num_evicted_tokens = 0;       // tokens the eviction algorithm removed from the cache so far
    size_t num_scheduled_tokens = 0;     // new tokens of this step
    std::vector<int32_t> block_table;    // physical block ids in logical order, slots of the new tokens included
    std::set<size_t> skipped_logical_blocks;             // blocks a sparse-attention mask hides from this step
    std::optional<size_t> score_aggregation_window;      // set by the scheduler once the SnapKV window is reached
    bool can_generate_tokens = false;                    // the prompt has been processed completely
};

struct AttentionInputs {
    std::vector<int32_t> past_lens;              // [B]
    std::vector<int32_t> subsequence_begins;     // [B + 1]
    std::vector<int32_t> block_indices;          // [sum of used blocks]
    std::vector<int32_t> block_indices_begins;   // [B + 1]
    std::vector<int32_t> score_aggregation_window;   // [B], empty when scores are not aggregated
    int32_t max_context_len = 0;
    int32_t num_tokens = 0;
};

// model_runner.hpp:802-856 for the per-sequence scalars, 1420-1481 for the block indices: a skipped
// logical block neither counts toward past_lens nor appears in block_indices.
inline AttentionInputs build_attention_inputs(const std::vector<ScheduledSequence>& seqs, size_t block_size, bool aggregate_attention_scores) {
    AttentionInputs in;
    in.subsequence_begins.push_back(0);
    in.block_indices_begins.push_back(0);
    for (const ScheduledSequence& s : seqs) {
        if (s.num_processed_tokens < s.num_evicted_tokens) throw std::invalid_argument("more evicted than processed tokens");
        const size_t expected_kv_cache_size = s.num_processed_tokens - s.num_evicted_tokens;
        const size_t num_blocks = s.block_table.size();
        const size_t ignored = s.skipped_logical_blocks.size();
        if (num_blocks < ignored) throw std::invalid_argument("more skipped blocks than blocks");
        if (expected_kv_cache_size < ignored * block_size) throw std::invalid_argument("skipped blocks exceed the cache occupancy");
        in.past_lens.push_back((int32_t)(expected_kv_cache_size - ignored * block_size));
        in.subsequence_begins.push_back(in.subsequence_begins.back() + (int32_t)s.num_scheduled_tokens);
        in.block_indices_begins.push_back(in.block_indices_begins.back() + (int32_t)(num_blocks - ignored));
        for (size_t j = 0; j < num_blocks; ++j)
            if (!s.skipped_logical_blocks.count(j)) in.block_indices.push_back(s.block_table[j]);
        if (aggregate_attention_scores) in.score_aggregation_window.push_back(s.score_aggregation_window ? (int32_t)*s.score_aggregation_window : 1);
        const size_t context = s.num_processed_tokens + s.num_scheduled_tokens;   // model_runner.hpp:497,533
        if ((int32_t)context > in.max_context_len) in.max_context_len = (int32_t)context;
    }
    in.num_tokens = in.subsequence_begins.back();
    return in;
}

struct RotationInputs {
    std::vector<int32_t> rotated_block_indices;   // physical ids
    std::vector<int32_t> rotation_deltas;         // LUT rows, one per rotated block
};

// `rotated` maps seq_id -> (logical block index, LUT row) in the order the eviction algorithm
// produced them; the physical ids are emitted sequence by sequence in ascending seq_id, the order
// in which the deltas are filled (model_runner.hpp:1503-1505).
inline RotationInputs build_rotation_inputs(const std::map<uint64_t, std::vector<std::pair<size_t, int32_t>>>& rotated,
                                            const std::vector<ScheduledSequence>& seqs) {
    std::map<uint64_t, const ScheduledSequence*> by_id;
    for (const ScheduledSequence& s : seqs) by_id[s.seq_id] = &s;
    RotationInputs out;
    for (const auto& entry : rotated) {   // std::map iterates in ascending seq_id
        auto it = by_id.find(entry.first);
        if (it == by_id.end()) throw std::invalid_argument("rotation data for a sequence that is not scheduled");
        for (const auto& lb : entry.second) {
            if (lb.first >= it->second->block_table.size()) throw std::invalid_argument("rotated logical block outside the block table");
            out.rotated_block_indices.push_back(it->second->block_table[lb.first]);
            out.rotation_deltas.push_back(lb.second);
        }
    }
    return out;
}

struct ScoreSpan {
    size_t begin = 0, end = 0;   // [begin, end) inside the operator's score output
};

// model_runner.hpp:1518-1568: every scheduled sequence owns a slot of
// context_len - evicted - skipped * block_size floats; only sequences whose prompt is finished, or
// that have a SnapKV window this step, hand their span to the eviction algorithm.
inline std::map<uint64_t, ScoreSpan> collect_attention_scores(const std::vector<ScheduledSequence>& seqs, size_t block_size) {
    std::map<uint64_t, ScoreSpan> spans;
    size_t offset = 0;
    for (const ScheduledSequence& s : seqs) {
        const size_t context_len = s.num_processed_tokens + s.num_scheduled_tokens;
        const size_t len = context_len - s.num_evicted_tokens - s.skipped_logical_blocks.size() * block_size;
        if (s.can_generate_tokens || s.score_aggregation_window.has_value()) spans[s.seq_id] = ScoreSpan{offset, offset + len};
        offset += len;
    }
    return spans;
}

// Row i: cos(i * block_size * theta_j) for j < head/2, then -sin(i * block_size * theta_j), with
// theta_j = rope_theta^(-2j / head): the rotate-half layout of the model_rotation_trig_lut input.
inline std::vector<float> make_rotation_trig_lut(size_t rows, size_t block_size, size_t head_size, double rope_theta = 10000.0) {
    if (!(rope_theta > 0)) throw std::invalid_argument("rope_theta must be positive");
    std::vector<float> lut(rows * head_size, 0.f);
    const size_t num_freqs = head_size / 2;
    for (size_t i = 0; i < rows; ++i)
        for (size_t j = 0; j < num_freqs; ++j) {
            const double exponent = -static_cast<double>(2 * j) / head_size;
            const double base_angle = std::pow(rope_theta, exponent);
            lut[i * head_size + j] = (float)std::cos(i * block_size * base_angle);
            lut[i * head_size + num_freqs + j] = (float)-std::sin(i * block_size * base_angle);
        }
    return lut;
}

}  // namespace genai_b200
