// Internal launch interface between the C ABI (pa_api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "pa_common.cuh"

namespace pa {

// Everything a kernel needs, passed by value.  All pointers are device memory.
struct KernelArgs {
    CacheGeom g;
    const void* query;
    const void* key;
    const void* value;
    void* output;
    int num_tokens;
    void* key_cache;
    void* value_cache;
    int num_blocks;
    const int32_t* past_lens;
    const int32_t* subsequence_begins;
    const int32_t* block_indices;
    const int32_t* block_indices_begins;
    int num_sequences;
    int max_context_len;
    float scale;
    const int32_t* score_aggregation_window;
    float* scores;
    const int32_t* rotated_block_indices;
    const int32_t* rotation_deltas;
    int num_rotated_blocks;
    const float* rotation_trig_lut;
    int rotation_lut_rows;
    uint32_t* status;      // device status word (PA_DEV_* bits)
    // scratch owned by the handle
    float* part_o;         // split partial outputs  [item][split][G][D]
    float* part_ml;        // split partial (max, sum) [item][split][G][2]
    float* lse;            // log-sum-exp per (token, q head), natural log, of the scaled logits
    float* score_part;     // per kv-head score partials [Hkv][scores_len]
    int64_t* score_offsets;// [num_sequences + 1] prefix sum of past_len + new tokens
    int split_tokens;      // context tokens handled by one decode CTA
    int max_splits;        // ceil(max_context_len / split_tokens)
    long long scores_len;
};

cudaError_t launch_write_kv(const KernelArgs& a, cudaStream_t stream);
cudaError_t launch_rotate(const KernelArgs& a, cudaStream_t stream);
cudaError_t launch_copy_blocks(void* key_cache, void* value_cache, long long block_bytes, int num_blocks,
                               const int32_t* pairs, int num_pairs, uint32_t* status, cudaStream_t stream);

// Attention over rows with exactly one new token (decode rows).  Launches the split-K kernel and
// the merge kernel.  Rows with more than one new token are skipped by these kernels.
cudaError_t launch_decode(const KernelArgs& a, cudaStream_t stream, int* launches);
size_t decode_smem_bytes(const CacheGeom& g);

// Attention over rows with more than one new token (prefill chunks).
cudaError_t launch_prefill(const KernelArgs& a, cudaStream_t stream, int* launches);

// SnapKV-style score output: scores[pos] = sum over q heads and the last W rows of each chunk of
// the softmax probabilities, using the log-sum-exp the attention kernels exported.
cudaError_t launch_scores(const KernelArgs& a, cudaStream_t stream, int* launches);

}  // namespace pa
