// Internal launch interface between the sampler C ABI (sampler_api.cu) and the kernel.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sampler_b200.h"

namespace sampler {

// Kernel arguments, passed by value.  All pointers are device memory.
struct StepArgs {
    float* logits;
    long long num_logit_rows;
    long long vocab;
    int num_rows;
    const sampler_row_params* rows;
    const int64_t* hist_offsets;
    const int32_t* hist_ids;
    const uint32_t* hist_meta;
    int64_t* out_token;
    float* out_log_prob;
    uint32_t* status;  // bit 0: history id out of range, bit 1: logits_row out of range, bit 2: raw log-prob without scratch,
                       // bit 3: top_k above the heap capacity (and below the vocabulary), bit 4: the sorted walk did not end
    float* hist_raw;   // raw logits of the history entries (rows that report raw log-probabilities), may be null
    // further draws of a row (all null: none): CSR offsets, their uniform numbers, their outputs
    const int64_t* extra_offsets;
    const float* extra_rand_u;
    int64_t* extra_out_token;
    float* extra_out_log_prob;
    // grammar bitmasks (both null: none)
    const int32_t* token_bitmasks;
    const int32_t* bitmask_index;
    long long bitmask_words;
};

cudaError_t launch_sampler(const StepArgs& a, cudaStream_t stream);
size_t sampler_smem_bytes();

// Full-vocabulary multinomial rows (sampler_exact.cu).  `scratch` holds one row of probabilities per
// CTA of the persistent grid: sampler_exact_scratch_bytes(ctas, vocab) bytes.
cudaError_t launch_sampler_exact(const StepArgs& a, float* scratch, int ctas, cudaStream_t stream);
size_t sampler_exact_scratch_bytes(int ctas, long long vocab);
size_t sampler_exact_smem_bytes();
cudaError_t launch_expf_selftest(const float* in, float* out, long long n, cudaStream_t stream);
constexpr int kSamplerMaxTopK = 1024;   // heap capacity of the top-k path

}  // namespace sampler
