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
    uint32_t* status;  // bit 0: history id out of range, bit 1: logits_row out of range, bit 2: raw log-prob without scratch
    float* hist_raw;   // raw logits of the history entries (rows that report raw log-probabilities), may be null
};

cudaError_t launch_sampler(const StepArgs& a, cudaStream_t stream);
size_t sampler_smem_bytes();

}  // namespace sampler
