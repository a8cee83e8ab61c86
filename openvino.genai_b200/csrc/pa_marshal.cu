// Device-side input marshalling: turns device-resident per-sequence block tables plus this step's
// schedule into the operator's tensors (past_lens, subsequence_begins, block_indices,
// block_indices_begins, max_context_len), i.e. what ModelRunner::forward builds on the host every step
// by walking std::maps per layer, group and block
// (src/cpp/src/continuous_batching/model_runner.hpp:802-856, 1316-1380, 1420-1481):
//   past_lens[s]            = processed - evicted - skipped blocks * block_size
//   subsequence_begins      = prefix sum of the scheduled tokens
//   block_indices           = every sequence's table in logical order without its skipped blocks
//   block_indices_begins    = prefix sum of the used blocks
//   max_context_len         = max over sequences of processed + scheduled
// Two launches: one block plans (validation, counts, prefix sums), a grid copies the block ids.
// Integer work, bound by the ids it moves (4 bytes read + 4 bytes written per used block).
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kPlanThreads = 1024;
constexpr int kFillChunk = 1024;   // logical blocks per CTA of the copy

__device__ __forceinline__ int skipped_below(const uint32_t* mask, int words, int upto) {   // set bits among logical blocks [0, upto)
    int n = 0;
    const int full = min(upto >> 5, words);
    for (int w = 0; w < full; ++w) n += __popc(mask[w]);
    if ((upto & 31) && full < words) n += __popc(mask[full] & ((1u << (upto & 31)) - 1u));
    return n;
}

__global__ void __launch_bounds__(kPlanThreads) marshal_plan_kernel(MarshalArgs a) {
    __shared__ int sh_tok[32], sh_blk[32], sh_max[32];
    __shared__ int run_tok, run_blk, run_max;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { run_tok = 0; run_blk = 0; run_max = 0; }
    __syncthreads();
    for (int base = 0; base < a.num_sequences; base += kPlanThreads) {
        const int s = base + tid;
        int n_tok = 0, n_blk = 0, ctx = 0, past = 0;
        if (s < a.num_sequences) {
            const int slot = a.slot ? a.slot[s] : s;
            const int processed = a.num_processed_tokens[s];
            const int evicted = a.num_evicted_tokens ? a.num_evicted_tokens[s] : 0;
            const int scheduled = a.num_scheduled_tokens[s];
            bool ok = slot >= 0 && slot < a.num_slots && processed >= 0 && evicted >= 0 && scheduled >= 0 && processed >= evicted;
            int len = 0, skipped = 0;
            if (ok) {
                len = a.block_table_len[slot];
                ok = len >= 0 && len <= a.table_stride;
            }
            if (ok && a.skip_mask) skipped = skipped_below(a.skip_mask + (long long)s * a.skip_words, a.skip_words, len);
            // the host code asserts these (model_runner.hpp:1449, 808-816); here the sequence is flagged and given nothing
            if (ok) ok = (long long)processed - evicted >= (long long)skipped * a.block_size;
            if (!ok) {
                atomicOr(a.status, PA_DEV_BAD_BEGINS);
            } else {
                n_tok = scheduled;
                n_blk = len - skipped;
                past = processed - evicted - skipped * a.block_size;
                ctx = processed + scheduled;
            }
            a.past_lens[s] = past;
        }
        // block-wide inclusive scans of tokens and blocks, maximum of the contexts
        int it = n_tok, ib = n_blk, mx = ctx;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ut = __shfl_up_sync(0xffffffffu, it, o), ub = __shfl_up_sync(0xffffffffu, ib, o);
            if (lane >= o) { it += ut; ib += ub; }
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (lane == 31) { sh_tok[warp] = it; sh_blk[warp] = ib; }
        if (lane == 0) sh_max[warp] = mx;
        __syncthreads();
        int off_t = run_tok, off_b = run_blk;
        for (int w = 0; w < warp; ++w) { off_t += sh_tok[w]; off_b += sh_blk[w]; }
        if (s < a.num_sequences) {
            a.subsequence_begins[s] = off_t + it - n_tok;
            a.block_indices_begins[s] = off_b + ib - n_blk;
        }
        __syncthreads();
        if (tid == kPlanThreads - 1) {
            run_tok = off_t + it;
            run_blk = off_b + ib;
            int m = run_max;
            for (int w = 0; w < 32; ++w) m = max(m, sh_max[w]);
            run_max = m;
        }
        __syncthreads();
    }
    if (tid == 0) {
        a.subsequence_begins[a.num_sequences] = run_tok;
        a.block_indices_begins[a.num_sequences] = run_blk;
        a.totals[0] = run_tok;            // num_tokens
        a.totals[1] = run_blk;            // num_block_indices
        a.totals[2] = run_max;            // max_context_len
        if (run_blk > a.block_indices_capacity) atomicOr(a.status, PA_DEV_BAD_BEGINS);
    }
}

// grid (chunks of the longest table, sequences)
__global__ void __launch_bounds__(256) marshal_fill_kernel(MarshalArgs a) {
    const int s = blockIdx.y;
    const int first = blockIdx.x * kFillChunk;
    const int begin = a.block_indices_begins[s], used = a.block_indices_begins[s + 1] - begin;
    if (used <= 0) return;
    const int slot = a.slot ? a.slot[s] : s;
    const int len = a.block_table_len[slot];
    if (first >= len) return;
    const uint32_t* mask = a.skip_mask ? a.skip_mask + (long long)s * a.skip_words : nullptr;
    __shared__ int skipped_before_chunk;
    if (threadIdx.x == 0) skipped_before_chunk = mask ? skipped_below(mask, a.skip_words, first) : 0;
    __syncthreads();
    const int32_t* table = a.block_table + (long long)slot * a.table_stride;
    for (int j = first + threadIdx.x; j < min(len, first + kFillChunk); j += blockDim.x) {
        int rank = j - skipped_before_chunk;
        if (mask) {
            const uint32_t word = (j >> 5) < a.skip_words ? mask[j >> 5] : 0u;
            if ((word >> (j & 31)) & 1u) continue;
            // skipped blocks between the chunk start and j
            for (int w = first >> 5; w < (j >> 5); ++w) rank -= __popc(mask[w]);
            rank -= __popc(word & ((1u << (j & 31)) - 1u));
        }
        const long long dst = (long long)begin + rank;
        if (rank >= 0 && rank < used && dst < a.block_indices_capacity) a.block_indices[dst] = table[j];
    }
}

}  // namespace

cudaError_t launch_marshal(const MarshalArgs& a, cudaStream_t stream, int* launches) {
    if (a.num_sequences <= 0) return cudaSuccess;
    marshal_plan_kernel<<<1, kPlanThreads, 0, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const int chunks = (a.table_stride + kFillChunk - 1) / kFillChunk;
    if (chunks > 0) {
        marshal_fill_kernel<<<dim3(chunks, a.num_sequences), 256, 0, stream>>>(a);
        e = cudaGetLastError();
    }
    if (launches) *launches += chunks > 0 ? 2 : 1;
    return e;
}

}  // namespace pa
