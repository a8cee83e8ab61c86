// Internal launch interface between the C ABI (pa_api.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "pa_common.cuh"

namespace pa {

// Rows of one prefill work item: (new token, q head of one GQA group) pairs of one kv head.
constexpr int kPrefillItemRows = 256;

// Header of the plan area in the handle's scratch.
struct PlanHeader {
    int total_tiles;   // 32-token tiles of all decode streams (rows x head tiles)
    int total_ptiles;  // kPrefillItemRows-row q tiles of all prefill chunks (per kv head)
    int next_pitem;    // work counter of the prefill kernel: next (q tile, kv head) item to hand out
    int pitems_sorted; // 1: pitem_order lists the q tiles by decreasing context length
};

constexpr int kPrefillSortCap = 2048;  // q tiles (per kv head) up to which the plan step orders them

// Where a decode worker's slice of the global tile sequence starts, prepared by the plan step so
// that the worker's first load is one 32-byte record instead of a binary search.
struct __align__(16) WorkerStart {
    int s;            // decode row that holds the slice's first tile; -1: not prepared, search
    int p0;           // tile_prefix[s]
    int r_tiles;      // tiles of row s (per head tile)
    int total_tiles;  // of the step, all streams
    int ctx;          // past_lens[s] + 1
    int tb, nb;       // block table of the row: begin and length
    int t0;           // row of the token in query / output
};

constexpr int kDecodeMinSlice = 4;   // a worker is given at least this many tiles
constexpr int kDecodeSharedPhantom = 12;    // SM-shared decode: what one more stream in a CTA's slice costs, in tiles

// The slices of the global tile sequence: worker w (a warp of decode_kernel, a CTA of decode_shared_kernel) takes the
// w-th of equal slices; small steps use fewer workers, so that every slice has at least kDecodeMinSlice tiles.
struct DecodeSlices {
    int workers1, per1;   // workers [0, workers1), per1 tiles each
    int total;
    __host__ __device__ long long begin(int w) const {
        const long long b = (long long)w * per1;
        return b < total ? b : total;
    }
    __host__ __device__ long long end(int w) const {
        if (w >= workers1) return total;
        const long long e = begin(w) + per1;
        return e < total ? e : total;
    }
    __host__ __device__ int worker_of(long long tile) const { return (int)(tile / per1); }   // tile < total
};
__host__ __device__ inline DecodeSlices decode_slices(int total_tiles, int all_workers) {
    DecodeSlices d{1, 1, total_tiles};
    const int want = (total_tiles + kDecodeMinSlice - 1) / kDecodeMinSlice;
    d.workers1 = all_workers < want ? all_workers : want;
    if (d.workers1 < 1) d.workers1 = 1;
    d.per1 = (total_tiles + d.workers1 - 1) / d.workers1;
    if (d.per1 < 1) d.per1 = 1;
    return d;
}

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
    int num_block_indices;
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
    // Decode plan.  A "stream" is (decode row, head tile); row s has tile_prefix[s+1] - tile_prefix[s]
    // tiles of 32 context tokens per head tile.  The global tile sequence is row-major, then head
    // tile, then position; worker w processes its w-th equal slice.
    PlanHeader* plan;      // decode plan header
    int* tile_prefix;      // [num_sequences + 1] exclusive prefix sum of tiles per row (one head tile)
    int* stream_done;      // [num_sequences * HK] partials of the stream published so far
    int* ptile_prefix;     // [num_sequences + 1] exclusive prefix sum of prefill q tiles per row (one kv head)
    int* pitem_order;      // [kPrefillSortCap] q tiles, longest context first (valid when plan->pitems_sorted); may be null
    int decode_all_workers;      // workers (warps of decode_kernel, CTAs of decode_shared_kernel) the decode launch will have (0: the plan prepares no start records)
    int decode_phantom;          // tiles added to every stream in the sequence the slices are cut in (SM-shared decode: a stream costs a CTA time beyond its tiles)
    int test_drop_copy;          // test hook: worker 0 issues no copy for its first tile and polls 2^10 times only
    WorkerStart* worker_start;   // [decode_all_workers], may be null
    long long max_tiles;   // upper bound of total_tiles known on the host
    int rows_per_tile;     // q heads per head tile: min(G, 16)
    float* part_o;         // partial outputs    [slot = stream + worker][rows_per_tile][D]
    float* part_ml;        // partial (max, sum) [slot][rows_per_tile][2]
    uint8_t* cta_q;        // SM-shared decode: staged query rows of the runs of each CTA
    float* lse;            // log-sum-exp per (token, q head), natural log, of the scaled logits
    int64_t* score_offsets;// [num_sequences + 1] prefix sum of past_len + new tokens
    int* stile_prefix;     // [num_sequences + 1] prefix sum of key tiles of the sequences that want scores
    float* score_part;     // [Hkv][scores_len] per-kv-head column sums of the window probabilities
    float* score_raw;      // [head tiles][scores_len][8 or 16] scaled logits (base 2) the decode kernel leaves for rows
                           // with one new token and a non-zero window (8 slots per head tile when the GQA group has at
                           // most 8 heads); null: every sequence goes through the score kernel
    long long scores_len;
};

// Device-side marshalling of the operator's inputs (pa_marshal.cu); all pointers are device memory.
struct MarshalArgs {
    const int32_t* block_table;          // [num_slots][table_stride] physical ids in logical order
    const int32_t* block_table_len;      // [num_slots]
    int table_stride, num_slots;
    const int32_t* slot;                 // [B] table row of every scheduled sequence (null: row s)
    const int32_t* num_processed_tokens; // [B]
    const int32_t* num_evicted_tokens;   // [B] or null
    const int32_t* num_scheduled_tokens; // [B]
    const uint32_t* skip_mask;           // [B][skip_words] bit j: logical block j is hidden this step; or null
    int skip_words;
    int num_sequences, block_size;
    int32_t* past_lens;                  // [B]
    int32_t* subsequence_begins;         // [B + 1]
    int32_t* block_indices;              // [block_indices_capacity]
    int32_t* block_indices_begins;       // [B + 1]
    int32_t* totals;                     // [3] num_tokens, num_block_indices, max_context_len
    int block_indices_capacity;
    uint32_t* status;
};
cudaError_t launch_marshal(const MarshalArgs& a, cudaStream_t stream, int* launches);

// Writes the chunk's new keys / values into the paged cache and, in the same launch, builds the
// decode plan (chunk list, zeroed counters) when `with_plan` is set.
cudaError_t launch_write_kv(const KernelArgs& a, cudaStream_t stream, bool with_plan);
cudaError_t launch_rotate(const KernelArgs& a, cudaStream_t stream);
cudaError_t launch_copy_blocks(void* key_cache, void* value_cache, long long block_bytes, int num_blocks,
                               const int32_t* pairs, int num_pairs, uint32_t* status, cudaStream_t stream);

// Attention over rows with exactly one new token (decode rows): one persistent launch that walks
// the plan's work queue.  Rows with more than one new token are not in the plan.
// When ev0/ev1 are given they are recorded immediately before / after the kernel.
cudaError_t launch_decode(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0 = nullptr,
                          cudaEvent_t ev1 = nullptr);

// Upper bound of the decode kernel's worker (warp) count, for sizing the partial-result scratch.
int decode_max_workers(int sm_count);
// Warps the decode launch of this step will have (the plan step prepares one start record each); *first_workers
// receives those of the first wave.
int decode_launch_workers(const KernelArgs& a, int sm_count);
// SM-shared decode (pa_decode_shared.cu): one CTA per SM whose warps take tiles from a shared counter
bool decode_shared_supported(const CacheGeom& g);
size_t decode_shared_scratch_bytes(int sm_count);
int decode_shared_chapter_tiles(const CacheGeom& g);   // tiles a CTA stages block ids for at a time
int decode_shared_max_chapters();   // PA_B200_DECODE_SHARED_CHAPTERS, default 2: longer slices go to the warp-per-slice kernel
int decode_shared_phantom();   // PA_B200_DECODE_PHANTOM, default kDecodeSharedPhantom
int decode_shared_ctas(const KernelArgs& a, int sm_count);
cudaError_t launch_decode_shared(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches, cudaEvent_t ev0 = nullptr,
                                 cudaEvent_t ev1 = nullptr);

// Attention over rows with more than one new token (prefill chunks): generic CUDA-core kernel.
cudaError_t launch_prefill(const KernelArgs& a, cudaStream_t stream, int* launches);

// The same on tcgen05 / TMEM for the shapes it supports (u8 cache, head size 128); walks the
// plan's q-tile list.  `max_items` is the host's upper bound of q tiles x kv heads.
bool prefill_tc_supported(const CacheGeom& g);
// f16 / bf16 caches: mma.sync kernel over the same work items (pa_prefill_mma.cu)
bool prefill_mma_supported(const CacheGeom& g);
cudaError_t launch_prefill_mma(const KernelArgs& a, cudaStream_t stream, long long max_items, int* launches);
cudaError_t launch_prefill_tc(const KernelArgs& a, cudaStream_t stream, int sm_count, long long max_items, int* launches);

// SnapKV-style score output: scores[pos] = sum over q heads and the last W rows of each chunk of
// the softmax probabilities, using the log-sum-exp the attention kernels exported.
cudaError_t launch_scores(const KernelArgs& a, cudaStream_t stream, int sm_count, int* launches);

constexpr int kScoreTile = 32;   // keys per tile of the score kernel

#ifdef __CUDACC__
// One sequence's slice of the scheduler metadata, checked before anything is indexed with it:
// 0 <= begins[s] <= begins[s + 1] <= the array it indexes, past_len >= 0 and a block table long
// enough for past_len + new tokens.  A sequence that fails sets PA_DEV_BAD_BEGINS or
// PA_DEV_BAD_PAST_LEN and is given no work (n = 0): nothing is read or written through its numbers.
struct SeqView {
    int t0, n;      // rows of the sequence in query / key / value / output
    int past;
    int tb, nb;     // its block table inside block_indices
};
__device__ __forceinline__ bool seq_view(const KernelArgs& a, int s, SeqView& v) {
    const int t0 = a.subsequence_begins[s], t1 = a.subsequence_begins[s + 1];
    const int tb = a.block_indices_begins[s], te = a.block_indices_begins[s + 1];
    const int past = a.past_lens[s];
    v = SeqView{0, 0, 0, 0, 0};
    if (t0 < 0 || t1 < t0 || t1 > a.num_tokens || tb < 0 || te < tb || te > a.num_block_indices) {
        atomicOr(a.status, PA_DEV_BAD_BEGINS);
        return false;
    }
    if (past < 0 || (long long)(te - tb) * a.g.bs < (long long)past + (t1 - t0)) {
        atomicOr(a.status, PA_DEV_BAD_PAST_LEN);
        return false;
    }
    v = SeqView{t0, t1 - t0, past, tb, te - tb};
    return true;
}

// Per-sequence offsets into `scores` (prefix sum of past_len + new tokens) and the prefix sum of the
// score kernel's work (key tiles x row tiles) over the sequences it serves.  Run by one warp of the
// cache-write launch, because the decode kernel needs the offsets to leave its logits behind.
__device__ inline void build_score_plan(const KernelArgs& a) {
    long long run = 0;
    int run_t = 0;
    const int lane = threadIdx.x & 31;
    for (int base = 0; base < a.num_sequences; base += 32) {
        const int s = base + lane;
        long long len = 0;
        int tiles = 0;
        if (s < a.num_sequences) {
            SeqView sv;
            const bool valid = seq_view(a, s, sv);
            const int n = sv.n, past = sv.past;
            // an invalid sequence still takes the slot its raw numbers describe, so that the offsets of the
            // sequences after it stay where the caller expects them
            len = valid ? (long long)past + n
                        : (long long)max(a.past_lens[s], 0) + max(a.subsequence_begins[s + 1] - a.subsequence_begins[s], 0);
            const bool ok = valid && n > 0;
            // cost of a sequence: key tiles x 16-row tiles of (window row, q head of the group) pairs
            const int W = ok ? min(max(a.score_aggregation_window[s], 0), n) : 0;
            const int G = a.g.Hq / a.g.Hkv;
            // rows with one new token are served from the logits the decode kernel left in score_raw
            const bool from_decode = a.score_raw != nullptr && n == 1;
            if (W > 0 && !from_decode) tiles = (int)((len + kScoreTile - 1) / kScoreTile) * ((W * G + 15) / 16);
        }
        long long incl = len;
        int incl_t = tiles;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long v = __shfl_up_sync(0xffffffffu, incl, o);
            const int vt = __shfl_up_sync(0xffffffffu, incl_t, o);
            if (lane >= o) { incl += v; incl_t += vt; }
        }
        if (s < a.num_sequences) { a.score_offsets[s] = run + incl - len; a.stile_prefix[s] = run_t + incl_t - tiles; }
        run += __shfl_sync(0xffffffffu, incl, 31);
        run_t += __shfl_sync(0xffffffffu, incl_t, 31);
    }
    if (lane == 0) { a.score_offsets[a.num_sequences] = run; a.stile_prefix[a.num_sequences] = run_t; }
}
#endif

}  // namespace pa
