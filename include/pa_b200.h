/*
 * pa_b200.h - C ABI of the B200 (sm_100a) PagedAttention operator.
 *
 * The entry points below are what an OpenVINO `ov::op::Op::evaluate()` shim (or the
 * ModelRunner itself) binds in place of the PagedAttentionExtension operator that the
 * reference inserts with ov::pass::SDPAToPagedAttention
 * (src/cpp/src/continuous_batching/pipeline_impl.cpp:73-92) and runs inside
 * ov::InferRequest::infer() (src/cpp/src/continuous_batching/model_runner.hpp:953).
 * Argument names and meaning follow the model-level tensors that ModelRunner::forward
 * fills (model_runner.hpp:505-522, 802-853, 1420-1509).
 *
 * Conventions
 *  - Plain C: pointers, sizes, integer status codes.  No exceptions cross this boundary.
 *  - The caller owns every buffer it passes.  The handle owns only its own scratch.
 *  - Device kernels never trap and never spin without a bound: a bad block index or a
 *    non-monotonic prefix sum sets a bit in a device status word and the offending row is
 *    skipped; pa_b200_last_device_status() reads the word.
 *  - One handle serves one engine thread (ContinuousBatchingImpl::step() is single
 *    threaded, pipeline_impl.cpp:378-533).  Calls on one handle are ordered on the
 *    handle's stream (or the stream passed in the args).
 */
#ifndef PA_B200_H
#define PA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PA_B200_ABI_VERSION 1

typedef enum pa_status {
    PA_OK = 0,
    PA_ERR_INVALID_ARG = 1,  /* NULL pointer, negative size, struct_size mismatch         */
    PA_ERR_UNSUPPORTED = 2,  /* sliding_window / alibi / unsupported head size or dtype   */
    PA_ERR_CUDA = 3,         /* a CUDA runtime call failed; see pa_b200_last_error()      */
    PA_ERR_BAD_INDEX = 4,    /* device status word reported an out-of-range block index   */
    PA_ERR_NO_DEVICE = 5,    /* no sm_100 device / library built without a usable kernel  */
    PA_ERR_TOO_LARGE = 6     /* request exceeds a stated fixed capacity                   */
} pa_status;

typedef enum pa_dtype {
    PA_DTYPE_F32 = 0,
    PA_DTYPE_F16 = 1,
    PA_DTYPE_BF16 = 2,
    PA_DTYPE_U8 = 3 /* cache only: by-token asymmetric u8, one (scale, zero-point) f32 pair per token per head */
} pa_dtype;

/* Bits of the device status word. */
#define PA_DEV_BAD_BLOCK_INDEX 0x1u   /* block_indices[i] outside [0, num_blocks)           */
#define PA_DEV_BAD_BEGINS 0x2u        /* subsequence_begins / block_indices_begins invalid  */
#define PA_DEV_BAD_PAST_LEN 0x4u      /* past_lens < 0 or block table too short             */
#define PA_DEV_BAD_ROTATION 0x8u      /* rotated block id or LUT row out of range           */
/* Every wait of a kernel on a copy it issued is bounded.  A wait that runs out sets one of the bits below and
 * the waiting warps leave (tensor memory freed, nothing left in flight); the step's output is then incomplete. */
#define PA_DEV_WAIT_TIMEOUT_SCORES 0x20000000u  /* score kernel: a staged key record never arrived             */
#define PA_DEV_WAIT_TIMEOUT_PREFILL 0x40000000u /* tcgen05 prefill kernel: a barrier wait ran out               */
#define PA_DEV_WAIT_TIMEOUT_DECODE 0x80000000u  /* decode kernel: a staged (block, head) record never arrived   */

/* Static attributes of one attention layer.  Replaces what KVCacheManager reads from the
 * compiled model's key_cache.N / value_cache.N ports
 * (src/cpp/src/continuous_batching/cache/kv_cache_manager.hpp:56-113). */
typedef struct pa_model_desc {
    uint32_t struct_size; /* sizeof(pa_model_desc) */
    int32_t num_q_heads;
    int32_t num_kv_heads;
    int32_t head_size;   /* 64 or 128 */
    int32_t block_size;  /* tokens per physical block: 16 or 32 */
    int32_t act_dtype;   /* pa_dtype of query/key/value/output: F16, BF16 or F32 */
    int32_t cache_dtype; /* pa_dtype of key_cache/value_cache: F16, BF16 or U8   */
} pa_model_desc;

/* What the caller's cache allocator must honour.  genai treats the cache as opaque bytes and
 * only copies whole blocks (kv_cache_manager.hpp:278-335), so the element order inside a block
 * is this library's choice:
 *   f16/bf16  key   [num_blocks][Hkv][block_size][D]
 *             value [num_blocks][Hkv][block_size][D]
 *   u8        key   [num_blocks][Hkv]{ u8 data[block_size][D], f32 scale[block_size], f32 zp[block_size] }
 *             value [num_blocks][Hkv]{ u8 data[D][block_size], f32 scale[block_size], f32 zp[block_size] }
 *             (value data is token-minor so that P.V contracts over contiguous bytes)
 * The declared 4-D shape for u8 is [num_blocks, Hkv, block_size, D + 8], same byte count. */
typedef struct pa_cache_layout {
    uint32_t struct_size;
    int32_t elem_dtype;          /* element type to declare on the port (F16, BF16, U8) */
    int64_t key_shape[4];        /* [0 (= any number of blocks), Hkv, block_size, D or D+8] */
    int64_t value_shape[4];
    int64_t key_block_bytes;     /* bytes of one physical block, all heads */
    int64_t value_block_bytes;
    int32_t base_alignment;      /* required alignment of the cache base pointers, bytes */
} pa_cache_layout;

/* One operator invocation (one layer, one step).  Field names = the reference's tensor names. */
typedef struct pa_forward_args {
    uint32_t struct_size; /* sizeof(pa_forward_args) */

    /* Activations, row-major [num_tokens, H*D], element type = pa_model_desc.act_dtype. */
    const void* query;  /* [num_tokens, Hq*D]  */
    const void* key;    /* [num_tokens, Hkv*D] new keys, written to the cache by this call   */
    const void* value;  /* [num_tokens, Hkv*D] new values                                    */
    void* output;       /* [num_tokens, Hq*D]  */
    int32_t num_tokens;

    /* Paged cache, device memory, layout per pa_b200_query_cache_layout(). */
    void* key_cache;
    void* value_cache;
    int32_t num_blocks; /* physical blocks in each cache tensor */

    /* Scheduler metadata (model_runner.hpp:509-516).  i32. */
    const int32_t* past_lens;            /* [num_sequences]     */
    const int32_t* subsequence_begins;   /* [num_sequences + 1] */
    const int32_t* block_indices;        /* [num_block_indices] */
    const int32_t* block_indices_begins; /* [num_sequences + 1] */
    int32_t num_sequences;
    int32_t num_block_indices;
    int32_t max_context_len;             /* max over sequences of past_len + new tokens */

    float scale;                         /* 0 => 1/sqrt(head_size) */
    int32_t sliding_window;              /* must be 0 (PA_ERR_UNSUPPORTED otherwise) */
    const float* alibi_slopes;           /* must be NULL */

    /* Eviction support (model_runner.hpp:838-848, 1483-1568).  All optional. */
    const int32_t* score_aggregation_window; /* [num_sequences] or NULL                       */
    float* scores;                           /* [sum_s (past_len_s + new_s)] or NULL          */
    int64_t scores_len;
    const int32_t* rotated_block_indices;    /* [num_rotated_blocks] physical ids or NULL     */
    const int32_t* rotation_deltas;          /* [num_rotated_blocks, 1] rows of the trig LUT  */
    int32_t num_rotated_blocks;
    const float* rotation_trig_lut;          /* [rotation_lut_rows, head_size] cos | -sin     */
    int32_t rotation_lut_rows;

    void* stream; /* cudaStream_t, NULL => the handle's stream */
} pa_forward_args;

typedef struct pa_handle pa_handle;

/* Library / device probing. */
int pa_b200_abi_version(void);
const char* pa_b200_last_error(void); /* thread-local text of the last PA_ERR_CUDA / INVALID_ARG */

/* Cache layout query: what KVCacheManager would read from the model ports
 * (kv_cache_manager.hpp:74-113). */
int pa_b200_query_cache_layout(const pa_model_desc* desc, pa_cache_layout* out);

/* Handle life cycle.  `device` is a CUDA ordinal.  The handle allocates its scratch with
 * cudaMalloc at creation and when a later call needs more (never inside a kernel). */
int pa_b200_create(const pa_model_desc* desc, int device, pa_handle** out);
int pa_b200_destroy(pa_handle* h);

/* Scratch bytes a forward call of this shape needs (split-K partials, score partials,
 * device copies of host metadata).  pa_b200_reserve() grows the handle's scratch to it so that
 * later calls of that shape do not allocate. */
int64_t pa_b200_workspace_bytes(const pa_handle* h, int32_t num_tokens, int32_t num_sequences,
                                int32_t max_context_len, int64_t scores_len);
int pa_b200_reserve(pa_handle* h, int32_t num_tokens, int32_t num_sequences, int32_t max_context_len,
                    int64_t scores_len, int32_t num_block_indices);

/* The operator: every pointer in `args` is DEVICE memory.  Asynchronous on the stream.
 * Replaces the PagedAttentionExtension node executed by infer() (model_runner.hpp:953). */
int pa_b200_forward(pa_handle* h, const pa_forward_args* args);

/* Same operator for a caller that holds HOST tensors, as ModelRunner does for everything
 * except the cache (model_runner.hpp:505-522 fills host ov::Tensors): query/key/value/output,
 * the metadata, the rotation inputs and `scores` are HOST pointers; key_cache/value_cache stay
 * device pointers.  Copies in, runs, copies out, synchronises, and returns PA_ERR_BAD_INDEX if
 * the device status word is non-zero. */
int pa_b200_forward_host(pa_handle* h, const pa_forward_args* args);

/* Reads (and clears) the device status word; synchronises the handle's stream. */
int pa_b200_last_device_status(pa_handle* h, uint32_t* status_bits);

/* Number of kernels this handle has launched since creation (for launch accounting). */
int64_t pa_b200_launch_count(const pa_handle* h);

/* Which kernel served the prefill chunks of the handle's last forward call (for tests and launch accounting): */
enum pa_prefill_kernel {
    PA_PREFILL_NONE = 0,     /* the step had no row with more than one new token */
    PA_PREFILL_GENERIC = 1,  /* CUDA cores, one warp per (token, q head) */
    PA_PREFILL_MMA_SYNC = 2, /* mma.sync m16n8k16 */
    PA_PREFILL_TCGEN05 = 3   /* tcgen05.mma with accumulators in tensor memory */
};
int pa_b200_last_prefill_kernel(const pa_handle* h);

/* Measurement support: while enabled, every forward call records a CUDA event pair around its
 * split-K decode kernel on the stream it launches on.  get_kernel_timing waits for the recorded
 * pairs, returns their summed duration and count, and clears them (at most 4096 pairs are kept). */
int pa_b200_set_kernel_timing(pa_handle* h, int enabled);
int pa_b200_get_kernel_timing(pa_handle* h, double* total_ms, int64_t* timed_launches);

/* Stand-alone cache operations used by the operator and by the cache manager.
 *  - write: scatter `num_tokens` new K/V rows into their slots (quantising for u8).
 *  - rotate: re-rotate the keys of the listed blocks in place (pipeline_impl.cpp:810-882).
 *  - copy_blocks: copy-on-write block copies (kv_cache_manager.hpp:278-335);
 *    src_dst_pairs is [num_pairs][2] i32 in device memory. */
int pa_b200_write_kv(pa_handle* h, const pa_forward_args* args);
int pa_b200_rotate_blocks(pa_handle* h, const pa_forward_args* args);
int pa_b200_copy_blocks(pa_handle* h, void* key_cache, void* value_cache, int32_t num_blocks,
                        const int32_t* src_dst_pairs, int32_t num_pairs, void* stream);

/* KV cache pool that grows in place.
 *
 * KVCacheManager::allocate_cache_if_needed grows a layer's cache by creating a larger tensor and copying all
 * blocks (src/cpp/src/continuous_batching/cache/kv_cache_manager.hpp:159-262): twice the memory while it
 * copies, and new tensor addresses to re-bind.  This pool reserves the address range of `max_blocks` once and
 * maps physical memory into it as it grows: key_cache / value_cache never move, written blocks keep their
 * bytes, nothing is copied, new blocks read as zeros.  One pool per layer (the layout is the one
 * pa_b200_query_cache_layout reports).  grow() to a size not above the current one does nothing, as in the
 * reference; beyond max_blocks it fails with PA_ERR_TOO_LARGE; when the device is out of memory it fails
 * with the reference's message.  Calls are host-synchronous; grow while no kernel writes the new range. */
typedef struct pa_cache_pool pa_cache_pool;
const char* pa_b200_cache_pool_last_error(void);
int pa_b200_cache_pool_create(const pa_model_desc* desc, int device, int64_t max_blocks, int64_t initial_blocks, pa_cache_pool** out);
int pa_b200_cache_pool_grow(pa_cache_pool* pool, int64_t num_blocks);
int pa_b200_cache_pool_get(pa_cache_pool* pool, void** key_cache, void** value_cache, int64_t* num_blocks);
int pa_b200_cache_pool_destroy(pa_cache_pool* pool);

/* Device-side marshalling of the operator's scheduler inputs.
 *
 * ModelRunner::forward builds past_lens / subsequence_begins / block_indices / block_indices_begins on the
 * host every step, walking layers x groups x blocks of std::maps
 * (src/cpp/src/continuous_batching/model_runner.hpp:802-856, 1316-1380, 1420-1481).  Here the block tables
 * live on the device ([num_slots][table_stride] physical ids per layer, updated by the cache manager when
 * a sequence gains, loses or shares a block) and one call turns them plus the step's schedule into the
 * operator's tensors:
 *   past_lens[s]         = processed - evicted - skipped_blocks * block_size      (model_runner.hpp:804-818)
 *   subsequence_begins   = prefix sum of num_scheduled_tokens                     (:599, :820)
 *   block_indices        = each sequence's table, logical order, skipped blocks left out (:1420-1481)
 *   block_indices_begins = prefix sum of the used blocks                          (:600, :822)
 *   totals               = { num_tokens, num_block_indices, max_context_len = max(processed + scheduled) }
 * A sequence whose numbers do not hold together (more evicted than processed, more skipped blocks than
 * the cache holds, a table longer than table_stride - the host code asserts these) sets
 * PA_DEV_BAD_BEGINS and is given no tokens and no blocks.  All pointers are device memory;
 * asynchronous on the stream.  `totals` may be read back by the caller or handed on as device scalars. */
typedef struct pa_marshal_args {
    uint32_t struct_size;
    const int32_t* block_table;           /* [num_slots][table_stride] */
    const int32_t* block_table_len;       /* [num_slots] blocks in use, slots of this step's new tokens included */
    int32_t table_stride;
    int32_t num_slots;
    const int32_t* slot;                  /* [num_sequences] table row of each scheduled sequence, NULL = row s */
    const int32_t* num_processed_tokens;  /* [num_sequences] */
    const int32_t* num_evicted_tokens;    /* [num_sequences] or NULL */
    const int32_t* num_scheduled_tokens;  /* [num_sequences] */
    const uint32_t* skip_mask;            /* [num_sequences][skip_words], bit j = logical block j hidden, or NULL */
    int32_t skip_words;
    int32_t num_sequences;
    int32_t* past_lens;                   /* out [num_sequences] */
    int32_t* subsequence_begins;          /* out [num_sequences + 1] */
    int32_t* block_indices;               /* out [block_indices_capacity] */
    int32_t* block_indices_begins;        /* out [num_sequences + 1] */
    int32_t* totals;                      /* out [3] */
    int32_t block_indices_capacity;
    void* stream;
} pa_marshal_args;
int pa_b200_marshal_inputs(pa_handle* h, const pa_marshal_args* args);

/* Allocation-free decode step.  It has no counterpart in the reference.
 *
 * For callers that cannot allocate device memory where they run the operator - code inside an
 * allocator or memory-pool callback, a server whose device memory is fully handed out at start-up,
 * a latency-critical loop that must not take the allocator's lock - this entry point needs no
 * handle and calls no cudaMalloc / cudaFree: its scratch is one file-scope device array of
 * PA_B200_STATIC_SCRATCH_BYTES that every GPU loading the library holds until the process exits.
 *
 * Same results as pa_b200_forward for a step in which every sequence has exactly one new token,
 * without score output and without rotation inputs (PA_ERR_UNSUPPORTED otherwise).  All pointers
 * are device memory; the launches go to args->stream (NULL = the default stream).
 *  - The host can only check num_tokens == num_sequences; the per-sequence token counts live in
 *    device memory.  A sequence whose subsequence_begins give it a count other than one is skipped
 *    on the device: nothing is written to the cache for it and its output rows stay untouched.
 *  - A step whose scratch need exceeds the fixed array is rejected with PA_ERR_TOO_LARGE (the
 *    message gives both sizes).  With G = Hq / Hkv the need is a few KB of counters plus
 *    (num_sequences * Hkv * ceil(G/16) + 16 * SM count) * min(G,16) * (head_size + 2) * 4 bytes:
 *    about 6 MB for 64 sequences of the 32/8-head, 128-dim shape on a 148-SM GPU, about 20 MB with more than 16 query
 *    heads per KV head (the array holds 32 MB).
 *  - The first call on a device looks up the array's device address; make that call before any
 *    stream capture.
 *  - All calls on a device share the array: two calls that overlap on the GPU (different streams)
 *    race.  Every call rewrites the parts that must start from a known state.
 *  - Block-index errors are still skipped on the device, but this entry point has no way to
 *    report the device status word; use pa_b200_forward to diagnose inputs. */
#define PA_B200_STATIC_SCRATCH_BYTES (32u << 20)
int pa_b200_decode_step_static(const pa_model_desc* desc, const pa_forward_args* args, int device);

#ifdef __cplusplus
}
#endif
#endif /* PA_B200_H */
