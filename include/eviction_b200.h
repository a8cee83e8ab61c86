/*
 * eviction_b200.h - C ABI of the eviction scoring that consumes the operator's score output on the
 * device, so that the per-step score vectors (sum over layers of every sequence's context length in
 * floats) never travel to the host.
 *
 * Replaces, for the SUM and NORM_SUM aggregation modes, what the pipeline does on the host each step
 * (src/cpp/src/continuous_batching/pipeline_impl.cpp:884-959):
 *   EvictionScoreManager::register_new_token_scores   cache/cache_eviction.cpp:71-128
 *       max-pool (window 7, pipeline_impl.cpp:900) of the scores past the start area, accumulated in
 *       double precision per tracked token; NORM_SUM also keeps per-token occurrence counters
 *       (:139-160, :204-224)
 *   CacheEvictionAlgorithm::evict_logical_blocks       cache/cache_eviction.cpp:302-412
 *       block scores = in-order sums over the block of score (/ counter) (:457-483), the
 *       num_evictable - keep blocks with the lowest (score, index) (:485-519), ascending; their
 *       tokens leave the tracked scores (:14-48)
 * Results are the reference's bit for bit: the same doubles in the same order of operations, hence
 * the same block lists.  KVCrush, Adaptive R-KV and skipped (sparse-attention) blocks stay on the
 * host path (EVICTION_ERR_UNSUPPORTED).
 *
 * State lives on the device, one record per (layer, sequence slot): scores f64[max_tracked_tokens],
 * counters u32[max_tracked_tokens], tracked length, SnapKV rows registered so far.
 */
#ifndef EVICTION_B200_H
#define EVICTION_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum eviction_status {
    EVICTION_OK = 0,
    EVICTION_ERR_INVALID_ARG = 1,
    EVICTION_ERR_UNSUPPORTED = 2,
    EVICTION_ERR_CUDA = 3,
    EVICTION_ERR_TOO_LARGE = 4 /* device status: a sequence tracks more tokens than max_tracked_tokens */
} eviction_status;

#define EVICTION_AGG_SUM 0
#define EVICTION_AGG_NORM_SUM 1

/* CacheEvictionConfig (src/cpp/include/openvino/genai/cache_eviction.hpp) plus the sizes of the device state. */
typedef struct eviction_config_b200 {
    uint32_t struct_size;
    int32_t start_size;        /* tokens, multiple of block_size: never evicted, not tracked        */
    int32_t recent_size;       /* tokens, multiple of block_size: not evicted yet                   */
    int32_t max_cache_size;    /* tokens, multiple of block_size                                    */
    int32_t block_size;
    int32_t aggregation;       /* EVICTION_AGG_*                                                    */
    int32_t snapkv_window_size;/* 0 = off                                                           */
    int32_t max_pool_window;   /* 7 in the pipeline                                                 */
    int32_t num_layers;
    int32_t num_slots;         /* sequences that can be tracked at once                             */
    int32_t max_tracked_tokens;/* per (layer, slot): max_cache_size + the largest chunk + block_size */
    int32_t max_evicted_blocks;/* row length of evicted_blocks                                      */
} eviction_config_b200;

typedef struct eviction_handle eviction_handle;

/* One step of one layer.  Every pointer is device memory except the handle. */
typedef struct eviction_step_args {
    uint32_t struct_size;
    int32_t layer;
    int32_t num_sequences;
    const float* scores;              /* the operator's score output of this layer                                   */
    const int64_t* span_begin;        /* [num_sequences] first float of the sequence's span (model_runner.hpp:1529-1537) */
    const int32_t* span_len;          /* [num_sequences] context_len - evicted tokens; <= 0: the sequence hands nothing on */
    const int32_t* slot;              /* [num_sequences] state record of the sequence                                 */
    const int32_t* num_snapkv_scores; /* [num_sequences] rows aggregated into this step's scores (0 outside the window) */
    int32_t do_evict;                 /* also run evict_logical_blocks after registering                              */
    int32_t* evicted_count;           /* out [num_sequences]                                                          */
    int32_t* evicted_blocks;          /* out [num_sequences][max_evicted_blocks] logical block ids, ascending         */
    void* stream;
} eviction_step_args;

const char* eviction_b200_last_error(void);
int eviction_b200_create(const eviction_config_b200* cfg, int device, eviction_handle** out);
int eviction_b200_destroy(eviction_handle* h);
/* Forgets a slot's state in every layer (a new sequence takes the slot). */
int eviction_b200_reset_slot(eviction_handle* h, int32_t slot, void* stream);
int eviction_b200_step(eviction_handle* h, const eviction_step_args* args);
/* Reads (and clears) the device status word: bit 0 = max_tracked_tokens or max_evicted_blocks exceeded,
 * bit 1 = slot out of range, bit 2 = more SnapKV rows than the window, bit 3 = a span shorter than the tracked scores. */
int eviction_b200_last_device_status(eviction_handle* h, uint32_t* bits);
/* Test support: copies a slot's tracked scores / counters to HOST arrays of max_tracked_tokens; returns the tracked length. */
int eviction_b200_read_slot(eviction_handle* h, int32_t layer, int32_t slot, double* scores, uint32_t* counters, int32_t* length);

#ifdef __cplusplus
}
#endif
#endif /* EVICTION_B200_H */
