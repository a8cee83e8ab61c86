/*
 * sampler_b200.h - C ABI of the B200 (sm_100a) Sampler step: logit processors + token selection.
 *
 * Replaces the numeric half of ov::genai::Sampler::sample
 * (src/cpp/src/sampling/sampler.cpp:1708-1810): for every scheduled row it applies, in the
 * reference's order (src/cpp/src/sampling/logit_processor.hpp:28-112),
 *     stop-token mask (min_new_tokens) -> repetition -> presence -> frequency penalties
 *     -> [multinomial only] top-k -> temperature -> min-p -> top-p
 * and then selects a token: strict-> argmax with lowest-index ties for greedy
 * (sampler.cpp:939-977), or the multinomial draw of sampler.cpp:979-1095 given the uniform
 * number the request's own std::mt19937 produced.  The whole batch is one kernel launch.
 *
 * What stays on the host (and is mirrored by the C++ class in csrc/host/sampler_host.hpp): the
 * per-request RNG engine, the token-count maps, stop conditions.  Structured-output masks,
 * beam search, tree search and logprobs > 0 are outside this entry point (SAMPLER_ERR_UNSUPPORTED).
 */
#ifndef SAMPLER_B200_H
#define SAMPLER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum sampler_status {
    SAMPLER_OK = 0,
    SAMPLER_ERR_INVALID_ARG = 1,
    SAMPLER_ERR_UNSUPPORTED = 2,
    SAMPLER_ERR_CUDA = 3,
    SAMPLER_ERR_BAD_TOKEN_ID = 4, /* a history id outside [0, vocab): the reference throws "input_ids token out of bounds" */
    SAMPLER_ERR_TOO_LARGE = 5
} sampler_status;

/* History entry flags (one entry per distinct token id of a row). */
#define SAMPLER_HIST_IN_PROMPT 0x1u    /* id is in the unique prompt ids (repetition penalty)             */
#define SAMPLER_HIST_GENERATED 0x2u    /* id has an entry in the generated-token map (all three penalties) */
#define SAMPLER_HIST_STOP_MASK 0x4u    /* id is a stop token and generated_len < min_new_tokens: -inf      */

/* Per-row parameters: the GenerationConfig fields LogitProcessor reads
 * (src/cpp/include/openvino/genai/generation_config.hpp:649-709), same defaults and same
 * activation rules (logit_processor.hpp:59-104). */
typedef struct sampler_row_params {
    int64_t logits_row;        /* row of `logits` to sample from (rows are not assumed to be in request order) */
    int64_t top_k;             /* active iff 0 < top_k < INT64_MAX; >= vocab leaves the full vocabulary   */
    int32_t do_sample;         /* 0 = greedy, 1 = multinomial                                           */
    float temperature;         /* 1.0 = off                                                            */
    float top_p;               /* 1.0 = off                                                            */
    float min_p;               /* 0.0 = off                                                            */
    float repetition_penalty;  /* 1.0 = off                                                            */
    float presence_penalty;    /* 0.0 = off                                                            */
    float frequency_penalty;   /* 0.0 = off                                                            */
    float rand_u;              /* the request's next std::uniform_real_distribution<float>(0,1) draw    */
} sampler_row_params;

typedef struct sampler_step_args {
    uint32_t struct_size;       /* sizeof(sampler_step_args) */
    float* logits;              /* [num_logit_rows, vocab] f32, penalties are applied IN PLACE (sampler.cpp:927-937) */
    int64_t num_logit_rows;
    int64_t vocab;
    int32_t num_rows;           /* rows to sample = entries of `rows` */
    const sampler_row_params* rows;
    /* CSR history: entries hist_offsets[r] .. hist_offsets[r+1] belong to row r. */
    const int64_t* hist_offsets;  /* [num_rows + 1] */
    const int32_t* hist_ids;      /* distinct token ids */
    const uint32_t* hist_meta;    /* (generated count << 3) | SAMPLER_HIST_* flags */
    int64_t* out_token;           /* [num_rows] */
    float* out_log_prob;          /* [num_rows] */
    void* stream;                 /* cudaStream_t, NULL => the handle's stream */
} sampler_step_args;

typedef struct sampler_handle sampler_handle;

const char* sampler_b200_last_error(void);

/* `max_rows` and `max_vocab` size the handle's scratch (candidate lists); calls beyond them grow it. */
int sampler_b200_create(int device, int32_t max_rows, int64_t max_vocab, sampler_handle** out);
int sampler_b200_destroy(sampler_handle* h);

/* One Sampler step over DEVICE buffers, asynchronous on the stream. */
int sampler_b200_step(sampler_handle* h, const sampler_step_args* args);

/* Same step for HOST buffers: logits, row parameters, history and outputs are host pointers;
 * copies in (logits included), runs, copies the mutated logits' sampled rows' results out,
 * synchronises.  Returns SAMPLER_ERR_BAD_TOKEN_ID if the kernel met an out-of-range history id. */
int sampler_b200_step_host(sampler_handle* h, const sampler_step_args* args, int copy_logits_back);

/* Reads (and clears) the device status word: bit 0 = out-of-range history id. */
int sampler_b200_last_device_status(sampler_handle* h, uint32_t* status_bits);

int64_t sampler_b200_launch_count(const sampler_handle* h);

#ifdef __cplusplus
}
#endif
#endif /* SAMPLER_B200_H */
