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
 * per-request RNG engine, the token-count maps, stop conditions, and the grammar matcher that fills a
 * request's next-token bitmask (the mask itself is applied here).  Beam search and tree search are
 * outside this entry point.
 *
 * logprobs > 0 (logit_processor.hpp:36-47): the reference first takes log(sum(exp(raw logits)))
 * over the whole vocabulary (FullVocabLogSumExpTransform, logit_transformers.hpp:264-277), lets the
 * penalties and filters work on a copy, and reports raw_logit[token] - that log-partition as the
 * token's log-probability (sampler.cpp:967-974, 1022-1029, 1076-1081).  A row asks for this with
 * SAMPLER_ROW_RAW_LOG_PROB; the selected token is the same as without it.  Unlike the reference
 * the logits row is still left with the penalties applied.
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

/* Bits of sampler_row_params.do_sample. */
#define SAMPLER_ROW_MULTINOMIAL 0x1   /* multinomial sampling (GenerationConfig::is_multinomial); clear = greedy */
#define SAMPLER_ROW_RAW_LOG_PROB 0x2  /* logprobs > 0: report raw_logit[token] - log-partition of the raw row   */

/* Per-row parameters: the GenerationConfig fields LogitProcessor reads
 * (src/cpp/include/openvino/genai/generation_config.hpp:649-709), same defaults and same
 * activation rules (logit_processor.hpp:59-104). */
typedef struct sampler_row_params {
    int64_t logits_row;        /* row of `logits` to sample from (rows are not assumed to be in request order) */
    int64_t top_k;             /* active iff 0 < top_k < INT64_MAX; >= vocab leaves the full vocabulary; an active
                                  top_k below the vocabulary must be <= 1024 (status bit 3 otherwise)         */
    int32_t do_sample;         /* 0 = greedy, 1 = multinomial; SAMPLER_ROW_* bits                       */
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
    float* hist_raw;              /* scratch, one float per history entry (same length as hist_ids): the raw logits the
                                     penalties overwrite.  Needed by sampler_b200_step when a row that has history sets
                                     SAMPLER_ROW_RAW_LOG_PROB (else status bit 2 and a NaN log-probability); may be NULL
                                     otherwise; ignored by sampler_b200_step_host, which stages its own. */
    /* Further draws from a row's distribution: a request with num_return_sequences = n draws n tokens from the
     * distribution of its first sampled token, one uniform number each from the same engine, and forks
     * (sampler.cpp:1539-1549, 1065-1089, 1163-1182).  Row r keeps its own draw (rand_u -> out_token[r]) and makes
     * extra_offsets[r + 1] - extra_offsets[r] more with the numbers extra_rand_u[extra_offsets[r] ..], written to
     * extra_out_token / extra_out_log_prob at the same positions.  Greedy rows make none.  All four NULL: no row
     * draws more than once.  A caller compiled against the struct without these members and the ones below
     * (struct_size ends at hist_raw) is served as if they were NULL. */
    const int64_t* extra_offsets;   /* [num_rows + 1] */
    const float* extra_rand_u;      /* [extra_offsets[num_rows]] */
    int64_t* extra_out_token;       /* [extra_offsets[num_rows]] */
    float* extra_out_log_prob;      /* [extra_offsets[num_rows]] */
    /* Structured output: the grammar's next-token bitmask (sampling/structured_output/xgrammar_backend.cpp:148-165,
     * 187-207), applied after the stop-token mask and before the penalties (logit_processor.hpp:47-57): token t is
     * allowed iff bit (t & 31) of word t / 32 is set, every other logit becomes -inf.  Masks are rows of
     * token_bitmasks, each bitmask_words = ceil(vocab / 32) int32 words; bitmask_index[r] names row r's mask,
     * -1 for a request without a grammar (or whose matcher has terminated).  Both NULL: no row has one. */
    const int32_t* token_bitmasks;  /* [num masks][bitmask_words] */
    const int32_t* bitmask_index;   /* [num_rows] */
    int64_t bitmask_words;
} sampler_step_args;

/* struct_size of the layout that ends at hist_raw */
#define SAMPLER_STEP_ARGS_SIZE_V1 ((uint32_t)offsetof(sampler_step_args, extra_offsets))

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

/* Reads (and clears) the device status word: bit 0 = out-of-range history id, bit 1 = logits_row out of
 * range, bit 2 = SAMPLER_ROW_RAW_LOG_PROB on a row with history but no hist_raw scratch, bit 3 = a
 * multinomial row with 1024 < top_k < vocab (the top-k heap lives in shared memory and holds 1024
 * candidates; such a row gets token -1 and sampler_b200_step_host returns SAMPLER_ERR_UNSUPPORTED),
 * bit 4 = internal: the sorted walk of a top-p row did not terminate. */
int sampler_b200_last_device_status(sampler_handle* h, uint32_t* status_bits);

int64_t sampler_b200_launch_count(const sampler_handle* h);

/* Diagnostic: evaluates the device restatement of the host libm's expf (the function every
 * TemperatureLogitTransform element goes through, logit_transformers.hpp:327-356) on `n` HOST floats.
 * The full-vocabulary path is exact only where this returns the host's expf bits; the tests compare. */
int sampler_b200_selftest_expf(sampler_handle* h, const float* in, float* out, int64_t n);

#ifdef __cplusplus
}
#endif
#endif /* SAMPLER_B200_H */
