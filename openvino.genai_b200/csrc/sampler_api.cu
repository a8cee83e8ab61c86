// C ABI of the Sampler step (include/sampler_b200.h): argument checks, staging for the
// host-tensor entry point, launch.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <string>

#include "sampler_kernels.h"

namespace {

thread_local std::string g_sampler_error;

int sfail(int code, const std::string& msg) {
    g_sampler_error = msg;
    return code;
}

#define S_CUDA(expr)                                                                           \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess)                                                                 \
            return sfail(SAMPLER_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

size_t up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

}  // namespace

struct sampler_handle {
    int device = 0;
    cudaStream_t stream = nullptr;
    uint32_t* status = nullptr;
    uint8_t* stage_dev = nullptr;
    uint8_t* stage_host = nullptr;  // pinned
    size_t stage_bytes = 0;
    float* exact_scratch = nullptr;   // one row of probabilities per CTA of the full-vocabulary kernel
    size_t exact_bytes = 0;
    int exact_ctas = 0;               // persistent grid of that kernel: two CTAs per SM
    int64_t launches = 0;
};

namespace {

int ensure_stage(sampler_handle* h, size_t bytes) {
    if (bytes <= h->stage_bytes) return SAMPLER_OK;
    S_CUDA(cudaStreamSynchronize(h->stream));
    if (h->stage_dev) S_CUDA(cudaFree(h->stage_dev));
    if (h->stage_host) S_CUDA(cudaFreeHost(h->stage_host));
    h->stage_dev = nullptr; h->stage_host = nullptr; h->stage_bytes = 0;
    const size_t want = up(bytes + bytes / 8, 1 << 20);
    S_CUDA(cudaMalloc((void**)&h->stage_dev, want));
    S_CUDA(cudaMallocHost((void**)&h->stage_host, want));
    h->stage_bytes = want;
    return SAMPLER_OK;
}

// Scratch of the full-vocabulary kernel: grows (with a stream synchronisation) when a step has a larger vocabulary.
int ensure_exact_scratch(sampler_handle* h, int32_t rows, int64_t vocab) {
    const int ctas = std::min<int64_t>(rows, h->exact_ctas);
    const size_t need = sampler::sampler_exact_scratch_bytes(ctas, vocab);
    if (need <= h->exact_bytes) return SAMPLER_OK;
    S_CUDA(cudaStreamSynchronize(h->stream));
    S_CUDA(cudaDeviceSynchronize());
    if (h->exact_scratch) S_CUDA(cudaFree(h->exact_scratch));
    h->exact_scratch = nullptr; h->exact_bytes = 0;
    S_CUDA(cudaMalloc((void**)&h->exact_scratch, need));
    h->exact_bytes = need;
    return SAMPLER_OK;
}

// Both launches of a step: penalties / greedy / top-k rows, then the full-vocabulary multinomial rows.
int launch_step(sampler_handle* h, const sampler::StepArgs& k, cudaStream_t stream, bool any_full_vocab) {
    S_CUDA(sampler::launch_sampler(k, stream));
    h->launches += 1;
    if (any_full_vocab) {
        int rc = ensure_exact_scratch(h, k.num_rows, k.vocab);
        if (rc != SAMPLER_OK) return rc;
        S_CUDA(sampler::launch_sampler_exact(k, h->exact_scratch, h->exact_ctas, stream));
        h->launches += 1;
    }
    return SAMPLER_OK;
}

bool row_is_full_vocab(const sampler_row_params& p, int64_t vocab) {
    if (!(p.do_sample & SAMPLER_ROW_MULTINOMIAL)) return false;
    const bool top_k_active = p.top_k > 0 && p.top_k < INT64_MAX;
    return !(top_k_active && p.top_k < vocab);
}

int validate(const sampler_handle* h, const sampler_step_args* a) {
    if (!h) return sfail(SAMPLER_ERR_INVALID_ARG, "NULL handle");
    if (!a || (a->struct_size != sizeof(sampler_step_args) && a->struct_size != SAMPLER_STEP_ARGS_SIZE_V1))
        return sfail(SAMPLER_ERR_INVALID_ARG, "sampler_step_args: NULL or struct_size mismatch");
    if (a->struct_size == sizeof(sampler_step_args) && a->extra_offsets && (!a->extra_rand_u || !a->extra_out_token || !a->extra_out_log_prob))
        return sfail(SAMPLER_ERR_INVALID_ARG, "extra draws: offsets without numbers or outputs");
    if (a->struct_size == sizeof(sampler_step_args) && a->token_bitmasks && a->bitmask_index && a->bitmask_words != (a->vocab + 31) / 32)
        return sfail(SAMPLER_ERR_INVALID_ARG, "bitmask_words must be ceil(vocab / 32)");
    if (a->num_rows < 0 || a->vocab <= 0 || a->num_logit_rows < 0) return sfail(SAMPLER_ERR_INVALID_ARG, "bad size");
    if (a->vocab > 0x7fffffffLL) return sfail(SAMPLER_ERR_TOO_LARGE, "vocab above 2^31 - 1");
    if (a->num_rows > 0 && (!a->logits || !a->rows || !a->out_token || !a->out_log_prob)) return sfail(SAMPLER_ERR_INVALID_ARG, "NULL pointer");
    if (a->hist_offsets && (!a->hist_ids || !a->hist_meta)) return sfail(SAMPLER_ERR_INVALID_ARG, "history arrays incomplete");
    return SAMPLER_OK;
}

sampler::StepArgs kernel_args(sampler_handle* h, const sampler_step_args* a) {
    sampler::StepArgs k;
    k.logits = a->logits; k.num_logit_rows = a->num_logit_rows; k.vocab = a->vocab; k.num_rows = a->num_rows;
    k.rows = a->rows; k.hist_offsets = a->hist_offsets; k.hist_ids = a->hist_ids; k.hist_meta = a->hist_meta;
    k.out_token = a->out_token; k.out_log_prob = a->out_log_prob; k.status = h->status; k.hist_raw = a->hist_raw;
    const bool extras = a->struct_size == sizeof(sampler_step_args) && a->extra_offsets != nullptr;
    k.extra_offsets = extras ? a->extra_offsets : nullptr;
    k.extra_rand_u = extras ? a->extra_rand_u : nullptr;
    k.extra_out_token = extras ? a->extra_out_token : nullptr;
    k.extra_out_log_prob = extras ? a->extra_out_log_prob : nullptr;
    const bool masks = a->struct_size == sizeof(sampler_step_args) && a->token_bitmasks != nullptr && a->bitmask_index != nullptr;
    k.token_bitmasks = masks ? a->token_bitmasks : nullptr;
    k.bitmask_index = masks ? a->bitmask_index : nullptr;
    k.bitmask_words = masks ? a->bitmask_words : 0;
    return k;
}

}  // namespace

extern "C" {

const char* sampler_b200_last_error(void) { return g_sampler_error.c_str(); }

int sampler_b200_destroy(sampler_handle* h);
int sampler_b200_create(int device, int32_t max_rows, int64_t max_vocab, sampler_handle** out) {
    if (!out) return sfail(SAMPLER_ERR_INVALID_ARG, "NULL out pointer");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || device < 0 || device >= count) return sfail(SAMPLER_ERR_INVALID_ARG, "no such CUDA device");
    cudaDeviceProp prop;
    S_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return sfail(SAMPLER_ERR_UNSUPPORTED, "this library is built for sm_100a only");
    S_CUDA(cudaSetDevice(device));
    sampler_handle* h = new sampler_handle();
    h->device = device;
    cudaError_t e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 256);
    if (e != cudaSuccess) {
        delete h;
        return sfail(SAMPLER_ERR_CUDA, std::string("sampler_b200_create: ") + cudaGetErrorString(e));
    }
    h->exact_ctas = 2 * prop.multiProcessorCount;
    if (max_rows > 0 && max_vocab > 0) {   // otherwise sized on first use
        const int rc = ensure_exact_scratch(h, max_rows, max_vocab);
        if (rc != SAMPLER_OK) { sampler_b200_destroy(h); return rc; }
    }
    *out = h;
    return SAMPLER_OK;
}

int sampler_b200_destroy(sampler_handle* h) {
    if (!h) return SAMPLER_OK;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    if (h->status) cudaFree(h->status);
    if (h->stage_dev) cudaFree(h->stage_dev);
    if (h->stage_host) cudaFreeHost(h->stage_host);
    if (h->exact_scratch) cudaFree(h->exact_scratch);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return SAMPLER_OK;
}

int sampler_b200_step(sampler_handle* h, const sampler_step_args* a) {
    int rc = validate(h, a);
    if (rc != SAMPLER_OK) return rc;
    if (a->num_rows == 0) return SAMPLER_OK;
    S_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    // the row parameters live on the device: the second launch is always made and leaves at once when no row needs it
    return launch_step(h, kernel_args(h, a), stream, true);
}

int sampler_b200_step_host(sampler_handle* h, const sampler_step_args* a, int copy_logits_back) {
    int rc = validate(h, a);
    if (rc != SAMPLER_OK) return rc;
    if (a->num_rows == 0) return SAMPLER_OK;
    S_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    const size_t n = (size_t)a->num_rows;
    const size_t logits_bytes = (size_t)a->num_logit_rows * a->vocab * sizeof(float);
    const size_t hist_n = a->hist_offsets ? (size_t)a->hist_offsets[n] : 0;
    size_t off = 0;
    const size_t o_rows = off;  off += up(n * sizeof(sampler_row_params));
    const size_t o_hoff = off;  off += up((n + 1) * sizeof(int64_t));
    const size_t o_hid = off;   off += up(hist_n * sizeof(int32_t));
    const size_t o_hmeta = off; off += up(hist_n * sizeof(uint32_t));
    const size_t small_in = off;
    const size_t o_tok = off;   off += up(n * sizeof(int64_t));
    const size_t o_lp = off;    off += up(n * sizeof(float));
    const size_t o_hraw = off;  off += up(hist_n * sizeof(float));
    const bool extras = a->struct_size == sizeof(sampler_step_args) && a->extra_offsets != nullptr;
    const size_t extra_n = extras ? (size_t)a->extra_offsets[n] : 0;
    const size_t o_xoff = off;  off += up(extras ? (n + 1) * sizeof(int64_t) : 0);
    const size_t o_xu = off;    off += up(extra_n * sizeof(float));
    const size_t o_xtok = off;  off += up(extra_n * sizeof(int64_t));
    const size_t o_xlp = off;   off += up(extra_n * sizeof(float));
    const bool masks = a->struct_size == sizeof(sampler_step_args) && a->token_bitmasks && a->bitmask_index;
    int32_t num_masks = 0;
    if (masks)
        for (size_t i = 0; i < n; ++i) num_masks = std::max(num_masks, a->bitmask_index[i] + 1);
    const size_t mask_bytes = masks ? (size_t)num_masks * (size_t)a->bitmask_words * sizeof(int32_t) : 0;
    const size_t o_midx = off;  off += up(masks ? n * sizeof(int32_t) : 0);
    const size_t o_mask = off;  off += up(mask_bytes);
    const size_t o_logits = off; off += up(logits_bytes);
    rc = ensure_stage(h, off);
    if (rc != SAMPLER_OK) return rc;
    std::memcpy(h->stage_host + o_rows, a->rows, n * sizeof(sampler_row_params));
    if (a->hist_offsets) {
        std::memcpy(h->stage_host + o_hoff, a->hist_offsets, (n + 1) * sizeof(int64_t));
        std::memcpy(h->stage_host + o_hid, a->hist_ids, hist_n * sizeof(int32_t));
        std::memcpy(h->stage_host + o_hmeta, a->hist_meta, hist_n * sizeof(uint32_t));
    }
    S_CUDA(cudaMemcpyAsync(h->stage_dev, h->stage_host, small_in, cudaMemcpyHostToDevice, stream));
    if (extras) {
        std::memcpy(h->stage_host + o_xoff, a->extra_offsets, (n + 1) * sizeof(int64_t));
        std::memcpy(h->stage_host + o_xu, a->extra_rand_u, extra_n * sizeof(float));
        S_CUDA(cudaMemcpyAsync(h->stage_dev + o_xoff, h->stage_host + o_xoff, o_xtok - o_xoff, cudaMemcpyHostToDevice, stream));
    }
    S_CUDA(cudaMemcpyAsync(h->stage_dev + o_logits, a->logits, logits_bytes, cudaMemcpyHostToDevice, stream));
    if (masks) {
        std::memcpy(h->stage_host + o_midx, a->bitmask_index, n * sizeof(int32_t));
        if (mask_bytes) std::memcpy(h->stage_host + o_mask, a->token_bitmasks, mask_bytes);
        S_CUDA(cudaMemcpyAsync(h->stage_dev + o_midx, h->stage_host + o_midx, o_mask + up(mask_bytes) - o_midx, cudaMemcpyHostToDevice, stream));
    }
    sampler_step_args d;
    std::memset(&d, 0, sizeof(d));
    std::memcpy(&d, a, a->struct_size);
    d.struct_size = sizeof(d);
    if (extras) {
        d.extra_offsets = (const int64_t*)(h->stage_dev + o_xoff);
        d.extra_rand_u = (const float*)(h->stage_dev + o_xu);
        d.extra_out_token = (int64_t*)(h->stage_dev + o_xtok);
        d.extra_out_log_prob = (float*)(h->stage_dev + o_xlp);
    }
    if (masks) {
        d.bitmask_index = (const int32_t*)(h->stage_dev + o_midx);
        d.token_bitmasks = (const int32_t*)(h->stage_dev + o_mask);
    }
    d.logits = (float*)(h->stage_dev + o_logits);
    d.rows = (const sampler_row_params*)(h->stage_dev + o_rows);
    d.hist_offsets = a->hist_offsets ? (const int64_t*)(h->stage_dev + o_hoff) : nullptr;
    d.hist_ids = (const int32_t*)(h->stage_dev + o_hid);
    d.hist_meta = (const uint32_t*)(h->stage_dev + o_hmeta);
    d.out_token = (int64_t*)(h->stage_dev + o_tok);
    d.out_log_prob = (float*)(h->stage_dev + o_lp);
    d.hist_raw = (float*)(h->stage_dev + o_hraw);
    bool any_full_vocab = false;
    for (size_t i = 0; i < n && !any_full_vocab; ++i) any_full_vocab = row_is_full_vocab(a->rows[i], a->vocab);
    rc = launch_step(h, kernel_args(h, &d), stream, any_full_vocab);
    if (rc != SAMPLER_OK) return rc;
    S_CUDA(cudaMemcpyAsync(a->out_token, d.out_token, n * sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
    S_CUDA(cudaMemcpyAsync(a->out_log_prob, d.out_log_prob, n * sizeof(float), cudaMemcpyDeviceToHost, stream));
    if (extras && extra_n) {
        S_CUDA(cudaMemcpyAsync(a->extra_out_token, d.extra_out_token, extra_n * sizeof(int64_t), cudaMemcpyDeviceToHost, stream));
        S_CUDA(cudaMemcpyAsync(a->extra_out_log_prob, d.extra_out_log_prob, extra_n * sizeof(float), cudaMemcpyDeviceToHost, stream));
    }
    if (copy_logits_back) S_CUDA(cudaMemcpyAsync(a->logits, d.logits, logits_bytes, cudaMemcpyDeviceToHost, stream));
    uint32_t bits = 0;
    S_CUDA(cudaMemcpyAsync(&bits, h->status, 4, cudaMemcpyDeviceToHost, stream));
    S_CUDA(cudaStreamSynchronize(stream));
    if (bits) {
        S_CUDA(cudaMemsetAsync(h->status, 0, 4, stream));
        const int code = (bits & 1u) ? SAMPLER_ERR_BAD_TOKEN_ID : (bits & 8u) ? SAMPLER_ERR_UNSUPPORTED : (bits & 16u) ? SAMPLER_ERR_CUDA : SAMPLER_ERR_INVALID_ARG;
        return sfail(code, "device status word " + std::to_string(bits));
    }
    return SAMPLER_OK;
}

int sampler_b200_last_device_status(sampler_handle* h, uint32_t* status_bits) {
    if (!h || !status_bits) return sfail(SAMPLER_ERR_INVALID_ARG, "NULL argument");
    S_CUDA(cudaSetDevice(h->device));
    S_CUDA(cudaStreamSynchronize(h->stream));
    S_CUDA(cudaMemcpy(status_bits, h->status, 4, cudaMemcpyDeviceToHost));
    if (*status_bits) S_CUDA(cudaMemset(h->status, 0, 4));
    return SAMPLER_OK;
}

int64_t sampler_b200_launch_count(const sampler_handle* h) { return h ? h->launches : -1; }

int sampler_b200_selftest_expf(sampler_handle* h, const float* in, float* out, int64_t n) {
    if (!h || !in || !out || n < 0) return sfail(SAMPLER_ERR_INVALID_ARG, "NULL argument");
    if (n == 0) return SAMPLER_OK;
    S_CUDA(cudaSetDevice(h->device));
    float* d = nullptr;
    S_CUDA(cudaMalloc((void**)&d, 2 * (size_t)n * sizeof(float)));
    cudaError_t e = cudaMemcpyAsync(d, in, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, h->stream);
    if (e == cudaSuccess) e = sampler::launch_expf_selftest(d, d + n, n, h->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, d + n, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost, h->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    cudaFree(d);
    if (e != cudaSuccess) return sfail(SAMPLER_ERR_CUDA, std::string("selftest: ") + cudaGetErrorString(e));
    return SAMPLER_OK;
}

}  // extern "C"
