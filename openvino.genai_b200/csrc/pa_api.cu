// C ABI of the PagedAttention operator (include/pa_b200.h): argument checking, scratch
// management, launch sequencing, and the host-tensor entry point.
#include <cuda_runtime.h>

#include <algorithm>
#include <climits>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "pa_kernels.h"

namespace {

thread_local std::string g_last_error;

int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

#define PA_CUDA(expr)                                                                        \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return fail(PA_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e));    \
    } while (0)

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

size_t act_bytes(int dt) { return dt == PA_DTYPE_F32 ? 4 : 2; }

}  // namespace

namespace pa {
void set_last_error(const std::string& msg) { g_last_error = msg; }
}  // namespace pa

struct pa_handle {
    pa_model_desc desc;
    pa::CacheGeom g;
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    uint8_t* ws = nullptr;       // kernel scratch
    size_t ws_bytes = 0;
    uint32_t* status = nullptr;  // device status word
    uint8_t* stage_dev = nullptr;  // device copies of host tensors (forward_host)
    size_t stage_dev_bytes = 0;
    uint8_t* stage_host = nullptr;  // pinned
    size_t stage_host_bytes = 0;
    int64_t launches = 0;
    int last_prefill_kernel = PA_PREFILL_NONE;
    bool force_generic_prefill = false;        // env PA_B200_GENERIC_PREFILL=1: cross-check path
    bool test_drop_copy = false;               // env PA_B200_TEST_DROP_FIRST_COPY=1: the decode kernel's bounded wait is made to run out
    bool timing = false;                       // record events around the split-K decode kernel
    std::vector<cudaEvent_t> ev;               // pairs, created on demand
    size_t ev_used = 0;
};

namespace {

int validate_desc(const pa_model_desc* d) {
    if (!d || d->struct_size != sizeof(pa_model_desc)) return fail(PA_ERR_INVALID_ARG, "pa_model_desc: NULL or struct_size mismatch");
    if (d->num_q_heads <= 0 || d->num_kv_heads <= 0 || d->num_q_heads % d->num_kv_heads != 0)
        return fail(PA_ERR_INVALID_ARG, "num_q_heads must be a positive multiple of num_kv_heads");
    if (d->head_size != 64 && d->head_size != 128) return fail(PA_ERR_UNSUPPORTED, "head_size must be 64 or 128");
    if (d->block_size != 16 && d->block_size != 32) return fail(PA_ERR_UNSUPPORTED, "block_size must be 16 or 32");
    if (d->act_dtype != PA_DTYPE_F32 && d->act_dtype != PA_DTYPE_F16 && d->act_dtype != PA_DTYPE_BF16)
        return fail(PA_ERR_UNSUPPORTED, "act_dtype must be f32, f16 or bf16");
    if (d->cache_dtype != PA_DTYPE_F16 && d->cache_dtype != PA_DTYPE_BF16 && d->cache_dtype != PA_DTYPE_U8)
        return fail(PA_ERR_UNSUPPORTED, "cache_dtype must be f16, bf16 or u8");
    return PA_OK;
}

pa::CacheGeom make_geom(const pa_model_desc& d) {
    pa::CacheGeom g;
    g.Hq = d.num_q_heads; g.Hkv = d.num_kv_heads; g.D = d.head_size; g.bs = d.block_size;
    g.act = d.act_dtype; g.cache = d.cache_dtype;
    g.head_bytes = pa::head_record_bytes(d.cache_dtype, d.block_size, d.head_size);
    g.block_bytes = g.head_bytes * d.num_kv_heads;
    return g;
}

// Scratch layout of one forward call.
struct Plan {
    long long max_tiles;
    size_t off_hdr, off_prefix, off_pprefix, off_porder, off_wstart, off_done, off_part_o, off_part_ml, off_cta_q, off_lse, off_score_off, off_stile, off_score_part, off_score_raw, total;
    bool has_score_raw;
};

Plan make_plan(const pa_handle* h, int num_tokens, int num_sequences, int max_context_len, int64_t scores_len,
               int num_block_indices = -1) {
    Plan p;
    const pa::CacheGeom& g = h->g;
    const int G = g.Hq / g.Hkv, gtiles = (G + 15) / 16, HK = g.Hkv * gtiles, RT = std::min(G, 16);
    const long long B = std::max(num_sequences, 0);
    // upper bound of the step's context tiles, known without reading device metadata
    long long tiles = B * ((std::max(max_context_len, 1) + 31) / 32);
    if (num_block_indices >= 0) tiles = std::min(tiles, (long long)num_block_indices * g.bs / 32 + B);
    p.max_tiles = tiles * HK;
    const long long slots = B * HK + pa::decode_max_workers(h->sm_count);  // slot = stream + slice
    size_t off = 0;
    p.off_hdr = off;       off += 256;
    p.off_prefix = off;    off += align_up((size_t)(B + 1) * sizeof(int), 256);
    p.off_pprefix = off;   off += align_up((size_t)(B + 1) * sizeof(int), 256);
    p.off_porder = off;    off += align_up((size_t)pa::kPrefillSortCap * sizeof(int), 256);
    p.off_wstart = off;    off += align_up((size_t)pa::decode_max_workers(h->sm_count) * sizeof(pa::WorkerStart), 256);
    p.off_done = off;      off += align_up((size_t)std::max(B, 1LL) * HK * sizeof(int), 256);
    p.off_part_o = off;    off += align_up((size_t)slots * RT * g.D * sizeof(float), 256);
    p.off_part_ml = off;   off += align_up((size_t)slots * RT * 2 * sizeof(float), 256);
    p.off_cta_q = off;     off += pa::decode_shared_supported(g) ? align_up(pa::decode_shared_scratch_bytes(h->sm_count), 256) : 0;
    p.off_lse = off;       off += align_up((size_t)std::max(num_tokens, 1) * g.Hq * sizeof(float), 256);
    p.off_score_off = off; off += align_up((size_t)(B + 1) * sizeof(int64_t), 256);
    p.off_stile = off;     off += align_up((size_t)(B + 1) * sizeof(int), 256);
    p.off_score_part = off; off += align_up((size_t)std::max<int64_t>(scores_len, 0) * g.Hkv * sizeof(float), 256);
    // scaled logits of the decode rows, [head tiles][scores_len][8 or 16]: kept only while they stay below 1 GiB; beyond
    // that every sequence goes through the score kernel, which reads the keys again instead
    const size_t raw_bytes = (size_t)std::max<int64_t>(scores_len, 0) * HK * (RT <= 8 ? 8 : 16) * sizeof(float);
    p.has_score_raw = raw_bytes > 0 && raw_bytes <= ((size_t)1 << 30);
    p.off_score_raw = off; off += p.has_score_raw ? align_up(raw_bytes, 256) : 0;
    p.total = off;
    return p;
}

int ensure_ws(pa_handle* h, size_t bytes) {
    if (bytes <= h->ws_bytes) return PA_OK;
    PA_CUDA(cudaStreamSynchronize(h->stream));
    if (h->ws) PA_CUDA(cudaFree(h->ws));
    h->ws = nullptr; h->ws_bytes = 0;
    const size_t want = align_up(bytes + bytes / 4, 1 << 20);
    PA_CUDA(cudaMalloc((void**)&h->ws, want));
    h->ws_bytes = want;
    return PA_OK;
}

int ensure_stage(pa_handle* h, size_t bytes) {
    if (bytes <= h->stage_dev_bytes) return PA_OK;
    PA_CUDA(cudaStreamSynchronize(h->stream));
    if (h->stage_dev) PA_CUDA(cudaFree(h->stage_dev));
    if (h->stage_host) PA_CUDA(cudaFreeHost(h->stage_host));
    h->stage_dev = nullptr; h->stage_host = nullptr; h->stage_dev_bytes = h->stage_host_bytes = 0;
    const size_t want = align_up(bytes + bytes / 4, 1 << 20);
    PA_CUDA(cudaMalloc((void**)&h->stage_dev, want));
    PA_CUDA(cudaMallocHost((void**)&h->stage_host, want));
    h->stage_dev_bytes = h->stage_host_bytes = want;
    return PA_OK;
}

int validate_args(const pa_handle* h, const pa_forward_args* a) {
    if (!h) return fail(PA_ERR_INVALID_ARG, "NULL handle");
    if (!a || a->struct_size != sizeof(pa_forward_args)) return fail(PA_ERR_INVALID_ARG, "pa_forward_args: NULL or struct_size mismatch");
    if (a->sliding_window != 0) return fail(PA_ERR_UNSUPPORTED, "sliding_window is not supported");
    if (a->alibi_slopes != nullptr) return fail(PA_ERR_UNSUPPORTED, "alibi_slopes is not supported");
    if (a->num_tokens < 0 || a->num_sequences < 0 || a->num_blocks < 0 || a->num_block_indices < 0 || a->max_context_len < 0)
        return fail(PA_ERR_INVALID_ARG, "negative size");
    if (a->num_sequences > 65535) return fail(PA_ERR_TOO_LARGE, "more than 65535 sequences in one call");
    if (a->num_tokens > 0 && (!a->query || !a->key || !a->value || !a->output)) return fail(PA_ERR_INVALID_ARG, "NULL activation pointer");
    if (a->num_sequences > 0 && (!a->past_lens || !a->subsequence_begins || !a->block_indices_begins || !a->key_cache || !a->value_cache))
        return fail(PA_ERR_INVALID_ARG, "NULL metadata or cache pointer");
    if (a->num_block_indices > 0 && !a->block_indices) return fail(PA_ERR_INVALID_ARG, "NULL block_indices");
    if (a->num_rotated_blocks < 0) return fail(PA_ERR_INVALID_ARG, "negative num_rotated_blocks");
    if (a->num_rotated_blocks > 0 && (!a->rotated_block_indices || !a->rotation_deltas || !a->rotation_trig_lut || a->rotation_lut_rows <= 0))
        return fail(PA_ERR_INVALID_ARG, "rotation inputs incomplete");
    if ((a->scores != nullptr) != (a->score_aggregation_window != nullptr))
        return fail(PA_ERR_INVALID_ARG, "scores and score_aggregation_window must be given together");
    if (a->scores && a->scores_len < 0) return fail(PA_ERR_INVALID_ARG, "negative scores_len");
    return PA_OK;
}

pa::KernelArgs make_kernel_args(pa_handle* h, const pa_forward_args* a, const Plan& p) {
    pa::KernelArgs k;
    std::memset(&k, 0, sizeof(k));
    k.g = h->g;
    k.query = a->query; k.key = a->key; k.value = a->value; k.output = a->output;
    k.num_tokens = a->num_tokens;
    k.key_cache = a->key_cache; k.value_cache = a->value_cache; k.num_blocks = a->num_blocks;
    k.past_lens = a->past_lens; k.subsequence_begins = a->subsequence_begins;
    k.block_indices = a->block_indices; k.block_indices_begins = a->block_indices_begins;
    k.num_block_indices = a->num_block_indices;
    k.num_sequences = a->num_sequences; k.max_context_len = a->max_context_len;
    k.scale = a->scale;
    k.score_aggregation_window = a->score_aggregation_window;
    k.scores = a->scores; k.scores_len = a->scores_len;
    k.rotated_block_indices = a->rotated_block_indices; k.rotation_deltas = a->rotation_deltas;
    k.num_rotated_blocks = a->num_rotated_blocks;
    k.rotation_trig_lut = a->rotation_trig_lut; k.rotation_lut_rows = a->rotation_lut_rows;
    k.status = h->status;
    k.part_o = (float*)(h->ws + p.off_part_o);
    k.part_ml = (float*)(h->ws + p.off_part_ml);
    k.cta_q = (uint8_t*)(h->ws + p.off_cta_q);
    k.lse = (float*)(h->ws + p.off_lse);
    k.score_offsets = (int64_t*)(h->ws + p.off_score_off);
    k.stile_prefix = (int*)(h->ws + p.off_stile);
    k.score_part = (float*)(h->ws + p.off_score_part);
    k.score_raw = a->scores && a->score_aggregation_window && p.has_score_raw ? (float*)(h->ws + p.off_score_raw) : nullptr;
    k.plan = (pa::PlanHeader*)(h->ws + p.off_hdr);
    k.tile_prefix = (int*)(h->ws + p.off_prefix);
    k.stream_done = (int*)(h->ws + p.off_done);
    k.ptile_prefix = (int*)(h->ws + p.off_pprefix);
    k.pitem_order = (int*)(h->ws + p.off_porder);
    k.worker_start = (pa::WorkerStart*)(h->ws + p.off_wstart);
    k.decode_all_workers = 0;
    k.max_tiles = p.max_tiles;
    k.rows_per_tile = std::min(h->g.Hq / h->g.Hkv, 16);
    return k;
}

int run_forward(pa_handle* h, const pa_forward_args* a, cudaStream_t stream) {
    if (a->num_sequences == 0 || a->num_tokens == 0) return PA_OK;
    Plan p = make_plan(h, a->num_tokens, a->num_sequences, a->max_context_len, a->scores_len, a->num_block_indices);
    int rc = ensure_ws(h, p.total);
    if (rc != PA_OK) return rc;
    pa::KernelArgs k = make_kernel_args(h, a, p);
    k.test_drop_copy = h->test_drop_copy ? 1 : 0;
    // SM-shared kernel while a CTA's slice fits two of its chapters; longer slices go to the warp-per-slice kernel, whose
    // fixed slices cost nothing per chapter and balance well when every warp has hundreds of tiles
    const bool shared_decode = pa::decode_shared_supported(h->g) && k.max_tiles <= (long long)h->sm_count * pa::decode_shared_chapter_tiles(h->g) * pa::decode_shared_max_chapters();
    if (shared_decode) {   // one CTA per SM is the worker; its warps share the slice
        k.decode_phantom = pa::decode_shared_phantom();
        k.max_tiles += (long long)a->num_sequences * h->g.Hkv * k.decode_phantom;
        k.decode_all_workers = pa::decode_shared_ctas(k, h->sm_count);
    } else {
        k.decode_all_workers = pa::decode_launch_workers(k, h->sm_count);   // the plan step prepares one start record per worker
    }
    int launches = 0;
    if (a->num_rotated_blocks > 0) { PA_CUDA(pa::launch_rotate(k, stream)); ++launches; }
    PA_CUDA(pa::launch_write_kv(k, stream, /*with_plan=*/true)); ++launches;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    if (h->timing && h->ev_used + 2 <= 8192) {
        while (h->ev.size() < h->ev_used + 2) {
            cudaEvent_t e;
            PA_CUDA(cudaEventCreate(&e));
            h->ev.push_back(e);
        }
        ev0 = h->ev[h->ev_used]; ev1 = h->ev[h->ev_used + 1];
        h->ev_used += 2;
    }
    if (shared_decode) PA_CUDA(pa::launch_decode_shared(k, stream, h->sm_count, &launches, ev0, ev1));
    else PA_CUDA(pa::launch_decode(k, stream, h->sm_count, &launches, ev0, ev1));
    h->last_prefill_kernel = PA_PREFILL_NONE;
    if (a->num_tokens > a->num_sequences) {
        const int G = h->g.Hq / h->g.Hkv;
        const long long max_items = ((long long)a->num_tokens * G / pa::kPrefillItemRows + a->num_sequences) * h->g.Hkv;
        if (pa::prefill_tc_supported(h->g) && !h->force_generic_prefill) {
            PA_CUDA(pa::launch_prefill_tc(k, stream, h->sm_count, max_items, &launches));
            h->last_prefill_kernel = PA_PREFILL_TCGEN05;
        } else if (pa::prefill_mma_supported(h->g) && !h->force_generic_prefill) {
            PA_CUDA(pa::launch_prefill_mma(k, stream, max_items, &launches));
            h->last_prefill_kernel = PA_PREFILL_MMA_SYNC;
        } else {
            PA_CUDA(pa::launch_prefill(k, stream, &launches));
            h->last_prefill_kernel = PA_PREFILL_GENERIC;
        }
    }
    if (a->scores) PA_CUDA(pa::launch_scores(k, stream, h->sm_count, &launches));
    h->launches += launches;
    return PA_OK;
}

}  // namespace

extern "C" {

int pa_b200_abi_version(void) { return PA_B200_ABI_VERSION; }

const char* pa_b200_last_error(void) { return g_last_error.c_str(); }

int pa_b200_query_cache_layout(const pa_model_desc* desc, pa_cache_layout* out) {
    int rc = validate_desc(desc);
    if (rc != PA_OK) return rc;
    if (!out || out->struct_size != sizeof(pa_cache_layout)) return fail(PA_ERR_INVALID_ARG, "pa_cache_layout: NULL or struct_size mismatch");
    pa::CacheGeom g = make_geom(*desc);
    out->elem_dtype = desc->cache_dtype;
    const int64_t inner = desc->cache_dtype == PA_DTYPE_U8 ? desc->head_size + 8 : desc->head_size;
    const int64_t shape[4] = {0, desc->num_kv_heads, desc->block_size, inner};
    for (int i = 0; i < 4; ++i) { out->key_shape[i] = shape[i]; out->value_shape[i] = shape[i]; }
    out->key_block_bytes = g.block_bytes;
    out->value_block_bytes = g.block_bytes;
    out->base_alignment = 256;
    return PA_OK;
}

int pa_b200_create(const pa_model_desc* desc, int device, pa_handle** out) {
    int rc = validate_desc(desc);
    if (rc != PA_OK) return rc;
    if (!out) return fail(PA_ERR_INVALID_ARG, "NULL out pointer");
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return fail(PA_ERR_NO_DEVICE, "no CUDA device");
    if (device < 0 || device >= count) return fail(PA_ERR_INVALID_ARG, "device ordinal out of range");
    cudaDeviceProp prop;
    PA_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(PA_ERR_NO_DEVICE, "this library is built for sm_100a only");
    PA_CUDA(cudaSetDevice(device));
    pa_handle* h = new pa_handle();
    h->desc = *desc;
    h->g = make_geom(*desc);
    h->device = device;
    h->sm_count = prop.multiProcessorCount;
    if (const char* e = std::getenv("PA_B200_GENERIC_PREFILL")) h->force_generic_prefill = std::atoi(e) != 0;
    if (const char* e = std::getenv("PA_B200_TEST_DROP_FIRST_COPY")) h->test_drop_copy = std::atoi(e) != 0;
    cudaError_t e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->status, 256);
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, 256);
    if (e != cudaSuccess) {
        delete h;
        return fail(PA_ERR_CUDA, std::string("pa_b200_create: ") + cudaGetErrorString(e));
    }
    *out = h;
    return PA_OK;
}

int pa_b200_destroy(pa_handle* h) {
    if (!h) return PA_OK;
    cudaSetDevice(h->device);
    if (h->stream) cudaStreamSynchronize(h->stream);
    if (h->ws) cudaFree(h->ws);
    if (h->status) cudaFree(h->status);
    if (h->stage_dev) cudaFree(h->stage_dev);
    if (h->stage_host) cudaFreeHost(h->stage_host);
    for (cudaEvent_t e : h->ev) cudaEventDestroy(e);
    if (h->stream) cudaStreamDestroy(h->stream);
    delete h;
    return PA_OK;
}

int64_t pa_b200_workspace_bytes(const pa_handle* h, int32_t num_tokens, int32_t num_sequences, int32_t max_context_len,
                                int64_t scores_len) {
    if (!h) return -1;
    return (int64_t)make_plan(h, num_tokens, num_sequences, max_context_len, scores_len).total;
}

int pa_b200_reserve(pa_handle* h, int32_t num_tokens, int32_t num_sequences, int32_t max_context_len, int64_t scores_len,
                    int32_t num_block_indices) {
    if (!h) return fail(PA_ERR_INVALID_ARG, "NULL handle");
    PA_CUDA(cudaSetDevice(h->device));
    int rc = ensure_ws(h, make_plan(h, num_tokens, num_sequences, max_context_len, scores_len, num_block_indices).total);
    if (rc != PA_OK) return rc;
    const size_t ab = act_bytes(h->g.act);
    size_t stage = (size_t)num_tokens * (2 * h->g.Hq + 2 * h->g.Hkv) * h->g.D * ab + (size_t)(3 * num_sequences + 2 + num_block_indices) * 4 +
                   (size_t)std::max<int64_t>(scores_len, 0) * 4 + (size_t)num_sequences * 4 + 16 * 256;
    return ensure_stage(h, stage);
}

int pa_b200_forward(pa_handle* h, const pa_forward_args* a) {
    int rc = validate_args(h, a);
    if (rc != PA_OK) return rc;
    PA_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    return run_forward(h, a, stream);
}

int pa_b200_write_kv(pa_handle* h, const pa_forward_args* a) {
    int rc = validate_args(h, a);
    if (rc != PA_OK) return rc;
    PA_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    Plan p = make_plan(h, a->num_tokens, a->num_sequences, a->max_context_len, 0);
    rc = ensure_ws(h, p.total);
    if (rc != PA_OK) return rc;
    pa::KernelArgs k = make_kernel_args(h, a, p);
    PA_CUDA(pa::launch_write_kv(k, stream, /*with_plan=*/false));
    h->launches += 1;
    return PA_OK;
}

int pa_b200_rotate_blocks(pa_handle* h, const pa_forward_args* a) {
    int rc = validate_args(h, a);
    if (rc != PA_OK) return rc;
    PA_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    Plan p = make_plan(h, 1, 1, 1, 0);
    rc = ensure_ws(h, p.total);
    if (rc != PA_OK) return rc;
    pa::KernelArgs k = make_kernel_args(h, a, p);
    if (a->num_rotated_blocks > 0) {
        PA_CUDA(pa::launch_rotate(k, stream));
        h->launches += 1;
    }
    return PA_OK;
}

int pa_b200_copy_blocks(pa_handle* h, void* key_cache, void* value_cache, int32_t num_blocks, const int32_t* src_dst_pairs,
                        int32_t num_pairs, void* stream) {
    if (!h || !key_cache || !value_cache || num_pairs < 0 || (num_pairs > 0 && !src_dst_pairs))
        return fail(PA_ERR_INVALID_ARG, "pa_b200_copy_blocks: bad argument");
    PA_CUDA(cudaSetDevice(h->device));
    cudaStream_t s = stream ? (cudaStream_t)stream : h->stream;
    PA_CUDA(pa::launch_copy_blocks(key_cache, value_cache, h->g.block_bytes, num_blocks, src_dst_pairs, num_pairs, h->status, s));
    if (num_pairs > 0) h->launches += 1;
    return PA_OK;
}

int pa_b200_last_device_status(pa_handle* h, uint32_t* status_bits) {
    if (!h || !status_bits) return fail(PA_ERR_INVALID_ARG, "NULL argument");
    PA_CUDA(cudaSetDevice(h->device));
    PA_CUDA(cudaStreamSynchronize(h->stream));
    PA_CUDA(cudaMemcpy(status_bits, h->status, 4, cudaMemcpyDeviceToHost));
    if (*status_bits) PA_CUDA(cudaMemset(h->status, 0, 4));
    return PA_OK;
}

int pa_b200_marshal_inputs(pa_handle* h, const pa_marshal_args* a) {
    if (!h) return fail(PA_ERR_INVALID_ARG, "NULL handle");
    if (!a || a->struct_size != sizeof(pa_marshal_args)) return fail(PA_ERR_INVALID_ARG, "pa_marshal_args: NULL or struct_size mismatch");
    if (a->num_sequences < 0 || a->table_stride < 0 || a->num_slots < 0 || a->skip_words < 0 || a->block_indices_capacity < 0)
        return fail(PA_ERR_INVALID_ARG, "negative size");
    if (a->num_sequences == 0) return PA_OK;
    if (!a->block_table || !a->block_table_len || !a->num_processed_tokens || !a->num_scheduled_tokens || !a->past_lens || !a->subsequence_begins ||
        !a->block_indices_begins || !a->totals || (a->block_indices_capacity > 0 && !a->block_indices))
        return fail(PA_ERR_INVALID_ARG, "NULL pointer");
    PA_CUDA(cudaSetDevice(h->device));
    pa::MarshalArgs m{};
    m.block_table = a->block_table; m.block_table_len = a->block_table_len; m.table_stride = a->table_stride; m.num_slots = a->num_slots;
    m.slot = a->slot; m.num_processed_tokens = a->num_processed_tokens; m.num_evicted_tokens = a->num_evicted_tokens;
    m.num_scheduled_tokens = a->num_scheduled_tokens; m.skip_mask = a->skip_mask; m.skip_words = a->skip_mask ? a->skip_words : 0;
    m.num_sequences = a->num_sequences; m.block_size = h->g.bs;
    m.past_lens = a->past_lens; m.subsequence_begins = a->subsequence_begins; m.block_indices = a->block_indices;
    m.block_indices_begins = a->block_indices_begins; m.totals = a->totals; m.block_indices_capacity = a->block_indices_capacity;
    m.status = h->status;
    int launches = 0;
    PA_CUDA(pa::launch_marshal(m, a->stream ? (cudaStream_t)a->stream : h->stream, &launches));
    h->launches += launches;
    return PA_OK;
}

int64_t pa_b200_launch_count(const pa_handle* h) { return h ? h->launches : -1; }
int pa_b200_last_prefill_kernel(const pa_handle* h) { return h ? h->last_prefill_kernel : -1; }

int pa_b200_set_kernel_timing(pa_handle* h, int enabled) {
    if (!h) return fail(PA_ERR_INVALID_ARG, "NULL handle");
    h->timing = enabled != 0;
    return PA_OK;
}

int pa_b200_get_kernel_timing(pa_handle* h, double* total_ms, int64_t* timed_launches) {
    if (!h || !total_ms || !timed_launches) return fail(PA_ERR_INVALID_ARG, "NULL argument");
    PA_CUDA(cudaSetDevice(h->device));
    double total = 0.0;
    for (size_t i = 0; i + 1 < h->ev_used; i += 2) {
        PA_CUDA(cudaEventSynchronize(h->ev[i + 1]));
        float ms = 0.f;
        PA_CUDA(cudaEventElapsedTime(&ms, h->ev[i], h->ev[i + 1]));
        total += ms;
    }
    *total_ms = total;
    *timed_launches = (int64_t)(h->ev_used / 2);
    h->ev_used = 0;
    return PA_OK;
}

// Host-tensor entry point.  Everything except the cache is packed into one pinned staging
// buffer, moved with a single host->device copy, and the results come back with one
// device->host copy per output tensor.
int pa_b200_forward_host(pa_handle* h, const pa_forward_args* a) {
    int rc = validate_args(h, a);
    if (rc != PA_OK) return rc;
    if (a->num_sequences == 0 || a->num_tokens == 0) return PA_OK;
    PA_CUDA(cudaSetDevice(h->device));
    cudaStream_t stream = a->stream ? (cudaStream_t)a->stream : h->stream;
    const pa::CacheGeom& g = h->g;
    const size_t ab = act_bytes(g.act);
    const size_t q_bytes = (size_t)a->num_tokens * g.Hq * g.D * ab;
    const size_t kv_bytes = (size_t)a->num_tokens * g.Hkv * g.D * ab;
    const size_t B = (size_t)a->num_sequences;

    struct Item { const void* src; size_t bytes; size_t off; };
    Item in[11];
    int n_in = 0;
    size_t off = 0;
    auto add = [&](const void* src, size_t bytes) {
        in[n_in] = Item{src, bytes, off};
        off += align_up(bytes, 256);
        return in[n_in++].off;
    };
    // metadata first (always staged through the handle's pinned buffer), then the activations, which are
    // copied straight from the caller's buffers when those are page-locked themselves
    const size_t o_past = add(a->past_lens, B * 4);
    const size_t o_sub = add(a->subsequence_begins, (B + 1) * 4);
    const size_t o_bi = add(a->block_indices, (size_t)a->num_block_indices * 4);
    const size_t o_bib = add(a->block_indices_begins, (B + 1) * 4);
    size_t o_saw = 0, o_rbi = 0, o_rd = 0, o_lut = 0;
    if (a->score_aggregation_window) o_saw = add(a->score_aggregation_window, B * 4);
    if (a->num_rotated_blocks > 0) {
        o_rbi = add(a->rotated_block_indices, (size_t)a->num_rotated_blocks * 4);
        o_rd = add(a->rotation_deltas, (size_t)a->num_rotated_blocks * 4);
        o_lut = add(a->rotation_trig_lut, (size_t)a->rotation_lut_rows * g.D * 4);
    }
    const int n_meta = n_in;
    const size_t meta_bytes = off;
    const size_t o_q = add(a->query, q_bytes);
    const size_t o_k = add(a->key, kv_bytes);
    const size_t o_v = add(a->value, kv_bytes);
    const size_t in_bytes = off;
    const size_t o_out = off;
    off += align_up(q_bytes, 256);
    const size_t o_scores = off;
    if (a->scores) off += align_up((size_t)a->scores_len * 4, 256);
    rc = ensure_stage(h, off);
    if (rc != PA_OK) return rc;

    auto page_locked = [](const void* p) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, p) != cudaSuccess) { cudaGetLastError(); return false; }
        return at.type == cudaMemoryTypeHost;
    };
    const bool direct = page_locked(a->query) && page_locked(a->key) && page_locked(a->value);
    const int n_staged = direct ? n_meta : n_in;
    for (int i = 0; i < n_staged; ++i)
        if (in[i].bytes) std::memcpy(h->stage_host + in[i].off, in[i].src, in[i].bytes);
    PA_CUDA(cudaMemcpyAsync(h->stage_dev, h->stage_host, direct ? meta_bytes : in_bytes, cudaMemcpyHostToDevice, stream));
    if (direct)
        for (int i = n_meta; i < n_in; ++i)
            if (in[i].bytes) PA_CUDA(cudaMemcpyAsync(h->stage_dev + in[i].off, in[i].src, in[i].bytes, cudaMemcpyHostToDevice, stream));

    pa_forward_args d = *a;
    uint8_t* base = h->stage_dev;
    d.query = base + o_q; d.key = base + o_k; d.value = base + o_v; d.output = base + o_out;
    d.past_lens = (const int32_t*)(base + o_past);
    d.subsequence_begins = (const int32_t*)(base + o_sub);
    d.block_indices = (const int32_t*)(base + o_bi);
    d.block_indices_begins = (const int32_t*)(base + o_bib);
    d.score_aggregation_window = a->score_aggregation_window ? (const int32_t*)(base + o_saw) : nullptr;
    d.scores = a->scores ? (float*)(base + o_scores) : nullptr;
    if (a->num_rotated_blocks > 0) {
        d.rotated_block_indices = (const int32_t*)(base + o_rbi);
        d.rotation_deltas = (const int32_t*)(base + o_rd);
        d.rotation_trig_lut = (const float*)(base + o_lut);
    }
    rc = run_forward(h, &d, stream);
    if (rc != PA_OK) return rc;
    PA_CUDA(cudaMemcpyAsync(a->output, base + o_out, q_bytes, cudaMemcpyDeviceToHost, stream));
    if (a->scores) PA_CUDA(cudaMemcpyAsync(a->scores, base + o_scores, (size_t)a->scores_len * 4, cudaMemcpyDeviceToHost, stream));
    // the status word comes back through the pinned staging buffer (a pageable target would make the copy synchronous)
    uint32_t* bits_host = reinterpret_cast<uint32_t*>(h->stage_host);
    PA_CUDA(cudaMemcpyAsync(bits_host, h->status, 4, cudaMemcpyDeviceToHost, stream));
    PA_CUDA(cudaStreamSynchronize(stream));
    const uint32_t bits = *bits_host;
    if (bits) {
        PA_CUDA(cudaMemsetAsync(h->status, 0, 4, stream));
        return fail(PA_ERR_BAD_INDEX, "device status word 0x" + std::to_string(bits));
    }
    return PA_OK;
}

}  // extern "C"
