// Allocation-free decode step: pa_b200_decode_step_static (include/pa_b200.h).
//
// Some callers may not allocate device memory at the point where they run the operator: code that
// runs inside a memory-pool or allocator callback, a serving loop whose device memory is fully
// handed out up front, or a latency-critical step that must not take the allocator's lock.  For
// them the scratch the decode path needs (plan, per-stream counters, partial results of context
// slices) lives in one file-scope device array of fixed size that every GPU loading this library
// holds until the process exits.
//
// In host code the array's NAME is only a host-side stand-in for the symbol; it is not a device
// address.  The device address is obtained once per device, with that device current, through
// cudaGetSymbolAddress, and that pointer is what the kernels receive.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <mutex>
#include <string>

#include "pa_kernels.h"

namespace pa {
void set_last_error(const std::string& msg);  // pa_api.cu
}

namespace {

constexpr size_t kStaticScratchBytes = PA_B200_STATIC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// The scratch itself.  Shared by every call on the device; it keeps the previous call's contents.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

struct DeviceSetup {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int sm_count = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

size_t up256(size_t x) { return (x + 255) / 256 * 256; }

int fail_static(int code, const std::string& msg) {
    pa::set_last_error(msg);
    return code;
}

}  // namespace

extern "C" int pa_b200_decode_step_static(const pa_model_desc* desc, const pa_forward_args* a, int device) {
    if (!desc || desc->struct_size != sizeof(pa_model_desc) || !a || a->struct_size != sizeof(pa_forward_args))
        return fail_static(PA_ERR_INVALID_ARG, "pa_b200_decode_step_static: NULL argument or struct_size mismatch");
    if (device < 0 || device >= kMaxDevices) return fail_static(PA_ERR_INVALID_ARG, "device ordinal out of range");
    if (desc->num_q_heads <= 0 || desc->num_kv_heads <= 0 || desc->num_q_heads % desc->num_kv_heads != 0 ||
        (desc->head_size != 64 && desc->head_size != 128) || (desc->block_size != 16 && desc->block_size != 32) ||
        (desc->cache_dtype != PA_DTYPE_F16 && desc->cache_dtype != PA_DTYPE_BF16 && desc->cache_dtype != PA_DTYPE_U8) ||
        (desc->act_dtype != PA_DTYPE_F32 && desc->act_dtype != PA_DTYPE_F16 && desc->act_dtype != PA_DTYPE_BF16))
        return fail_static(PA_ERR_UNSUPPORTED, "pa_b200_decode_step_static: unsupported model description");
    if (a->sliding_window != 0 || a->alibi_slopes) return fail_static(PA_ERR_UNSUPPORTED, "sliding_window / alibi are not supported");
    if (a->scores || a->score_aggregation_window || a->num_rotated_blocks != 0)
        return fail_static(PA_ERR_UNSUPPORTED, "the allocation-free entry point covers plain decode steps only (no scores, no rotation)");
    if (a->num_tokens != a->num_sequences || a->num_sequences < 0)
        return fail_static(PA_ERR_UNSUPPORTED, "the allocation-free entry point needs exactly one new token per sequence");
    if (a->num_sequences == 0) return PA_OK;
    if (a->num_sequences > 65535) return fail_static(PA_ERR_TOO_LARGE, "more than 65535 sequences in one call");
    if (!a->query || !a->key || !a->value || !a->output || !a->key_cache || !a->value_cache || !a->past_lens || !a->subsequence_begins ||
        !a->block_indices || !a->block_indices_begins)
        return fail_static(PA_ERR_INVALID_ARG, "NULL pointer");

    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail_static(PA_ERR_CUDA, std::string("cudaSetDevice: ") + cudaGetErrorString(e));

    // ---- set-up, once per device, with that device current ----------------------------------------
    DeviceSetup& st = g_setup[device];
    {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        if (!st.ready) {
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr)
                return fail_static(PA_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess) return fail_static(PA_ERR_CUDA, std::string("cudaDeviceGetAttribute: ") + cudaGetErrorString(e));
            int major = 0;
            e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
            if (e != cudaSuccess || major != 10) return fail_static(PA_ERR_NO_DEVICE, "this library is built for sm_100a only");
            st.scratch = static_cast<unsigned char*>(ptr);
            st.sm_count = sms;
            st.ready = true;
        }
    }

    // ---- carve the fixed scratch ---------------------------------------------------------------------
    pa::CacheGeom g;
    g.Hq = desc->num_q_heads; g.Hkv = desc->num_kv_heads; g.D = desc->head_size; g.bs = desc->block_size;
    g.act = desc->act_dtype; g.cache = desc->cache_dtype;
    g.head_bytes = pa::head_record_bytes(desc->cache_dtype, desc->block_size, desc->head_size);
    g.block_bytes = g.head_bytes * desc->num_kv_heads;
    const int G = g.Hq / g.Hkv, gtiles = (G + 15) / 16, HK = g.Hkv * gtiles, RT = std::min(G, 16);
    const long long B = a->num_sequences;
    long long tiles = B * ((std::max(a->max_context_len, 1) + 31) / 32);
    if (a->num_block_indices >= 0) tiles = std::min(tiles, (long long)a->num_block_indices * g.bs / 32 + B);
    const long long slots = B * HK + pa::decode_max_workers(st.sm_count);
    size_t off = 0;
    const size_t o_status = off; off += 256;
    const size_t o_hdr = off;    off += 256;
    const size_t o_prefix = off; off += up256((size_t)(B + 1) * sizeof(int));
    const size_t o_pprefix = off; off += up256((size_t)(B + 1) * sizeof(int));
    const size_t o_done = off;   off += up256((size_t)B * HK * sizeof(int));
    const size_t o_part_o = off; off += up256((size_t)slots * RT * g.D * sizeof(float));
    const size_t o_part_ml = off; off += up256((size_t)slots * RT * 2 * sizeof(float));
    if (off > kStaticScratchBytes)
        return fail_static(PA_ERR_TOO_LARGE, "pa_b200_decode_step_static: this step needs " + std::to_string(off) +
                                                 " bytes of scratch, the fixed array holds " + std::to_string(kStaticScratchBytes) +
                                                 "; use pa_b200_forward for larger batches");

    pa::KernelArgs k;
    std::memset(&k, 0, sizeof(k));
    k.g = g;
    k.query = a->query; k.key = a->key; k.value = a->value; k.output = a->output;
    k.num_tokens = a->num_tokens;
    k.key_cache = a->key_cache; k.value_cache = a->value_cache; k.num_blocks = a->num_blocks;
    k.past_lens = a->past_lens; k.subsequence_begins = a->subsequence_begins;
    k.block_indices = a->block_indices; k.block_indices_begins = a->block_indices_begins;
    k.num_block_indices = a->num_block_indices;
    k.num_sequences = a->num_sequences; k.max_context_len = a->max_context_len;
    k.scale = a->scale;
    unsigned char* base = st.scratch;  // device address from cudaGetSymbolAddress, never the symbol's name
    k.status = reinterpret_cast<uint32_t*>(base + o_status);
    k.plan = reinterpret_cast<pa::PlanHeader*>(base + o_hdr);
    k.worker_start = nullptr;      // the workers locate their slices themselves on this path
    k.decode_all_workers = 0;
    k.tile_prefix = reinterpret_cast<int*>(base + o_prefix);
    k.ptile_prefix = reinterpret_cast<int*>(base + o_pprefix);
    k.stream_done = reinterpret_cast<int*>(base + o_done);
    k.part_o = reinterpret_cast<float*>(base + o_part_o);
    k.part_ml = reinterpret_cast<float*>(base + o_part_ml);
    k.lse = nullptr;
    k.max_tiles = tiles * HK;
    k.rows_per_tile = RT;

    // The plan step of the first launch rewrites the header, the prefix sums and the per-stream
    // counters, which is everything that must start from a known state; partial results are
    // written before they are read.
    cudaStream_t stream = (cudaStream_t)a->stream;
    e = pa::launch_write_kv(k, stream, /*with_plan=*/true);
    if (e != cudaSuccess) return fail_static(PA_ERR_CUDA, std::string("write_kv launch: ") + cudaGetErrorString(e));
    int launches = 0;
    e = pa::launch_decode(k, stream, st.sm_count, &launches);
    if (e != cudaSuccess) return fail_static(PA_ERR_CUDA, std::string("decode launch: ") + cudaGetErrorString(e));
    return PA_OK;
}
