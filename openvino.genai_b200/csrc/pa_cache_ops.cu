// Cache maintenance kernels of the PagedAttention operator: writing a chunk's new keys / values
// into their paged slots (with by-token u8 quantisation), re-rotating the keys of listed blocks,
// and block copies for copy-on-write.  All three are HBM-bound byte movers; one warp owns one
// (token, kv head) row so the min/max for the quantiser is a warp shuffle.
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

// Locates the sequence that owns flattened token `t` by binary search in subsequence_begins.
__device__ __forceinline__ int find_sequence(const int32_t* begins, int num_seq, int t) {
    int lo = 0, hi = num_seq;  // begins[lo] <= t < begins[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (begins[mid] <= t) lo = mid; else hi = mid;
    }
    return lo;
}

// Number of 32-token context tiles of one decode row (0 for rows that are not decode rows), plus the phantom tiles
// of the slicing sequence where the decode kernel asks for them.
__device__ __forceinline__ int seq_tiles(const KernelArgs& a, int s) {
    SeqView v;
    if (!seq_view(a, s, v) || v.n != 1) return 0;
    return (v.past + 1 + 31) / 32 + a.decode_phantom;
}

// Builds the decode plan with one block of 256 threads: the exclusive prefix sum of the per-row
// tile counts (workers slice the global tile sequence through it) and zeroed per-stream counters.
__device__ void build_decode_plan(const KernelArgs& a) {
    __shared__ int sh_warp[8];
    __shared__ int sh_run;
    __shared__ int sh_warp_p[8];
    __shared__ int sh_run_p;
    constexpr int kPrefixCap = 2048;           // rows whose prefix sums are also kept in shared memory
    __shared__ int sh_prefix[kPrefixCap + 1];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int B = a.num_sequences;
    const int G = a.g.Hq / a.g.Hkv, HK = a.g.Hkv * ((G + 15) / 16);
    if (tid == 0) { sh_run = 0; sh_run_p = 0; }
    __syncthreads();
    for (int base = 0; base < B; base += 256) {
        const int s = base + tid;
        const int n = s < B ? seq_tiles(a, s) : 0;
        // prefill chunks: q tiles of kPrefillItemRows (new token, q head of one group) pairs
        int np = 0;
        if (s < B) {
            SeqView sv;
            if (n == 0 && seq_view(a, s, sv) && sv.n > 1) np = (sv.n * G + kPrefillItemRows - 1) / kPrefillItemRows;
        }
        int v = n, vp = np;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, v, o), up = __shfl_up_sync(0xffffffffu, vp, o);
            if (lane >= o) { v += u; vp += up; }
        }
        if (lane == 31) { sh_warp[wid] = v; sh_warp_p[wid] = vp; }
        __syncthreads();
        int off = sh_run, offp = sh_run_p;
        for (int w = 0; w < wid; ++w) { off += sh_warp[w]; offp += sh_warp_p[w]; }
        if (s < B) {
            a.tile_prefix[s] = off + v - n;
            a.ptile_prefix[s] = offp + vp - np;
            if (s <= kPrefixCap) sh_prefix[s] = off + v - n;
        }
        __syncthreads();
        if (tid == 255) { sh_run = off + v; sh_run_p = offp + vp; }
        __syncthreads();
    }
    for (int i = tid; i < B * HK; i += 256) a.stream_done[i] = 0;
    // start records of the decode workers: the row that holds each slice's first tile
    if (a.worker_start && a.decode_all_workers > 0) {
        const int total_tiles = sh_run * HK;
        if (B <= kPrefixCap) {
            if (tid == 0) sh_prefix[B] = sh_run;
            __syncthreads();
            const DecodeSlices sl = decode_slices(total_tiles, a.decode_all_workers);
            for (int w = tid; w < a.decode_all_workers; w += 256) {
                WorkerStart ws{-1, 0, 0, total_tiles, 0, 0, 0, 0};
                const long long g_tile = sl.begin(w);
                if (w < sl.workers1 && g_tile < sl.end(w)) {
                    const int key = (int)(g_tile / HK);
                    int lo = 0, hi = B;   // sh_prefix[lo] <= key < sh_prefix[hi]
                    while (hi - lo > 1) {
                        const int mid = (lo + hi) >> 1;
                        if (sh_prefix[mid] <= key) lo = mid; else hi = mid;
                    }
                    const int tb = a.block_indices_begins[lo];
                    ws = WorkerStart{lo, sh_prefix[lo], sh_prefix[lo + 1] - sh_prefix[lo], total_tiles, a.past_lens[lo] + 1, tb,
                                     a.block_indices_begins[lo + 1] - tb, a.subsequence_begins[lo]};
                } else {
                    ws.s = -2;   // no tiles for this worker
                }
                a.worker_start[w] = ws;
            }
        } else {
            for (int w = tid; w < a.decode_all_workers; w += 256) a.worker_start[w] = WorkerStart{-1, 0, 0, total_tiles, 0, 0, 0, 0};
        }
    }
    // The prefill kernel hands out (q tile, kv head) items from a counter.  Longest context first keeps
    // the last items short, so the CTAs finish together; sequence order leaves a long item for the end.
    const int total_p = sh_run_p;
    const bool sort_items = a.pitem_order != nullptr && total_p > 1 && total_p <= kPrefillSortCap;
    if (sort_items) {
        __shared__ int sh_cost[kPrefillSortCap];
        if (tid == 0) a.ptile_prefix[B] = total_p;
        __syncthreads();   // the prefix sums written above are visible to the whole block
        for (int t = tid; t < total_p; t += 256) {
            int lo = 0, hi = B;   // ptile_prefix[lo] <= t < ptile_prefix[hi]
            while (hi - lo > 1) {
                const int mid = (lo + hi) >> 1;
                if (a.ptile_prefix[mid] <= t) lo = mid; else hi = mid;
            }
            const int p0 = a.ptile_prefix[lo], np = a.ptile_prefix[lo + 1] - p0;
            const int qt = np - 1 - (t - p0);   // the kernel's mapping: late (heavy) q tiles first
            const int n_new = a.subsequence_begins[lo + 1] - a.subsequence_begins[lo];
            const int r_hi = min(n_new * G, (qt + 1) * kPrefillItemRows) - 1;
            sh_cost[t] = a.past_lens[lo] + r_hi / G + 1;   // context of the q tile's last row
        }
        __syncthreads();
        for (int t = tid; t < total_p; t += 256) {
            const int c = sh_cost[t];
            int rank = 0;
            for (int u = 0; u < total_p; ++u) {
                const int cu = sh_cost[u];
                rank += (cu > c || (cu == c && u < t)) ? 1 : 0;
            }
            a.pitem_order[rank] = t;
        }
    }
    if (tid == 0) {
        a.tile_prefix[B] = sh_run;
        a.plan->total_tiles = sh_run * HK;
        a.ptile_prefix[B] = sh_run_p;
        a.plan->total_ptiles = sh_run_p;
        a.plan->next_pitem = 0;
        a.plan->pitems_sorted = sort_items ? 1 : 0;
    }
}

// One warp per (token, kv head).  Lane l owns dims {l + 32*i}.  With PLAN set, the last block of
// the grid builds the decode plan instead.
template <int D, bool PLAN>
__global__ void __launch_bounds__(256) write_kv_kernel(KernelArgs a) {
    constexpr int PER = D / 32;
    // No early griddepcontrol.launch_dependents here: decode CTAs placed while blocks of this grid still hold
    // shared memory do not all fit, and the decode kernel's static slices then run in two waves.
    if constexpr (PLAN) {
        if (blockIdx.x == gridDim.x - 1) {
            build_decode_plan(a);
            return;
        }
        // with a score output the block before the last prepares the score offsets and work list
        if (a.scores && a.score_aggregation_window && blockIdx.x == gridDim.x - 2) {
            if (threadIdx.x < 32) build_score_plan(a);
            return;
        }
    }
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int total = a.num_tokens * a.g.Hkv;
    if (warp >= total) return;
    const int t = warp / a.g.Hkv, h = warp % a.g.Hkv;
    const int s = find_sequence(a.subsequence_begins, a.num_sequences, t);
    SeqView sv;
    if (!seq_view(a, s, sv)) return;
    const int t0 = sv.t0, past = sv.past, tb = sv.tb;
    if (t < t0 || t >= t0 + sv.n) {   // prefix sums that are not monotone, or that leave tokens uncovered
        if (lane == 0) atomicOr(a.status, PA_DEV_BAD_BEGINS);
        return;
    }
    const int pos = past + (t - t0);
    const int block = a.block_indices[tb + pos / a.g.bs];
    if (block < 0 || block >= a.num_blocks) {
        if (lane == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
        return;
    }
    const int slot = pos % a.g.bs;
    const long long src = ((long long)t * a.g.Hkv + h) * D;
    const long long rec = (long long)block * a.g.block_bytes + (long long)h * a.g.head_bytes;
    float k[PER], v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        k[i] = load_act(a.key, src + lane + 32 * i, a.g.act);
        v[i] = load_act(a.value, src + lane + 32 * i, a.g.act);
    }
    if (a.g.cache == PA_DTYPE_U8) {
        uint8_t* kr = (uint8_t*)a.key_cache + rec;
        uint8_t* vr = (uint8_t*)a.value_cache + rec;
        float kmn = k[0], kmx = k[0], vmn = v[0], vmx = v[0];
#pragma unroll
        for (int i = 1; i < PER; ++i) {
            kmn = fminf(kmn, k[i]); kmx = fmaxf(kmx, k[i]);
            vmn = fminf(vmn, v[i]); vmx = fmaxf(vmx, v[i]);
        }
        kmn = warp_min(kmn); kmx = warp_max(kmx); vmn = warp_min(vmn); vmx = warp_max(vmx);
        float ks, kz, ki, vs, vz, vi;
        quant_params(kmn, kmx, ks, kz, ki);
        quant_params(vmn, vmx, vs, vz, vi);
        float* kp = (float*)(kr + (long long)a.g.bs * D);
        float* vp = (float*)(vr + (long long)a.g.bs * D);
        if (lane == 0) {
            kp[slot] = ks; kp[a.g.bs + slot] = kz;
            vp[slot] = vs; vp[a.g.bs + slot] = vz;
        }
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            kr[(long long)slot * D + d] = (uint8_t)quant_one(k[i], ki, kz);   // key data   [bs][D]
            vr[(long long)d * a.g.bs + slot] = (uint8_t)quant_one(v[i], vi, vz);  // value data [D][bs]
        }
    } else {
        uint16_t* kr = (uint16_t*)((uint8_t*)a.key_cache + rec) + (long long)slot * D;
        uint16_t* vr = (uint16_t*)((uint8_t*)a.value_cache + rec) + (long long)slot * D;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int d = lane + 32 * i;
            if (a.g.cache == PA_DTYPE_F16) {
                kr[d] = __half_as_ushort(__float2half_rn(k[i]));
                vr[d] = __half_as_ushort(__float2half_rn(v[i]));
            } else {
                kr[d] = __bfloat16_as_ushort(__float2bfloat16_rn(k[i]));
                vr[d] = __bfloat16_as_ushort(__float2bfloat16_rn(v[i]));
            }
        }
    }
}

// HALF / EL lanes per (rotated block, kv head, token).  Lane l owns the pairs (j, j + D/2) for
// j in EL*l .. EL*l + EL-1.  k'[j] = fma(-k[j+D/2], s, k[j]*c);  k'[j+D/2] = fma(k[j], s, k[j+D/2]*c)
// with c = lut[row][j], s = lut[row][D/2 + j].  EL = 8: the three divisions of a token's new scale and
// zero-point (every lane of the token computes them) are spread over sixteen elements per lane.
template <int D>
__global__ void __launch_bounds__(256) rotate_kernel(KernelArgs a) {
    constexpr int HALF = D / 2;
    constexpr int EL = 8;                  // pairs per lane: an 8-byte (u8) or 16-byte (f16 / bf16) vector per half
    constexpr int LPT = HALF / EL;         // lanes per token: 8 (D = 128) or 4 (D = 64)
    // One CTA per rotated block; its sub-warps walk the block's (kv head, token) units.
    const int l = threadIdx.x % LPT;
    const int r = blockIdx.x;
    const int units = a.g.Hkv * a.g.bs;
    const int block = a.rotated_block_indices[r];
    const int row = a.rotation_deltas[r];
    const bool bad = block < 0 || block >= a.num_blocks || row < 0 || row >= a.rotation_lut_rows;
    if (bad && threadIdx.x == 0) atomicOr(a.status, PA_DEV_BAD_ROTATION);
    const float* lut = a.rotation_trig_lut + (long long)(bad ? 0 : row) * D;
    float cv[EL], sv[EL];
#pragma unroll
    for (int i = 0; i < EL; i += 4) {
        const float4 c4 = *reinterpret_cast<const float4*>(lut + EL * l + i), s4 = *reinterpret_cast<const float4*>(lut + HALF + EL * l + i);
        cv[i] = c4.x; cv[i + 1] = c4.y; cv[i + 2] = c4.z; cv[i + 3] = c4.w;
        sv[i] = s4.x; sv[i + 1] = s4.y; sv[i + 2] = s4.z; sv[i + 3] = s4.w;
    }
    for (int base = 0; base < units; base += blockDim.x / LPT) {   // warp-uniform trip count
    const int unit = base + threadIdx.x / LPT;
    const bool live = unit < units;
    const int uu = live ? unit : units - 1;
    const int tok = uu % a.g.bs, h = uu / a.g.bs;
    const bool work = live && !bad;
    uint8_t* rec = (uint8_t*)a.key_cache + (long long)(bad ? 0 : block) * a.g.block_bytes + (long long)h * a.g.head_bytes;
    float* params = (float*)(rec + (long long)a.g.bs * D);
    float lo[EL], hi[EL];
#pragma unroll
    for (int i = 0; i < EL; ++i) { lo[i] = 0.f; hi[i] = 0.f; }
    if (work) {
        if (a.g.cache == PA_DTYPE_U8) {
            const float sc = params[tok], zp = params[a.g.bs + tok];
            const uint2 wl = *reinterpret_cast<const uint2*>(rec + (long long)tok * D + EL * l);
            const uint2 wh = *reinterpret_cast<const uint2*>(rec + (long long)tok * D + HALF + EL * l);
            const uint32_t wlv[2] = {wl.x, wl.y}, whv[2] = {wh.x, wh.y};
#pragma unroll
            for (int i = 0; i < EL; ++i) {
                lo[i] = dequant_one((wlv[i >> 2] >> (8 * (i & 3))) & 0xffu, sc, zp);
                hi[i] = dequant_one((whv[i >> 2] >> (8 * (i & 3))) & 0xffu, sc, zp);
            }
        } else {
            const uint16_t* p = (const uint16_t*)rec + (long long)tok * D;
            const uint4 wl = *reinterpret_cast<const uint4*>(p + EL * l), wh = *reinterpret_cast<const uint4*>(p + HALF + EL * l);
            const uint32_t wlv[4] = {wl.x, wl.y, wl.z, wl.w}, whv[4] = {wh.x, wh.y, wh.z, wh.w};
#pragma unroll
            for (int i = 0; i < EL; ++i) {
                const unsigned short el = (unsigned short)(wlv[i >> 1] >> (16 * (i & 1))), eh = (unsigned short)(whv[i >> 1] >> (16 * (i & 1)));
                if (a.g.cache == PA_DTYPE_F16) {
                    lo[i] = __half2float(__ushort_as_half(el));
                    hi[i] = __half2float(__ushort_as_half(eh));
                } else {
                    lo[i] = __bfloat162float(__ushort_as_bfloat16(el));
                    hi[i] = __bfloat162float(__ushort_as_bfloat16(eh));
                }
            }
        }
    }
    float nlo[EL], nhi[EL];
#pragma unroll
    for (int i = 0; i < EL; ++i) {
        nlo[i] = __fmaf_rn(-hi[i], sv[i], __fmul_rn(lo[i], cv[i]));
        nhi[i] = __fmaf_rn(lo[i], sv[i], __fmul_rn(hi[i], cv[i]));
    }
    if (a.g.cache == PA_DTYPE_U8) {
        float mn = fminf(nlo[0], nhi[0]), mx = fmaxf(nlo[0], nhi[0]);
#pragma unroll
        for (int i = 1; i < EL; ++i) {
            mn = fminf(mn, fminf(nlo[i], nhi[i]));
            mx = fmaxf(mx, fmaxf(nlo[i], nhi[i]));
        }
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) {   // over the token's lanes (every lane of the warp takes part)
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        float sc, zp, inv;
        quant_params(mn, mx, sc, zp, inv);
        __syncwarp();   // every lane has read the old parameters
        if (work) {
            if (l == 0) { params[tok] = sc; params[a.g.bs + tok] = zp; }
            uint32_t wlv[2] = {0, 0}, whv[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < EL; ++i) {
                wlv[i >> 2] |= quant_one(nlo[i], inv, zp) << (8 * (i & 3));
                whv[i >> 2] |= quant_one(nhi[i], inv, zp) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(rec + (long long)tok * D + EL * l) = make_uint2(wlv[0], wlv[1]);
            *reinterpret_cast<uint2*>(rec + (long long)tok * D + HALF + EL * l) = make_uint2(whv[0], whv[1]);
        }
    } else if (work) {
        uint16_t* p = (uint16_t*)rec + (long long)tok * D;
        uint32_t wlv[4] = {0, 0, 0, 0}, whv[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < EL; ++i) {
            unsigned short el, eh;
            if (a.g.cache == PA_DTYPE_F16) {
                el = __half_as_ushort(__float2half_rn(nlo[i]));
                eh = __half_as_ushort(__float2half_rn(nhi[i]));
            } else {
                el = __bfloat16_as_ushort(__float2bfloat16_rn(nlo[i]));
                eh = __bfloat16_as_ushort(__float2bfloat16_rn(nhi[i]));
            }
            wlv[i >> 1] |= (uint32_t)el << (16 * (i & 1));
            whv[i >> 1] |= (uint32_t)eh << (16 * (i & 1));
        }
        *reinterpret_cast<uint4*>(p + EL * l) = make_uint4(wlv[0], wlv[1], wlv[2], wlv[3]);
        *reinterpret_cast<uint4*>(p + HALF + EL * l) = make_uint4(whv[0], whv[1], whv[2], whv[3]);
    }
    }
}

// Block copies: grid.x = pair, grid.y = slice of the block.  16-byte vectors.
__global__ void __launch_bounds__(256) copy_blocks_kernel(uint8_t* key_cache, uint8_t* value_cache, long long block_bytes,
                                                          int num_blocks, const int32_t* pairs, uint32_t* status) {
    const int src = pairs[2 * blockIdx.x], dst = pairs[2 * blockIdx.x + 1];
    if (src < 0 || src >= num_blocks || dst < 0 || dst >= num_blocks) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, PA_DEV_BAD_BLOCK_INDEX);
        return;
    }
    if (src == dst) return;
    const long long vecs = block_bytes / 16;
    const uint4* ks = (const uint4*)(key_cache + (long long)src * block_bytes);
    uint4* kd = (uint4*)(key_cache + (long long)dst * block_bytes);
    const uint4* vs = (const uint4*)(value_cache + (long long)src * block_bytes);
    uint4* vd = (uint4*)(value_cache + (long long)dst * block_bytes);
    for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.y * blockDim.x) {
        kd[i] = ks[i];
        vd[i] = vs[i];
    }
}

}  // namespace

cudaError_t launch_write_kv(const KernelArgs& a, cudaStream_t stream, bool with_plan) {
    if (a.num_tokens <= 0 && !with_plan) return cudaSuccess;
    const long long warps = (long long)a.num_tokens * a.g.Hkv;
    const int grid = (int)((warps * 32 + 255) / 256) + (with_plan ? 1 : 0) + (with_plan && a.scores && a.score_aggregation_window ? 1 : 0);
    if (a.g.D == 128) {
        if (with_plan) write_kv_kernel<128, true><<<grid, 256, 0, stream>>>(a);
        else write_kv_kernel<128, false><<<grid, 256, 0, stream>>>(a);
    } else {
        if (with_plan) write_kv_kernel<64, true><<<grid, 256, 0, stream>>>(a);
        else write_kv_kernel<64, false><<<grid, 256, 0, stream>>>(a);
    }
    return cudaGetLastError();
}

cudaError_t launch_rotate(const KernelArgs& a, cudaStream_t stream) {
    if (a.num_rotated_blocks <= 0) return cudaSuccess;
    const int grid = a.num_rotated_blocks;
    if (a.g.D == 128) rotate_kernel<128><<<grid, 256, 0, stream>>>(a);
    else rotate_kernel<64><<<grid, 256, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_copy_blocks(void* key_cache, void* value_cache, long long block_bytes, int num_blocks,
                               const int32_t* pairs, int num_pairs, uint32_t* status, cudaStream_t stream) {
    if (num_pairs <= 0) return cudaSuccess;
    dim3 grid(num_pairs, 8);
    copy_blocks_kernel<<<grid, 256, 0, stream>>>((uint8_t*)key_cache, (uint8_t*)value_cache, block_bytes, num_blocks, pairs, status);
    return cudaGetLastError();
}

}  // namespace pa
