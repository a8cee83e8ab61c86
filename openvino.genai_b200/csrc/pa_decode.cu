// Paged decode attention for sm_100a: rows with exactly one new token.
//
// Work split: one CTA per (sequence, kv head, context split).  Inside the CTA each of the four
// warps owns a private multi-stage shared-memory ring and walks its own 32-token tiles of the
// block table, so the main loop needs no block-wide barrier:
//   * u8 cache   - lane 0 issues one TMA-engine bulk copy per (block, head) record (data +
//                  per-token scale / zero-point, contiguous and 16-byte aligned), completion on
//                  an mbarrier; bytes are turned into exact f16 in registers
//                  (byte | 0x6400 = 1024 + byte) and the zero-point is folded algebraically:
//                     q.k  = ks * (q.k_u8 - kz * sum(q))
//                     p.v  = sum_t (p*vs)_t * v_u8 - sum_t (p*vs)_t * vz_t
//   * f16 / bf16 - all lanes issue 16-byte cp.async into an XOR-swizzled tile read by ldmatrix.
// Q.K^T and P.V run on mma.sync m16n8k16 with the GQA group as the M dimension, so a KV byte is
// read from HBM once for all q heads that share it.  Softmax is online per warp; the four warps
// are merged through shared memory, the context splits through a small fp32 scratch and a
// merge kernel.  The kernel is bound by HBM: 2*Hkv*(D+8) bytes per context token for u8.
#include "pa_common.cuh"
#include "pa_kernels.h"

namespace pa {

namespace {

constexpr int kTile = 32;       // context tokens per pipeline stage
constexpr int kDecodeWarps = 4;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

template <int D, int BS, int CACHE>
struct DecodeCfg {
    static constexpr bool U8 = CACHE == PA_DTYPE_U8;
    static constexpr bool BF16 = CACHE == PA_DTYPE_BF16;
    static constexpr int REC = U8 ? BS * (D + 8) : BS * D * 2;  // bytes of one (block, head) record
    static constexpr int NREC = kTile / BS;                     // records per tile
    static constexpr int HALF_STAGE = NREC * REC;               // K part (V part has the same size)
    static constexpr int STAGE = 2 * HALF_STAGE;
    static constexpr int NSTAGE = 3;
    static constexpr int RING = NSTAGE * STAGE;                 // per warp
    static constexpr int SMEM = kDecodeWarps * RING + kDecodeWarps * NSTAGE * 8;
};

struct SeqInfo {
    int t0, past, ctx, nb;
    const int32_t* table;
};

template <int D, int BS, int CACHE, bool HI>
__global__ void __launch_bounds__(kDecodeWarps * 32) decode_kernel(KernelArgs a) {
    using Cfg = DecodeCfg<D, BS, CACHE>;
    constexpr bool U8 = Cfg::U8;
    constexpr bool BF16 = Cfg::BF16;
    constexpr int NKK = D / 16;   // k-steps of Q.K^T
    constexpr int NDT = D / 8;    // n-tiles of P.V
    constexpr int ROWS = HI ? 2 : 1;

    extern __shared__ __align__(128) uint8_t smem[];

    const int s = blockIdx.z;
    const int t0 = a.subsequence_begins[s];
    const int n_new = a.subsequence_begins[s + 1] - t0;
    if (n_new != 1) return;  // prefill chunks are handled elsewhere
    const int past = a.past_lens[s];
    const int tb = a.block_indices_begins[s];
    const int nb = a.block_indices_begins[s + 1] - tb;
    if (past < 0 || nb < 0 || (long long)nb * BS < (long long)past + 1) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicOr(a.status, PA_DEV_BAD_PAST_LEN);
        return;
    }
    const int ctx = past + 1;
    const int split = blockIdx.x;
    const int tok_begin = split * a.split_tokens;
    if (tok_begin >= ctx) return;
    const int tok_end = min(ctx, tok_begin + a.split_tokens);
    const int nsplit = (ctx + a.split_tokens - 1) / a.split_tokens;
    const int32_t* table = a.block_indices + tb;

    const int G = a.g.Hq / a.g.Hkv;
    const int gtiles = (G + 15) / 16;
    const int hk = blockIdx.y / gtiles;
    const int hbase = hk * G + (blockIdx.y % gtiles) * 16;  // first q head of this CTA
    const int hcount = min(16, hk * G + G - hbase);          // q heads of this CTA (<= 8 unless HI)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, c = lane & 3;

    uint8_t* ring = smem + warp * Cfg::RING;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kDecodeWarps * Cfg::RING) + warp * Cfg::NSTAGE;
    if constexpr (U8) {
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < Cfg::NSTAGE; ++i) mbar_init(&bars[i], 1);
            mbar_fence_init();
        }
        __syncwarp();
    }

    // ---- Q fragments ---------------------------------------------------------------------
    // u8: the contraction index is permuted so that one 16-byte shared load of a key row feeds
    // four k-steps: k-step kk = 4*half + i covers dims 64*half + 16*c + 4*i + {0..3} for lane c.
    uint32_t qa[NKK][4];
    float qsum[ROWS], qscale[ROWS];  // sum of the f16 q row (u8 zero-point term); logit scale in log2 units
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int hrow = g + 8 * r;
        const bool live = hrow < hcount;
        const long long qoff = ((long long)t0 * a.g.Hq + hbase + hrow) * D;
        float q[D / 4];
        float amax = 0.f;
#pragma unroll
        for (int e = 0; e < D / 4; ++e) {
            int d;
            if constexpr (U8) d = 64 * (e / 16) + 16 * c + (e % 16);
            else d = 16 * (e / 4) + 2 * c + (e & 1) + 8 * ((e >> 1) & 1);
            q[e] = live ? load_act(a.query, qoff + d, a.g.act) : 0.f;
            amax = fmaxf(amax, fabsf(q[e]));
        }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        // keep |q| inside the f16 range with an exact power-of-two prescale
        float qmul = 1.f;
        if (!BF16 && amax > 32768.f && amax < INFINITY) {
            int ex;
            frexpf(amax, &ex);
            qmul = ldexpf(1.f, 15 - ex);
        }
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < D / 4; e += 2) {
            uint32_t packed;
            if constexpr (BF16) {
                packed = pack_bf2(q[e], q[e + 1]);
            } else {
                packed = pack_h2(q[e] * qmul, q[e + 1] * qmul);
                __half2 h = *reinterpret_cast<__half2*>(&packed);
                sum += __low2float(h) + __high2float(h);
            }
            const int kk = e / 4;
            qa[kk][r + 2 * ((e >> 1) & 1)] = packed;
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        qsum[r] = sum;
        const float sm_scale = a.scale != 0.f ? a.scale : rsqrtf((float)D);
        qscale[r] = sm_scale * kLog2e / qmul;
    }
    if constexpr (!HI) {
#pragma unroll
        for (int kk = 0; kk < NKK; ++kk) { qa[kk][1] = 0u; qa[kk][3] = 0u; }
    }

    // ---- tile schedule of this warp ------------------------------------------------------------
    const int first_tile = tok_begin / kTile;
    const int num_tiles = (tok_end - tok_begin + kTile - 1) / kTile;
    const int my_tiles = num_tiles > warp ? (num_tiles - warp + kDecodeWarps - 1) / kDecodeWarps : 0;
    const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)hk * a.g.head_bytes;
    const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)hk * a.g.head_bytes;
    bool bad_index = false;

    auto issue = [&](int it) {
        const int tile = first_tile + warp + it * kDecodeWarps;
        uint8_t* st = ring + (it % Cfg::NSTAGE) * Cfg::STAGE;
        if constexpr (U8) {
            if (lane == 0) {
                int blocks[Cfg::NREC];
                uint32_t bytes = 0;
#pragma unroll
                for (int r = 0; r < Cfg::NREC; ++r) {
                    const int bi = tile * Cfg::NREC + r;
                    int blk = -1;
                    if (bi < nb && bi * BS < tok_end) {
                        blk = table[bi];
                        if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                        bytes += 2 * Cfg::REC;
                    }
                    blocks[r] = blk;
                }
                uint64_t* bar = &bars[it % Cfg::NSTAGE];
                mbar_expect_tx(bar, bytes);
#pragma unroll
                for (int r = 0; r < Cfg::NREC; ++r)
                    if (blocks[r] >= 0) {
                        bulk_g2s(st + r * Cfg::REC, kc + (long long)blocks[r] * a.g.block_bytes, Cfg::REC, bar);
                        bulk_g2s(st + Cfg::HALF_STAGE + r * Cfg::REC, vc + (long long)blocks[r] * a.g.block_bytes, Cfg::REC, bar);
                    }
            }
        } else {
            constexpr int CPR = D / 8;  // 16-byte chunks per token row
#pragma unroll
            for (int r = 0; r < Cfg::NREC; ++r) {
                const int bi = tile * Cfg::NREC + r;
                if (bi < nb && bi * BS < tok_end) {
                    int blk = table[bi];
                    if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                    const uint8_t* ksrc = kc + (long long)blk * a.g.block_bytes;
                    const uint8_t* vsrc = vc + (long long)blk * a.g.block_bytes;
#pragma unroll
                    for (int i = lane; i < BS * CPR; i += 32) {
                        const int row = r * BS + i / CPR, ch = i % CPR;
                        const int dst = row * (2 * D) + ((ch ^ (row & 7)) << 4);
                        cp_async16(st + dst, ksrc + (long long)i * 16);
                        cp_async16(st + Cfg::HALF_STAGE + dst, vsrc + (long long)i * 16);
                    }
                }
            }
        }
    };

    // ---- running state ----------------------------------------------------------------------------
    float oacc[NDT][2 * ROWS];
#pragma unroll
    for (int i = 0; i < NDT; ++i)
#pragma unroll
        for (int r = 0; r < 2 * ROWS; ++r) oacc[i][r] = 0.f;
    float m_run[ROWS], l_run[ROWS], z_run[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { m_run[r] = -INFINITY; l_run[r] = 0.f; z_run[r] = 0.f; }

#pragma unroll
    for (int p = 0; p < Cfg::NSTAGE - 1; ++p) {
        if (p < my_tiles) issue(p);
        if constexpr (!U8) cp_async_commit();
    }

    bool timed_out = false;
    for (int it = 0; it < my_tiles; ++it) {
        __syncwarp();  // every lane is done with the stage that is refilled next
        if (it + Cfg::NSTAGE - 1 < my_tiles) issue(it + Cfg::NSTAGE - 1);
        if constexpr (U8) {
            if (!mbar_wait_bounded(&bars[it % Cfg::NSTAGE], (it / Cfg::NSTAGE) & 1)) { timed_out = true; break; }
        } else {
            cp_async_commit();
            cp_async_wait<Cfg::NSTAGE - 1>();
            __syncwarp();
        }
        const uint8_t* st = ring + (it % Cfg::NSTAGE) * Cfg::STAGE;
        const int tile_base = (first_tile + warp + it * kDecodeWarps) * kTile;
        const int valid = tok_end - tile_base;  // tokens of this tile inside the split (may exceed 32)

        if constexpr (!U8) {
            if (valid < kTile) {  // stale rows of a partly filled block may hold NaN bit patterns
                constexpr int CPR = D / 8;
                for (int i = lane; i < (kTile - valid) * CPR; i += 32) {
                    const int row = valid + i / CPR, ch = i % CPR;
                    *reinterpret_cast<uint4*>(const_cast<uint8_t*>(st) + Cfg::HALF_STAGE + row * 2 * D + (ch << 4)) = make_uint4(0, 0, 0, 0);
                }
                __syncwarp();
            }
        }

        // ---- S = Q.K^T over four 8-token n-tiles ------------------------------------------------
        float sacc[4][2 * ROWS];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
            for (int r = 0; r < 2 * ROWS; ++r) sacc[j][r] = 0.f;
            float acc4[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (U8) {
                const int row = 8 * (g >> 1) + 2 * j + (g & 1);
                const uint8_t* kp = st + (row / BS) * Cfg::REC + (row % BS) * D + 16 * c;
#pragma unroll
                for (int h = 0; h < D / 64; ++h) {
                    const uint4 w = *reinterpret_cast<const uint4*>(kp + 64 * h);
                    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        mma16816<false, HI>(acc4, qa[4 * h + i], u8x2_to_h2_lo(ww[i]), u8x2_to_h2_hi(ww[i]));
                }
            } else {
#pragma unroll
                for (int p = 0; p < NKK / 2; ++p) {
                    const int row = 8 * j + (lane & 7), ch = 4 * p + (lane >> 3);
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(st + row * 2 * D + ((ch ^ (row & 7)) << 4)));
                    mma16816<BF16, HI>(acc4, qa[2 * p], b[0], b[1]);
                    mma16816<BF16, HI>(acc4, qa[2 * p + 1], b[2], b[3]);
                }
            }
            sacc[j][0] = acc4[0]; sacc[j][1] = acc4[1];
            if constexpr (HI) { sacc[j][2] = acc4[2]; sacc[j][3] = acc4[3]; }
        }

        // ---- scale, mask, online softmax -----------------------------------------------------------
        float vsc[4][2], vzp[4][2];
        float tmax[ROWS];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) tmax[r] = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tk = U8 ? 8 * c + 2 * j : 8 * j + 2 * c;  // tile token of accumulator column 0
            float ks0 = 1.f, ks1 = 1.f, kz0 = 0.f, kz1 = 0.f;
            if constexpr (U8) {
                const uint8_t* kp = st + (tk / BS) * Cfg::REC + BS * D;
                const float2 ks = *reinterpret_cast<const float2*>(kp + 4 * (tk % BS));
                const float2 kz = *reinterpret_cast<const float2*>(kp + 4 * BS + 4 * (tk % BS));
                ks0 = ks.x; ks1 = ks.y; kz0 = kz.x; kz1 = kz.y;
                const uint8_t* vp = st + Cfg::HALF_STAGE + (tk / BS) * Cfg::REC + BS * D;
                const float2 vs = *reinterpret_cast<const float2*>(vp + 4 * (tk % BS));
                const float2 vz = *reinterpret_cast<const float2*>(vp + 4 * BS + 4 * (tk % BS));
                vsc[j][0] = vs.x; vsc[j][1] = vs.y; vzp[j][0] = vz.x; vzp[j][1] = vz.y;
            }
            const bool ok0 = tk < valid, ok1 = tk + 1 < valid;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) {
                float s0 = sacc[j][2 * r], s1 = sacc[j][2 * r + 1];
                if constexpr (U8) {
                    s0 = (s0 - kz0 * qsum[r]) * ks0;
                    s1 = (s1 - kz1 * qsum[r]) * ks1;
                }
                s0 = ok0 ? s0 * qscale[r] : -INFINITY;
                s1 = ok1 ? s1 * qscale[r] : -INFINITY;
                sacc[j][2 * r] = s0; sacc[j][2 * r + 1] = s1;
                tmax[r] = fmaxf(tmax[r], fmaxf(s0, s1));
            }
        }
        uint32_t pa_frag[2][4];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float mx = tmax[r];
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[r], mx);       // finite: every tile has >= 1 valid token
            const float alpha = exp2f(m_run[r] - m_new);   // 0 on the first tile
            m_run[r] = m_new;
            l_run[r] *= alpha;
            z_run[r] *= alpha;
#pragma unroll
            for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] *= alpha; oacc[i][2 * r + 1] *= alpha; }
            float lsum = 0.f, zsum = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tk = U8 ? 8 * c + 2 * j : 8 * j + 2 * c;
                const float p0 = exp2f(sacc[j][2 * r] - m_new), p1 = exp2f(sacc[j][2 * r + 1] - m_new);
                lsum += p0 + p1;
                uint32_t packed;
                if constexpr (U8) {
                    packed = pack_h2(tk < valid ? p0 * vsc[j][0] : 0.f, tk + 1 < valid ? p1 * vsc[j][1] : 0.f);
                    const __half2 h = *reinterpret_cast<__half2*>(&packed);
                    zsum += (tk < valid ? __low2float(h) * vzp[j][0] : 0.f) + (tk + 1 < valid ? __high2float(h) * vzp[j][1] : 0.f);
                } else if constexpr (BF16) {
                    packed = pack_bf2(p0, p1);
                } else {
                    packed = pack_h2(p0, p1);
                }
                pa_frag[j >> 1][r + 2 * (j & 1)] = packed;
            }
            l_run[r] += lsum;
            z_run[r] += zsum;
        }
        if constexpr (!HI) { pa_frag[0][1] = pa_frag[0][3] = pa_frag[1][1] = pa_frag[1][3] = 0u; }

        // ---- O += P.V -----------------------------------------------------------------------------
        if constexpr (U8) {
#pragma unroll
            for (int i = 0; i < NDT; ++i) {
                const int d = 8 * i + g;
                const uint8_t* vp = st + Cfg::HALF_STAGE + ((8 * c) / BS) * Cfg::REC + d * BS + ((8 * c) % BS);
                const uint2 w = *reinterpret_cast<const uint2*>(vp);
                float acc4[4];
                acc4[0] = oacc[i][0]; acc4[1] = oacc[i][1];
                if constexpr (HI) { acc4[2] = oacc[i][2]; acc4[3] = oacc[i][3]; }
                mma16816<false, HI>(acc4, pa_frag[0], u8x2_to_h2_lo(w.x), u8x2_to_h2_hi(w.x));
                mma16816<false, HI>(acc4, pa_frag[1], u8x2_to_h2_lo(w.y), u8x2_to_h2_hi(w.y));
                oacc[i][0] = acc4[0]; oacc[i][1] = acc4[1];
                if constexpr (HI) { oacc[i][2] = acc4[2]; oacc[i][3] = acc4[3]; }
            }
        } else {
#pragma unroll
            for (int kt = 0; kt < 2; ++kt)
#pragma unroll
                for (int q = 0; q < NDT / 2; ++q) {
                    const int row = 16 * kt + 8 * ((lane >> 3) & 1) + (lane & 7), ch = 2 * q + (lane >> 4);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(st + Cfg::HALF_STAGE + row * 2 * D + ((ch ^ (row & 7)) << 4)));
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int i = 2 * q + e;
                        float acc4[4];
                        acc4[0] = oacc[i][0]; acc4[1] = oacc[i][1];
                        if constexpr (HI) { acc4[2] = oacc[i][2]; acc4[3] = oacc[i][3]; }
                        mma16816<BF16, HI>(acc4, pa_frag[kt], b[2 * e], b[2 * e + 1]);
                        oacc[i][0] = acc4[0]; oacc[i][1] = acc4[1];
                        if constexpr (HI) { oacc[i][2] = acc4[2]; oacc[i][3] = acc4[3]; }
                    }
                }
        }
    }
    if constexpr (!U8) cp_async_wait<0>();
    if (timed_out || bad_index) {
        if (lane == 0) atomicOr(a.status, bad_index ? PA_DEV_BAD_BLOCK_INDEX : 0x80000000u);
    }

    // ---- fold the zero-point term, reduce the row sums over the four lanes of a row ---------------
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        float l = l_run[r], z = z_run[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1); l += __shfl_xor_sync(0xffffffffu, l, 2);
        z += __shfl_xor_sync(0xffffffffu, z, 1); z += __shfl_xor_sync(0xffffffffu, z, 2);
        l_run[r] = l;
#pragma unroll
        for (int i = 0; i < NDT; ++i) { oacc[i][2 * r] -= z; oacc[i][2 * r + 1] -= z; }
    }

    // ---- merge the four warps through shared memory (the rings are free now) ----------------------
    __syncthreads();
    constexpr int HROWS = 8 * ROWS;
    float* sm_o = reinterpret_cast<float*>(smem);              // [warp][HROWS][D]
    float* sm_m = sm_o + kDecodeWarps * HROWS * D;             // [warp][HROWS]
    float* sm_l = sm_m + kDecodeWarps * HROWS;                 // [warp][HROWS]
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int hrow = g + 8 * r;
#pragma unroll
        for (int i = 0; i < NDT; ++i) {
            float2 v = make_float2(oacc[i][2 * r], oacc[i][2 * r + 1]);
            *reinterpret_cast<float2*>(&sm_o[(warp * HROWS + hrow) * D + 8 * i + 2 * c]) = v;
        }
        if (c == 0) { sm_m[warp * HROWS + hrow] = m_run[r]; sm_l[warp * HROWS + hrow] = l_run[r]; }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < hcount * D; idx += blockDim.x) {
        const int hrow = idx / D, d = idx % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) m = fmaxf(m, sm_m[w * HROWS + hrow]);
        float o = 0.f, l = 0.f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float mw = sm_m[w * HROWS + hrow];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - m);
            o += f * sm_o[(w * HROWS + hrow) * D + d];
            l += f * sm_l[w * HROWS + hrow];
        }
        const int hq = hbase + hrow;
        if (nsplit == 1) {
            store_act(a.output, ((long long)t0 * a.g.Hq + hq) * D + d, a.g.act, o / l);
            if (d == 0 && a.lse) a.lse[(long long)t0 * a.g.Hq + hq] = (m + log2f(l)) * kLn2;
        } else {
            const long long slot = ((long long)s * a.g.Hq + hq) * a.max_splits + split;
            a.part_o[slot * D + d] = o;
            if (d == 0) { a.part_ml[slot * 2] = m; a.part_ml[slot * 2 + 1] = l; }
        }
    }
}

// Combines the context splits of one (sequence, q head): grid (Hq, num_sequences), D threads.
template <int D>
__global__ void __launch_bounds__(D) decode_merge_kernel(KernelArgs a) {
    const int s = blockIdx.y, hq = blockIdx.x, d = threadIdx.x;
    const int t0 = a.subsequence_begins[s];
    if (a.subsequence_begins[s + 1] - t0 != 1) return;
    const int past = a.past_lens[s];
    if (past < 0) return;
    const int nsplit = (past + 1 + a.split_tokens - 1) / a.split_tokens;
    if (nsplit <= 1 || nsplit > a.max_splits) return;
    const long long base = ((long long)s * a.g.Hq + hq) * a.max_splits;
    float m = -INFINITY;
    for (int i = 0; i < nsplit; ++i) m = fmaxf(m, a.part_ml[(base + i) * 2]);
    float o = 0.f, l = 0.f;
    for (int i = 0; i < nsplit; ++i) {
        const float f = exp2f(a.part_ml[(base + i) * 2] - m);
        o += f * a.part_o[(base + i) * D + d];
        l += f * a.part_ml[(base + i) * 2 + 1];
    }
    store_act(a.output, ((long long)t0 * a.g.Hq + hq) * D + d, a.g.act, o / l);
    if (d == 0 && a.lse) a.lse[(long long)t0 * a.g.Hq + hq] = (m + log2f(l)) * kLn2;
}

template <int D, int BS, int CACHE>
cudaError_t launch_decode_t(const KernelArgs& a, cudaStream_t stream, int* launches) {
    using Cfg = DecodeCfg<D, BS, CACHE>;
    const int G = a.g.Hq / a.g.Hkv;
    const int gtiles = (G + 15) / 16;
    dim3 grid(a.max_splits, a.g.Hkv * gtiles, a.num_sequences);
    const bool hi = G > 8;
    auto kern = hi ? decode_kernel<D, BS, CACHE, true> : decode_kernel<D, BS, CACHE, false>;
    static bool attr_set[2] = {false, false};
    if (!attr_set[hi]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
        if (e != cudaSuccess) return e;
        attr_set[hi] = true;
    }
    kern<<<grid, kDecodeWarps * 32, Cfg::SMEM, stream>>>(a);
    ++*launches;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (a.max_splits > 1) {
        decode_merge_kernel<D><<<dim3(a.g.Hq, a.num_sequences), D, 0, stream>>>(a);
        ++*launches;
        e = cudaGetLastError();
    }
    return e;
}

template <int D, int BS>
cudaError_t launch_decode_c(const KernelArgs& a, cudaStream_t stream, int* launches) {
    switch (a.g.cache) {
        case PA_DTYPE_U8: return launch_decode_t<D, BS, PA_DTYPE_U8>(a, stream, launches);
        case PA_DTYPE_F16: return launch_decode_t<D, BS, PA_DTYPE_F16>(a, stream, launches);
        case PA_DTYPE_BF16: return launch_decode_t<D, BS, PA_DTYPE_BF16>(a, stream, launches);
    }
    return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_decode(const KernelArgs& a, cudaStream_t stream, int* launches) {
    if (a.num_sequences <= 0) return cudaSuccess;
    if (a.g.D == 128 && a.g.bs == 32) return launch_decode_c<128, 32>(a, stream, launches);
    if (a.g.D == 128 && a.g.bs == 16) return launch_decode_c<128, 16>(a, stream, launches);
    if (a.g.D == 64 && a.g.bs == 32) return launch_decode_c<64, 32>(a, stream, launches);
    if (a.g.D == 64 && a.g.bs == 16) return launch_decode_c<64, 16>(a, stream, launches);
    return cudaErrorInvalidValue;
}

}  // namespace pa
