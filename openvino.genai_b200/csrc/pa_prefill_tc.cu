// Prefill-chunk attention on the 5th-generation tensor cores (tcgen05 + TMEM) for the u8 and the f16
// cache, head sizes 128 and 64.
//
// A work item is a q tile of 256 rows = (new token, q head of one GQA group) pairs of one
// (sequence, kv head), so a K/V byte is read once for the whole group.  The item is split into two
// halves A and B of 128 rows (UMMA M) that share the key / value operand tiles.  One persistent
// CTA per SM runs four roles that meet only through mbarriers:
//   loader    (1 thread)   TMA-engine bulk copies of the (block, head) records of 64-token tiles
//                          into a two-stage raw ring;
//   converter (4 warps)    raw bytes -> f16 operand tiles in 128-byte-swizzled layout:
//                          K' = byte * f16(k scale) as [64 tokens][128 dims], V'^T = byte *
//                          f16(v scale) as [128 dims][64 tokens] (the cache keeps value bytes
//                          token-minor, so both are K-major operands), two stages each;
//   mma       (1 warp, one elected lane issues) tcgen05.mma: S_X = Q_X.K'^T into TMEM, O_X += P_X.V' in
//                          TMEM, for X = A, B; as soon as half X has published P of tile j the S of tile
//                          j + 1 and then its P.V are queued, so the tensor core works on one half while the
//                          other half's softmax runs;
//   softmax   (2 x 4 warps) thread r owns row r of its half: reads S from TMEM, masks (diagonal
//                          tiles only), keeps a lazy running maximum, writes P = 2^(scale*(s-m)) as
//                          f16 into TMEM (the A operand of P.V); rescales O in TMEM only when a row maximum
//                          grew by more than 2^4; normalises and stores the output at the end.
// The zero-points ride on the tensor core: Q and K' carry 16 extra dims holding the row's sum of q
// and minus scale * zero-point split into f16 pieces, so S comes out with the offset term already
// subtracted; V'^T carries extra rows holding scale * zero-point (subtracted from O in the
// epilogue) and an all-ones row whose P.V column is the softmax denominator.
// The f16 cache needs no conversion: its four "converter" warps copy the token rows of a tile with
// 16-byte cp.async straight into the swizzled operand tiles (rows beyond the context are zero-filled).
// Key and value rows are both token-major there, so K' is a K-major operand and V' an MN-major one
// with the same shared-memory image; the softmax denominator comes from a second, 16-column P.V
// product against a constant tile whose first row is all ones.  The raw ring, the extra dims and
// the loader's copies do not exist in that variant.
// The CTA has four warpgroups (softmax A, softmax B, converter / copy, {mma, loader, two idle warps}) that re-divide the
// register file with setmaxnreg once their roles start: 160 registers per softmax thread, 104 per converter thread, 88 for
// the rest (one warp of each warpgroup shares a scheduler's 16 K registers).
// Every wait is bounded; a wait that runs out raises a flag that all roles poll.
// Tensor-bound for long contexts: 4 * Hq * D flops per (new token, context token) pair.
#include <algorithm>
#include <cstdio>

#include "pa_common.cuh"
#include "pa_kernels.h"
#include "tc05.cuh"

namespace pa {

namespace {

constexpr int kRows = 128;     // rows of one half = UMMA M
constexpr int kDx = 16;        // extra dims / extra V^T rows that carry the zero-point terms
constexpr int kKv = 64;        // context tokens per KV tile = UMMA N of Q.K^T
constexpr int kTmemCols = 512; // head size 128: S_A [0,64) S_B [64,128) O_A [128,272) O_B [272,416) P_A [416,448) P_B [448,480)
constexpr int kStages = 2;     // operand stages of the u8 variant (its raw ring has two more); the f16 variant has kStages16
constexpr int kStages16 = 4;
constexpr int kItemSlots = 4;   // depth of the queue that hands work items from the loader to the other roles
constexpr float kLazy = 4.f;   // log2 of the growth of a row maximum that forces a rescale of O
constexpr float kLog2eP = 1.4426950408889634f;
constexpr float kLn2P = 0.6931471805599453f;

constexpr int kSoftmaxWarps = 8, kConvWarps = 4;
constexpr int kWarpMma = kSoftmaxWarps + kConvWarps, kWarpLoad = kWarpMma + 1;
constexpr int kThreads = 512;   // four warpgroups: softmax A, softmax B, converter / copy warps, {mma, loader, two idle warps}
// Registers per thread after the roles have re-divided the register file among the warpgroups (one warp of each shares a
// scheduler's 16 K registers: 160 + 160 + 104 + 88 = 512 x 32)
#ifndef PA_TC_REG_SOFTMAX
#define PA_TC_REG_SOFTMAX 160
#define PA_TC_REG_CONV 104
#define PA_TC_REG_MISC 88
#endif
template <int R> __device__ __forceinline__ void reg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R)); }
template <int R> __device__ __forceinline__ void reg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R)); }
static_assert(kPrefillItemRows == 2 * kRows, "an item is two UMMA row tiles");

// One work item as every role sees it.
struct Item {
    int s, hk, t0, n_new, past;
    int row0;            // first (token, head) pair of half A
    int ctx_hi[2];       // context the last row of each half sees (0: the half has no rows)
    int nt[2];           // 64-token tiles of each half
    int ntiles;          // max of the two
    const int32_t* table;
};

template <int BS, int CT, int D>
struct PrefillSmem16;
template <int BS, int CT, int D>
struct PrefillSmem;

template <int BS, int D>
struct PrefillSmem<BS, PA_DTYPE_U8, D> {
    static constexpr int NO = D + kDx;   // UMMA N of P.V
    static constexpr int NST = kStages;
    static constexpr int REC = BS * (D + 8);
    static constexpr int NREC = kKv / BS;
    static constexpr int RSTRIDE = REC + 64;       // records 64 bytes out of phase: conflict-free 16-byte reads across records
    alignas(1024) uint8_t q[2][kRows * D * 2];     // per half: D / 64 swizzle atoms of [128 rows][64 dims]
    alignas(1024) uint8_t k[kStages][kKv * D * 2];    // D / 64 atoms of [64 tokens][64 dims]
    alignas(1024) uint8_t vt[kStages][NO * kKv * 2];  // [D + 16 dims][64 tokens], groups of 8 rows
    alignas(128) uint8_t qx[2][kRows * kDx * 2];   // unswizzled [128 rows][16 dims]
    alignas(128) uint8_t kx[kStages][kKv * kDx * 2];  // unswizzled [64 tokens][16 dims]
    alignas(128) uint8_t raw_k[kStages][NREC * RSTRIDE];
    alignas(128) uint8_t raw_v[kStages][NREC * RSTRIDE];
    alignas(16) uint2 v_tab[kConvWarps][kKv / 2];  // per converter warp: (scale, -1024 * scale) f16 pairs of two tokens
    alignas(8) uint64_t raw_full[kStages];   // loader -> converter (transaction bytes)
    alignas(8) uint64_t raw_free[kStages];   // converter -> loader
    alignas(8) uint64_t k_full[kStages];     // converter -> mma
    alignas(8) uint64_t v_full[kStages];
    alignas(8) uint64_t k_free[kStages];     // mma (commit) -> converter
    alignas(8) uint64_t v_free[kStages];
    alignas(8) uint64_t q_full[2];           // softmax -> mma, per item
    alignas(8) uint64_t s_full[2];           // mma (commit) -> softmax
    alignas(8) uint64_t p_full[2];           // softmax -> mma: P written, O rescaled
    alignas(8) uint64_t o_done[2];           // mma (commit) -> softmax: P.V complete
    alignas(8) uint64_t item_full[kItemSlots];   // loader -> every other warp
    alignas(8) uint64_t item_free[kItemSlots];   // every other warp -> loader: the slot has been read
    int item_ring[kItemSlots];
    Item item_desc[kItemSlots];   // the loader locates an item once for every role
    uint32_t tmem_base;
    volatile int abort;
};

// f16 / bf16 cache: operand tiles only.  The bf16 variant has no denominator columns (P takes their place in tensor memory
// as two bf16 pieces, and the rows sum their own probabilities).
template <int BS, int D>
struct PrefillSmem<BS, PA_DTYPE_F16, D> : PrefillSmem16<BS, PA_DTYPE_F16, D> {};
template <int BS, int D>
struct PrefillSmem<BS, PA_DTYPE_BF16, D> : PrefillSmem16<BS, PA_DTYPE_BF16, D> {};

template <int BS, int CT, int D>
struct PrefillSmem16 {
    static constexpr int NO = CT == PA_DTYPE_BF16 ? D : D + kDx;
    static constexpr int NREC = kKv / BS;
    static constexpr int NST = kStages16;
    alignas(1024) uint8_t q[2][kRows * D * 2];        // per half: D / 64 swizzle atoms of [128 rows][64 dims]
    alignas(1024) uint8_t k[NST][kKv * D * 2];    // D / 64 atoms of [64 tokens][64 dims], K-major
    alignas(1024) uint8_t vt[NST][kKv * D * 2];   // the same image read as an MN-major operand: atoms of 64 dims, 8-token groups 1024 bytes apart
    alignas(128) uint8_t ones[16 * 16 * 2];           // unswizzled K-major [16 rows][16 tokens]: row 0 all ones
    alignas(8) uint64_t k_full[NST];     // copy warps -> mma
    alignas(8) uint64_t v_full[NST];
    alignas(8) uint64_t k_free[NST];     // mma (commit) -> copy warps
    alignas(8) uint64_t v_free[NST];
    alignas(8) uint64_t q_full[2];
    alignas(8) uint64_t s_full[2];
    alignas(8) uint64_t p_full[2];
    alignas(8) uint64_t o_done[2];
    alignas(8) uint64_t item_full[kItemSlots];
    alignas(8) uint64_t item_free[kItemSlots];
    int item_ring[kItemSlots];
    Item item_desc[kItemSlots];   // the loader locates an item once for every role
    uint32_t tmem_base;
    volatile int abort;
};

__device__ __forceinline__ void cp_async16_zfill(void* dst_smem, const void* src_gmem, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ uint32_t sw128(uint32_t row, uint32_t chunk) { return row * 128u + ((chunk ^ (row & 7u)) << 4); }
// unswizzled K-major tile of 16 dims: 8-row groups 256 bytes apart, the two 8-dim halves 128 apart
__device__ __forceinline__ uint32_t plain16(uint32_t row, uint32_t half) { return (row >> 3) * 256u + half * 128u + (row & 7u) * 16u; }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t ex2_h2(uint32_t x) {
    uint32_t y;
    asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
__device__ __forceinline__ uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t y;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(y) : "r"(a), "r"(b), "r"(c));
    return y;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
    uint32_t y;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
    return y;
}
// f32 -> f16 through the packed conversion: the scalar form runs on the quarter-rate special
// function unit, which the softmax warps keep busy with exponentials
__device__ __forceinline__ __half f2h(float x) { return __ushort_as_half((unsigned short)(pack_h2(x, 0.f) & 0xffffu)); }
// z = h + m + l up to 2^-33 |z|, every piece an f16
__device__ __forceinline__ void split3(float z, __half& h, __half& m, __half& l) {
    h = f2h(z);
    const float r = z - __half2float(h);
    m = f2h(r);
    l = f2h(r - __half2float(m));
}
__device__ __forceinline__ uint32_t h2_bits(__half a, __half b) {
    return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
}
// 16 cache bytes -> 16 f16 values 1024 + byte
__device__ __forceinline__ void bytes16_to_h(const uint4 w, uint4& lo4, uint4& hi4) {
    lo4.x = __byte_perm(w.x, 0x64646464u, 0x4140); lo4.y = __byte_perm(w.x, 0x64646464u, 0x4342);
    lo4.z = __byte_perm(w.y, 0x64646464u, 0x4140); lo4.w = __byte_perm(w.y, 0x64646464u, 0x4342);
    hi4.x = __byte_perm(w.z, 0x64646464u, 0x4140); hi4.y = __byte_perm(w.z, 0x64646464u, 0x4342);
    hi4.z = __byte_perm(w.w, 0x64646464u, 0x4140); hi4.w = __byte_perm(w.w, 0x64646464u, 0x4342);
}
// (1024 + byte) -> byte * scale, rounded once.  The fused form needs -1024 * scale inside the f16
// range; scales of 32 and more take the two-step form.
__device__ __forceinline__ void scale16(uint4& lo4, uint4& hi4, __half sc) {
    const uint32_t s2 = h2_bits(sc, sc);
    uint32_t* w0 = reinterpret_cast<uint32_t*>(&lo4);
    uint32_t* w1 = reinterpret_cast<uint32_t*>(&hi4);
    if (fabsf(__half2float(sc)) < 32.f) {
        const uint32_t c2 = hmul2_bits(s2, 0xE400E400u);   // -1024 * scale, exact
#pragma unroll
        for (int k = 0; k < 4; ++k) { w0[k] = hfma2_bits(w0[k], s2, c2); w1[k] = hfma2_bits(w1[k], s2, c2); }
    } else {
#pragma unroll
        for (int k = 0; k < 4; ++k) { w0[k] = hmul2_bits(hadd2_bits(w0[k], 0xE400E400u), s2); w1[k] = hmul2_bits(hadd2_bits(w1[k], 0xE400E400u), s2); }
    }
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for the whole warp, after every lane's preceding writes.
__device__ __forceinline__ void warp_arrive(uint64_t* bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}


__device__ __forceinline__ Item locate_item(const KernelArgs& a, int item, int G, int Hkv) {
    Item it;
    // q tiles in the plan's order (longest context first) when it made one, else in sequence order
    const int gq = a.plan->pitems_sorted ? __ldcg(a.pitem_order + item / Hkv) : item / Hkv;
    it.hk = item % Hkv;
    int lo = 0, hi = a.num_sequences;  // ptile_prefix[lo] <= gq < ptile_prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldcg(a.ptile_prefix + mid) <= gq) lo = mid; else hi = mid;
    }
    it.s = lo;
    const int p0 = __ldcg(a.ptile_prefix + lo), np = __ldcg(a.ptile_prefix + lo + 1) - p0;
    const int qt = np - 1 - (gq - p0);           // heavy (late) tiles first
    it.t0 = a.subsequence_begins[lo];
    it.n_new = a.subsequence_begins[lo + 1] - it.t0;
    it.past = a.past_lens[lo];
    it.table = a.block_indices + a.block_indices_begins[lo];
    it.row0 = qt * kPrefillItemRows;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        const int r0 = it.row0 + x * kRows;
        if (r0 < it.n_new * G) {
            const int tok_hi = min(it.n_new - 1, (r0 + kRows - 1) / G);
            it.ctx_hi[x] = it.past + tok_hi + 1;
            it.nt[x] = (it.ctx_hi[x] + kKv - 1) / kKv;
        } else {
            it.ctx_hi[x] = 0;
            it.nt[x] = 0;
        }
    }
    it.ntiles = max(it.nt[0], it.nt[1]);
    return it;
}

template <int BS, int CT, int D>
__global__ void __launch_bounds__(kThreads, 1) prefill_tc_kernel(KernelArgs a) {
    using Smem = PrefillSmem<BS, CT, D>;
    constexpr bool U8 = CT == PA_DTYPE_U8, BF = CT == PA_DTYPE_BF16;
    constexpr int kD = D, kNo = Smem::NO, kTmemP = 2 * kKv + 2 * kNo, NST = Smem::NST;
    constexpr int kPCols = BF ? kKv : kKv / 2;   // tensor-memory columns of one half's P: f16, or bf16 high + low pieces
    constexpr int kFmt = BF ? 1 : 0;
    static_assert(!U8 || NST == 2, "the converter and the loader of the u8 variant index two stages");
    static_assert(kTmemP + 2 * kPCols <= kTmemCols, "S, O and P of both halves fit the tensor memory");
    extern __shared__ uint8_t smem_raw_[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw_) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.g.Hq / a.g.Hkv;
    const int Hkv = a.g.Hkv;
    const int total_items = a.plan->total_ptiles * Hkv;
    const float qscale = (a.scale != 0.f ? a.scale : rsqrtf((float)kD)) * kLog2eP;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < NST; ++i) {
            if constexpr (U8) {
                mbar_init(&sm.raw_full[i], 1);
                mbar_init(&sm.raw_free[i], kConvWarps);
            }
            mbar_init(&sm.k_full[i], kConvWarps);
            mbar_init(&sm.v_full[i], kConvWarps);
            mbar_init(&sm.k_free[i], 1);
            mbar_init(&sm.v_free[i], 1);
        }
#pragma unroll
        for (int x = 0; x < 2; ++x) {
            mbar_init(&sm.q_full[x], kRows / 32);
            mbar_init(&sm.s_full[x], 1);
            mbar_init(&sm.p_full[x], kRows / 32);
            mbar_init(&sm.o_done[x], 1);
        }
#pragma unroll
        for (int i = 0; i < kItemSlots; ++i) {
            mbar_init(&sm.item_full[i], 1);
            mbar_init(&sm.item_free[i], kWarpMma + 1);
        }
        mbar_fence_init();
        sm.abort = 0;
    }
    if constexpr (U8) {
        // rows 132..143 of V'^T stay zero for the whole kernel
        if (tid < NST * (kNo - kD - 4) * 8) {
            const int st = tid / ((kNo - kD - 4) * 8), i = tid % ((kNo - kD - 4) * 8);
            *reinterpret_cast<uint4*>(sm.vt[st] + (kD + 4) * 128 + i * 16) = make_uint4(0, 0, 0, 0);
        }
    } else {
        // row 0 of the constant tile (16-byte units 0 and 8: its two halves along the tokens) is all ones
        if (!BF && tid < 32) {
            const uint32_t one2 = tid == 0 || tid == 8 ? 0x3C003C00u : 0u;
            *reinterpret_cast<uint4*>(sm.ones + tid * 16) = make_uint4(one2, one2, one2, one2);
        }
    }
    if (warp == 0) tc05::tmem_alloc(&sm.tmem_base, kTmemCols);
    tc05::fence_proxy_async_smem();
    tc05::fence_before_thread_sync();
    __syncthreads();
    tc05::fence_after_thread_sync();
    const uint32_t tmem = sm.tmem_base;

    // A wait that runs out raises sm.abort; every waiter polls the flag, so all roles unwind.
    // `cat` names the wait for the optional cycle accounting (-DPA_PREFILL_PROF).
#ifdef PA_PREFILL_PROF
    long long prof[5] = {0, 0, 0, 0, 0};
    const long long prof_begin = clock64();
    __shared__ long long trace[5][8][4];   // role, event, tile 64..67 of this CTA
#define PA_TRACE(role, ev, tile) do { if (lane == 0 && (tile) >= 64 && (tile) < 68) trace[role][ev][(tile) - 64] = clock64(); } while (0)
#else
#define PA_TRACE(role, ev, tile) do { } while (0)
#endif
    auto wait = [&](uint64_t* bar, uint32_t parity, int cat) -> bool {
#ifdef PA_PREFILL_PROF
        const long long w0 = clock64();
#endif
        bool ok = false;
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            if (mbar_try_wait(bar, parity)) { ok = true; break; }
            if ((i & 255u) == 255u && sm.abort) return false;
        }
#ifdef PA_PREFILL_PROF
        prof[cat] += clock64() - w0;
#endif
        (void)cat;
        if (ok) return true;
        sm.abort = 1;
        atomicOr(a.status, PA_DEV_WAIT_TIMEOUT_PREFILL);
        return false;
    };
    auto wait_warp = [&](uint64_t* bar, uint32_t parity, int cat) -> bool { return __all_sync(0xffffffffu, wait(bar, parity, cat)) != 0; };
    // Work items come from a global counter: the loader draws them and publishes each through a
    // small ring, so that all roles of the CTA walk the same sequence.  -1 ends the sequence, -2
    // reports a wait that ran out.
    auto fetch_item = [&](uint32_t k, Item& it) -> int {
        const int slot = k & (kItemSlots - 1);
        if (!wait_warp(&sm.item_full[slot], (k / kItemSlots) & 1, 0)) return -2;
        const int item = sm.item_ring[slot];
        if (item >= 0) it = sm.item_desc[slot];
        warp_arrive(&sm.item_free[slot]);
        return item;
    };

    if (warp >= kWarpMma) reg_dec<PA_TC_REG_MISC>();   // the fourth warpgroup: mma, loader and two warps that only keep it whole
    if (warp < kSoftmaxWarps) {
        // ======================= softmax + epilogue of half X ==========================================
        reg_inc<PA_TC_REG_SOFTMAX>();
        const int X = warp >> 2, r = tid & (kRows - 1);
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;   // this warp's TMEM lanes
        const uint32_t tmem_s = tmem + kKv * X + lane_base, tmem_o = tmem + 2 * kKv + kNo * X + lane_base;
        uint8_t* const sq = sm.q[X];
        const uint32_t tmem_p = tmem + kTmemP + kPCols * X + lane_base;
        uint32_t n = 0;   // tiles of this half so far, over all items
        for (uint32_t ik = 0;; ++ik) {
            Item it;
            const int item = fetch_item(ik, it);
            if (item == -2) goto done;
            if (item < 0) break;
            if (it.nt[X] == 0) continue;
            const int flat = it.row0 + X * kRows + r;
            const int tok = flat / G, hq = it.hk * G + flat % G;
            const bool row_live = tok < it.n_new;
            const int my_ctx = row_live ? it.past + tok + 1 : it.ctx_hi[X];
            const long long grow_off = ((long long)(it.t0 + (row_live ? tok : 0)) * a.g.Hq + hq);

            // ---- Q -> f16 swizzled A operand; the row's sum goes into the extra dims.  Every S of this
            // half's previous item has completed, so the tile is free. ------------------------------
            float qs = qscale;   // the row's softmax scale: the kernel's, divided by the row's prescale
            {
                // large queries (bf16 / f32 beyond the f16 range, or f16 rows whose sum would leave it): an exact power-of-two
                // prescale keeps the packed row and its sum inside the f16 range (the decode kernel does the same), and the
                // softmax scale of the row takes it back out
                float qmul = 1.f;
                if (!BF && row_live) {   // (the bf16 variant runs on bf16 activations only: its rows go in as they are)
                    float amax = 0.f;
#pragma unroll 4
                    for (int c = 0; c < kD / 8; ++c) {
                        float v[8];
                        load_act_vec<8>(a.query, grow_off * kD + 8 * c, a.g.act, v);
#pragma unroll
                        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
                    }
                    if (amax > 256.f && amax < INFINITY) {   // 128 terms of at most 2^8 each keep the row sum below the f16 maximum too
                        int ex;
                        frexpf(amax, &ex);
                        qmul = ldexpf(1.f, 8 - ex);
                    }
                }
                qs = qscale / qmul;
                float qsum = 0.f;
#pragma unroll 4
                for (int c = 0; c < kD / 8; ++c) {
                    float v[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = 0.f;
                    if (row_live) load_act_vec<8>(a.query, grow_off * kD + 8 * c, a.g.act, v);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] *= qmul;
                    uint4 w;
                    if constexpr (BF) {
                        w.x = pack_bf2(v[0], v[1]); w.y = pack_bf2(v[2], v[3]); w.z = pack_bf2(v[4], v[5]); w.w = pack_bf2(v[6], v[7]);
                    } else {
                        w.x = pack_h2(v[0], v[1]); w.y = pack_h2(v[2], v[3]); w.z = pack_h2(v[4], v[5]); w.w = pack_h2(v[6], v[7]);
                    }
                    if constexpr (U8) {
                        const __half2* h = reinterpret_cast<const __half2*>(&w);
#pragma unroll
                        for (int e = 0; e < 4; ++e) qsum += __low2float(h[e]) + __high2float(h[e]);
                    }
                    *reinterpret_cast<uint4*>(sq + (c / 8) * (kRows * 128) + sw128(r, c % 8)) = w;
                }
                if constexpr (U8) {
                    const __half qh = f2h(qsum), ql = f2h(qsum - __half2float(qh));
                    const __half zero = __ushort_as_half(0);
                    *reinterpret_cast<uint4*>(sm.qx[X] + plain16(r, 0)) = make_uint4(h2_bits(qh, qh), h2_bits(qh, ql), h2_bits(ql, zero), 0u);
                    *reinterpret_cast<uint4*>(sm.qx[X] + plain16(r, 1)) = make_uint4(0u, 0u, 0u, 0u);
                }
                tc05::fence_proxy_async_smem();
                warp_arrive(&sm.q_full[X]);
            }

            float m_run = -INFINITY;   // running maximum of q.k' (before the softmax scale)
            float l_own = 0.f;         // bf16 variant: the row's own sum of probabilities
            for (int j = 0; j < it.nt[X]; ++j, ++n) {
                const int col0 = j * kKv;
                if (!wait_warp(&sm.s_full[X], n & 1, 0)) goto done;
                if ((warp & 3) == 0) PA_TRACE(X, 0, n);
                tc05::fence_after_thread_sync();
                float sv[kKv];   // q.k' in units of 1 / qs
                {
                    uint32_t s0[32], s1[32];
                    tc05::ld_32x32b_x32(tmem_s, s0);
                    tc05::ld_32x32b_x32(tmem_s + 32, s1);
                    tc05::wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; ++c) { sv[c] = __uint_as_float(s0[c]); sv[32 + c] = __uint_as_float(s1[c]); }
                }
                if ((warp & 3) == 0) PA_TRACE(X, 1, n);
#ifdef PA_EXP_NOSOFTMAX
                float alpha = 1.f;
                bool rescale = false;
                uint32_t pw[kKv / 2];
#pragma unroll
                for (int c = 0; c < kKv; c += 2) pw[c >> 1] = __float_as_uint(sv[c]) ^ __float_as_uint(sv[c + 1]);
                m_run = 0.f;
#else
                if (col0 + kKv > my_ctx) {     // diagonal tile: hide what this row cannot see
                    const int nvis = my_ctx - col0;   // may be <= 0
#pragma unroll
                    for (int c = 0; c < kKv; ++c) sv[c] = c < nvis ? sv[c] : -INFINITY;
                }
                float mx = -INFINITY;
#pragma unroll
                for (int c = 0; c < kKv; c += 2) mx = max3(mx, sv[c], sv[c + 1]);
                float alpha = 1.f;
                bool rescale = false;
                if (j == 0) {
                    m_run = mx;      // finite: column 0 of tile 0 is visible to every row
                } else {
                    const bool grow = (mx - m_run) * qs > kLazy;
                    rescale = __any_sync(0xffffffffu, grow);
                    if (grow) { alpha = ex2((m_run - mx) * qs); m_run = mx; }
                }
                if constexpr (BF) l_own *= alpha;
                // P = 2^(qs * (s - m)) in f16 pairs: the exponent is rounded to f16 first, which costs
                // at most 2^-12 of the exponent's magnitude in relative error of p
                const float mq = m_run * qs;
                uint32_t pw[kKv / 2];
                uint32_t pl[BF ? kKv / 2 : 1];   // bf16 variant: the low pieces, p = high + low up to 2^-17 p
#pragma unroll
                for (int c = 0; c < kKv; c += 2) {
#if defined(PA_EXP_NOEXP)
                    pw[c >> 1] = __byte_perm(__float_as_uint(fmaf(sv[c], qs, -mq)), __float_as_uint(fmaf(sv[c + 1], qs, -mq)), 0x7632);
#elif defined(PA_EXP_NOCVT)
                    pw[c >> 1] = ex2_h2(__byte_perm(__float_as_uint(fmaf(sv[c], qs, -mq)), __float_as_uint(fmaf(sv[c + 1], qs, -mq)), 0x7632));
#else
                    // the packed f16 exponential is good to 2^-9.9 relative: inside the u8 cache's error bound, not inside the
                    // f16 cache's, whose P goes through the f32 exponential and is rounded once
                    if constexpr (U8) {
                        pw[c >> 1] = ex2_h2(pack_h2(fmaf(sv[c], qs, -mq), fmaf(sv[c + 1], qs, -mq)));
                    } else if constexpr (BF) {
                        const float p0 = ex2(fmaf(sv[c], qs, -mq)), p1 = ex2(fmaf(sv[c + 1], qs, -mq));
                        l_own += p0 + p1;
                        const uint32_t hi = pack_bf2(p0, p1);
                        pw[c >> 1] = hi;
                        pl[c >> 1] = pack_bf2(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
                    } else {
                        pw[c >> 1] = pack_h2(ex2(fmaf(sv[c], qs, -mq)), ex2(fmaf(sv[c + 1], qs, -mq)));
                    }
#endif
                }
#endif
                // P.V of the previous tile of this half still reads the P tile and writes O
                if ((warp & 3) == 0) PA_TRACE(X, 2, n);
                if (n > 0) {
                    if (!wait_warp(&sm.o_done[X], (n - 1) & 1, 1)) goto done;
                    tc05::fence_after_thread_sync();
                }
                if ((warp & 3) == 0) PA_TRACE(X, 3, n);
                if (rescale) {
#pragma unroll
                    for (int q4 = 0; q4 < kD / 32; ++q4) {
                        uint32_t t[32];
                        tc05::ld_32x32b_x32(tmem_o + 32 * q4, t);
                        tc05::wait_ld();
#pragma unroll
                        for (int c = 0; c < 32; ++c) t[c] = __float_as_uint(__uint_as_float(t[c]) * alpha);
                        tc05::st_32x32b_x32(tmem_o + 32 * q4, t);
                    }
                    if constexpr (!BF) {
                        uint32_t t[16];
                        tc05::ld_32x32b_x16(tmem_o + kD, t);
                        tc05::wait_ld();
#pragma unroll
                        for (int c = 0; c < 16; ++c) t[c] = __float_as_uint(__uint_as_float(t[c]) * alpha);
                        tc05::st_32x32b_x16(tmem_o + kD, t);
                    }
                    tc05::wait_st();
                }
                tc05::st_32x32b_x32(tmem_p, pw);   // row r of the A operand: lane r, two tokens per column
                if constexpr (BF) tc05::st_32x32b_x32(tmem_p + kKv / 2, pl);
                tc05::wait_st();
                tc05::fence_before_thread_sync();
                warp_arrive(&sm.p_full[X]);
                if ((warp & 3) == 0) PA_TRACE(X, 4, n);
            }
            // ---- epilogue: out = (O - z) / l; z = the three zero-point columns, l = the all-ones column (u8 cache);
            // the f16 cache has no z and its l is the first column of the 16-column product
            if (!wait_warp(&sm.o_done[X], (n - 1) & 1, 2)) goto done;
            tc05::fence_after_thread_sync();
            {
                float z = 0.f, l_run = l_own;
                if constexpr (!BF) {
                    uint32_t zr[16];
                    tc05::ld_32x32b_x16(tmem_o + kD, zr);
                    tc05::wait_ld();
                    if constexpr (U8) z = __uint_as_float(zr[0]) + __uint_as_float(zr[1]) + __uint_as_float(zr[2]);
                    l_run = __uint_as_float(zr[U8 ? 3 : 0]);
                }
                const float inv = 1.f / l_run;
#pragma unroll
                for (int q4 = 0; q4 < kD / 32; ++q4) {
                    uint32_t t[32];
                    tc05::ld_32x32b_x32(tmem_o + 32 * q4, t);
                    tc05::wait_ld();
                    if (row_live) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8) {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = (__uint_as_float(t[c + e]) - z) * inv;
                            store_act_vec8(a.output, grow_off * kD + 32 * q4 + c, a.g.act, v);
                        }
                    }
                }
                if (row_live && a.lse) a.lse[grow_off] = (m_run * qs + log2f(l_run)) * kLn2P;
            }
            tc05::fence_before_thread_sync();
        }
    } else if (warp < kWarpMma) {
        // ======================= converter: raw records -> f16 operand tiles =============================
        reg_dec<PA_TC_REG_CONV>();
        const int ctid = tid - kSoftmaxWarps * 32, cwarp = warp - kSoftmaxWarps;
        if constexpr (U8) {
        uint32_t t = 0;   // tiles so far, over all items
        for (uint32_t ik = 0;; ++ik) {
            Item it;
            const int item = fetch_item(ik, it);
            if (item == -2) goto done;
            if (item < 0) break;
            const int ctx_hi = max(it.ctx_hi[0], it.ctx_hi[1]);
            for (int j = 0; j < it.ntiles; ++j, ++t) {
                const int st = t & 1;
                const uint32_t use = t >> 1;
                const int live_tokens = min(kKv, ctx_hi - j * kKv);
                const uint8_t* raw_k = sm.raw_k[st];
                const uint8_t* raw_v = sm.raw_v[st];
                if (!wait_warp(&sm.raw_full[st], use & 1, 0)) goto done;
                if (cwarp == 0) PA_TRACE(2, 0, t);
                if (use > 0 && !wait_warp(&sm.k_free[st], (use - 1) & 1, 1)) goto done;
                if (cwarp == 0) PA_TRACE(2, 1, t);
                // K' = byte * f16(k scale): unit u = 16 dims of one token
#ifndef PA_EXP_NOCONV
#pragma unroll
                for (int i = 0; i < kD / 32; ++i) {
                    const int u = ctid + 128 * i;
                    const int token = u / (kD / 16), seg = u % (kD / 16);
                    uint4 lo4 = make_uint4(0u, 0u, 0u, 0u), hi4 = lo4;
                    if (token < live_tokens) {
                        const uint8_t* rec = raw_k + (token / BS) * Smem::RSTRIDE;
                        const __half ksh = f2h(*reinterpret_cast<const float*>(rec + BS * kD + 4 * (token % BS)));
                        bytes16_to_h(*reinterpret_cast<const uint4*>(rec + (token % BS) * kD + 16 * seg), lo4, hi4);
                        scale16(lo4, hi4, ksh);
                    }
                    uint8_t* atom = sm.k[st] + (seg >> 2) * (kKv * 128);
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg) & 7)) = lo4;
                    *reinterpret_cast<uint4*>(atom + sw128(token, (2 * seg + 1) & 7)) = hi4;
                }
#endif
                if (ctid < kKv) {
                    const int token = ctid;
                    const bool ok = token < live_tokens;
                    const float* kp = reinterpret_cast<const float*>(raw_k + (token / BS) * Smem::RSTRIDE + BS * kD);
                    const float ksf = __half2float(f2h(kp[token % BS]));
                    __half zh, zm, zl;
                    split3(ok ? -(ksf * kp[BS + token % BS]) : 0.f, zh, zm, zl);
                    const __half zero = __ushort_as_half(0);
                    *reinterpret_cast<uint4*>(sm.kx[st] + plain16(token, 0)) = make_uint4(h2_bits(zh, zm), h2_bits(zl, zh), h2_bits(zm, zero), 0u);
                    *reinterpret_cast<uint4*>(sm.kx[st] + plain16(token, 1)) = make_uint4(0u, 0u, 0u, 0u);
                }
                tc05::fence_proxy_async_smem();
                warp_arrive(&sm.k_full[st]);
                if (cwarp == 0) PA_TRACE(2, 2, t);

                if (use > 0 && !wait_warp(&sm.v_free[st], (use - 1) & 1, 2)) goto done;
                if (cwarp == 0) PA_TRACE(2, 3, t);
                // this warp's table of (scale, -1024 * scale) for the tile's token pairs
                __syncwarp();
                float vs0 = 0.f, vs1 = 0.f;
                {
                    const int t0k = 2 * lane, t1k = 2 * lane + 1;
                    if (t0k < live_tokens) vs0 = *reinterpret_cast<const float*>(raw_v + (t0k / BS) * Smem::RSTRIDE + BS * kD + 4 * (t0k % BS));
                    if (t1k < live_tokens) vs1 = *reinterpret_cast<const float*>(raw_v + (t1k / BS) * Smem::RSTRIDE + BS * kD + 4 * (t1k % BS));
                }
                const uint32_t s2 = pack_h2(vs0, vs1);
                sm.v_tab[cwarp][lane] = make_uint2(s2, hmul2_bits(s2, 0xE400E400u));
                const bool big = __any_sync(0xffffffffu, !(fabsf(vs0) < 32.f) || !(fabsf(vs1) < 32.f));
                __syncwarp();
                // V'^T = byte * f16(v scale): unit = 16 tokens of one dim
                const int tg = ctid & 3;
                uint2 tab[8];
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    const uint4 t4 = *reinterpret_cast<const uint4*>(&sm.v_tab[cwarp][8 * tg + k]);
                    tab[k] = make_uint2(t4.x, t4.y);
                    tab[k + 1] = make_uint2(t4.z, t4.w);
                }
                constexpr int UPR = BS / 16;   // 16-token units per record
#ifndef PA_EXP_NOCONV
#pragma unroll
                for (int i = 0; i < kD / 32; ++i) {
                    const int d = (ctid >> 2) + 32 * i;
                    uint4 lo4, hi4;
                    bytes16_to_h(*reinterpret_cast<const uint4*>(raw_v + (tg / UPR) * Smem::RSTRIDE + d * BS + 16 * (tg % UPR)), lo4, hi4);
                    uint32_t w[8] = {lo4.x, lo4.y, lo4.z, lo4.w, hi4.x, hi4.y, hi4.z, hi4.w};
                    if (!big) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) w[k] = hfma2_bits(w[k], tab[k].x, tab[k].y);
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) w[k] = hmul2_bits(hadd2_bits(w[k], 0xE400E400u), tab[k].x);
                    }
                    *reinterpret_cast<uint4*>(sm.vt[st] + sw128(d, 2 * tg)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(sm.vt[st] + sw128(d, 2 * tg + 1)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
#endif
                if (ctid < kKv) {
                    const int token = ctid;
                    const bool ok = token < live_tokens;
                    const float* vp = reinterpret_cast<const float*>(raw_v + (token / BS) * Smem::RSTRIDE + BS * kD);
                    const float vsf = __half2float(f2h(vp[token % BS]));
                    __half zh, zm, zl;
                    split3(ok ? vsf * vp[BS + token % BS] : 0.f, zh, zm, zl);
                    const uint32_t off = (token & 7) * 2;
                    uint8_t* vt = sm.vt[st];
                    *reinterpret_cast<__half*>(vt + sw128(kD + 0, token >> 3) + off) = zh;
                    *reinterpret_cast<__half*>(vt + sw128(kD + 1, token >> 3) + off) = zm;
                    *reinterpret_cast<__half*>(vt + sw128(kD + 2, token >> 3) + off) = zl;
                    *reinterpret_cast<__half*>(vt + sw128(kD + 3, token >> 3) + off) = __ushort_as_half(ok ? (unsigned short)0x3C00u : (unsigned short)0u);
                }
                tc05::fence_proxy_async_smem();
                warp_arrive(&sm.v_full[st]);
                warp_arrive(&sm.raw_free[st]);
                if (cwarp == 0) PA_TRACE(2, 4, t);
            }
        }
        } else {
            // ---- f16 cache: token rows -> operand tiles with cp.async; thread = 16-byte chunk `ch` of the rows trow + TP u.
            // The copies of tile t are in flight while tile t - 1 is handed over: K_t is issued, then K_(t-1) is
            // awaited, fenced for the tensor core's proxy and published, then the same for V.
            (void)cwarp;
            constexpr int CH = kD / 8, TP = kConvWarps * 32 / CH, NU = kKv / TP;   // chunks of a row, tokens per pass, passes
            const int ch = ctid % CH, trow = ctid / CH;
            const uint32_t dst0 = (uint32_t)(ch >> 3) * (kKv * 128);
            uint32_t t = 0;
            bool bad_index = false;
            for (uint32_t ik = 0;; ++ik) {
                Item it;
                const int item = fetch_item(ik, it);
                if (item == -2) goto done;
                if (item < 0) break;
                const int ctx_hi = max(it.ctx_hi[0], it.ctx_hi[1]);
                const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)it.hk * a.g.head_bytes + 16 * ch;
                const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)it.hk * a.g.head_bytes + 16 * ch;
                for (int j = 0; j < it.ntiles; ++j, ++t) {
                    const int st = t % NST, stp = (t + NST - 1) % NST;
                    const uint32_t use = t / NST;
                    const int live_tokens = min(kKv, ctx_hi - j * kKv);
                    long long off[NU];   // byte offset of this thread's chunk of token trow + TP u; -1: beyond the context
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const int token = trow + TP * u;
                        off[u] = -1;
                        if (token < live_tokens) {
                            int blk = it.table[j * Smem::NREC + token / BS];
                            if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                            off[u] = (long long)blk * a.g.block_bytes + (long long)(token % BS) * (kD * 2);
                        }
                    }
                    if (use > 0 && !wait_warp(&sm.k_free[st], (use - 1) & 1, 1)) goto done;
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const bool ok = off[u] >= 0;
#ifndef PA_EXP_NOCOPY16
                        cp_async16_zfill(sm.k[st] + dst0 + sw128(trow + TP * u, ch & 7), kc + (ok ? off[u] : 0), ok ? 16u : 0u);
#endif
                    }
                    cp_async_commit();
                    if (t > 0) {
                        cp_async_wait<2>();   // pending at most V_(t-1), K_t
                        tc05::fence_proxy_async_smem();
                        warp_arrive(&sm.k_full[stp]);
                    }
                    if (use > 0 && !wait_warp(&sm.v_free[st], (use - 1) & 1, 2)) goto done;
#pragma unroll
                    for (int u = 0; u < NU; ++u) {
                        const bool ok = off[u] >= 0;
#ifndef PA_EXP_NOCOPY16
                        cp_async16_zfill(sm.vt[st] + dst0 + sw128(trow + TP * u, ch & 7), vc + (ok ? off[u] : 0), ok ? 16u : 0u);
#endif
                    }
                    cp_async_commit();
                    if (t > 0) {
                        cp_async_wait<2>();   // pending at most K_t, V_t
                        tc05::fence_proxy_async_smem();
                        warp_arrive(&sm.v_full[stp]);
                    }
                }
            }
            if (t > 0) {
                cp_async_wait<1>();
                tc05::fence_proxy_async_smem();
                warp_arrive(&sm.k_full[(t - 1) % NST]);
                cp_async_wait<0>();
                tc05::fence_proxy_async_smem();
                warp_arrive(&sm.v_full[(t - 1) % NST]);
            }
            if (__any_sync(0xffffffffu, bad_index) && lane == 0) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
        }
    } else if (warp == kWarpMma) {
        // ======================= mma issue ================================================================
        // The whole warp runs the loop (uniform control flow keeps the descriptors in uniform registers);
        // one elected lane issues the tensor-core instructions.
        {
            constexpr uint32_t idesc_s = tc05::instr_desc_f16(kRows, kKv, kFmt, 0, 0);   // A and B K-major
            constexpr uint32_t idesc_o = U8 ? tc05::instr_desc_f16(kRows, kNo, 0, 0, 0) : tc05::instr_desc_f16(kRows, kD, kFmt, 0, 1);   // f16 / bf16 cache: V' MN-major
            constexpr uint32_t idesc_l = tc05::instr_desc_f16(kRows, kDx, 0, 0, 0);   // f16 cache: P . ones
            // operand descriptors are built once; a step along K or to another buffer only moves the
            // start-address field (bits [0,14) of the low word, in 16-byte units, no carry out of it)
            const uint64_t dq = tc05::smem_desc_sw128(smem_u32(sm.q[0]), 1024), dk = tc05::smem_desc_sw128(smem_u32(sm.k[0]), 1024);
            // MN-major V' of the f16 cache: 8-token groups 1024 bytes apart, the two 64-dim atoms kKv * 128 bytes apart
            const uint64_t dv = U8 ? tc05::smem_desc_sw128(smem_u32(sm.vt[0]), 1024) : tc05::smem_desc_sw128(smem_u32(sm.vt[0]), 1024, kKv * 128);
            uint64_t dqx = 0, dkx = 0, dones = 0;
            uint32_t qx_step = 0, kx_step = 0;
            if constexpr (U8) {
                dqx = tc05::smem_desc_plain(smem_u32(sm.qx[0]), 128, 256);
                dkx = tc05::smem_desc_plain(smem_u32(sm.kx[0]), 128, 256);
                qx_step = sizeof(sm.qx[0]) >> 4;
                kx_step = sizeof(sm.kx[0]) >> 4;
            } else if constexpr (!BF) {
                dones = tc05::smem_desc_plain(smem_u32(sm.ones), 128, 256);
            }
            constexpr uint32_t q_step = sizeof(sm.q[0]) >> 4, k_step = sizeof(sm.k[0]) >> 4, v_step = sizeof(sm.vt[0]) >> 4;
            auto issue_s = [&](int X, int st) {
                const uint64_t da0 = dq + X * q_step, db0 = dk + st * k_step;
                const uint32_t d = tmem + kKv * X;
                if (tc05::elect_one()) {
#pragma unroll
                for (int kk = 0; kk < kD / 16; ++kk) {
                    const uint32_t a_off = ((kk >> 2) * (kRows * 128) + (kk & 3) * 32) >> 4, b_off = ((kk >> 2) * (kKv * 128) + (kk & 3) * 32) >> 4;
                    if (kk == 0) tc05::mma_ss<0>(d, da0 + a_off, db0 + b_off, idesc_s);
                    else tc05::mma_ss<1>(d, da0 + a_off, db0 + b_off, idesc_s);
                }
                if constexpr (U8) tc05::mma_ss<1>(d, dqx + X * qx_step, dkx + st * kx_step, idesc_s);
                tc05::commit(&sm.s_full[X]);
                }
                __syncwarp();
            };
            auto issue_pv = [&](int X, int st, bool acc) {
                const uint32_t pa = tmem + kTmemP + kPCols * X;   // 16 tokens of P = 8 columns
                const uint64_t db0 = dv + st * v_step;
                const uint32_t d = tmem + 2 * kKv + kNo * X;
                if (tc05::elect_one()) {
                if constexpr (U8) {
                    if (acc) tc05::mma_ts<1>(d, pa, db0, idesc_o);
                    else tc05::mma_ts<0>(d, pa, db0, idesc_o);
#pragma unroll
                    for (int kk = 1; kk < kKv / 16; ++kk) tc05::mma_ts<1>(d, pa + 8 * kk, db0 + 2 * kk, idesc_o);
                } else if constexpr (BF) {
                    // high pieces of P, then the low pieces against the same value rows
                    if (acc) tc05::mma_ts<1>(d, pa, db0, idesc_o);
                    else tc05::mma_ts<0>(d, pa, db0, idesc_o);
#pragma unroll
                    for (int kk = 1; kk < kKv / 16; ++kk) tc05::mma_ts<1>(d, pa + 8 * kk, db0 + 128 * kk, idesc_o);
#pragma unroll
                    for (int kk = 0; kk < kKv / 16; ++kk) tc05::mma_ts<1>(d, pa + kKv / 2 + 8 * kk, db0 + 128 * kk, idesc_o);
                } else {
                    // 16 tokens further along K = 16 rows of 128 bytes; the denominators go to the 16 columns after O
#ifdef PA_EXP_NOONES
                    if (acc) { tc05::mma_ts<1>(d, pa, db0, idesc_o); }
                    else { tc05::mma_ts<0>(d, pa, db0, idesc_o); }
#pragma unroll
                    for (int kk = 1; kk < kKv / 16; ++kk) {
                        tc05::mma_ts<1>(d, pa + 8 * kk, db0 + 128 * kk, idesc_o);
                    }
#else
                    if (acc) { tc05::mma_ts<1>(d, pa, db0, idesc_o); tc05::mma_ts<1>(d + kD, pa, dones, idesc_l); }
                    else { tc05::mma_ts<0>(d, pa, db0, idesc_o); tc05::mma_ts<0>(d + kD, pa, dones, idesc_l); }
#pragma unroll
                    for (int kk = 1; kk < kKv / 16; ++kk) {
                        tc05::mma_ts<1>(d, pa + 8 * kk, db0 + 128 * kk, idesc_o);
                        tc05::mma_ts<1>(d + kD, pa + 8 * kk, dones, idesc_l);
                    }
#endif
                }
                tc05::commit(&sm.o_done[X]);
                }
                __syncwarp();
            };
            uint32_t t = 0, n[2] = {0, 0}, iq[2] = {0, 0};
            for (uint32_t ik = 0;; ++ik) {
                Item it;
                const int item = fetch_item(ik, it);
                if (item == -2) goto done;
                if (item < 0) break;
                // first S of the item.  The S region of a half is free: its softmax published the last P of
                // the previous item (waited below) after reading that tile's S.
#pragma unroll
                for (int X = 0; X < 2; ++X)
                    if (it.nt[X] > 0) {
                        if (!wait_warp(&sm.q_full[X], iq[X] & 1, 0)) goto done;
                        ++iq[X];
                    }
                if (!wait_warp(&sm.k_full[t % NST], (t / NST) & 1, 1)) goto done;
                tc05::fence_after_thread_sync();
#pragma unroll
                for (int X = 0; X < 2; ++X)
                    if (it.nt[X] > 0) issue_s(X, t % NST);
                if (tc05::elect_one()) tc05::commit(&sm.k_free[t % NST]);
                for (int j = 0; j < it.ntiles; ++j, ++t) {
                    const int st = t % NST, st1 = (t + 1) % NST;
                    const bool more = j + 1 < it.ntiles;
                    PA_TRACE(3, 0, t);
                    // The converter finishes V' of tile j before K' of tile j + 1, so the latter's barrier
                    // covers both; only the item's last tile waits for its V' directly.
                    if (more) {
                        if (!wait_warp(&sm.k_full[st1], ((t + 1) / NST) & 1, 1)) goto done;
                    } else {
                        if (!wait_warp(&sm.v_full[st], (t / NST) & 1, 3)) goto done;
                    }
                    PA_TRACE(3, 3, t);
#pragma unroll
                    for (int X = 0; X < 2; ++X)
                        if (j < it.nt[X]) {
                            // P of tile j is in TMEM, so S of tile j has been read: both MMAs may go
                            if (!wait_warp(&sm.p_full[X], (n[X] + j) & 1, 4)) goto done;
                            PA_TRACE(3, 4 + 2 * X, t);
                            tc05::fence_after_thread_sync();
                            // the next logits first: the half's softmax warps wait for them, nobody waits for this P.V yet
                            if (j + 1 < it.nt[X]) issue_s(X, st1);
                            issue_pv(X, st, j > 0);
                            PA_TRACE(3, 5 + 2 * X, t);
                        }
                    if (tc05::elect_one()) {
                        if (more) tc05::commit(&sm.k_free[st1]);
                        tc05::commit(&sm.v_free[st]);
                    }
                }
                n[0] += it.nt[0];
                n[1] += it.nt[1];
            }
            // every commit has landed before the CTA's shared memory is given up
            if (t > 0) wait_warp(&sm.v_free[(t - 1) % NST], ((t - 1) / NST) & 1, 0);
        }
    } else if (warp == kWarpLoad) {
        // ======================= loader: TMA-engine copies of the tiles' records =========================
        if (lane == 0) {
            uint32_t t = 0;
            bool bad_index = false;
            for (uint32_t ik = 0;; ++ik) {
                const int slot = ik & (kItemSlots - 1);
                if (ik >= kItemSlots && !wait(&sm.item_free[slot], ((ik / kItemSlots) - 1) & 1, 1)) goto done;
                if constexpr (!U8) {
                    // Nothing throttles this loader (it copies no tiles), and an item drawn early is an item another CTA cannot
                    // take: the next one is drawn when every role has started the previous one, which is still several tiles
                    // before the copy warps need it.
                    if (ik >= 1 && !wait(&sm.item_free[(ik - 1) & (kItemSlots - 1)], ((ik - 1) / kItemSlots) & 1, 1)) goto done;
                }
                int item = atomicAdd(&a.plan->next_pitem, 1);
                if (item >= total_items) item = -1;
                Item it{};
                if (item >= 0) {
                    it = locate_item(a, item, G, Hkv);
                    sm.item_desc[slot] = it;
                }
                sm.item_ring[slot] = item;
                mbar_arrive(&sm.item_full[slot]);
                if (item < 0) break;
                if constexpr (U8) {
                const int ctx_hi = max(it.ctx_hi[0], it.ctx_hi[1]);
                const uint8_t* kc = (const uint8_t*)a.key_cache + (long long)it.hk * a.g.head_bytes;
                const uint8_t* vc = (const uint8_t*)a.value_cache + (long long)it.hk * a.g.head_bytes;
                for (int j = 0; j < it.ntiles; ++j, ++t) {
                    const int st = t & 1;
                    const uint32_t use = t >> 1;
                    if (use > 0 && !wait(&sm.raw_free[st], (use - 1) & 1, 0)) goto done;
                    PA_TRACE(4, 0, t);
                    uint32_t bytes = 0;
                    int blocks[Smem::NREC];
#pragma unroll
                    for (int r = 0; r < Smem::NREC; ++r) {
                        const int bi = j * Smem::NREC + r;
                        int blk = -1;
                        if (bi * BS < ctx_hi) {
                            blk = it.table[bi];
                            if (blk < 0 || blk >= a.num_blocks) { blk = 0; bad_index = true; }
                            bytes += 2 * Smem::REC;
                        }
                        blocks[r] = blk;
                    }
#ifdef PA_EXP_NOLOAD
                    bytes = 0;
#endif
                    mbar_expect_tx(&sm.raw_full[st], bytes);
#pragma unroll
                    for (int r = 0; r < Smem::NREC; ++r)
                        if (blocks[r] >= 0 && bytes) {
                            bulk_g2s(sm.raw_k[st] + r * Smem::RSTRIDE, kc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.raw_full[st]);
                            bulk_g2s(sm.raw_v[st] + r * Smem::RSTRIDE, vc + (long long)blocks[r] * a.g.block_bytes, Smem::REC, &sm.raw_full[st]);
                        }
                }
                }
            }
            if (bad_index) atomicOr(a.status, PA_DEV_BAD_BLOCK_INDEX);
        }
    }
done:
#ifdef PA_PREFILL_PROF
    __syncthreads();
    if (blockIdx.x == 0 && tid == 0) {
        const long long base = trace[3][0][0];
        for (int role = 0; role < 5; ++role)
            for (int tl = 0; tl < 4; ++tl)
                printf("trace role %d tile %d: %lld %lld %lld %lld %lld %lld %lld %lld\n", role, 64 + tl, trace[role][0][tl] - base, trace[role][1][tl] - base,
                       trace[role][2][tl] - base, trace[role][3][tl] - base, trace[role][4][tl] - base, trace[role][5][tl] - base, trace[role][6][tl] - base,
                       trace[role][7][tl] - base);
    }
    if (blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 4 || warp == kSoftmaxWarps || warp >= kWarpMma))
        printf("prefill prof warp %d total %lld waits %lld %lld %lld %lld %lld\n", warp, clock64() - prof_begin, prof[0], prof[1], prof[2], prof[3], prof[4]);
#endif
    if constexpr (!U8) cp_async_wait<0>();   // an aborted copy warp leaves no copy in flight
    tc05::fence_before_thread_sync();
    __syncthreads();
    if (warp == 0) tc05::tmem_dealloc(tmem, kTmemCols);
}

}  // namespace

bool prefill_tc_supported(const CacheGeom& g) {
    // the bf16 cache with bf16 activations only: other queries would need a second, low piece of every row
    const bool cache_ok = g.cache == PA_DTYPE_U8 || g.cache == PA_DTYPE_F16 || (g.cache == PA_DTYPE_BF16 && g.act == PA_DTYPE_BF16);
    return cache_ok && (g.D == 128 || g.D == 64) && (g.bs == 32 || g.bs == 16) && g.Hq % g.Hkv == 0;
}

namespace {
template <int BS, int CT, int D>
cudaError_t launch_tc_t(const KernelArgs& a, cudaStream_t stream, int grid) {
    const int bytes = (int)sizeof(PrefillSmem<BS, CT, D>) + 1024;
    cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<BS, CT, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    prefill_tc_kernel<BS, CT, D><<<grid, kThreads, bytes, stream>>>(a);
    return cudaGetLastError();
}
template <int CT, int D>
cudaError_t launch_tc_bs(const KernelArgs& a, cudaStream_t stream, int grid) {
    return a.g.bs == 32 ? launch_tc_t<32, CT, D>(a, stream, grid) : launch_tc_t<16, CT, D>(a, stream, grid);
}
}  // namespace

cudaError_t launch_prefill_tc(const KernelArgs& a, cudaStream_t stream, int sm_count, long long max_items, int* launches) {
    if (max_items <= 0) return cudaSuccess;
    const int grid = (int)std::min<long long>(max_items, sm_count);
    cudaError_t e;
    if (a.g.cache == PA_DTYPE_U8) e = a.g.D == 128 ? launch_tc_bs<PA_DTYPE_U8, 128>(a, stream, grid) : launch_tc_bs<PA_DTYPE_U8, 64>(a, stream, grid);
    else if (a.g.cache == PA_DTYPE_F16) e = a.g.D == 128 ? launch_tc_bs<PA_DTYPE_F16, 128>(a, stream, grid) : launch_tc_bs<PA_DTYPE_F16, 64>(a, stream, grid);
    else e = a.g.D == 128 ? launch_tc_bs<PA_DTYPE_BF16, 128>(a, stream, grid) : launch_tc_bs<PA_DTYPE_BF16, 64>(a, stream, grid);
    if (e != cudaSuccess) return e;
    ++*launches;
    return cudaSuccess;
}

}  // namespace pa
