// Shared device helpers of the sm_100a PagedAttention kernels: element conversion, the
// by-token u8 quantiser, mbarrier / bulk-copy / cp.async / mma.sync wrappers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/pa_b200.h"

namespace pa {

constexpr int kWarp = 32;

// ---- geometry of the paged cache (see pa_cache_layout in pa_b200.h) -------------------------
struct CacheGeom {
    int Hq, Hkv, D, bs;
    int act, cache;
    long long head_bytes;   // one (block, head) record
    long long block_bytes;  // one physical block, all heads
};

__host__ __device__ inline long long head_record_bytes(int cache_dtype, int bs, int D) {
    return cache_dtype == PA_DTYPE_U8 ? (long long)bs * (D + 8) : (long long)bs * D * 2;
}

// ---- activations ---------------------------------------------------------------------------
template <int ACT> struct ActT;
template <> struct ActT<PA_DTYPE_F32> { using type = float; };
template <> struct ActT<PA_DTYPE_F16> { using type = __half; };
template <> struct ActT<PA_DTYPE_BF16> { using type = __nv_bfloat16; };

__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }

__device__ __forceinline__ void from_float(float& d, float x) { d = x; }
__device__ __forceinline__ void from_float(__half& d, float x) { d = __float2half_rn(x); }
__device__ __forceinline__ void from_float(__nv_bfloat16& d, float x) { d = __float2bfloat16_rn(x); }

__device__ __forceinline__ float load_act(const void* p, long long i, int act) {
    if (act == PA_DTYPE_F32) return ((const float*)p)[i];
    if (act == PA_DTYPE_F16) return __half2float(((const __half*)p)[i]);
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// N consecutive activations starting at element i (i a multiple of N, N*2 bytes <= 32 and the
// tensor's base 16-byte aligned) with 16-byte / 8-byte / 4-byte loads.
template <int N>
__device__ __forceinline__ void load_act_vec(const void* p, long long i, int act, float (&out)[N]) {
    static_assert(N == 2 || N == 4 || N == 8 || N == 16, "vector widths");
    if (act == PA_DTYPE_F32) {
        if constexpr (N >= 4) {
#pragma unroll
            for (int k = 0; k < N / 4; ++k) {
                const float4 v = *reinterpret_cast<const float4*>((const float*)p + i + 4 * k);
                out[4 * k] = v.x; out[4 * k + 1] = v.y; out[4 * k + 2] = v.z; out[4 * k + 3] = v.w;
            }
        } else {
            const float2 v = *reinterpret_cast<const float2*>((const float*)p + i);
            out[0] = v.x; out[1] = v.y;
        }
        return;
    }
    uint32_t w[N / 2];
    const uint16_t* src = (const uint16_t*)p + i;
    if constexpr (N >= 8) {
#pragma unroll
        for (int k = 0; k < N / 8; ++k) {
            const uint4 v = *reinterpret_cast<const uint4*>(src + 8 * k);
            w[4 * k] = v.x; w[4 * k + 1] = v.y; w[4 * k + 2] = v.z; w[4 * k + 3] = v.w;
        }
    } else if constexpr (N == 4) {
        const uint2 v = *reinterpret_cast<const uint2*>(src);
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = *reinterpret_cast<const uint32_t*>(src);
    }
#pragma unroll
    for (int k = 0; k < N / 2; ++k) {
        if (act == PA_DTYPE_F16) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[k]));
            out[2 * k] = f.x; out[2 * k + 1] = f.y;
        } else {
            out[2 * k] = __uint_as_float(w[k] << 16);
            out[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
        }
    }
}

__device__ __forceinline__ void store_act(void* p, long long i, int act, float v) {
    if (act == PA_DTYPE_F32) ((float*)p)[i] = v;
    else if (act == PA_DTYPE_F16) ((__half*)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}

// 8 consecutive activations starting at element i (i a multiple of 8, base 16-byte aligned).
__device__ __forceinline__ void store_act_vec8(void* p, long long i, int act, const float (&v)[8]) {
    if (act == PA_DTYPE_F32) {
        float4* dst = reinterpret_cast<float4*>((float*)p + i);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
        return;
    }
    uint4 w;
    if (act == PA_DTYPE_F16) {
        __half2 h0 = __floats2half2_rn(v[0], v[1]), h1 = __floats2half2_rn(v[2], v[3]);
        __half2 h2 = __floats2half2_rn(v[4], v[5]), h3 = __floats2half2_rn(v[6], v[7]);
        w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
        w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
    } else {
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
        w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
        w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
    }
    *reinterpret_cast<uint4*>((uint16_t*)p + i) = w;
}

// ---- by-token asymmetric u8 quantiser --------------------------------------------------------
// scale = (max - min) / 255 (1 for a constant row), zp = -min / scale,
// q = clamp(rint(fma(x, 1/scale, zp)), 0, 255).  Every step is individually rounded so that the
// bytes are reproducible on any IEEE machine.
__device__ __forceinline__ void quant_params(float mn, float mx, float& scale, float& zp, float& inv) {
    float s = __fdiv_rn(__fsub_rn(mx, mn), 255.0f);
    if (!(s > 0.f) || isinf(s) || isnan(s)) s = 1.0f;
    scale = s;
    zp = __fdiv_rn(-mn, s);
    inv = __fdiv_rn(1.0f, s);
}

__device__ __forceinline__ unsigned quant_one(float x, float inv, float zp) {
    float q = rintf(__fmaf_rn(x, inv, zp));
    q = fminf(255.0f, fmaxf(0.0f, q));
    return (unsigned)q;
}

__device__ __forceinline__ float dequant_one(unsigned q, float scale, float zp) {
    return __fmul_rn(__fsub_rn((float)q, zp), scale);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---- shared-memory addressing, mbarrier, bulk copy (TMA engine), cp.async ---------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls and reports false so the caller can flag an error
// and leave instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// 1-D bulk copy global -> shared through the TMA engine.  Both addresses 16-byte aligned, size a
// multiple of 16 bytes.  Completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src_gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst_smem)), "l"(src_gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tensor-core fragments (mma.sync m16n8k16, f32 accumulate) --------------------------------
// Only rows 0..7 of the 16-row A operand are live when HI == false: the upper accumulator half is
// then computed from zeros and dropped, which saves its registers.
template <bool BF16, bool HI>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (HI) {
        if constexpr (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                         : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                         : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        float t2, t3;
        if constexpr (BF16)
            asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                         : "+f"(c[0]), "+f"(c[1]), "=f"(t2), "=f"(t3)
                         : "r"(a[0]), "r"(0u), "r"(a[2]), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
        else
            asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                         : "+f"(c[0]), "+f"(c[1]), "=f"(t2), "=f"(t3)
                         : "r"(a[0]), "r"(0u), "r"(a[2]), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
        (void)t2; (void)t3;
    }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

// Two cache bytes -> two exact f16 values.  0x6400 is 1024.0 in f16 with a unit ulp, so
// (0x6400 | byte) is 1024 + byte; subtracting 1024 leaves the integer exactly.
__device__ __forceinline__ uint32_t u8x2_to_h2_lo(uint32_t w) {
    uint32_t r = __byte_perm(w, 0x64646464u, 0x4140);
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), __half2half2(__ushort_as_half((unsigned short)0x6400)));
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t u8x2_to_h2_hi(uint32_t w) {
    uint32_t r = __byte_perm(w, 0x64646464u, 0x4342);
    __half2 h = __hsub2(*reinterpret_cast<__half2*>(&r), __half2half2(__ushort_as_half((unsigned short)0x6400)));
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

}  // namespace pa
