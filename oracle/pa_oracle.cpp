// TEST INFRASTRUCTURE - CPU restatement of the PagedAttentionExtension operator contract.
//
// PARITY UNPINNED: the reference executes this operator inside the un-vendored OpenVINO
// runtime (openvino~=2026.4.0.0.dev, pyproject.toml:56); no source, golden vector or runnable
// copy of it exists under the reference tree.  What the reference does pin is the tensor
// contract at its call sites, which this file follows:
//   past_lens / subsequence_begins / block_indices / block_indices_begins / max_context_len
//     src/cpp/src/continuous_batching/model_runner.hpp:505-522, 802-853, 1420-1481
//   score_aggregation_window and the per-sequence layout of `scores`
//     model_runner.hpp:838-848, 1518-1568; cache/cache_eviction.cpp:110-135, 638-657
//   rotated_block_indices / rotation_deltas / rotation_trig_lut (cos | -sin halves)
//     model_runner.hpp:1483-1509; pipeline_impl.cpp:256-290; cache/cache_eviction.cpp:543-573
// Arithmetic decisions that no reference file states (fp32 math, u8 rounding, K-only rotation,
// scores = sum over heads and window rows) are written beside the code that takes them.
//
// Only tests, the smoke check and the bench's CPU-baseline leg may call this file.  It is the
// checker, never the product path.
//
// All pointers are HOST memory.  The argument struct is the product's pa_forward_args.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../include/pa_b200.h"

namespace {

inline float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t f;
    if (exp == 0) {
        if (man == 0) {
            f = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            man &= 0x3ffu;
            f = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        f = sign | 0x7f800000u | (man << 13);
    } else {
        f = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float out;
    std::memcpy(&out, &f, 4);
    return out;
}

inline uint16_t float_to_half(float x) {  // round to nearest even
    uint32_t f;
    std::memcpy(&f, &x, 4);
    uint32_t sign = (f >> 16) & 0x8000u;
    uint32_t a = f & 0x7fffffffu;
    if (a >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((a > 0x7f800000u) ? 0x200u : 0));
    if (a >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to inf
    if (a < 0x33000001u) return (uint16_t)sign;               // rounds to zero
    int exp = (int)(a >> 23);
    uint32_t man = (a & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < 113) {  // subnormal half
        shift = 126 - exp;  // 14..24
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(exp - 112) << 10;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (exp >= 113) q &= 0x3ffu;
    uint32_t r = base + q;
    if (rem > halfway || (rem == halfway && (r & 1u))) ++r;
    return (uint16_t)(sign | r);
}

inline float bf16_to_float(uint16_t h) {
    uint32_t f = (uint32_t)h << 16;
    float out;
    std::memcpy(&out, &f, 4);
    return out;
}

inline uint16_t float_to_bf16(float x) {  // round to nearest even
    uint32_t f;
    std::memcpy(&f, &x, 4);
    if ((f & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((f >> 16) | 0x40u);
    uint32_t lsb = (f >> 16) & 1u;
    f += 0x7fffu + lsb;
    return (uint16_t)(f >> 16);
}

inline float load_act(const void* p, int64_t i, int dt) {
    switch (dt) {
        case PA_DTYPE_F32: return ((const float*)p)[i];
        case PA_DTYPE_F16: return half_to_float(((const uint16_t*)p)[i]);
        default: return bf16_to_float(((const uint16_t*)p)[i]);
    }
}

inline void store_act(void* p, int64_t i, int dt, float v) {
    switch (dt) {
        case PA_DTYPE_F32: ((float*)p)[i] = v; break;
        case PA_DTYPE_F16: ((uint16_t*)p)[i] = float_to_half(v); break;
        default: ((uint16_t*)p)[i] = float_to_bf16(v); break;
    }
}

struct Geometry {
    int Hq, Hkv, D, bs, act, cache;
    int64_t head_bytes;   // bytes of one (block, head) record in either cache
    int64_t block_bytes;  // bytes of one physical block
    float scale;
};

Geometry make_geometry(const pa_model_desc* d, float scale) {
    Geometry g;
    g.Hq = d->num_q_heads; g.Hkv = d->num_kv_heads; g.D = d->head_size; g.bs = d->block_size;
    g.act = d->act_dtype; g.cache = d->cache_dtype;
    g.head_bytes = (g.cache == PA_DTYPE_U8) ? (int64_t)g.bs * (g.D + 8) : (int64_t)g.bs * g.D * 2;
    g.block_bytes = g.head_bytes * g.Hkv;
    g.scale = scale != 0.f ? scale : 1.0f / std::sqrt((float)g.D);
    return g;
}

// ---- cache element access ----------------------------------------------------------------
// u8 record of one (block, head):  data, then f32 scale[bs], then f32 zp[bs].
// key data is [bs][D]; value data is [D][bs].
inline uint8_t* rec(void* cache, const Geometry& g, int64_t block, int head) {
    return (uint8_t*)cache + block * g.block_bytes + (int64_t)head * g.head_bytes;
}

// Decision: dequantised value = (q - zp) * scale, the subtraction rounded before the product.
inline float dequant(uint8_t q, float scale, float zp) { return ((float)q - zp) * scale; }

inline float read_k(void* cache, const Geometry& g, int64_t block, int head, int slot, int d) {
    uint8_t* r = rec(cache, g, block, head);
    if (g.cache == PA_DTYPE_U8) {
        const float* sc = (const float*)(r + (int64_t)g.bs * g.D);
        const float* zp = sc + g.bs;
        return dequant(r[(int64_t)slot * g.D + d], sc[slot], zp[slot]);
    }
    uint16_t h = ((uint16_t*)r)[(int64_t)slot * g.D + d];
    return g.cache == PA_DTYPE_F16 ? half_to_float(h) : bf16_to_float(h);
}

inline float read_v(void* cache, const Geometry& g, int64_t block, int head, int slot, int d) {
    uint8_t* r = rec(cache, g, block, head);
    if (g.cache == PA_DTYPE_U8) {
        const float* sc = (const float*)(r + (int64_t)g.bs * g.D);
        const float* zp = sc + g.bs;
        return dequant(r[(int64_t)d * g.bs + slot], sc[slot], zp[slot]);
    }
    uint16_t h = ((uint16_t*)r)[(int64_t)slot * g.D + d];
    return g.cache == PA_DTYPE_F16 ? half_to_float(h) : bf16_to_float(h);
}

// By-token asymmetric u8 quantisation of one head row of D floats.
// Decision: scale = (max - min) / 255 (1 if the row is constant), zp = -min / scale,
// q = clamp(rint(fma(x, 1/scale, zp)), 0, 255), rint = round half to even.
inline void quant_params(const float* x, int D, float* scale, float* zp, float* inv) {
    float mn = x[0], mx = x[0];
    for (int i = 1; i < D; ++i) { mn = std::min(mn, x[i]); mx = std::max(mx, x[i]); }
    float s = (mx - mn) / 255.0f;
    if (!(s > 0.f) || !std::isfinite(s)) s = 1.0f;
    *scale = s;
    *zp = -mn / s;
    *inv = 1.0f / s;
}

inline uint8_t quant_one(float x, float inv, float zp) {
    float q = std::nearbyintf(std::fmaf(x, inv, zp));
    q = std::min(255.0f, std::max(0.0f, q));
    return (uint8_t)q;
}

void write_row(void* cache, const Geometry& g, int64_t block, int head, int slot, const float* x, bool is_value) {
    uint8_t* r = rec(cache, g, block, head);
    if (g.cache == PA_DTYPE_U8) {
        float* sc = (float*)(r + (int64_t)g.bs * g.D);
        float* zp = sc + g.bs;
        float s, z, inv;
        quant_params(x, g.D, &s, &z, &inv);
        sc[slot] = s;
        zp[slot] = z;
        for (int d = 0; d < g.D; ++d) {
            uint8_t q = quant_one(x[d], inv, z);
            if (is_value) r[(int64_t)d * g.bs + slot] = q; else r[(int64_t)slot * g.D + d] = q;
        }
    } else {
        uint16_t* p = (uint16_t*)r + (int64_t)slot * g.D;
        for (int d = 0; d < g.D; ++d) p[d] = g.cache == PA_DTYPE_F16 ? float_to_half(x[d]) : float_to_bf16(x[d]);
    }
}

template <class F>
void parallel_for(int64_t n, int threads, F&& f) {
    if (threads <= 1 || n <= 1) { for (int64_t i = 0; i < n; ++i) f(i); return; }
    std::atomic<int64_t> next{0};
    std::vector<std::thread> pool;
    int nt = (int)std::min<int64_t>(threads, n);
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&] { for (int64_t i; (i = next.fetch_add(1)) < n;) f(i); });
    for (auto& th : pool) th.join();
}

bool metadata_ok(const pa_forward_args* a, const Geometry& g) {
    if (a->num_sequences < 0 || a->num_tokens < 0) return false;
    for (int s = 0; s < a->num_sequences; ++s) {
        int n = a->subsequence_begins[s + 1] - a->subsequence_begins[s];
        int nb = a->block_indices_begins[s + 1] - a->block_indices_begins[s];
        if (n < 0 || nb < 0 || a->past_lens[s] < 0) return false;
        int64_t need = ((int64_t)a->past_lens[s] + n + g.bs - 1) / g.bs;
        if (nb < need) return false;
        for (int b = 0; b < nb; ++b) {
            int id = a->block_indices[a->block_indices_begins[s] + b];
            if (id < 0 || id >= a->num_blocks) return false;
        }
    }
    return true;
}

}  // namespace

extern "C" {

// Step 1 of the operator: re-rotate the keys of the listed physical blocks, in place.
// Decision (no reference file states the arithmetic): keys only; rotate-half pairing
//   k'[j]       = k[j]*c_j - k[j+D/2]*s_j
//   k'[j+D/2]   = k[j+D/2]*c_j + k[j]*s_j
// with c = lut[row][j], s = lut[row][D/2+j] (the LUT's second half already holds -sin,
// cache_eviction.cpp:567-569), each line evaluated as fma(-+k, s, round(k*c)); a u8 block is
// dequantised, rotated and re-quantised token by token with fresh scale / zero-point.
int pa_oracle_rotate_blocks(const pa_model_desc* desc, const pa_forward_args* a) {
    if (!a->rotated_block_indices || a->num_rotated_blocks <= 0) return PA_OK;
    Geometry g = make_geometry(desc, a->scale);
    const int half = g.D / 2;
    std::vector<float> x(g.D), y(g.D);
    for (int r = 0; r < a->num_rotated_blocks; ++r) {
        int64_t block = a->rotated_block_indices[r];
        int row = a->rotation_deltas[r];
        if (block < 0 || block >= a->num_blocks || row < 0 || row >= a->rotation_lut_rows) return PA_ERR_BAD_INDEX;
        const float* lut = a->rotation_trig_lut + (int64_t)row * g.D;
        for (int h = 0; h < g.Hkv; ++h)
            for (int t = 0; t < g.bs; ++t) {
                for (int d = 0; d < g.D; ++d) x[d] = read_k(a->key_cache, g, block, h, t, d);
                for (int j = 0; j < half; ++j) {
                    float c = lut[j], s = lut[half + j];
                    float k0 = x[j], k1 = x[j + half];
                    y[j] = std::fmaf(-k1, s, k0 * c);
                    y[j + half] = std::fmaf(k0, s, k1 * c);
                }
                write_row(a->key_cache, g, block, h, t, y.data(), false);
            }
    }
    return PA_OK;
}

// Step 2: write the chunk's new keys / values into slots past .. past+n-1 of each sequence.
int pa_oracle_write_kv(const pa_model_desc* desc, const pa_forward_args* a) {
    Geometry g = make_geometry(desc, a->scale);
    if (!metadata_ok(a, g)) return PA_ERR_BAD_INDEX;
    std::vector<float> x(g.D);
    for (int s = 0; s < a->num_sequences; ++s) {
        int t0 = a->subsequence_begins[s], n = a->subsequence_begins[s + 1] - t0;
        const int32_t* table = a->block_indices + a->block_indices_begins[s];
        for (int j = 0; j < n; ++j) {
            int pos = a->past_lens[s] + j;
            int64_t block = table[pos / g.bs];
            int slot = pos % g.bs;
            for (int h = 0; h < g.Hkv; ++h) {
                int64_t base = ((int64_t)(t0 + j) * g.Hkv + h) * g.D;
                for (int d = 0; d < g.D; ++d) x[d] = load_act(a->key, base + d, g.act);
                write_row(a->key_cache, g, block, h, slot, x.data(), false);
                for (int d = 0; d < g.D; ++d) x[d] = load_act(a->value, base + d, g.act);
                write_row(a->value_cache, g, block, h, slot, x.data(), true);
            }
        }
    }
    return PA_OK;
}

// Step 3: causal grouped-query attention of every new token over positions 0 .. past+j, read
// back from the cache (so a chunk sees its own keys at cache precision), fp32 throughout:
//   logit = scale * dot(q, k);  p = exp(logit - max) / sum;  out = sum p * v
// scores[pos] = sum over q heads and over the last W rows of the chunk of p[h][row][pos],
// W = min(score_aggregation_window[s], n); W == 0 writes zeros (cache_eviction.cpp:131-135
// ignores them but model_runner.hpp:1536-1537 still counts their slots).
int pa_oracle_attend(const pa_model_desc* desc, const pa_forward_args* a, int threads) {
    Geometry g = make_geometry(desc, a->scale);
    if (!metadata_ok(a, g)) return PA_ERR_BAD_INDEX;
    const int G = g.Hq / g.Hkv;
    std::vector<int64_t> score_off(a->num_sequences + 1, 0);
    for (int s = 0; s < a->num_sequences; ++s)
        score_off[s + 1] = score_off[s] + a->past_lens[s] + (a->subsequence_begins[s + 1] - a->subsequence_begins[s]);
    const bool want_scores = a->scores && a->score_aggregation_window;
    if (want_scores) {
        if (a->scores_len < score_off[a->num_sequences]) return PA_ERR_INVALID_ARG;
        std::fill(a->scores, a->scores + a->scores_len, 0.f);
    }
    // scores are accumulated per (sequence, kv head) into private rows and summed in head
    // order afterwards so the result does not depend on the thread schedule.
    std::vector<std::vector<float>> partial(want_scores ? (size_t)a->num_sequences * g.Hkv : 0);

    parallel_for((int64_t)a->num_sequences * g.Hkv, threads, [&](int64_t item) {
        int s = (int)(item / g.Hkv), hk = (int)(item % g.Hkv);
        int t0 = a->subsequence_begins[s], n = a->subsequence_begins[s + 1] - t0;
        int past = a->past_lens[s];
        int ctx = past + n;
        const int32_t* table = a->block_indices + a->block_indices_begins[s];
        int W = want_scores ? std::min(std::max(a->score_aggregation_window[s], 0), n) : 0;
        std::vector<float> kd((size_t)ctx * g.D), vd((size_t)ctx * g.D);
        for (int pos = 0; pos < ctx; ++pos) {
            int64_t block = table[pos / g.bs];
            int slot = pos % g.bs;
            for (int d = 0; d < g.D; ++d) {
                kd[(size_t)pos * g.D + d] = read_k(a->key_cache, g, block, hk, slot, d);
                vd[(size_t)pos * g.D + d] = read_v(a->value_cache, g, block, hk, slot, d);
            }
        }
        std::vector<float> logit(ctx), q(g.D), acc(g.D);
        std::vector<float>* sc = nullptr;
        if (want_scores) { sc = &partial[item]; sc->assign(ctx, 0.f); }
        for (int j = 0; j < n; ++j) {
            int visible = past + j + 1;
            for (int hq = hk * G; hq < (hk + 1) * G; ++hq) {
                int64_t qbase = ((int64_t)(t0 + j) * g.Hq + hq) * g.D;
                for (int d = 0; d < g.D; ++d) q[d] = load_act(a->query, qbase + d, g.act);
                float mx = -INFINITY;
                for (int pos = 0; pos < visible; ++pos) {
                    const float* kr = &kd[(size_t)pos * g.D];
                    float dot = 0.f;
                    for (int d = 0; d < g.D; ++d) dot += q[d] * kr[d];
                    logit[pos] = dot * g.scale;
                    mx = std::max(mx, logit[pos]);
                }
                double sum = 0.0;
                for (int pos = 0; pos < visible; ++pos) { logit[pos] = std::exp(logit[pos] - mx); sum += logit[pos]; }
                float inv = (float)(1.0 / sum);
                std::fill(acc.begin(), acc.end(), 0.f);
                for (int pos = 0; pos < visible; ++pos) {
                    float p = logit[pos] * inv;
                    const float* vr = &vd[(size_t)pos * g.D];
                    for (int d = 0; d < g.D; ++d) acc[d] += p * vr[d];
                    if (sc && j >= n - W) (*sc)[pos] += p;
                }
                for (int d = 0; d < g.D; ++d) store_act(a->output, qbase + d, g.act, acc[d]);
            }
        }
    });
    if (want_scores)
        for (int s = 0; s < a->num_sequences; ++s)
            for (int hk = 0; hk < g.Hkv; ++hk) {
                const auto& p = partial[(size_t)s * g.Hkv + hk];
                float* dst = a->scores + score_off[s];
                for (size_t i = 0; i < p.size(); ++i) dst[i] += p[i];
            }
    return PA_OK;
}

// The whole operator: rotate listed blocks, write the chunk, attend.
int pa_oracle_forward(const pa_model_desc* desc, const pa_forward_args* a, int threads) {
    if (a->sliding_window != 0 || a->alibi_slopes != nullptr) return PA_ERR_UNSUPPORTED;
    int rc = pa_oracle_rotate_blocks(desc, a);
    if (rc != PA_OK) return rc;
    rc = pa_oracle_write_kv(desc, a);
    if (rc != PA_OK) return rc;
    return pa_oracle_attend(desc, a, threads);
}

// Element-level readers used by tests to build caches and to gather dense K/V for an
// independent second opinion (torch scaled_dot_product_attention on the CPU).
void pa_oracle_gather_dense(const pa_model_desc* desc, void* key_cache, void* value_cache, const int32_t* table,
                            int ctx, int kv_head, float* k_out, float* v_out) {
    Geometry g = make_geometry(desc, 0.f);
    for (int pos = 0; pos < ctx; ++pos) {
        int64_t block = table[pos / g.bs];
        int slot = pos % g.bs;
        for (int d = 0; d < g.D; ++d) {
            k_out[(size_t)pos * g.D + d] = read_k(key_cache, g, block, kv_head, slot, d);
            v_out[(size_t)pos * g.D + d] = read_v(value_cache, g, block, kv_head, slot, d);
        }
    }
}

int pa_oracle_hardware_threads() { return (int)std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"
