// TEST INFRASTRUCTURE - not part of the shipped library.
//
// CPU restatement of the reference engine's block-quantized MoE FFN arithmetic (hyukudan/strix-halo-engine-lab),
// written from its declared contracts so that the CUDA path can be compared bit for bit. Every function names the
// reference file:line it follows. Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may load
// this file; the product library never links or calls it.
//
// Parity status: PINNED. tests/test_oracle_pins.py checks this file against (a) the known-answer literals of the
// reference's own tests (router digest 0x168f06b494ae3b13, cancellation / subnormal Q8_0 fixtures, tie / NaN / -0
// router literals), (b) outputs of the reference's own CPU code compiled from its sources (oracle/_ref, built by
// oracle/Makefile) on seeded inputs, and (c) the committed vectors under tests/golden/ generated from that build.
// The group-limited routing step (n_group > 1) has no counterpart in the reference: that step alone is unpinned.
//
// Build: g++ -O2 -std=c++17 -ffp-contract=off -pthread -shared -fPIC (oracle/Makefile). Contraction MUST stay off:
// every float operation below is one IEEE-754 binary32 operation.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <atomic>
#include <functional>
#include <limits>
#include <thread>
#include <vector>

#include "../include/b200moe.h"

#if defined(__FAST_MATH__)
#error "the oracle needs strict IEEE semantics"
#endif

namespace {

using u8 = std::uint8_t;
using u16 = std::uint16_t;
using u32 = std::uint32_t;
using u64 = std::uint64_t;
using i8 = std::int8_t;
using i32 = std::int32_t;

inline float bits_f(u32 b) { float f; std::memcpy(&f, &b, 4); return f; }
inline u32 f_bits(float f) { u32 b; std::memcpy(&b, &f, 4); return b; }
inline bool is_finite(float x) { return (f_bits(x) & 0x7f800000u) != 0x7f800000u; }

// fp16 -> fp32, exact incl. subnormals (src/cpu/core/reference.cpp:15-24).
inline float half_f(u16 h) {
    const u32 sign = (u32)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u;
    if (e == 0) { const float v = std::ldexp((float)m, -24); return sign ? -v : v; }
    if (e == 31) return bits_f(sign | 0x7f800000u | (m << 13));
    return bits_f(sign | ((e + 112u) << 23) | (m << 13));
}
inline u16 ld16(const u8* p) { return (u16)(p[0] | (p[1] << 8)); }

// ---- A8 (src/cpu/core/reference.cpp:35-55; src/ds41_formats.cpp:146-165) ---------------------------------------
void quantize_group(const float* x, i8* codes, float* delta, i32* sum) {
    float amax = 0.0f;
    for (int j = 0; j < 32; ++j) amax = std::max(amax, std::fabs(x[j]));
    const bool tiny = amax > 0.0f && amax < 0x1p-119f;
    const float d = (amax == 0.0f || tiny) ? 1.0f : amax / 127.0f;
    i32 s = 0;
    for (int j = 0; j < 32; ++j) {
        const float r = tiny ? 0.0f : std::nearbyint(x[j] / d);
        const i8 c = (i8)std::min(127.0f, std::max(-127.0f, r));
        codes[j] = c;
        s += c;
    }
    *delta = d;
    *sum = s;
}

// ---- butterfly of 32 lane classes (src/ds41_formats.cpp:37-44; src/core/integer_math.hpp:43-47) -----------------
float butterfly32(float* v) {
    for (unsigned d = 16; d; d >>= 1) {
        float n[32];
        for (unsigned l = 0; l < 32; ++l) n[l] = v[l] + v[l ^ d];
        std::memcpy(v, n, sizeof n);
    }
    return v[0];
}

// ---- Q8_0 x A8 product, DS41 / CPU-backend contract (src/ds41_formats.cpp:188-197; reference.cpp:57-84) ---------
float product_q8_0(const u8* row, const i8* codes, const float* deltas, size_t width) {
    float lanes[32];
    for (auto& l : lanes) l = 0.0f;
    for (size_t g = 0; g < width / 32; ++g) {
        const u8* blk = row + g * 34;
        const float scale = half_f(ld16(blk));
        i32 dot = 0;
        for (int j = 0; j < 32; ++j) dot += (i32)(i8)blk[2 + j] * (i32)codes[g * 32 + j];
        const float sd = scale * deltas[g];
        lanes[g % 32] = lanes[g % 32] + (float)dot * sd;
    }
    return butterfly32(lanes);
}

// ---- Q2_K x A8 product, DS41 contract (src/ds41_formats.cpp:106-115 q2_k_group, :198-218 product_q2_k) ---------------
// 84-byte super-blocks {scales[16], qs[64], fp16 d, fp16 dmin}; group g of a block: half = g / 4, 2-bit codes at bit
// 2 * (g % 4) of qs[32 * half + l]; its two 16-weight halves carry (scale | min << 4) bytes 8 * half + 2 * (g % 4) + {0, 1}.
float product_q2_k(const u8* row, const i8* codes, const float* deltas, size_t width) {
    float lanes[32];
    for (auto& l : lanes) l = 0.0f;
    for (size_t g = 0; g < width / 32; ++g) {
        const u8* blk = row + g / 8 * 84;
        const unsigned within = (unsigned)(g % 8), half = within / 4, shift = 2 * (within % 4);
        i32 a = 0, b = 0;
        for (unsigned h = 0; h < 2; ++h) {
            i32 qx = 0, sx = 0;
            for (unsigned j = 16 * h; j < 16 * h + 16; ++j) {
                const i32 q = (blk[16 + 32 * half + j] >> shift) & 3, x = codes[g * 32 + j];
                qx += q * x;
                sx += x;
            }
            const u8 sc = blk[8 * half + 2 * (within % 4) + h];
            a += (i32)(sc & 15) * qx;
            b += (i32)(sc >> 4) * sx;
        }
        const float scaled = half_f(ld16(blk + 80)) * (float)a;
        const float offset = half_f(ld16(blk + 82)) * (float)b;
        lanes[g % 32] = lanes[g % 32] + (scaled - offset) * deltas[g];
    }
    return butterfly32(lanes);
}
inline float product_ds41(u32 type, const u8* row, const i8* codes, const float* deltas, size_t width) {
    return type == B200MOE_TYPE_Q2_K ? product_q2_k(row, codes, deltas, width) : product_q8_0(row, codes, deltas, width);
}

// ---- Q4_K 6-bit factors (src/cpu/core/routed_expert.cpp:65-71 == get_scale_min_k4, src/ggml_dequant.cpp:43-50) --
inline void q4k_factors(const u8* blk, unsigned j, unsigned* sc, unsigned* mn) {
    const u8* p = blk + 4;
    if (j < 4) { *sc = p[j] & 63u; *mn = p[j + 4] & 63u; }
    else { *sc = (p[j + 4] & 15u) | ((p[j - 4] >> 6) << 4); *mn = (p[j + 4] >> 4) | ((p[j] >> 6) << 4); }
}

// ---- Q4_K x A8 row, Qwen A8 contract (src/cpu/core/routed_expert.cpp:73-108; moe_q4k_a8_contract.cpp:126-141) ---
inline size_t row_bytes(u32 type, u32 width) {
    switch (type) {
        case B200MOE_TYPE_Q8_0: return (size_t)width / 32 * 34;
        case B200MOE_TYPE_Q5_1: return (size_t)width / 32 * 24;
        case B200MOE_TYPE_Q5_K: return (size_t)width / 256 * 176;
        case B200MOE_TYPE_Q2_K: return (size_t)width / 256 * 84;
        default: return (size_t)width / 256 * 144;
    }
}
// q5k: 176-byte super-blocks, 32 bytes of high bits at offset 16 (bit j of byte k = bit 4 of weight k of group j), the
// nibbles from offset 48 (routed_expert.cpp:75, :88-95); everything else is the Q4_K rule.
float row_kquant(const u8* row, u32 blocks, const i8* codes, const float* deltas, const i32* sums, bool q5k) {
    const size_t wb = q5k ? 176 : 144, qs = q5k ? 48 : 16;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (u32 b = 0; b < blocks; ++b) {
        const u8* blk = row + (size_t)b * wb;
        const float d = half_f(ld16(blk)), dm = half_f(ld16(blk + 2));
        float x[8];
        for (unsigned j = 0; j < 8; ++j) {
            const u8* q = blk + qs + 32 * (j >> 1);
            i32 dot = 0;
            for (int k = 0; k < 32; ++k) {
                int w = (j & 1) ? (q[k] >> 4) : (q[k] & 15);
                if (q5k) w |= ((blk[16 + k] >> j) & 1) << 4;
                dot += w * (i32)codes[256 * (size_t)b + 32 * j + k];
            }
            unsigned sc, mn;
            q4k_factors(blk, j, &sc, &mn);
            const float D = d * (float)sc, DM = dm * (float)mn;
            const float u = D * (float)dot;
            const float v = DM * (float)sums[8 * (size_t)b + j];
            const float t = u - v;
            x[j] = deltas[8 * (size_t)b + j] * t;
        }
        for (int p = 0; p < 4; ++p) { const float pair = x[2 * p] + x[2 * p + 1]; acc[p] = acc[p] + pair; }
    }
    const float s01 = acc[0] + acc[1], s23 = acc[2] + acc[3];
    return s01 + s23;
}

float row_q4k(const u8* row, u32 blocks, const i8* codes, const float* deltas, const i32* sums) {
    return row_kquant(row, blocks, codes, deltas, sums, false);
}

// ---- Q5_1 down row, four chains (src/cpu/core/routed_expert.cpp:110-144): combined = d * float(dot) + m * float(S_g) ----
float row_q5_1_chain4(const u8* row, u32 groups, const i8* codes, const float* deltas, const i32* sums) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (u32 g = 0; g < groups; ++g) {
        const u8* blk = row + (size_t)g * 24;
        const float d = half_f(ld16(blk)), m = half_f(ld16(blk + 2));
        u32 qh;
        std::memcpy(&qh, blk + 4, 4);
        i32 dot = 0;
        for (u32 k = 0; k < 32; ++k) {
            const u8 byte = blk[8 + (k & 15)];
            const int q = (k < 16 ? (byte & 15) : (byte >> 4)) | (int)(((qh >> k) & 1u) << 4);
            dot += q * (i32)codes[32 * (size_t)g + k];
        }
        const float first = d * (float)dot;
        const float combined = first + (m * (float)sums[g]);
        acc[g % 4] = acc[g % 4] + (deltas[g] * combined);
    }
    const float s01 = acc[0] + acc[1], s23 = acc[2] + acc[3];
    return s01 + s23;
}

// ---- Q8_0 down row, Qwen four-chain contract (src/cpu/core/routed_expert.cpp:110-144) ----------------------------
float row_q8_chain4(const u8* row, u32 groups, const i8* codes, const float* deltas) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (u32 g = 0; g < groups; ++g) {
        const u8* blk = row + (size_t)g * 34;
        const float d = half_f(ld16(blk));
        i32 dot = 0;
        for (int k = 0; k < 32; ++k) dot += (i32)(i8)blk[2 + k] * (i32)codes[32 * (size_t)g + k];
        const float first = d * (float)dot;
        acc[g % 4] = acc[g % 4] + deltas[g] * first;
    }
    const float s01 = acc[0] + acc[1], s23 = acc[2] + acc[3];
    return s01 + s23;
}

// ---- declared math of the DS41 family (include/strix/ds41_moe.hpp:31-100) ---------------------------------------
inline float pow2i(int k) { return bits_f((u32)(k + 127) << 23); }
float declared_exp(float x) {
    if (!(x == x)) return x;
    if (x > 88.0f) return std::numeric_limits<float>::infinity();
    if (x < -103.0f) return 0.0f;
    const float n = std::nearbyint(x * 1.44269504f);
    const float r = (x - n * 0.693359375f) - n * -2.12194440e-4f;
    float p = 1.98412698e-4f;
    p = p * r + 1.38888889e-3f;
    p = p * r + 8.33333333e-3f;
    p = p * r + 4.16666667e-2f;
    p = p * r + 1.66666667e-1f;
    p = p * r + 0.5f;
    p = p * r + 1.0f;
    p = p * r + 1.0f;
    const int k = (int)n, k1 = k / 2, k2 = k - k1;
    return (p * pow2i(k1)) * pow2i(k2);
}
float declared_log(float y) {
    const u32 b = f_bits(y);
    int k = (int)((b >> 23) & 0xffu) - 127;
    float m = bits_f((b & 0x7fffffu) | 0x3f800000u);
    if (m > 1.41421356f) { m = m * 0.5f; k = k + 1; }
    const float s = (m - 1.0f) / (m + 1.0f), s2 = s * s;
    float p = 0.111111111f;
    p = p * s2 + 0.142857143f;
    p = p * s2 + 0.2f;
    p = p * s2 + 0.333333333f;
    p = p * s2 + 1.0f;
    const float kf = (float)k;
    return kf * 0.693359375f + (kf * -2.12194440e-4f + (2.0f * s) * p);
}
float declared_log1p(float e) {
    const float u = 1.0f + e;
    if (u == 1.0f) return e;
    return declared_log(u) * (e / (u - 1.0f));
}
float sqrt_softplus(float z) { return std::sqrt(z > 20.0f ? z : declared_log1p(declared_exp(z))); }
float sigmoid_score(float z) { return 1.0f / (1.0f + declared_exp(-z)); }

// SwiGLU with the shared clamp trait (include/strix/ds41_moe.hpp:57-60; moe/activation_policy.hpp:22-24).
float swiglu_ds41(float g, float u, float limit) {
    const float cg = g > limit ? limit : g;
    const float cu = u < -limit ? -limit : (u > limit ? limit : u);
    return (cg / (1.0f + declared_exp(-cg))) * cu;
}

// ---- gfx1151 expf twin at zero correction tables (src/cpu/core/routed_expert.cpp:208-261) ------------------------
// With empty / zero tables v_exp(a) = float(exp2(double(a))) (routed_expert.cpp:212-228; the real probe tables are
// not part of the reference repository, its bench uses zero tables: scripts/bench/residency/cpu_expert_bench.cpp:78-89).
float gfx1151_expf(float x) {
    const float kLog2e = bits_f(0x3fb8aa3bu), kLog2eLo = bits_f(0x32a5705fu);
    const float ph = x * kLog2e;
    const float e = std::nearbyint(ph);
    float pl = std::fmaf(x, kLog2e, -ph);
    pl = std::fmaf(x, kLog2eLo, pl);
    const float a = (ph - e) + pl;
    float y;
    if (std::fabs(a) < 1.0f) y = std::scalbn((float)std::exp2((double)a), (int)e);
    else y = a != a ? a : 0.0f;
    if (bits_f(0xc2ce8ed0u) > x) y = 0.0f;
    if (bits_f(0x42b17218u) < x) y = bits_f(0x7f800000u);
    return y;
}
float swiglu_qwen(float g, float u) {  // routed_expert.cpp:151-153
    const float ex = gfx1151_expf(-g);
    return (g / (1.0f + ex)) * u;
}

// ---- router selection (include/strix/moe/route_policy.hpp:80-129) -----------------------------------------------
inline u32 ordered_key(float v) {
    u32 u = f_bits(v);
    if (u == 0x80000000u) u = 0;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
inline bool better(u32 key, float a, u32 ai, float b, u32 bi) {
    if (key == B200MOE_KEY_FLOAT_SERIAL) return a > b;
    const u32 ka = ordered_key(a), kb = ordered_key(b);
    return ka > kb || (ka == kb && ai < bi);
}
// k serial passes over `n` candidates with choice c[]; `allowed` (optional) masks candidates.
void k_pass(u32 key, const float* c, u32 n, const u8* allowed, u32 k, u32* out) {
    std::vector<u8> taken(n, 0);
    for (u32 pass = 0; pass < k; ++pass) {
        u32 pick = n;
        float best = 0.0f;
        for (u32 e = 0; e < n; ++e) {
            if (taken[e] || (allowed && !allowed[e])) continue;
            if (pick == n || better(key, c[e], e, best, pick)) { pick = e; best = c[e]; }
        }
        if (pick == n) { out[pass] = n; continue; }  // fewer candidates than passes (masked selection only)
        taken[pick] = 1;
        out[pass] = pick;
    }
}

// Work-sharing over host threads (results never depend on the split: every item is computed independently).
void parallel_for(size_t n, const std::function<void(size_t)>& fn) {
    unsigned threads = std::max(1u, std::thread::hardware_concurrency());
    if (n < 2 || threads == 1) { for (size_t i = 0; i < n; ++i) fn(i); return; }
    if (threads > n) threads = (unsigned)n;
    std::atomic<size_t> next{0};
    auto work = [&] { for (;;) { const size_t i = next.fetch_add(1, std::memory_order_relaxed); if (i >= n) break; fn(i); } };
    std::vector<std::thread> pool;
    for (unsigned t = 1; t < threads; ++t) pool.emplace_back(work);
    work();
    for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

float orc_half_to_float(u16 h) { return half_f(h); }
float orc_declared_exp(float x) { return declared_exp(x); }
float orc_declared_log1p(float x) { return declared_log1p(x); }
float orc_sqrt_softplus(float z) { return sqrt_softplus(z); }
float orc_gfx1151_expf(float x) { return gfx1151_expf(x); }
float orc_swiglu_ds41(float g, float u, float limit) { return swiglu_ds41(g, u, limit); }
float orc_swiglu_qwen(float g, float u) { return swiglu_qwen(g, u); }

// rows x width -> codes / deltas / sums with the given strides (elements). Returns 1 for a width not divisible by 32
// and writes nothing then (tests/cpu_backend_host_tests.cpp:65-92).
int orc_quantize_a8(const float* x, u32 rows, u32 width, u32 x_stride, i8* codes, float* deltas, i32* sums, u32 stride) {
    if (width % 32) return 1;
    if (!x_stride) x_stride = width;
    if (!stride) stride = width;
    for (u32 r = 0; r < rows; ++r)
        for (u32 g = 0; g < width / 32; ++g) {
            i32 s;
            quantize_group(x + (size_t)r * x_stride + 32 * g, codes + (size_t)r * stride + 32 * g,
                           deltas + (size_t)r * (stride / 32) + g, &s);
            if (sums) sums[(size_t)r * (stride / 32) + g] = s;
        }
    return 0;
}

// RMSNorm of the CPU backend (src/cpu/core/reference.cpp:86-103; lane count src/cpu/core/backend.hpp:91): L = 256 lanes
// (128 below n = 512), lane l = fma(x[i], x[i], .) over i = l, l + L, ..., halving tree, r = 1 / sqrt(sum / n + eps),
// y = (x * r) * w or x * r. y may alias x.
int orc_rmsnorm_f32(const float* x, const float* w, u32 n, float eps, float* y, u32 rows) {
    const u32 lanes = n >= 512 ? 256u : 128u;
    float partial[256];
    for (u32 row = 0; row < rows; ++row) {
        const float* xr = x + (size_t)row * n;
        float* yr = y + (size_t)row * n;
        for (u32 lane = 0; lane < lanes; ++lane) {
            float a = 0.0f;
            for (u32 i = lane; i < n; i += lanes) a = std::fma(xr[i], xr[i], a);
            partial[lane] = a;
        }
        for (u32 h = lanes / 2; h > 0; h >>= 1)
            for (u32 lane = 0; lane < h; ++lane) partial[lane] = partial[lane] + partial[lane + h];
        const float r = 1.0f / std::sqrt(partial[0] / (float)n + eps);
        for (u32 i = 0; i < n; ++i) yr[i] = w ? (xr[i] * r) * w[i] : xr[i] * r;
    }
    return 0;
}

// Q8_0 x A8 GEMV (src/cpu/core/reference.cpp:57-84).
int orc_gemv_q8_0_a8(const u8* weight, u32 row_bytes, u32 width, u32 count, u32 rows, const i8* codes, const float* deltas,
                     u32 x_stride, float* out, u32 out_stride, u32 accumulate) {
    if (width % 32) return 1;
    if (!x_stride) x_stride = width;
    if (!out_stride) out_stride = count;
    parallel_for((size_t)rows * count, [&](size_t i) {
            const u32 r = (u32)(i / count), o = (u32)(i % count);
            const float p = product_q8_0(weight + (size_t)o * row_bytes, codes + (size_t)r * x_stride,
                                         deltas + (size_t)r * (x_stride / 32), width);
            float& y = out[(size_t)r * out_stride + o];
            y = accumulate ? y + p : p;
    });
    return 0;
}

float orc_row_q4k(const u8* row, u32 blocks, const i8* codes, const float* deltas, const i32* sums) {
    return row_q4k(row, blocks, codes, deltas, sums);
}
float orc_row_q8_chain4(const u8* row, u32 groups, const i8* codes, const float* deltas) {
    return row_q8_chain4(row, groups, codes, deltas);
}

// Router logits in the declared dot order (src/ds41_moe.cpp:72-82) (+ logit_bias[e] after the butterfly).
void orc_router_logits(const float* x, u32 rows, u32 hidden, u32 x_stride, const float* w, u32 experts,
                       const float* logit_bias, float* logits) {
    if (!x_stride) x_stride = hidden;
    parallel_for((size_t)rows * experts, [&](size_t i) {
            const u32 r = (u32)(i / experts), e = (u32)(i % experts);
            float lanes[32];
            for (auto& l : lanes) l = 0.0f;
            const float* wr = w + (size_t)e * hidden;
            const float* xr = x + (size_t)r * x_stride;
            for (u32 i = 0; i < hidden; ++i) { const float prod = wr[i] * xr[i]; lanes[i % 32] = lanes[i % 32] + prod; }
            float z = butterfly32(lanes);
            if (logit_bias) z = z + logit_bias[e];
            logits[(size_t)r * experts + e] = z;
    });
}

// Score transform of one row (include/strix/moe/route_policy.hpp:133-156, Math = the DS41 declared math).
void orc_route_scores(u32 score, const float* logits, u32 n, float* scores) {
    if (score == B200MOE_SCORE_SOFTMAX) {
        float m = -std::numeric_limits<float>::infinity();
        for (u32 e = 0; e < n; ++e) m = logits[e] > m ? logits[e] : m;
        float sum = 0.0f;
        for (u32 e = 0; e < n; ++e) { scores[e] = declared_exp(logits[e] - m); sum = sum + scores[e]; }
        for (u32 e = 0; e < n; ++e) scores[e] = scores[e] / sum;
    } else if (score == B200MOE_SCORE_SIGMOID) {
        for (u32 e = 0; e < n; ++e) scores[e] = sigmoid_score(logits[e]);
    } else {
        for (u32 e = 0; e < n; ++e) scores[e] = sqrt_softplus(logits[e]);
    }
}

// Selection + weights of one row (route_policy.hpp:99-129). n_group > 1: the group-limited extension described in
// include/b200moe.h (no reference counterpart). Returns 1 on a policy the contract rejects.
int orc_route_select(const b200moe_route_policy* p, const float* scores, const float* bias, u32* ids, float* weights) {
    if (p->experts == 0 || p->top_k == 0 || p->top_k > p->experts) return 1;
    if (p->n_group == 0 || p->topk_group == 0 || p->topk_group > p->n_group || p->experts % p->n_group) return 1;
    std::vector<float> c(p->experts);
    for (u32 e = 0; e < p->experts; ++e) c[e] = p->selection_bias ? scores[e] + bias[e] : scores[e];
    std::vector<u8> allowed;
    if (p->n_group > 1) {
        const u32 per = p->experts / p->n_group;
        if (per < 2 || p->topk_group * per < p->top_k) return 1;
        std::vector<float> gs(p->n_group);
        for (u32 g = 0; g < p->n_group; ++g) {
            u32 two[2];
            k_pass(p->key, c.data() + (size_t)g * per, per, nullptr, 2, two);
            gs[g] = c[(size_t)g * per + two[0]] + c[(size_t)g * per + two[1]];
        }
        std::vector<u32> keep(p->topk_group);
        k_pass(p->key, gs.data(), p->n_group, nullptr, p->topk_group, keep.data());
        allowed.assign(p->experts, 0);
        for (u32 i = 0; i < p->topk_group; ++i)
            for (u32 j = 0; j < per; ++j) allowed[(size_t)keep[i] * per + j] = 1;
    }
    k_pass(p->key, c.data(), p->experts, allowed.empty() ? nullptr : allowed.data(), p->top_k, ids);
    if (p->order == B200MOE_ORDER_ASCENDING_ID) std::sort(ids, ids + p->top_k);
    const bool renorm = p->renormalize && (p->top_k > 1 || p->renorm_single);
    float sum = 0.0f;
    for (u32 k = 0; k < p->top_k; ++k) sum = sum + scores[ids[k]];
    const float den = sum + p->renorm_eps;
    for (u32 k = 0; k < p->top_k; ++k) {
        const float s = scores[ids[k]];
        weights[k] = (renorm ? s / den : s) * p->scale;
    }
    return 0;
}

// Whole router over rows (src/ds41_moe.cpp:63-97 with any policy). scores may be NULL.
int orc_router(const float* x, u32 rows, u32 hidden, const float* w, const float* logit_bias, const float* bias,
               const b200moe_route_policy* p, float* logits_io, float* scores_out, u32* ids, float* weights) {
    std::vector<float> logits((size_t)rows * p->experts);
    if (x) orc_router_logits(x, rows, hidden, hidden, w, p->experts, logit_bias, logits.data());
    else std::memcpy(logits.data(), logits_io, logits.size() * 4);
    if (x && logits_io) std::memcpy(logits_io, logits.data(), logits.size() * 4);
    int rc = 0;
    for (u32 r = 0; r < rows; ++r) {
        std::vector<float> s(p->experts);
        orc_route_scores(p->score, logits.data() + (size_t)r * p->experts, p->experts, s.data());
        if (scores_out) std::memcpy(scores_out + (size_t)r * p->experts, s.data(), s.size() * 4);
        rc |= orc_route_select(p, s.data(), bias, ids + (size_t)r * p->top_k, weights + (size_t)r * p->top_k);
    }
    return rc;
}

// Window routes (src/ds41_moe.cpp:11-61: build_window_routes then restrict_routes to [first, end), ids - base).
// Arrays sized as in include/b200moe.h. Returns the union count, or -1 when an id repeats in a row / is out of range.
int orc_routes(const u32* ids, u32 rows, u32 top_k, u32 experts, u32 split, u32 first, u32 end, u32 base,
               u32* out_experts, u32* begins, u32* out_rows, u32* out_slots, u32* order, u32* low_counts, u32* counts) {
    if (end == 0) end = experts;
    for (u32 r = 0; r < rows; ++r) {
        std::vector<std::pair<u32, u32>> row;
        for (u32 k = 0; k < top_k; ++k) {
            const u32 slot = r * top_k + k, e = ids[slot];
            if (e >= experts) return -1;
            for (auto& pr : row) if (pr.first == e) return -1;
            row.emplace_back(e, slot);
        }
        std::sort(row.begin(), row.end());
        u32 low = 0;
        for (u32 k = 0; k < top_k; ++k) { order[r * top_k + k] = row[k].second; low += row[k].first < split; }
        low_counts[r] = low;
    }
    u32 n_union = 0, n_entries = 0, max_rows = 0;
    begins[0] = 0;
    for (u32 e = first; e < end; ++e) {
        u32 cnt = 0;
        for (u32 s = 0; s < rows * top_k; ++s)
            if (ids[s] == e) { out_rows[n_entries] = s / top_k; out_slots[n_entries] = s; ++n_entries; ++cnt; }
        if (cnt) { out_experts[n_union++] = e - base; begins[n_union] = n_entries; max_rows = std::max(max_rows, cnt); }
    }
    counts[0] = n_union; counts[1] = max_rows; counts[2] = n_entries; counts[3] = 0;
    return (int)n_union;
}

// Routed experts of every (row, k) slot: gate/up products, SwiGLU, A8 of h, down -> raw[slot][hidden] (unweighted).
// Follows reference_window (src/ds41_moe.cpp:124-151) for Q8_0 gate/up and reference_run
// (src/cpu/core/routed_expert.cpp:264-300) for Q4_K gate/up. Only experts in [first, end) are evaluated (end 0 = all).
// status[row] |= 8 and raw left untouched for the WHOLE job when any h group is non-finite (Qwen family,
// routed_expert.hpp:17-19). Optional taps: gate_out / up_out [slot][inter], act codes / deltas / sums.
int orc_experts(const b200moe_shape* sh, const u8* gate, const u8* up, const u8* down, const u32* ids, u32 rows,
                const i8* x_codes, const float* x_deltas, const i32* x_sums, u32 first, u32 end, float* raw,
                float* gate_out, float* up_out, i8* act_codes, float* act_deltas, i32* act_sums, u32* status) {
    const u32 H = sh->hidden, I = sh->inter, K = sh->top_k;
    if (end == 0) end = sh->experts;
    const bool q5k = sh->gate_type == B200MOE_TYPE_Q5_K;
    const bool q4k = sh->gate_type == B200MOE_TYPE_Q4_K || q5k;  // the K-quant (Qwen A8) family
    const bool g2 = sh->gate_type == B200MOE_TYPE_Q2_K, d2 = sh->down_type == B200MOE_TYPE_Q2_K;
    if (!q4k && sh->gate_type != B200MOE_TYPE_Q8_0 && !g2) return 1;
    if (sh->down_type != B200MOE_TYPE_Q4_K && sh->down_type != B200MOE_TYPE_Q8_0 && sh->down_type != B200MOE_TYPE_Q5_1 && !d2) return 1;
    if (!q4k && sh->down_type != B200MOE_TYPE_Q8_0 && !d2) return 1;
    if (q4k && d2) return 1;
    if (H % ((q4k || g2) ? 256 : 32) || I % ((sh->down_type == B200MOE_TYPE_Q4_K || d2) ? 256 : 32)) return 1;
    const size_t grow = row_bytes(sh->gate_type, H), drow = row_bytes(sh->down_type, I);
    const u32 slots = rows * K;
    std::vector<i8> hc((size_t)slots * I);
    std::vector<float> hd((size_t)slots * (I / 32));
    std::vector<i32> hs((size_t)slots * (I / 32));
    std::atomic<int> bad{0};
    parallel_for(slots, [&](size_t si) {
        const u32 s = (u32)si, e = ids[s], r = s / K;
        if (e < first || e >= end) return;
        std::vector<float> h(I);
        const i8* xc = x_codes + (size_t)r * H;
        const float* xd = x_deltas + (size_t)r * (H / 32);
        const i32* xs = x_sums + (size_t)r * (H / 32);
        for (u32 o = 0; o < I; ++o) {
            const u8* gr = gate + ((size_t)e * I + o) * grow;
            const u8* ur = up + ((size_t)e * I + o) * grow;
            float g, u;
            if (q4k) { g = row_kquant(gr, H / 256, xc, xd, xs, q5k); u = row_kquant(ur, H / 256, xc, xd, xs, q5k); }
            else { g = product_ds41(sh->gate_type, gr, xc, xd, H); u = product_ds41(sh->gate_type, ur, xc, xd, H); }
            if (gate_out) gate_out[(size_t)s * I + o] = g;
            if (up_out) up_out[(size_t)s * I + o] = u;
            h[o] = q4k ? swiglu_qwen(g, u) : swiglu_ds41(g, u, sh->limit);
            if (q4k && (!is_finite(g) || !is_finite(u) || !is_finite(h[o]))) {
                bad.store(1);
                if (status) __atomic_fetch_or(&status[r], B200MOE_ROW_PROJECTION_NONFINITE, __ATOMIC_RELAXED);
            }
        }
        for (u32 g = 0; g < I / 32; ++g)
            quantize_group(h.data() + 32 * g, hc.data() + (size_t)s * I + 32 * g, &hd[(size_t)s * (I / 32) + g],
                           &hs[(size_t)s * (I / 32) + g]);
    });
    if (act_codes) std::memcpy(act_codes, hc.data(), hc.size());
    if (act_deltas) std::memcpy(act_deltas, hd.data(), hd.size() * 4);
    if (act_sums) std::memcpy(act_sums, hs.data(), hs.size() * 4);
    if (bad.load()) return 0;
    parallel_for(slots, [&](size_t si) {
        const u32 s = (u32)si, e = ids[s];
        if (e < first || e >= end) return;
        const i8* c = hc.data() + (size_t)s * I;
        const float* d = hd.data() + (size_t)s * (I / 32);
        const i32* sm = hs.data() + (size_t)s * (I / 32);
        for (u32 o = 0; o < H; ++o) {
            const u8* dr = down + ((size_t)e * H + o) * drow;
            float v;
            if (sh->down_type == B200MOE_TYPE_Q4_K) v = row_q4k(dr, I / 256, c, d, sm);
            else if (sh->down_type == B200MOE_TYPE_Q5_1) v = row_q5_1_chain4(dr, I / 32, c, d, sm);
            else if (q4k) v = row_q8_chain4(dr, I / 32, c, d);
            else v = product_ds41(sh->down_type, dr, c, d, I);
            raw[(size_t)s * H + o] = v;
        }
    });
    return 0;
}

// Combine (forms of include/b200moe.h). ids [rows * top_k]. shared / y_bf16 optional.
int orc_combine(u32 form, const float* raw, const float* shared, const float* weights, const u32* ids, u32 rows, u32 top_k,
                u32 hidden, u32 parts, u32 part_experts, int only_part, float* y, u16* y_bf16) {
    for (u32 r = 0; r < rows; ++r) {
        std::vector<std::pair<u32, u32>> ord;
        for (u32 k = 0; k < top_k; ++k) ord.emplace_back(ids[r * top_k + k], r * top_k + k);
        std::sort(ord.begin(), ord.end());
        for (u32 o = 0; o < hidden; ++o) {
            float out;
            if (form == B200MOE_COMBINE_FMA_SLOTS) {
                float acc = 0.0f;
                for (u32 k = 0; k < top_k; ++k) acc = std::fmaf(weights[r * top_k + k], raw[((size_t)r * top_k + k) * hidden + o], acc);
                out = shared ? acc + shared[(size_t)r * hidden + o] : acc;
            } else {
                if (parts == 0 || part_experts == 0) return 1;
                float total = shared ? shared[(size_t)r * hidden + o] : 0.0f;
                float single = 0.0f;
                for (u32 p = 0; p < parts; ++p) {
                    float sum = 0.0f;
                    for (u32 k = 0; k < top_k; ++k) {
                        const u32 part = std::min(ord[k].first / part_experts, parts - 1);
                        if (part != p) continue;
                        const float term = weights[ord[k].second] * raw[(size_t)ord[k].second * hidden + o];
                        sum = sum + term;
                    }
                    if ((int)p == only_part) single = sum;
                    total = total + sum;
                }
                out = only_part >= 0 ? single : total;
            }
            y[(size_t)r * hidden + o] = out;
            if (y_bf16) {
                const u32 b = f_bits(out);
                y_bf16[(size_t)r * hidden + o] = (u16)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
            }
        }
    }
    return 0;
}

// Float truth ("oracle B", after lab/moe_q8_0/moe_q8_0.hip:376-455): FP32 activations x dequantised weights
// (src/ggml_dequant.cpp:84, :119-131) with double accumulation, std::exp SiLU, weighted scatter-add. Reports how far
// the A8 contract itself sits from exact math; never used as the parity target.
static double deq_dot(u32 type, const u8* row, const float* x, u32 width) {
    double acc = 0.0;
    if (type == B200MOE_TYPE_Q8_0) {
        for (u32 g = 0; g < width / 32; ++g) {
            const u8* blk = row + (size_t)g * 34;
            const double d = half_f(ld16(blk));
            for (int j = 0; j < 32; ++j) acc += d * (double)(i8)blk[2 + j] * (double)x[32 * g + j];
        }
    } else if (type == B200MOE_TYPE_Q5_1) {
        for (u32 g = 0; g < width / 32; ++g) {
            const u8* blk = row + (size_t)g * 24;
            const double d = half_f(ld16(blk)), m = half_f(ld16(blk + 2));
            u32 qh;
            std::memcpy(&qh, blk + 4, 4);
            for (u32 k = 0; k < 32; ++k) {
                const u8 byte = blk[8 + (k & 15)];
                const int q = (k < 16 ? (byte & 15) : (byte >> 4)) | (int)(((qh >> k) & 1u) << 4);
                acc += (d * q + m) * (double)x[32 * g + k];
            }
        }
    } else {
        const bool q5k = type == B200MOE_TYPE_Q5_K;
        for (u32 b = 0; b < width / 256; ++b) {
            const u8* blk = row + (size_t)b * (q5k ? 176 : 144);
            const double d = half_f(ld16(blk)), dm = half_f(ld16(blk + 2));
            for (unsigned j = 0; j < 8; ++j) {
                unsigned sc, mn;
                q4k_factors(blk, j, &sc, &mn);
                const u8* q = blk + (q5k ? 48 : 16) + 32 * (j >> 1);
                for (int k = 0; k < 32; ++k) {
                    int w = (j & 1) ? (q[k] >> 4) : (q[k] & 15);
                    if (q5k) w |= ((blk[16 + k] >> j) & 1) << 4;
                    acc += (d * sc * w - dm * mn) * (double)x[256 * b + 32 * j + k];
                }
            }
        }
    }
    return acc;
}
int orc_float_truth(const b200moe_shape* sh, const u8* gate, const u8* up, const u8* down, const u32* ids, const float* weights,
                    u32 rows, const float* x, float* y) {
    const u32 H = sh->hidden, I = sh->inter, K = sh->top_k;
    const bool q4k = sh->gate_type == B200MOE_TYPE_Q4_K || sh->gate_type == B200MOE_TYPE_Q5_K;
    const size_t grow = row_bytes(sh->gate_type, H), drow = row_bytes(sh->down_type, I);
    parallel_for(rows, [&](size_t ri) {
        const u32 r = (u32)ri;
        std::vector<double> acc(H, 0.0);
        std::vector<float> h(I);
        for (u32 k = 0; k < K; ++k) {
            const u32 e = ids[r * K + k];
            for (u32 o = 0; o < I; ++o) {
                const double g = deq_dot(sh->gate_type, gate + ((size_t)e * I + o) * grow, x + (size_t)r * H, H);
                const double u = deq_dot(sh->gate_type, up + ((size_t)e * I + o) * grow, x + (size_t)r * H, H);
                double cg = g, cu = u;
                if (!q4k) { cg = g > sh->limit ? sh->limit : g; cu = u < -sh->limit ? -sh->limit : (u > sh->limit ? sh->limit : u); }
                h[o] = (float)(cg / (1.0 + std::exp(-cg)) * cu);
            }
            for (u32 o = 0; o < H; ++o)
                acc[o] += (double)weights[r * K + k] * deq_dot(sh->down_type, down + ((size_t)e * H + o) * drow, h.data(), I);
        }
        for (u32 o = 0; o < H; ++o) y[(size_t)r * H + o] = (float)acc[o];
    });
    return 0;
}

}  // extern "C"
