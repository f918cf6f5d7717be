// Device forms of the reference's declared scalar math. Each function is the published operation sequence of the
// cited host function, written with explicit round-to-nearest intrinsics so the bits do not depend on compiler flags.
#pragma once
#include "common.cuh"

namespace b200moe {

__device__ __forceinline__ float pow2i(int k) { return __uint_as_float(static_cast<u32>(k + 127) << 23); }

// exp(x) from basic IEEE operations (include/strix/ds41_moe.hpp:38-54): Cody-Waite reduction by ln 2, degree-7 Taylor
// polynomial in Horner form with separate multiply and add, two-step power-of-two scaling.
__device__ __forceinline__ float declared_exp(float x) {
    if (!(x == x)) return x;
    if (x > 88.0f) return __uint_as_float(0x7f800000u);
    if (x < -103.0f) return 0.0f;
    const float n = rintf(__fmul_rn(x, 1.44269504f));
    const float r = __fsub_rn(__fsub_rn(x, __fmul_rn(n, 0.693359375f)), __fmul_rn(n, -2.12194440e-4f));
    float p = 1.98412698e-4f;
    p = __fadd_rn(__fmul_rn(p, r), 1.38888889e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 8.33333333e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 4.16666667e-2f);
    p = __fadd_rn(__fmul_rn(p, r), 1.66666667e-1f);
    p = __fadd_rn(__fmul_rn(p, r), 0.5f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    p = __fadd_rn(__fmul_rn(p, r), 1.0f);
    const int k = static_cast<int>(n), k1 = k / 2, k2 = k - k1;
    return __fmul_rn(__fmul_rn(p, pow2i(k1)), pow2i(k2));
}
// ln of a positive normal float (include/strix/ds41_moe.hpp:65-79).
__device__ __forceinline__ float declared_log(float y) {
    const u32 bits = __float_as_uint(y);
    int k = static_cast<int>((bits >> 23) & 0xffu) - 127;
    float m = __uint_as_float((bits & 0x7fffffu) | 0x3f800000u);
    if (m > 1.41421356f) { m = __fmul_rn(m, 0.5f); k = k + 1; }
    const float s = __fdiv_rn(__fsub_rn(m, 1.0f), __fadd_rn(m, 1.0f)), s2 = __fmul_rn(s, s);
    float p = 0.111111111f;
    p = __fadd_rn(__fmul_rn(p, s2), 0.142857143f);
    p = __fadd_rn(__fmul_rn(p, s2), 0.2f);
    p = __fadd_rn(__fmul_rn(p, s2), 0.333333333f);
    p = __fadd_rn(__fmul_rn(p, s2), 1.0f);
    const float kf = static_cast<float>(k);
    return __fadd_rn(__fmul_rn(kf, 0.693359375f), __fadd_rn(__fmul_rn(kf, -2.12194440e-4f), __fmul_rn(__fmul_rn(2.0f, s), p)));
}
__device__ __forceinline__ float declared_log1p(float e) {  // ds41_moe.hpp:81-85
    const float u = __fadd_rn(1.0f, e);
    if (u == 1.0f) return e;
    return __fmul_rn(declared_log(u), __fdiv_rn(e, __fsub_rn(u, 1.0f)));
}
__device__ __forceinline__ float sqrt_softplus_score(float z) {  // ds41_moe.hpp:98-100, route_policy.hpp:78-81
    return __fsqrt_rn(z > 20.0f ? z : declared_log1p(declared_exp(z)));
}
__device__ __forceinline__ float sigmoid_score(float z) {  // route_policy.hpp:74-77
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, declared_exp(-z)));
}
// SwiGLU with the shared clamp trait (ds41_moe.hpp:57-60; moe/activation_policy.hpp:22-24). limit = +inf: no clamp.
__device__ __forceinline__ float swiglu_ds41(float gate, float up, float limit) {
    const float g = gate > limit ? limit : gate;
    const float u = up < -limit ? -limit : (up > limit ? limit : up);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, declared_exp(-g))), u);
}

// gfx1151 expf twin at zero correction tables (src/cpu/core/routed_expert.cpp:208-261): Cody-Waite split of
// x * log2(e) with two fused steps, v_exp(a) = float(exp2(double(a))) for |a| < 1, scaled by 2^e.
// The host evaluates exp2 in double with the C library; the device's double exp2 differs from it by at most one
// double ulp, which changes the rounded float only when the double lands within 2^-29 of a float rounding boundary.
__device__ __forceinline__ float gfx1151_expf(float x) {
    const float kLog2e = __uint_as_float(0x3fb8aa3bu), kLog2eLo = __uint_as_float(0x32a5705fu);
    const float ph = __fmul_rn(x, kLog2e);
    const float e = rintf(ph);
    float pl = __fmaf_rn(x, kLog2e, -ph);
    pl = __fmaf_rn(x, kLog2eLo, pl);
    const float a = __fadd_rn(__fsub_rn(ph, e), pl);
    float y;
    if (fabsf(a) < 1.0f) y = scalbnf(static_cast<float>(exp2(static_cast<double>(a))), static_cast<int>(e));
    else y = a != a ? a : 0.0f;
    if (__uint_as_float(0xc2ce8ed0u) > x) y = 0.0f;
    if (__uint_as_float(0x42b17218u) < x) y = __uint_as_float(0x7f800000u);
    return y;
}
__device__ __forceinline__ float swiglu_qwen(float g, float u) {  // routed_expert.cpp:151-153
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, gfx1151_expf(-g))), u);
}

}  // namespace b200moe
