// Shared host/device helpers of the B200 MoE FFN library.
//
// Every translation unit of the library is compiled with --fmad=false -prec-div=true -prec-sqrt=true -ftz=false: the
// arithmetic contracts are written as single IEEE-754 binary32 operations (the reference builds its exact kernels
// the same way, cmake/QwenCuda.cmake:49), so FP32 code written in the declared order gives the host reference's bits.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>

#include "../../include/b200moe.h"

namespace b200moe {

using u8 = std::uint8_t;
using u16 = std::uint16_t;
using u32 = std::uint32_t;
using u64 = std::uint64_t;
using i8 = std::int8_t;
using i32 = std::int32_t;

// ---- host: error text, launch accounting --------------------------------------------------------------------------
std::string& last_error_slot();
int fail(int code, const char* fmt, ...);
std::atomic<u64>& launch_counter();
// Checks the launch that was just enqueued; counts it. Returns B200MOE_OK or B200MOE_ERR_CUDA.
int after_launch(const char* what);
// True once a device with the sm_100a image is usable; otherwise records why and returns false.
bool device_ready();
// Raises a kernel's dynamic shared memory limit when `bytes` needs more than it has been given so far (per device).
int ensure_dynamic_smem(const void* kernel, u32 bytes);
// Asks for the largest shared-memory carve-out for a kernel that itself needs little (see api.cu).
int prefer_max_shared(const void* kernel);
// Multiprocessors of the current device (148 on a B200; queried, not assumed).
int device_sm_count();

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }
inline bool aligned(const void* p, std::size_t a) { return (reinterpret_cast<std::uintptr_t>(p) % a) == 0; }

#define B200_REQUIRE(cond, ...)                                                  \
    do {                                                                         \
        if (!(cond)) return ::b200moe::fail(B200MOE_ERR_INVALID_ARGUMENT, __VA_ARGS__); \
    } while (0)

constexpr u32 kQ8Block = 34, kQ4KBlock = 144, kQ5KBlock = 176, kQ51Block = 24, kQ2KBlock = 84;
inline u64 row_bytes_of(u32 type, u32 width) {
    switch (type) {
        case B200MOE_TYPE_Q8_0: return u64(width / 32) * kQ8Block;
        case B200MOE_TYPE_Q5_1: return u64(width / 32) * kQ51Block;
        case B200MOE_TYPE_Q5_K: return u64(width / 256) * kQ5KBlock;
        case B200MOE_TYPE_Q2_K: return u64(width / 256) * kQ2KBlock;
        default: return u64(width / 256) * kQ4KBlock;
    }
}
// gate / up of the Qwen A8 family (K-quant super-blocks, four-chain pair rule); down types whose term reads the code sums
inline bool is_kquant(u32 type) { return type == B200MOE_TYPE_Q4_K || type == B200MOE_TYPE_Q5_K; }
// tensors of the DS41 family (32 lane classes + butterfly, declared_exp SwiGLU with the clamp)
inline bool is_ds41_type(u32 type) { return type == B200MOE_TYPE_Q8_0 || type == B200MOE_TYPE_Q2_K; }
inline bool down_reads_sums(u32 type) { return type == B200MOE_TYPE_Q4_K || type == B200MOE_TYPE_Q5_1; }

// ---- device helpers ------------------------------------------------------------------------------------------------
#if defined(__CUDACC__)
__device__ __forceinline__ float half_bits_to_float(u32 h) {  // exact for every fp16 value, subnormals included
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h)));
}
__device__ __forceinline__ bool finite_f(float x) { return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u; }
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
// The declared butterfly: v[l] = v[l] + v[l ^ d], d = 16 .. 1 (src/core/integer_math.hpp:43-47). Addition is
// commutative bit for bit, so every lane ends with the tree's value.
__device__ __forceinline__ float butterfly32(float v) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
}
// One A8 group of 32 values held one per lane (src/cpu/core/reference.cpp:35-55). Returns the code; delta and sum
// are the same in every lane.
__device__ __forceinline__ int a8_quantize_lane(float x, float* delta_out, int* sum_out) {
    const float amax = warp_max(fabsf(x));  // NaN operands are ignored, as std::max(amax, |x|) ignores them
    const bool tiny = amax > 0.0f && amax < 0x1p-119f;
    const float delta = (amax == 0.0f || tiny) ? 1.0f : __fdiv_rn(amax, 127.0f);
    const float r = tiny ? 0.0f : rintf(__fdiv_rn(x, delta));
    const float lo = (-127.0f < r) ? r : -127.0f;  // std::max(-127, r): a NaN quotient gives -127
    const float cl = (lo < 127.0f) ? lo : 127.0f;
    const int code = static_cast<int>(cl);
    *delta_out = delta;
    *sum_out = warp_sum_i(code);
    return code;
}
__device__ __forceinline__ u16 bf16_rne_bits(float v) {  // src/cuda/models/qwen/qwen_moe.cu:333-334
    const u32 b = __float_as_uint(v);
    return static_cast<u16>((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}
#endif

}  // namespace b200moe
