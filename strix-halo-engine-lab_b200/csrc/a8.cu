// A8 activation quantiser: one warp per (row, 32-value group), one value per lane.
// Contract: src/cpu/core/reference.cpp:35-55 (= src/ds41_formats.cpp:146-165).
// HBM traffic per row: width * 4 B in (2 B for bfloat16), width * 1.25 B out: negligible beside the expert weights.
#include <algorithm>

#include "kernels.cuh"

namespace b200moe {
namespace {

template <bool BF16>
__global__ void __launch_bounds__(256) quantize_a8_kernel(const void* __restrict__ x, u32 rows, u32 groups, u32 x_stride,
                                                          i8* __restrict__ codes, float* __restrict__ deltas,
                                                          i32* __restrict__ sums, u32 stride, u32* __restrict__ status) {
    const u32 lane = threadIdx.x & 31u;
    const u64 item = u64(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= u64(rows) * groups) return;
    const u32 r = static_cast<u32>(item / groups), g = static_cast<u32>(item % groups);
    const u64 at = u64(r) * x_stride + 32u * g + lane;
    float v;
    if (BF16) v = __uint_as_float(static_cast<u32>(static_cast<const u16*>(x)[at]) << 16);
    else v = static_cast<const float*>(x)[at];
    float delta;
    int sum;
    const int code = a8_quantize_lane(v, &delta, &sum);
    codes[u64(r) * stride + 32u * g + lane] = static_cast<i8>(code);
    if (lane == 0) {
        deltas[u64(r) * (stride / 32) + g] = delta;
        if (sums) sums[u64(r) * (stride / 32) + g] = sum;
    }
    if (status) {
        const bool bad = __any_sync(0xffffffffu, !finite_f(v));
        if (bad && lane == 0) atomicOr(&status[r], B200MOE_ROW_NONFINITE_ACTIVATION);
    }
}

// bfloat16 bit patterns widened to FP32 (exact): the router reads FP32 rows.
__global__ void __launch_bounds__(256) widen_bf16_kernel(const u16* __restrict__ in, float* __restrict__ out, u64 count) {
    for (u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += u64(gridDim.x) * blockDim.x)
        out[i] = __uint_as_float(static_cast<u32>(in[i]) << 16);
}

}  // namespace

int launch_widen_bf16(const u16* in, float* out, u64 count, cudaStream_t stream) {
    if (count == 0) return B200MOE_OK;
    const u32 blocks = static_cast<u32>(std::min<u64>((count + 255) / 256, 148u * 16u));
    widen_bf16_kernel<<<blocks, 256, 0, stream>>>(in, out, count);
    return after_launch("widen_bf16");
}

int launch_quantize_a8(const b200moe_quantize_a8_view& v, cudaStream_t stream) {
    const u32 groups = v.width / 32;
    const u64 items = u64(v.rows) * groups;
    if (items == 0) return B200MOE_OK;
    const u32 x_stride = v.x_stride ? v.x_stride : v.width, stride = v.out.stride ? v.out.stride : v.width;
    const u32 blocks = static_cast<u32>((items + 7) / 8);
    if (v.x_is_bf16)
        quantize_a8_kernel<true><<<blocks, 256, 0, stream>>>(v.x, v.rows, groups, x_stride, v.out.codes, v.out.deltas, v.out.sums, stride, v.status);
    else
        quantize_a8_kernel<false><<<blocks, 256, 0, stream>>>(v.x, v.rows, groups, x_stride, v.out.codes, v.out.deltas, v.out.sums, stride, v.status);
    return after_launch("quantize_a8");
}

}  // namespace b200moe
