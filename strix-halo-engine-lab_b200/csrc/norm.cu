// RMSNorm in front of the FFN, fused with the A8 quantiser of its output (the rows the router and the experts read).
// One CTA per row, 256 threads = the 256 lanes of the host rule (src/cpu/core/reference.cpp:86-103): lane l runs
// a = fma(x[i], x[i], a) over i = l, l + L, ... (L = 128 below n = 512), the lanes fold by the halving tree, and
// s = 1 / sqrt(sum / n + eps) - IEEE division and square root. The second pass is warp-per-group: y = (x * s) * w for
// 32 consecutive values, written out and / or quantised by the A8 rule on the spot. HBM traffic: x once (the second
// pass hits L1 / L2), y and the A8 rows once.
#include "kernels.cuh"

namespace b200moe {
namespace {

__global__ void __launch_bounds__(256) rmsnorm_a8_kernel(b200moe_rmsnorm_view v) {
    __shared__ float partial[256];
    const u32 r = blockIdx.x, t = threadIdx.x, n = v.n;
    const u32 x_stride = v.x_stride ? v.x_stride : n, out_stride = v.out_stride ? v.out_stride : n;
    const float* __restrict__ x = v.x + u64(r) * x_stride;
    const u32 lanes = n >= 512u ? 256u : 128u;
    float a = 0.0f;
    if (t < lanes)
        for (u32 i = t; i < n; i += lanes) { const float xi = x[i]; a = __fmaf_rn(xi, xi, a); }
    partial[t] = a;
    __syncthreads();
    for (u32 h = lanes / 2; h > 0; h >>= 1) {
        if (t < h) partial[t] = __fadd_rn(partial[t], partial[t + h]);
        __syncthreads();
    }
    const float s = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial[0], static_cast<float>(n)), v.eps)));
    const u32 lane = t & 31u, warp = t >> 5, groups = n / 32;
    const u32 a8_stride = v.a8.stride ? v.a8.stride : v.a8.width;
    bool bad = false;
    for (u32 g = warp; g < groups; g += 8) {
        const u32 i = 32u * g + lane;
        float y = __fmul_rn(x[i], s);
        if (v.weight) y = __fmul_rn(y, v.weight[i]);
        if (v.out) v.out[u64(r) * out_stride + i] = y;
        if (v.a8.codes) {
            float delta;
            int sum;
            const int code = a8_quantize_lane(y, &delta, &sum);
            v.a8.codes[u64(r) * a8_stride + i] = static_cast<i8>(code);
            if (lane == 0) {
                v.a8.deltas[u64(r) * (a8_stride / 32) + g] = delta;
                if (v.a8.sums) v.a8.sums[u64(r) * (a8_stride / 32) + g] = sum;
            }
        }
        bad |= !finite_f(y);
    }
    if (v.status && __any_sync(0xffffffffu, bad) && lane == 0) atomicOr(&v.status[r], B200MOE_ROW_NONFINITE_ACTIVATION);
}

}  // namespace

int launch_rmsnorm_a8(const b200moe_rmsnorm_view& v, cudaStream_t stream) {
    if (v.rows == 0 || v.n == 0) return B200MOE_OK;
    rmsnorm_a8_kernel<<<v.rows, 256, 0, stream>>>(v);
    return after_launch("rmsnorm_a8");
}

}  // namespace b200moe
