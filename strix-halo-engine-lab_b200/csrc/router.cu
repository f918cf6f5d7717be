// Router: logits in the declared dot order, score transform, k-pass top-k selection and weights.
//
// Contracts: strix::ds41::reference_router's product order (src/ds41_moe.cpp:72-82), the score transforms and the
// selection / weight rule of the shared route policy (include/strix/moe/route_policy.hpp:80-156). Expert ids are only
// reproducible when the choice values are bit-identical, so the logits keep the declared order: lane class l sums
// elements l, l + 32, ... ascending with separate multiply and add, then the butterfly d = 16 .. 1.
//
// HBM: the logits kernel streams the FP32 router matrix once per RT-row tile ([experts][hidden] * 4 B); the select
// kernel touches rows * experts * 4 B. Both are small beside the expert weights.
#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

// One warp computes an RT x ET tile of logits over the whole hidden width; lane = lane class.
template <int RT, int ET>
__global__ void __launch_bounds__(128) router_logits_kernel(const float* __restrict__ x, u32 x_stride, u32 rows, u32 hidden,
                                                            const float* __restrict__ w, u32 experts,
                                                            const float* __restrict__ logit_bias, float* __restrict__ logits) {
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const u32 e0 = (blockIdx.x * 4u + warp) * ET, r0 = blockIdx.y * RT;
    if (e0 >= experts) return;
    float acc[RT][ET];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int e = 0; e < ET; ++e) acc[r][e] = 0.0f;
    const float* xr[RT];
    const float* wr[ET];
#pragma unroll
    for (int r = 0; r < RT; ++r) xr[r] = x + u64(min(r0 + r, rows - 1)) * x_stride;
#pragma unroll
    for (int e = 0; e < ET; ++e) wr[e] = w + u64(min(e0 + e, experts - 1)) * hidden;
#pragma unroll 4
    for (u32 i = lane; i < hidden; i += 32) {
        float xv[RT], wv[ET];
#pragma unroll
        for (int r = 0; r < RT; ++r) xv[r] = xr[r][i];
#pragma unroll
        for (int e = 0; e < ET; ++e) wv[e] = __ldg(wr[e] + i);
#pragma unroll
        for (int r = 0; r < RT; ++r)
#pragma unroll
            for (int e = 0; e < ET; ++e) acc[r][e] = __fadd_rn(acc[r][e], __fmul_rn(wv[e], xv[r]));
    }
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int e = 0; e < ET; ++e) {
            float z = butterfly32(acc[r][e]);
            if (lane == 0 && r0 + r < rows && e0 + e < experts) {
                if (logit_bias) z = __fadd_rn(z, logit_bias[e0 + e]);
                logits[u64(r0 + r) * experts + e0 + e] = z;
            }
        }
}

}  // namespace
}  // namespace b200moe

#include "router_select.cuh"

namespace b200moe {
namespace {

// One warp per row; shared memory per warp: scores[experts] + choice[experts] + 32 group scores.
__global__ void __launch_bounds__(128) router_select_kernel(const float* logits, float* scores_out, const float* __restrict__ bias,
                                                            b200moe_route_policy p, u32 rows, u32* __restrict__ ids,
                                                            float* __restrict__ weights) {
    extern __shared__ float smem[];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const u32 row = blockIdx.x * 4u + warp;
    if (row >= rows) return;
    select_detail::select_row(logits, scores_out, bias, p, row, lane, smem + warp * (2u * p.experts + 32u), ids, weights);
}

}  // namespace

int launch_router_logits(const b200moe_router_view& v, cudaStream_t stream, const b200moe_quantize_a8_view* fused_quantize) {
    const u32 E = v.policy.experts, xs = v.x_stride ? v.x_stride : v.hidden;
    if (v.rows == 0) return B200MOE_OK;
    if (fused_quantize) if (int rc = launch_quantize_a8(*fused_quantize, stream)) return rc;
#define B200_LOGITS(RT, ET)                                                                                   \
    router_logits_kernel<RT, ET><<<dim3((E + 4 * ET - 1) / (4 * ET), (v.rows + RT - 1) / RT), 128, 0, stream>>>( \
        v.x, xs, v.rows, v.hidden, v.weight, E, v.logit_bias, v.logits)
    if (v.rows == 1) B200_LOGITS(1, 1);
    else if (v.rows == 2) B200_LOGITS(2, 1);
    else if (v.rows <= 4) B200_LOGITS(4, 1);
    // 8 x 4 tiles read the router matrix a quarter as often, but only pay when they still leave every SM a dozen warps
    // (token blocks); a 64-row window over 256 experts is 512 such tiles - 3.5 warps per SM, latency bound (117 us
    // measured against 8 x 1 tiles on the same window)
    else if (v.rows <= 16 || u64((E + 3) / 4) * ((v.rows + 7) / 8) < 148u * 12u) B200_LOGITS(8, 1);
    else B200_LOGITS(8, 4);
#undef B200_LOGITS
    return after_launch("router_logits");
}

int launch_router_select(const b200moe_router_view& v, cudaStream_t stream) {
    if (v.rows == 0) return B200MOE_OK;
    const u32 smem = 4u * (2u * v.policy.experts + 32u) * sizeof(float);
    router_select_kernel<<<(v.rows + 3) / 4, 128, smem, stream>>>(v.logits, v.scores, v.bias, v.policy, v.rows, v.ids, v.weights);
    return after_launch("router_select");
}

}  // namespace b200moe
