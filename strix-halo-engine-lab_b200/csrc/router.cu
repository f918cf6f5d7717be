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

// Windows of more than 4 rows: a CTA owns 8 rows x 16 experts and walks the hidden width in chunks of 512 columns that
// all 128 threads stage into shared memory with 16-byte asynchronous copies, three chunks in flight; a warp keeps an
// 8 x 4 tile of lane-class sums. The x tile is then read from HBM / L2 once per 16 experts instead of once per expert (a
// 64-row window over 256 experts of width 7168 pulled 470 MB through L2 in the form above), and the copies of two chunks
// cover the arithmetic of one. Same products, same order: lane l of a warp meets columns l, l + 32, ... ascending.
constexpr u32 kTileRows = 8, kTileExperts = 16, kTileCols = 512, kTileStages = 3;
constexpr u32 kTileStageFloats = (kTileRows + kTileExperts) * kTileCols;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<u32>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

__global__ void __launch_bounds__(128) router_logits_tile_kernel(const float* __restrict__ x, u32 x_stride, u32 rows, u32 hidden,
                                                                 const float* __restrict__ w, u32 experts,
                                                                 const float* __restrict__ logit_bias, float* __restrict__ logits) {
    extern __shared__ __align__(16) float tile_smem[];
    const u32 tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const u32 r0 = blockIdx.y * kTileRows, e0 = blockIdx.x * kTileExperts;
    const u32 n_chunks = (hidden + kTileCols - 1) / kTileCols;
    auto issue = [&](u32 c) {
        if (c < n_chunks) {
            float* st = tile_smem + (c % kTileStages) * kTileStageFloats;
            const u32 col0 = c * kTileCols, nvec = (min(kTileCols, hidden - col0)) / 4;
            if (tid < nvec) {
#pragma unroll
                for (u32 j = 0; j < kTileRows + kTileExperts; ++j) {
                    const float* src = j < kTileRows ? x + u64(min(r0 + j, rows - 1)) * x_stride : w + u64(min(e0 + j - kTileRows, experts - 1)) * hidden;
                    cp_async16(st + j * kTileCols + 4 * tid, src + col0 + 4 * tid);
                }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");  // an empty group keeps the count of the wait below fixed
    };
    float acc[kTileRows][4];
#pragma unroll
    for (int r = 0; r < (int)kTileRows; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[r][e] = 0.0f;
    issue(0);
    issue(1);
    for (u32 c = 0; c < n_chunks; ++c) {
        issue(c + 2);
        asm volatile("cp.async.wait_group 2;" ::: "memory");
        __syncthreads();
        const float* st = tile_smem + (c % kTileStages) * kTileStageFloats;
        const u32 ncol = min(kTileCols, hidden - c * kTileCols);
#pragma unroll 4
        for (u32 col = lane; col < ncol; col += 32) {
            float xv[kTileRows], wv[4];
#pragma unroll
            for (int r = 0; r < (int)kTileRows; ++r) xv[r] = st[r * kTileCols + col];
#pragma unroll
            for (int e = 0; e < 4; ++e) wv[e] = st[(kTileRows + 4 * warp + e) * kTileCols + col];
#pragma unroll
            for (int r = 0; r < (int)kTileRows; ++r)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[r][e] = __fadd_rn(acc[r][e], __fmul_rn(wv[e], xv[r]));
        }
        __syncthreads();  // the stage is refilled by the copies issued two iterations on
    }
#pragma unroll
    for (int r = 0; r < (int)kTileRows; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float z = butterfly32(acc[r][e]);
            const u32 row = r0 + r, ex = e0 + 4 * warp + e;
            if (lane == 0 && row < rows && ex < experts) {
                if (logit_bias) z = __fadd_rn(z, logit_bias[ex]);
                logits[u64(row) * experts + ex] = z;
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
    else if (aligned(v.x, 16) && aligned(v.weight, 16) && xs % 4 == 0 && v.hidden % 4 == 0) {
        constexpr u32 smem = kTileStages * kTileStageFloats * sizeof(float);
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(router_logits_tile_kernel), smem)) return rc;
        router_logits_tile_kernel<<<dim3((E + kTileExperts - 1) / kTileExperts, (v.rows + kTileRows - 1) / kTileRows), 128, smem, stream>>>(
            v.x, xs, v.rows, v.hidden, v.weight, E, v.logit_bias, v.logits);
    } else if (v.rows <= 16) B200_LOGITS(8, 1);
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
