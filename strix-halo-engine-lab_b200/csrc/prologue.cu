// Layer prologue of decode windows (up to 8 rows) in ONE launch: A8 of the activations, router logits, score
// transform + top-k selection + weights, and the window routes.
//
// Contracts are those of the stand-alone kernels (a8.cu, router.cu, routes.cu): logits in the declared lane-strided
// order without fused multiply-add (src/ds41_moe.cpp:72-82), the route policy's transforms and k-pass selection
// (include/strix/moe/route_policy.hpp:99-156), build_window_routes (src/ds41_moe.cpp:11-61). Bits do not change.
//
// Shape: blocks [0, logit_blocks) take eight experts each, one warp per expert. A warp copies its expert's current
// 2048-wide run to shared memory asynchronously, the block does the same with that run of every activation row, then
// each lane walks its lane class in ascending order. The
// block that finishes last (a ticket counter in the workspace) runs selection (one warp per row) and the routes.
// Blocks past logit_blocks quantise the activations. Everything the expert kernels need is ready after this launch.
#include "kernels.cuh"
#include "router_select.cuh"
#include "routes_small.cuh"

namespace b200moe {
namespace {

// Eight experts (= warps) per logits block. Fewer experts per block spread the logits over more CTAs but every CTA stages the
// window's activation rows itself: measured on B200 at config 2, batch 8, 4 and 2 experts per block cost 80.6 and 92.5 us per
// step against 76.2 us with 8 (no difference at batch 1).
constexpr u32 kRunElems = 2048, kWarps = 8;

__device__ __forceinline__ u32 smem_addr(const void* p) { return static_cast<u32>(__cvta_generic_to_shared(p)); }

struct PrologueArgs {
    b200moe_router_view r;
    b200moe_quantize_a8_view q;
    b200moe_routes_view routes;
    u32 routes_end;
    u32 logit_blocks;
    u32* ticket;  // zero before the first launch; the block that finishes last puts it back to zero
};

template <int RT>
__global__ void __launch_bounds__(kWarps * 32) prologue_decode_kernel(PrologueArgs a) {
    extern __shared__ __align__(16) float xs[];  // [rows + kWarps][kRunElems] while the logits run, select scratch afterwards
    __shared__ u32 s_last;
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;

    if (blockIdx.x >= a.logit_blocks) {  // ---- A8 quantiser: one warp per (row, 32-value group)
        const b200moe_quantize_a8_view& qv = a.q;
        const u32 groups = qv.width / 32;
        const u64 item = u64(blockIdx.x - a.logit_blocks) * kWarps + warp;
        if (item >= u64(qv.rows) * groups) return;
        const u32 r = static_cast<u32>(item / groups), g = static_cast<u32>(item % groups);
        const u32 xst = qv.x_stride ? qv.x_stride : qv.width, st = qv.out.stride ? qv.out.stride : qv.width;
        const float v = static_cast<const float*>(qv.x)[u64(r) * xst + 32u * g + lane];
        float delta;
        int sum;
        const int code = a8_quantize_lane(v, &delta, &sum);
        qv.out.codes[u64(r) * st + 32u * g + lane] = static_cast<i8>(code);
        if (lane == 0) {
            qv.out.deltas[u64(r) * (st / 32) + g] = delta;
            if (qv.out.sums) qv.out.sums[u64(r) * (st / 32) + g] = sum;
        }
        if (qv.status && __any_sync(0xffffffffu, !finite_f(v)) && lane == 0) atomicOr(&qv.status[r], B200MOE_ROW_NONFINITE_ACTIVATION);
        return;
    }

    // ---- router logits: warp = expert
    const b200moe_router_view& rv = a.r;
    const u32 E = rv.policy.experts, H = rv.hidden, rows = rv.rows;
    const u32 x_stride = rv.x_stride ? rv.x_stride : H;
    const u32 e = blockIdx.x * kWarps + warp;
    const float* wr = rv.weight + u64(min(e, E - 1)) * H;
    const bool vec4 = (reinterpret_cast<uintptr_t>(rv.x) % 16 == 0) && x_stride % 4 == 0 && H % 4 == 0;
    const bool wvec4 = (reinterpret_cast<uintptr_t>(rv.weight) % 16 == 0) && H % 4 == 0;
    float* ws = xs + rows * kRunElems + warp * kRunElems;  // this warp's expert row run
    float acc[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) acc[r] = 0.0f;
    // Both operands are staged with asynchronous copies from short rolled loops: every request of the run is in flight
    // at once, and the code stays small (this kernel runs once per step on cold instruction caches, so straight-line
    // unrolled code would pay a fetch miss per line).
    for (u32 c0 = 0; c0 < H; c0 += kRunElems) {
        const u32 n_el = min(kRunElems, H - c0);
        __syncthreads();  // the previous run has been consumed
        {
            const float* src = wr + c0;
            const u32 dst = smem_addr(ws);
            if (wvec4) {
                for (u32 i = lane; i < n_el / 4; i += 32)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 4u * i) : "memory");
            } else {
                for (u32 i = lane; i < n_el; i += 32)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * i), "l"(src + i) : "memory");
            }
        }
        for (u32 r = 0; r < rows; ++r) {
            const float* src = rv.x + u64(r) * x_stride + c0;
            const u32 dst = smem_addr(xs + r * kRunElems);
            if (vec4) {  // rows, strides and run starts are all multiples of four floats
                for (u32 i = threadIdx.x; i < n_el / 4; i += kWarps * 32)
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * i), "l"(src + 4u * i) : "memory");
            } else {
                for (u32 i = threadIdx.x; i < n_el; i += kWarps * 32)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * i), "l"(src + i) : "memory");
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
#pragma unroll 4
        for (u32 i = lane; i < n_el; i += 32) {  // the lane class in ascending order (src/ds41_moe.cpp:72-82)
            const float w = ws[i];
#pragma unroll
            for (int r = 0; r < RT; ++r)
                if (r < (int)rows) acc[r] = __fadd_rn(acc[r], __fmul_rn(w, xs[r * kRunElems + i]));
        }
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        float z = butterfly32(acc[r]);
        if (lane == 0 && r < (int)rows && e < E) {
            if (rv.logit_bias) z = __fadd_rn(z, rv.logit_bias[e]);
            rv.logits[u64(r) * E + e] = z;
        }
    }

    // ---- the last block to finish selects and builds the routes
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1u) == a.logit_blocks - 1) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) *a.ticket = 0;  // every block has taken its ticket: ready for the next launch without a memset
    for (u32 row = warp; row < rows; row += kWarps)
        select_detail::select_row(rv.logits, rv.scores, rv.bias, rv.policy, row, lane, xs + warp * (2u * E + 32u), rv.ids, rv.weights);
    __syncthreads();  // the ids written above are read below by the whole block
    if (a.routes.out.experts) routes_detail::routes_small_body(a.routes, a.routes_end);  // optional: a caller that routes elsewhere passes no outputs
}

}  // namespace

bool prologue_fusable(const b200moe_router_view& r, u32 top_k) {
    return r.rows >= 1 && r.rows <= 8 && u64(r.rows) * top_k <= routes_detail::kChunk && kWarps * (2u * r.policy.experts + 32u) * 4u <= 64u * 1024u;
}

int launch_prologue(const b200moe_router_view& r, const b200moe_quantize_a8_view& q, const b200moe_routes_view& routes, u32* ticket,
                    cudaStream_t stream) {
    PrologueArgs a{};
    a.r = r; a.q = q; a.routes = routes; a.routes_end = routes.end ? routes.end : routes.experts; a.ticket = ticket;
    a.logit_blocks = (r.policy.experts + kWarps - 1) / kWarps;
    const u32 quant_blocks = static_cast<u32>((u64(q.rows) * (q.width / 32) + kWarps - 1) / kWarps);
    const u32 smem = std::max<u32>((r.rows + kWarps) * kRunElems * 4u, kWarps * (2u * r.policy.experts + 32u) * 4u);
    const dim3 grid(a.logit_blocks + quant_blocks);
#define B200_PRO(RT)                                                                                            \
    {                                                                                                           \
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(prologue_decode_kernel<RT>), smem)) return rc; \
        if (int rc = prefer_max_shared(reinterpret_cast<const void*>(prologue_decode_kernel<RT>))) return rc;       \
        prologue_decode_kernel<RT><<<grid, kWarps * 32, smem, stream>>>(a);                                     \
    }
    if (r.rows <= 2) B200_PRO(2)
    else if (r.rows <= 4) B200_PRO(4)
    else B200_PRO(8)
#undef B200_PRO
    return after_launch("prologue_decode");
}

}  // namespace b200moe
