// Tensor parallelism of the dense SwiGLU block behind the C ABI: b200moe_tp_dense enqueues a rank's share of the block
// (column-parallel gate / up over whole super-blocks of inter, SwiGLU and the A8 of h local to the share, row-parallel down
// over the same K share) AND the exchange of the partial sums, on the caller's stream, with no host wait and no collective
// library: every rank stores its [rows][hidden] partial - FP32, or rounded to bfloat16, the payload the row-parallel
// all-reduce of such a block usually carries - straight into block `rank` of every peer's window (CUDA IPC mappings, plain
// peer stores over NVLink), raises its arrival flag there, and every rank then folds the W blocks in RANK ORDER,
// y = (((+0 + P_0) + P_1) + ...) + P_{W-1} in FP32. That is an all-reduce whose association order is fixed, so W GPUs and W virtual
// ranks on one GPU give the same bits - the reference's rule for its two-rank split of the shared expert
// (include/strix/ds41_shexp_tp.hpp:7-9; the join itself: src/core/tp_join.hpp:16-78).
//
// Flags, step counter, the two window halves and the bounded waits are those of ep.cu: the fold kernel polls the W flag
// words at most wait_polls times, then sets B200MOE_JOB_WAIT_ABORTED and writes nothing.
#include <algorithm>
#include <cstring>

#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kMaxWorld = 8;
constexpr u32 kDefaultWaitPolls = 1u << 22;
constexpr u64 kFlagBytes = 256;

u64 up256(u64 v) { return (v + 255) & ~u64(255); }

struct Tp {
    b200moe_shape shape;  // the rank's share: inter = its slice
    u32 world, rank, rows, bf16;
    unsigned char* win[kMaxWorld];
    u64 half;             // bytes of one parity half: world blocks of rows * hidden elements
    u32* counters;        // device: [0] step, [1] ticket
    u32 calls, wait_polls;
};

struct TpDev {
    unsigned char* win[kMaxWorld];
    u32 world, rank, bf16;
    u64 half_base, block_bytes;
};

__global__ void tp_begin_kernel(u32* counters) {
    counters[0] += 1;
    counters[1] = 0;
}

// The rank's partial to block `rank` of every window (its own included), then the arrival flags.
__global__ void __launch_bounds__(256) tp_scatter_kernel(TpDev d, const float* __restrict__ partial, u64 count, u32* counters) {
    __shared__ u32 s_last;
    for (u64 i = (u64(blockIdx.x) * blockDim.x + threadIdx.x) * 4; i < count; i += u64(gridDim.x) * blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(partial + i);
        if (d.bf16) {
            const uint2 packed = make_uint2(u32(bf16_rne_bits(v.x)) | (u32(bf16_rne_bits(v.y)) << 16), u32(bf16_rne_bits(v.z)) | (u32(bf16_rne_bits(v.w)) << 16));
            for (u32 r = 0; r < d.world; ++r) *reinterpret_cast<uint2*>(d.win[r] + d.half_base + d.rank * d.block_bytes + i * 2) = packed;
        } else {
            for (u32 r = 0; r < d.world; ++r) *reinterpret_cast<float4*>(d.win[r] + d.half_base + d.rank * d.block_bytes + i * 4) = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&counters[1], 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    const u32 step = *reinterpret_cast<volatile u32*>(&counters[0]);
    if (threadIdx.x < d.world) *reinterpret_cast<volatile u32*>(d.win[threadIdx.x] + 4u * d.rank) = step;
}

// Waits (bounded) for every rank's flag, then y = (((+0 + P_0) + P_1) + ...) + P_{W-1}.
__global__ void __launch_bounds__(256) tp_fold_kernel(const unsigned char* window, u64 half_base, u64 block_bytes, u32 world, u32 bf16, const u32* counters,
                                                      u32 polls, u64 count, float* __restrict__ y, u16* __restrict__ y_bf16, u32* summary) {
    __shared__ u32 s_ok;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const u32 step = counters[0];
        const volatile u32* f = reinterpret_cast<const volatile u32*>(window) + threadIdx.x;
        bool seen = false;
        for (u32 i = 0; i < polls && !seen; ++i) {
            seen = static_cast<int>(*f - step) >= 0;
            if (!seen) __nanosleep(200);
        }
        if (!seen) { s_ok = 0; if (summary) atomicOr(summary, B200MOE_JOB_WAIT_ABORTED); }
        __threadfence_system();
    }
    __syncthreads();
    if (!s_ok) return;  // fail closed: a partial never arrived
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float acc = 0.0f;
    for (u32 r = 0; r < world; ++r) {
        const unsigned char* blk = window + half_base + r * block_bytes;
        const float v = bf16 ? __uint_as_float(u32(reinterpret_cast<const u16*>(blk)[i]) << 16) : reinterpret_cast<const float*>(blk)[i];
        acc = __fadd_rn(acc, v);
    }
    y[i] = acc;
    if (y_bf16) y_bf16[i] = bf16_rne_bits(acc);
}

u64 partial_offset(const Tp& tp) { return up256(b200moe_layer_workspace_bytes(&tp.shape, tp.rows)); }

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

uint64_t b200moe_tp_window_bytes(uint32_t hidden, uint32_t world, uint32_t rows, uint32_t payload_bf16) {
    if (world == 0 || world > kMaxWorld || rows == 0 || hidden == 0) return 0;
    return kFlagBytes + 2 * up256(u64(world) * rows * hidden * (payload_bf16 ? 2 : 4));
}

int b200moe_tp_create(const b200moe_tp_desc* desc, void** out) {
    B200_REQUIRE(desc && out, "tp_create: null descriptor / output");
    B200_REQUIRE(desc->world >= 1 && desc->world <= kMaxWorld && desc->rank < desc->world, "tp_create: need 1 <= world <= 8 and rank < world");
    B200_REQUIRE(desc->shape.experts == 1 && desc->shape.top_k == 1, "tp_create: shape.experts and shape.top_k must be 1 (a dense block)");
    B200_REQUIRE(desc->rows >= 1 && desc->shape.hidden % 4 == 0, "tp_create: rows is 0 or hidden is not a multiple of 4");
    B200_REQUIRE(desc->windows, "tp_create: windows is null");
    for (u32 r = 0; r < desc->world; ++r) B200_REQUIRE(desc->windows[r] && aligned(desc->windows[r], 256), "tp_create: window %u is null or not 256-byte aligned", r);
    if (b200moe_layer_workspace_bytes(&desc->shape, desc->rows) == 0) return B200MOE_ERR_INVALID_ARGUMENT;  // the shape check's message stands
    if (!device_ready()) return B200MOE_ERR_CUDA;
    Tp* tp = new Tp{};
    tp->shape = desc->shape; tp->world = desc->world; tp->rank = desc->rank; tp->rows = desc->rows; tp->bf16 = desc->payload_bf16 ? 1u : 0u;
    tp->half = up256(u64(tp->world) * tp->rows * tp->shape.hidden * (tp->bf16 ? 2 : 4));
    tp->wait_polls = desc->wait_polls ? desc->wait_polls : kDefaultWaitPolls;
    for (u32 r = 0; r < tp->world; ++r) tp->win[r] = static_cast<unsigned char*>(desc->windows[r]);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&tp->counters), 256);
    if (e == cudaSuccess) e = cudaMemset(tp->counters, 0, 256);
    if (e != cudaSuccess) {
        const int rc = fail(B200MOE_ERR_CUDA, "tp_create: %s", cudaGetErrorString(e));
        b200moe_tp_destroy(tp);
        return rc;
    }
    *out = tp;
    return B200MOE_OK;
}

void b200moe_tp_destroy(void* handle) {
    Tp* tp = static_cast<Tp*>(handle);
    if (!tp) return;
    if (tp->counters) cudaFree(tp->counters);
    delete tp;
}

uint64_t b200moe_tp_workspace_bytes(const void* handle) {
    const Tp* tp = static_cast<const Tp*>(handle);
    return tp ? partial_offset(*tp) + up256(u64(tp->rows) * tp->shape.hidden * 4) + 256 : 0;
}

int b200moe_tp_dense(void* handle, const b200moe_tp_step_view* v, void* stream) {
    Tp* tp = static_cast<Tp*>(handle);
    B200_REQUIRE(tp && v, "tp_dense: null handle / view");
    B200_REQUIRE(v->rows >= 1 && v->rows <= tp->rows, "tp_dense: rows %u exceed the %u the windows were sized for", v->rows, tp->rows);
    B200_REQUIRE(v->y, "tp_dense: y is null");
    const u64 need = b200moe_tp_workspace_bytes(tp);
    if (!v->workspace || v->workspace_bytes < need)
        return fail(B200MOE_ERR_WORKSPACE, "tp_dense: workspace of %llu bytes needed, %llu given", (unsigned long long)need, (unsigned long long)v->workspace_bytes);
    B200_REQUIRE(aligned(v->workspace, 256), "tp_dense: workspace must be 256-byte aligned");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);
    unsigned char* ws = static_cast<unsigned char*>(v->workspace);
    float* partial = reinterpret_cast<float*>(ws + partial_offset(*tp));
    u32* summary = v->summary ? v->summary : reinterpret_cast<u32*>(ws + need - 256);
    const u32 parity = tp->calls++ & 1u;

    tp_begin_kernel<<<1, 1, 0, st>>>(tp->counters);
    if (int rc = after_launch("tp_begin")) return rc;
    cudaError_t ce = cudaMemsetAsync(summary, 0, sizeof(u32), st);
    if (ce != cudaSuccess) return fail(B200MOE_ERR_CUDA, "tp_dense: cudaMemsetAsync: %s", cudaGetErrorString(ce));

    b200moe_dense_view dv{};
    dv.shape = tp->shape; dv.weights = v->weights; dv.rows = v->rows; dv.x = v->x; dv.y = partial;
    dv.workspace = ws; dv.workspace_bytes = partial_offset(*tp);
    if (int rc = b200moe_dense_ffn(&dv, stream)) return rc;

    TpDev d{};
    for (u32 r = 0; r < tp->world; ++r) d.win[r] = tp->win[r];
    d.world = tp->world; d.rank = tp->rank; d.bf16 = tp->bf16;
    d.half_base = kFlagBytes + parity * tp->half;
    d.block_bytes = u64(tp->rows) * tp->shape.hidden * (tp->bf16 ? 2 : 4);
    const u64 count = u64(v->rows) * tp->shape.hidden;
    const u32 blocks = static_cast<u32>(std::min<u64>((count / 4 + 255) / 256, 296));
    tp_scatter_kernel<<<blocks, 256, 0, st>>>(d, partial, count, tp->counters);
    if (int rc = after_launch("tp_scatter")) return rc;
    tp_fold_kernel<<<static_cast<u32>((count + 255) / 256), 256, 0, st>>>(tp->win[tp->rank], d.half_base, d.block_bytes, tp->world, tp->bf16, tp->counters,
                                                                          tp->wait_polls, count, v->y, v->y_bf16, summary);
    return after_launch("tp_fold");
}

}  // extern "C"
