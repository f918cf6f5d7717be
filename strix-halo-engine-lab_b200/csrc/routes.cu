// Window routes: the expert-major CSR of (row, slot) entries that every expert kernel gathers through. Activations
// are never permuted in memory.
//
// Contract: strix::ds41::build_window_routes + restrict_routes (src/ds41_moe.cpp:11-61; device mirror
// include/strix/cuda/ds41_moe.hpp:41-72): union experts ascending, the entries of an expert in ascending row,
// slots[i] = row * top_k + k, order[row][*] = the row's slots in ascending expert id, low_counts[row] = ids < split.
// All integer work; results are exact and independent of the launch shape.
//
// Two forms: up to 1024 slots (decode windows) one block does everything; above that three launches over chunks of
// 1024 slots (per-chunk histograms, a scan over chunks and experts, then the stable fill).
#include "kernels.cuh"
#include "router_select.cuh"
#include "routes_small.cuh"

namespace b200moe {
namespace {

constexpr u32 kChunk = routes_detail::kChunk;

using routes_detail::block_exclusive_scan;
using routes_detail::entry_id;
using routes_detail::row_order;
using routes_detail::routes_small_body;

__global__ void __launch_bounds__(1024) routes_small_kernel(b200moe_routes_view v, u32 end) { routes_small_body(v, end); }

// Decode windows: the router's selection (one warp per row) and the routes of the selected ids in ONE block, so the
// layer prologue costs one launch less. Dynamic shared memory: rows * (2 * experts + 32) floats.
__global__ void __launch_bounds__(1024) select_routes_small_kernel(const float* logits, float* scores_out, const float* __restrict__ bias,
                                                                   b200moe_route_policy p, u32 rows, u32* ids, float* __restrict__ weights,
                                                                   b200moe_routes_view rv, u32 end) {
    extern __shared__ float sel_smem[];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    if (warp < rows) select_detail::select_row(logits, scores_out, bias, p, warp, lane, sel_smem + warp * (2u * p.experts + 32u), ids, weights);
    __syncthreads();  // the ids written above are read below by the whole block
    routes_small_body(rv, end);
}

// ---- chunked form --------------------------------------------------------------------------------------------------
// scratch: hist[chunks][experts], then ebegin[experts].
__global__ void __launch_bounds__(1024) routes_count_kernel(b200moe_routes_view v, u32 end, u32 chunks) {
    __shared__ u32 cnt[1024];
    const u32 t = threadIdx.x, n = v.rows * v.top_k, s = blockIdx.x * kChunk + t;
    cnt[t] = 0;
    __syncthreads();
    if (s < n) { const u32 e = entry_id(v.ids, s, v.top_k, v.experts, v.first, end); if (e != 0xffffffffu) atomicAdd(&cnt[e], 1u); }
    __syncthreads();
    if (t < v.experts) v.scratch[u64(blockIdx.x) * v.experts + t] = cnt[t];
    for (u32 r = blockIdx.x * blockDim.x + t; r < v.rows; r += gridDim.x * blockDim.x)
        row_order(v.ids, r, v.top_k, v.experts, v.split, v.out.order, v.out.low_counts, v.row_status);
}
__global__ void __launch_bounds__(1024) routes_scan_kernel(b200moe_routes_view v, u32 chunks) {
    __shared__ u32 warp_tot[32], total_s, union_s, maxc;
    const u32 t = threadIdx.x;
    if (t == 0) maxc = 0;
    u32 c = 0;
    if (t < v.experts)
        for (u32 k = 0; k < chunks; ++k) { u32* h = &v.scratch[u64(k) * v.experts + t]; const u32 x = *h; *h = c; c += x; }
    __syncthreads();
    const u32 begin = block_exclusive_scan(c, warp_tot, &total_s);
    const u32 uidx = block_exclusive_scan(c ? 1u : 0u, warp_tot, &union_s);
    if (t < v.experts) v.scratch[u64(chunks) * v.experts + t] = begin;
    if (c) { v.out.experts[uidx] = t - v.base; v.out.begins[uidx + 1] = begin + c; atomicMax(&maxc, c); }
    __syncthreads();
    if (t == 0) {
        v.out.begins[0] = 0;
        v.out.counts[0] = union_s; v.out.counts[1] = maxc; v.out.counts[2] = total_s; v.out.counts[3] = 0;
    }
}
__global__ void __launch_bounds__(1024) routes_fill_kernel(b200moe_routes_view v, u32 end, u32 chunks) {
    __shared__ u32 sid[1024];
    const u32 t = threadIdx.x, n = v.rows * v.top_k, s = blockIdx.x * kChunk + t;
    u32 e = 0xffffffffu;
    if (s < n) e = entry_id(v.ids, s, v.top_k, v.experts, v.first, end);
    sid[t] = e;
    __syncthreads();
    if (e == 0xffffffffu) return;
    u32 rank = 0;
    for (u32 i = 0; i < t; ++i) rank += sid[i] == e ? 1u : 0u;
    const u32 pos = v.scratch[u64(chunks) * v.experts + e] + v.scratch[u64(blockIdx.x) * v.experts + e] + rank;
    v.out.rows[pos] = s / v.top_k;
    v.out.slots[pos] = s;
}


// The routes of a dense block (one expert, top-1: every row is one entry of expert 0, slot = row) written directly, with
// the job's status words cleared in the same launch: what build_window_routes (src/ds41_moe.cpp:11-43) gives for ids = 0,
// without the sort and without the memsets in front of it.
__global__ void __launch_bounds__(256) dense_routes_kernel(b200moe_routes out, u32 rows, u32* row_status, u32* summary4) {
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) {
        out.rows[i] = i;
        out.slots[i] = i;
        if (out.order) out.order[i] = i;
        if (out.low_counts) out.low_counts[i] = 1u;  // id 0 < split 1
        if (row_status) row_status[i] = 0u;
    }
    if (i == 0) {
        out.experts[0] = 0u;
        out.begins[0] = 0u;
        out.begins[1] = rows;
        out.counts[0] = 1u; out.counts[1] = rows; out.counts[2] = rows; out.counts[3] = 0u;
        if (summary4) { summary4[0] = 0u; summary4[1] = 0u; summary4[2] = 0u; summary4[3] = 0u; }
    }
}

}  // namespace

u64 routes_scratch_words(u32 rows, u32 top_k, u32 experts) {
    const u64 n = u64(rows) * top_k, chunks = (n + kChunk - 1) / kChunk;
    return (chunks + 1) * experts + 4;
}

bool select_routes_fusable(const b200moe_router_view& r, u32 top_k) {
    return r.rows <= 32 && u64(r.rows) * top_k <= kChunk && u64(r.rows) * (2u * r.policy.experts + 32u) * 4u <= 96u * 1024u;
}
int launch_select_routes(const b200moe_router_view& r, const b200moe_routes_view& v, cudaStream_t stream) {
    if (r.rows == 0) return B200MOE_OK;
    const u32 smem = r.rows * (2u * r.policy.experts + 32u) * 4u;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(select_routes_small_kernel), smem)) return rc;
    select_routes_small_kernel<<<1, 1024, smem, stream>>>(r.logits, r.scores, r.bias, r.policy, r.rows, r.ids, r.weights, v, v.end ? v.end : v.experts);
    return after_launch("select_routes_small");
}

int launch_dense_routes(const b200moe_routes& out, u32 rows, u32* row_status, u32* summary4, cudaStream_t stream) {
    dense_routes_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(out, rows, row_status, summary4);
    return after_launch("dense_routes");
}

int launch_routes(const b200moe_routes_view& v, cudaStream_t stream) {
    const u64 n = u64(v.rows) * v.top_k;
    if (n == 0) return B200MOE_OK;
    const u32 end = v.end ? v.end : v.experts;
    if (n <= kChunk) {
        routes_small_kernel<<<1, 1024, 0, stream>>>(v, end);
        return after_launch("routes_small");
    }
    const u32 chunks = static_cast<u32>((n + kChunk - 1) / kChunk);
    routes_count_kernel<<<chunks, 1024, 0, stream>>>(v, end, chunks);
    if (int rc = after_launch("routes_count")) return rc;
    routes_scan_kernel<<<1, 1024, 0, stream>>>(v, chunks);
    if (int rc = after_launch("routes_scan")) return rc;
    routes_fill_kernel<<<chunks, 1024, 0, stream>>>(v, end, chunks);
    return after_launch("routes_fill");
}

}  // namespace b200moe
