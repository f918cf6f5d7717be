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

namespace b200moe {
namespace {

constexpr u32 kChunk = 1024;

// Exclusive scan of one value per thread over a 1024-thread block; `total` gets the sum. warp_tot: 32 words of smem.
__device__ __forceinline__ u32 block_exclusive_scan(u32 v, u32* warp_tot, u32* total) {
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    u32 inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, inc, d); if (lane >= (u32)d) inc += o; }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        u32 t = warp_tot[lane], ti = t;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, ti, d); if (lane >= (u32)d) ti += o; }
        warp_tot[lane] = ti - t;
        if (lane == 31) *total = ti;
    }
    __syncthreads();
    const u32 r = warp_tot[warp] + inc - v;
    __syncthreads();
    return r;
}

// Per row: the slots sorted by expert id (top_k <= 32, insertion sort), the low count and the route check.
__device__ void row_order(const u32* ids, u32 row, u32 top_k, u32 experts, u32 split, u32* order, u32* low_counts, u32* row_status) {
    u32 key[32], slot[32];
    u32 low = 0;
    bool bad = false;
    for (u32 k = 0; k < top_k; ++k) {
        const u32 s = row * top_k + k, e = ids[s];
        bad |= e >= experts;
        low += e < split ? 1u : 0u;
        u32 j = k;
        while (j > 0 && key[j - 1] > e) { key[j] = key[j - 1]; slot[j] = slot[j - 1]; --j; }
        bad |= (j > 0 && key[j - 1] == e);
        key[j] = e; slot[j] = s;
    }
    for (u32 k = 0; k < top_k; ++k) order[row * top_k + k] = slot[k];
    low_counts[row] = low;
    if (bad && row_status) atomicOr(&row_status[row], B200MOE_ROW_INVALID_ROUTE);
}

__device__ __forceinline__ bool owned(u32 e, u32 experts, u32 first, u32 end) { return e < experts && e >= first && e < end; }

// ---- one block, <= 1024 slots ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) routes_small_kernel(b200moe_routes_view v, u32 end) {
    __shared__ u32 cnt[1024], ebegin[1024], sid[1024], warp_tot[32], total_s, union_s, maxc;
    const u32 t = threadIdx.x, n = v.rows * v.top_k;
    cnt[t] = 0;
    if (t == 0) maxc = 0;
    __syncthreads();
    u32 e = 0xffffffffu;
    if (t < n) {
        e = v.ids[t];
        if (!owned(e, v.experts, v.first, end)) e = 0xffffffffu;
        else atomicAdd(&cnt[e], 1u);
    }
    sid[t] = e;
    for (u32 r = t; r < v.rows; r += blockDim.x) row_order(v.ids, r, v.top_k, v.experts, v.split, v.out.order, v.out.low_counts, v.row_status);
    __syncthreads();
    const u32 c = t < v.experts ? cnt[t] : 0u;
    const u32 begin = block_exclusive_scan(c, warp_tot, &total_s);
    const u32 uidx = block_exclusive_scan(c ? 1u : 0u, warp_tot, &union_s);
    ebegin[t] = begin;
    if (c) { v.out.experts[uidx] = t - v.base; v.out.begins[uidx + 1] = begin + c; atomicMax(&maxc, c); }
    __syncthreads();
    if (t == 0) {
        v.out.begins[0] = 0;
        v.out.counts[0] = union_s; v.out.counts[1] = maxc; v.out.counts[2] = total_s; v.out.counts[3] = 0;
    }
    if (e != 0xffffffffu) {
        u32 rank = 0;
        for (u32 i = 0; i < t; ++i) rank += sid[i] == e ? 1u : 0u;
        const u32 pos = ebegin[e] + rank;
        v.out.rows[pos] = t / v.top_k;
        v.out.slots[pos] = t;
    }
}

// ---- chunked form --------------------------------------------------------------------------------------------------
// scratch: hist[chunks][experts], then ebegin[experts].
__global__ void __launch_bounds__(1024) routes_count_kernel(b200moe_routes_view v, u32 end, u32 chunks) {
    __shared__ u32 cnt[1024];
    const u32 t = threadIdx.x, n = v.rows * v.top_k, s = blockIdx.x * kChunk + t;
    cnt[t] = 0;
    __syncthreads();
    if (s < n) { const u32 e = v.ids[s]; if (owned(e, v.experts, v.first, end)) atomicAdd(&cnt[e], 1u); }
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
    if (s < n) { e = v.ids[s]; if (!owned(e, v.experts, v.first, end)) e = 0xffffffffu; }
    sid[t] = e;
    __syncthreads();
    if (e == 0xffffffffu) return;
    u32 rank = 0;
    for (u32 i = 0; i < t; ++i) rank += sid[i] == e ? 1u : 0u;
    const u32 pos = v.scratch[u64(chunks) * v.experts + e] + v.scratch[u64(blockIdx.x) * v.experts + e] + rank;
    v.out.rows[pos] = s / v.top_k;
    v.out.slots[pos] = s;
}

}  // namespace

u64 routes_scratch_words(u32 rows, u32 top_k, u32 experts) {
    const u64 n = u64(rows) * top_k, chunks = (n + kChunk - 1) / kChunk;
    return (chunks + 1) * experts + 4;
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
