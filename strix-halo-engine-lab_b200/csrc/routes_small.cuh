// Routes of a decode window (up to 1024 slots, up to 1024 experts) built by ONE block of any size: device code shared by
// the stand-alone routes kernel (routes.cu) and the fused layer prologue (prologue.cu).
// Contract: strix::ds41::build_window_routes + restrict_routes (src/ds41_moe.cpp:11-61), see routes.cu.
#pragma once
#include "common.cuh"

namespace b200moe {
namespace routes_detail {

constexpr u32 kChunk = 1024;

// Exclusive scan of one value per thread over the block (blockDim a multiple of 32, at most 1024); `total` gets the
// sum. warp_tot: 32 words of shared memory.
__device__ __forceinline__ u32 block_exclusive_scan(u32 v, u32* warp_tot, u32* total) {
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    u32 inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, inc, d); if (lane >= (u32)d) inc += o; }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        u32 t = lane < nwarps ? warp_tot[lane] : 0u, ti = t;
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
__device__ inline void row_order(const u32* ids, u32 row, u32 top_k, u32 experts, u32 split, u32* order, u32* low_counts, u32* row_status) {
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
// The expert id slot s contributes an entry for, or 0xffffffff for none: the id must lie in the owned range and must not
// repeat an earlier slot of the same row. (The host builder throws on a repeated id, src/ds41_moe.cpp:22-23; here the row
// is flagged INVALID_ROUTE and only the first occurrence keeps its entry, so no expert ever has more entries than the
// window has rows and a flagged row cannot disturb the entries of a valid one.)
__device__ __forceinline__ u32 entry_id(const u32* ids, u32 s, u32 top_k, u32 experts, u32 first, u32 end) {
    const u32 e = ids[s];
    if (!owned(e, experts, first, end)) return 0xffffffffu;
    for (u32 i = s - s % top_k; i < s; ++i)
        if (ids[i] == e) return 0xffffffffu;
    return e;
}

// Windows of up to 256 slots (decode): every slot's thread counts what it needs directly from the ids in shared memory
// - O(slots) work per thread, three block barriers, no scans. Same outputs as the general body below.
__device__ inline void routes_tiny_body(const b200moe_routes_view& v, u32 end) {
    __shared__ u32 sid[256], srank[256], red[4];
    const u32 t = threadIdx.x, nt = blockDim.x, n = v.rows * v.top_k, K = v.top_k;
    if (t < 4) red[t] = 0;
    for (u32 s = t; s < n; s += nt) {
        sid[s] = entry_id(v.ids, s, K, v.experts, v.first, end);
    }
    __syncthreads();
    for (u32 s = t; s < n; s += nt) {  // rank among the slots of the same expert (ascending slot = ascending row)
        const u32 e = sid[s];
        u32 rank = 0;
        for (u32 i = 0; i < s; ++i) rank += sid[i] == e ? 1u : 0u;
        srank[s] = rank;
    }
    __syncthreads();
    for (u32 s = t; s < n; s += nt) {
        const u32 e = sid[s];
        // the row's order, low count and route check (every slot places itself)
        {
            const u32 row = s / K, raw = v.ids[s];
            u32 pos = 0, low = 0;
            bool bad = raw >= v.experts;
            for (u32 k = 0; k < K; ++k) {
                const u32 o = v.ids[row * K + k], so = row * K + k;
                pos += (o < raw || (o == raw && so < s)) ? 1u : 0u;
                bad |= (o == raw && so != s);
                low += o < v.split ? 1u : 0u;
            }
            v.out.order[row * K + pos] = s;
            if (s == row * K) v.out.low_counts[row] = low;
            if (bad && v.row_status) atomicOr(&v.row_status[row], B200MOE_ROW_INVALID_ROUTE);
        }
        if (e == 0xffffffffu) continue;
        u32 before = 0, uidx = 0, cnt = 0;
        for (u32 i = 0; i < n; ++i) {
            const u32 o = sid[i];
            before += o < e ? 1u : 0u;                          // 0xffffffff (not owned) is never below e
            uidx += (o < e && srank[i] == 0) ? 1u : 0u;
            cnt += o == e ? 1u : 0u;
        }
        const u32 rank = srank[s], pos = before + rank;
        v.out.rows[pos] = s / K;
        v.out.slots[pos] = s;
        if (rank == 0) {
            v.out.experts[uidx] = e - v.base;
            v.out.begins[uidx + 1] = before + cnt;
            atomicAdd(&red[0], 1u);
            atomicMax(&red[1], cnt);
            atomicAdd(&red[2], cnt);
        }
    }
    __syncthreads();
    if (t == 0) {
        v.out.begins[0] = 0;
        v.out.counts[0] = red[0]; v.out.counts[1] = red[1]; v.out.counts[2] = red[2]; v.out.counts[3] = 0;
    }
}

// The whole build by one block. Each thread owns a contiguous run of experts for the scans.
__device__ inline void routes_small_body(const b200moe_routes_view& v, u32 end) {
    __shared__ u32 cnt[1024], ebegin[1024], sid[1024], warp_tot[32], total_s, union_s, maxc;
    const u32 t = threadIdx.x, nt = blockDim.x, n = v.rows * v.top_k;
    if (n <= 256) { routes_tiny_body(v, end); return; }
    for (u32 i = t; i < 1024; i += nt) cnt[i] = 0;
    if (t == 0) maxc = 0;
    __syncthreads();
    for (u32 s = t; s < n; s += nt) {
        const u32 e = entry_id(v.ids, s, v.top_k, v.experts, v.first, end);
        if (e != 0xffffffffu) atomicAdd(&cnt[e], 1u);
        sid[s] = e;
    }
    for (u32 r = t; r < v.rows; r += nt) row_order(v.ids, r, v.top_k, v.experts, v.split, v.out.order, v.out.low_counts, v.row_status);
    __syncthreads();
    const u32 per = (v.experts + nt - 1) / nt, e0 = t * per, e1 = min(e0 + per, v.experts);
    u32 c_sum = 0, c_nz = 0, c_max = 0;
    for (u32 e = e0; e < e1; ++e) { const u32 c = cnt[e]; c_sum += c; c_nz += c ? 1u : 0u; c_max = max(c_max, c); }
    u32 begin = block_exclusive_scan(c_sum, warp_tot, &total_s);
    u32 uidx = block_exclusive_scan(c_nz, warp_tot, &union_s);
    if (c_max) atomicMax(&maxc, c_max);
    for (u32 e = e0; e < e1; ++e) {
        const u32 c = cnt[e];
        ebegin[e] = begin;
        if (c) { v.out.experts[uidx] = e - v.base; v.out.begins[uidx + 1] = begin + c; ++uidx; }
        begin += c;
    }
    __syncthreads();
    if (t == 0) {
        v.out.begins[0] = 0;
        v.out.counts[0] = union_s; v.out.counts[1] = maxc; v.out.counts[2] = total_s; v.out.counts[3] = 0;
    }
    for (u32 s = t; s < n; s += nt) {
        const u32 e = sid[s];
        if (e == 0xffffffffu) continue;
        u32 rank = 0;
        for (u32 i = 0; i < s; ++i) rank += sid[i] == e ? 1u : 0u;
        const u32 pos = ebegin[e] + rank;
        v.out.rows[pos] = s / v.top_k;
        v.out.slots[pos] = s;
    }
}

}  // namespace routes_detail
}  // namespace b200moe
