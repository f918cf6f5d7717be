// Skeleton shared by the segment-streaming kernels (gemv_q4k_wide.cu, gemv_q8_wide.cu): the virtual-expert work list a CTA
// builds in shared memory from the window routes, the split of that list over the grid by estimated cost, and the host
// helper that encodes a tensor map of weight rows. See gemv_q4k_wide.cu for the design.
#pragma once
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "q4k_row.cuh"

namespace b200moe {
namespace wide {

constexpr u32 kKE = 8;                                  // entries of a virtual expert
constexpr u32 kGroups = 2, kGroupWarps = 8;
constexpr u32 kConsumerWarps = kGroups * kGroupWarps;
constexpr u32 kThreads = (kConsumerWarps + kGroups) * 32;  // one producer warp per group
constexpr u32 kEndItem = 0xffffffffu;
constexpr u32 kCostFixed = 4, kCostEntry = 3;           // estimated cost of an item: fixed + per entry
constexpr u32 kSmemBudget = 227u * 1024u;
constexpr u32 kDefaultWaitLimit = 1u << 22;

struct VExpert {  // one word: expert index (10 bits, experts <= 1024), first entry in the routes (14 bits, slots <= 8192), entries (4 bits)
    u32 bits;
    __host__ __device__ static VExpert make(u32 expert, u32 begin, u32 ne) { return VExpert{expert | (begin << 10) | (ne << 24)}; }
    __host__ __device__ u32 expert() const { return bits & 0x3ffu; }
    __host__ __device__ u32 begin() const { return (bits >> 10) & 0x3fffu; }
    __host__ __device__ u32 ne() const { return bits >> 24; }
};

__device__ __forceinline__ u32 warp_inclusive_scan(u32 v, u32 lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, v, d); if (lane >= (u32)d) v += o; }
    return v;
}
__device__ __forceinline__ u32 virtual_cost(u32 ne) { return kCostFixed + kCostEntry * ne; }

// First item whose cumulative cost start is >= B (items: virtual expert major, chunks ascending; an item of virtual
// expert jv costs virtual_cost(ne) and starts at cum[jv] * nc + chunk * cost). B >= total * nc gives n_virtual * nc.
__device__ inline u32 item_at(const VExpert* table, const u32* cum, u32 n_virtual, u32 nc, u64 total_items_cost, u64 B) {
    if (B >= total_items_cost) return n_virtual * nc;
    u32 lo = 0, hi = n_virtual - 1;  // last jv with cum[jv] * nc <= B
    while (lo < hi) {
        const u32 mid = (lo + hi + 1) >> 1;
        if (u64(cum[mid]) * nc <= B) lo = mid; else hi = mid - 1;
    }
    const u32 c = virtual_cost(table[lo].ne());
    const u64 excl = u64(cum[lo]) * nc;
    return lo * nc + static_cast<u32>((B - excl + c - 1) / c);
}

// Builds the CTA's work list: `table` gets the virtual experts (an expert of the union with at most kKE of its entries; an
// expert with more entries appears several times), ctl[2] / ctl[3] the first item and the item count of this CTA's run
// (items = virtual expert major x n_chunks chunks, split over the grid by cumulative cost). `scratch` is shared memory that
// is free until the first copy is issued ((2 * max_union + 2 + vmax) words). Every thread of the block calls it; it holds two
// block barriers. n_union <= max_union.
__device__ __forceinline__ void build_work_list(const b200moe_routes& routes, u32 n_union, u32 max_union, u32 vmax, u32 n_chunks, u32* scratch,
                                                VExpert* table, u32* ctl) {
    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    u32* t_beg = scratch;
    u32* t_exp = t_beg + max_union + 1;
    u32* t_cum = t_exp + max_union;  // exclusive cost prefix of every virtual expert: only the work split reads it
    for (u32 j = tid; j <= n_union; j += blockDim.x) {
        t_beg[j] = __ldg(routes.begins + j);
        if (j < n_union) t_exp[j] = __ldg(routes.experts + j);
    }
    __syncthreads();
    if (warp == 0) {
        u32 n_virtual = 0, total = 0;
        for (u32 j0 = 0; j0 < n_union; j0 += 32) {
            const u32 j = j0 + lane;
            const u32 eb = j < n_union ? t_beg[j] : 0u, ne = j < n_union ? t_beg[j + 1] - eb : 0u;
            const u32 nv = (ne + kKE - 1) / kKE, cost = nv * kCostFixed + ne * kCostEntry;
            const u32 iv = warp_inclusive_scan(nv, lane), ic = warp_inclusive_scan(cost, lane);
            u32 pos = n_virtual + iv - nv, cum = total + ic - cost;
            for (u32 k = 0; k < nv && pos < vmax; ++k, ++pos) {
                const u32 part = min(kKE, ne - k * kKE);
                table[pos] = VExpert::make(t_exp[j], eb + k * kKE, part);
                t_cum[pos] = cum;
                cum += virtual_cost(part);
            }
            n_virtual += __shfl_sync(0xffffffffu, iv, 31);
            total += __shfl_sync(0xffffffffu, ic, 31);
        }
        if (n_virtual > vmax) n_virtual = vmax;
        __syncwarp();
        if (lane == 0) {
            const u64 all = u64(total) * n_chunks;
            const u32 lo = item_at(table, t_cum, n_virtual, n_chunks, all, all * blockIdx.x / gridDim.x);
            const u32 hi = item_at(table, t_cum, n_virtual, n_chunks, all, all * (blockIdx.x + 1) / gridDim.x);
            ctl[2] = lo;
            ctl[3] = hi - lo;
        }
    }
    __syncthreads();
}

inline int sm_count() {
    int dev = 0, v = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v;
}

// Tensor map of a [rows][row_bytes] tensor seen as 64-bit elements, boxes of box_bytes (a multiple of 16) x box_rows rows,
// no swizzle. The encoder is the driver's cuTensorMapEncodeTiled, looked up through the runtime (no link against
// the driver library). Encoded maps are kept per (device, tensor, geometry): encoding is host work of a few microseconds
// that a decode step would otherwise pay on every call.
inline int rows_map(const u8* base, u64 row_bytes, u64 rows, u32 box_bytes, u32 box_rows, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    if (!fn) return fail(B200MOE_ERR_CUDA, "streaming form: cuTensorMapEncodeTiled is not available from this driver");
    static std::mutex m;
    static std::map<std::tuple<int, const u8*, u64, u64, u32, u32>, CUtensorMap> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const auto key = std::make_tuple(dev, base, row_bytes, rows, box_bytes, box_rows);
    std::lock_guard<std::mutex> lock(m);
    const auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return B200MOE_OK; }
    const cuuint64_t dims[2] = {row_bytes / 8, rows};
    const cuuint64_t strides[1] = {row_bytes};  // bytes between rows: a multiple of 16 (144 per super-block)
    const cuuint32_t box[2] = {box_bytes / 8, box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<u8*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200MOE_ERR_CUDA, "streaming form: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    if (cache.size() >= 1024) cache.clear();
    cache.emplace(key, *out);
    return B200MOE_OK;
}


}  // namespace wide
}  // namespace b200moe
