// Skeleton shared by the segment-streaming kernels (gemv_q4k_wide.cu, gemv_q8_wide.cu): the virtual-expert work list a CTA
// builds in shared memory from the window routes, the claim word through which the grid deals the items out, and the host
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
// ---- the grid's claim word -------------------------------------------------------------------------------------------
// Items are dealt to the groups of all CTAs through ONE word of device memory, routes.counts[3] (zero between launches: the
// routes builders write 0, and a launch leaves 0 behind): bits 0..21 count the claims, bits 22..31 the CTAs that have made
// their last claim. The CTA that retires last puts the word back to zero, so the next launch (a graph replay included)
// needs no memset. Why not a fixed share per CTA: the time of an item depends on its entries in a way a cost estimate only
// approximates, and with a dozen items per group a mis-estimate leaves SMs idle for the last tenth of the kernel.
constexpr u32 kClaimBits = 22, kClaimMask = (1u << kClaimBits) - 1u;
__host__ __device__ constexpr u32 work_list_scratch_words(u32 max_union, u32 vmax) { return 2 * max_union + 2 + vmax + kKE; }
__device__ __forceinline__ u32 claim_item(u32* claim) { return atomicAdd(claim, 1u) & kClaimMask; }
// Called once per producer warp (lane 0) when it will claim no more; ctl[1] counts the CTA's producers that have finished.
__device__ __forceinline__ void retire_claims(u32* claim, u32* ctl) {
    if (atomicAdd(&ctl[1], 1u) != kGroups - 1u) return;
    const u32 before = atomicAdd(claim, 1u << kClaimBits);
    if ((before >> kClaimBits) == gridDim.x - 1u) atomicExch(claim, 0u);
}

// Builds the work list: `table` gets the virtual experts (an expert of the union with at most kKE of its entries; an expert
// with more entries appears several times) ORDERED BY ENTRIES, most first (stable within a count): items are claimed in
// table order, so the long items start first and the kernel's tail is made of short ones. ctl[3] = items (virtual expert
// major x n_chunks chunks). Every CTA builds the same list. `scratch` is shared memory that is free until the first copy is
// issued (work_list_scratch_words(max_union, vmax) words). Every thread of the block calls it; it holds four block barriers.
// n_union <= max_union.
__device__ __forceinline__ void build_work_list(const b200moe_routes& routes, u32 n_union, u32 max_union, u32 vmax, u32 n_chunks, u32* scratch,
                                                VExpert* table, u32* ctl) {
    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    u32* t_beg = scratch;
    u32* t_exp = t_beg + max_union + 1;
    VExpert* unsorted = reinterpret_cast<VExpert*>(t_exp + max_union);
    u32* s_hist = reinterpret_cast<u32*>(unsorted + vmax);
    for (u32 j = tid; j <= n_union; j += blockDim.x) {
        t_beg[j] = __ldg(routes.begins + j);
        if (j < n_union) t_exp[j] = __ldg(routes.experts + j);
    }
    __syncthreads();
    if (warp == 0) {
        u32 n_virtual = 0;
        for (u32 j0 = 0; j0 < n_union; j0 += 32) {
            const u32 j = j0 + lane;
            const u32 eb = j < n_union ? t_beg[j] : 0u, ne = j < n_union ? t_beg[j + 1] - eb : 0u;
            const u32 nv = (ne + kKE - 1) / kKE;
            const u32 iv = warp_inclusive_scan(nv, lane);
            u32 pos = n_virtual + iv - nv;
            for (u32 k = 0; k < nv && pos < vmax; ++k, ++pos) unsorted[pos] = VExpert::make(t_exp[j], eb + k * kKE, min(kKE, ne - k * kKE));
            n_virtual += __shfl_sync(0xffffffffu, iv, 31);
        }
        if (n_virtual > vmax) n_virtual = vmax;
        if (lane == 0) { ctl[2] = n_virtual; ctl[3] = n_virtual * n_chunks; }
    }
    __syncthreads();
    // counting sort by entries, descending: warp b places the virtual experts of kKE - b entries
    const u32 n_virtual = ctl[2];
    const u32 want = kKE - warp;
    if (warp < kKE) {
        u32 n = 0;
        for (u32 i0 = 0; i0 < n_virtual; i0 += 32) n += __popc(__ballot_sync(0xffffffffu, i0 + lane < n_virtual && unsorted[i0 + lane].ne() == want));
        if (lane == 0) s_hist[warp] = n;
    }
    __syncthreads();
    if (warp < kKE) {
        u32 pos = 0;
        for (u32 b = 0; b < warp; ++b) pos += s_hist[b];
        for (u32 i0 = 0; i0 < n_virtual; i0 += 32) {
            const bool mine = i0 + lane < n_virtual && unsorted[i0 + lane].ne() == want;
            const u32 m = __ballot_sync(0xffffffffu, mine);
            if (mine) table[pos + __popc(m & ((1u << lane) - 1u))] = unsorted[i0 + lane];
            pos += __popc(m);
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
