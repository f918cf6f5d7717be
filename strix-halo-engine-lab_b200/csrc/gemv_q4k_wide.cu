// Routed experts, Qwen A8 family, decode form for ANY row length: a persistent kernel that streams SEGMENTS of the
// weight rows - and of the activations they meet - through shared memory with the TMA engine.
//
// Same arithmetic as gemv_q4k.cu (the contract of src/cpu/core/routed_expert.hpp:9-15, bit for bit). What this form adds
// over gemv_q4k_stream.cu is that nothing is sized by the row length or by the window: hidden 7168 (4032-byte gate rows),
// inter 17408 (9792-byte down rows) and 64-row windows stream exactly like the small layers.
//
//  * Work item = (virtual expert, 64 weight rows): 32 gate + 32 up rows of one output group, or 64 down rows. A virtual
//    expert is an expert of the window's union with at most kKE = 8 of its entries; an expert with more entries appears
//    several times (its rows are then streamed again, out of L2). Every CTA builds the virtual list in shared memory from
//    the routes (one warp scan) and takes a contiguous run of items of about equal estimated cost.
//  * A stage = S = 3 super-blocks of the item's 64 rows (one or two tiled TMA copies of 432 bytes x 32 / 64 rows: the rows
//    lie 432 bytes apart in shared memory, an odd count of 16-byte units, which keeps the 128-bit reads of eight rows
//    conflict free) PLUS the same K range of the A8 rows of the item's entries (codes, deltas, sums: three bulk copies per
//    entry), all counted on one mbarrier. The consumers therefore find everything a stage needs in shared memory.
//  * Two groups of eight consumer warps share a CTA, each with its own ring of stages and its own producer warp; a group
//    takes the next unclaimed item of the CTA's run (a shared-memory counter), so the groups finish together. Lane =
//    (pair p, row): a lane walks its row's super-blocks in ascending order across the item's stages, the serial chains
//    acc_p += pair_p never leave their lane, and (a0 + a1) + (a2 + a3) is two xor-shuffles at the end of the item.
//  * gate/up: the group meets on an mbarrier once per item and eight warps run SwiGLU + the A8 rule of one entry each.
//
// Every wait is bounded (plan.wait_limit polls): a waiter that runs out raises the CTA's abort flag, every role leaves
// its loops, the producers wait (bounded) for the copies they still have in flight, B200MOE_JOB_WAIT_ABORTED is set in the
// job summary and the kernel returns - the host reads a status, the GPU never hangs.
//
// Roofline: HBM. Algorithmic bytes per item = 64 rows x K / 256 x 144 (+ the entries' A8 bytes).
#include <map>
#include <mutex>
#include <tuple>

#include "q4k_row.cuh"

namespace b200moe {

namespace {
using namespace q4k;

constexpr u32 kKE = 8;                                  // entries of a virtual expert
constexpr u32 kGroups = 2, kGroupWarps = 8;
constexpr u32 kConsumerWarps = kGroups * kGroupWarps;
constexpr u32 kThreads = (kConsumerWarps + kGroups) * 32;  // one producer warp per group
constexpr u32 kItemRows = 64;
constexpr u32 kEndItem = 0xffffffffu;
constexpr u32 kCostFixed = 4, kCostEntry = 3;           // estimated cost of an item: fixed + per entry
constexpr u32 kSmemBudget = 227u * 1024u;
constexpr u32 kDefaultWaitLimit = 1u << 22;

struct WidePlan {
    u32 S;              // super-blocks per stage
    u32 nb;             // super-blocks per row
    u32 nseg;           // stages per item
    u32 stages;         // ring depth per group
    u32 row_seg_bytes;  // S * 144
    u32 w_bytes;        // 64 * row_seg_bytes
    u32 x_entry_bytes;  // S * 320: codes, deltas, sums of one entry over the stage's K range
    u32 stage_bytes;
    u32 n_chunks;       // items per (virtual) expert
    u32 max_union;      // bound of the union
    u32 vmax;           // capacity of the virtual expert list
    u32 wait_limit;
    u32 stall_stage;    // test hook: group 0's producer stops before this stage (0xffffffff: never)
};

struct WideArgs {
    b200moe_routes routes;
    b200moe_a8_rows in;    // x (gate/up) or the A8 of h (down)
    b200moe_a8_rows act;   // gate/up output
    float* gate_out;
    float* up_out;
    float* raw;            // down output
    u32* row_status;
    u32* summary;
    u32 rows_per_expert;   // weight rows of one expert: inter (gate/up) or hidden (down)
    u32 out_width;         // inter (gate/up) or hidden (down)
};

struct VExpert { u32 expert, begin, ne, cum; };

__device__ __forceinline__ u32 warp_inclusive_scan(u32 v, u32 lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, v, d); if (lane >= (u32)d) v += o; }
    return v;
}
__device__ __forceinline__ u32 virtual_cost(u32 ne) { return kCostFixed + kCostEntry * ne; }

// First item whose cumulative cost start is >= B (items: virtual expert major, chunks ascending; an item of virtual
// expert jv costs virtual_cost(ne) and starts at cum[jv] * nc + chunk * cost). B >= total * nc gives n_virtual * nc.
__device__ u32 item_at(const VExpert* table, u32 n_virtual, u32 nc, u64 total_items_cost, u64 B) {
    if (B >= total_items_cost) return n_virtual * nc;
    u32 lo = 0, hi = n_virtual - 1;  // last jv with cum[jv] * nc <= B
    while (lo < hi) {
        const u32 mid = (lo + hi + 1) >> 1;
        if (u64(table[mid].cum) * nc <= B) lo = mid; else hi = mid - 1;
    }
    const u32 c = virtual_cost(table[lo].ne);
    const u64 excl = u64(table[lo].cum) * nc;
    return lo * nc + static_cast<u32>((B - excl + c - 1) / c);
}

// (a0 + a1) + (a2 + a3) over the four pair lanes of a row (lane = 8 * p + row); every lane of the row gets the value.
__device__ __forceinline__ float tree4(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 8));
    return __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
}

// One stage of one weight row (this lane's pair p of nbk super-blocks, ascending) against NR staged A8 rows. blk: the
// row's first super-block of the stage; xs: entry 0's area of the stage ({codes[S * 256], deltas[S * 8], sums[S * 8]},
// the next entry x_entry_bytes further). acc[r] is the lane's chain acc_p of entry r.
template <int NR>
__device__ __forceinline__ void stage_rows(const uint4* blk, u32 nbk, u32 p, const unsigned char* xs, u32 x_entry_bytes, u32 S, float* acc) {
#pragma unroll 1
    for (u32 b = 0; b < nbk; ++b, blk += kQ4KBlock / 16) {
        const uint4 hdr = blk[0], q0 = blk[1 + 2 * p], q1 = blk[2 + 2 * p];
        const Factors f = q4k_factors(hdr, p);
        const Nibbles n = split_nibbles(q0, q1);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const unsigned char* xe = xs + r * x_entry_bytes;
            const uint4* c = reinterpret_cast<const uint4*>(xe + 256u * b + 64u * p);
            const uint4 c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3];
            const float2 e = *reinterpret_cast<const float2*>(xe + 256u * S + 32u * b + 8u * p);
            const int2 sm = *reinterpret_cast<const int2*>(xe + 288u * S + 32u * b + 8u * p);
            int lo, hi;
            dots(n, c0, c1, c2, c3, &lo, &hi);
            acc[r] = __fadd_rn(acc[r], pair_value(f, lo, hi, e.x, e.y, small_int_to_float(sm.x), small_int_to_float(sm.y)));
        }
    }
}
__device__ __forceinline__ void stage_rows_n(u32 nr, const uint4* blk, u32 nbk, u32 p, const unsigned char* xs, u32 xeb, u32 S, float* acc) {
    switch (nr) {  // no per-entry branches inside the block loop
        case 1: stage_rows<1>(blk, nbk, p, xs, xeb, S, acc); break;
        case 2: stage_rows<2>(blk, nbk, p, xs, xeb, S, acc); break;
        case 3: stage_rows<3>(blk, nbk, p, xs, xeb, S, acc); break;
        default: stage_rows<4>(blk, nbk, p, xs, xeb, S, acc); break;
    }
}

template <bool DOWN>
__global__ void __launch_bounds__(kThreads, 1)
q4k_wide_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, WideArgs a, WidePlan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    if (DOWN && a.summary && *a.summary) return;  // a failed or aborted projection skips the whole stage (routed_expert.hpp:17-19)
    u32 n_union = a.routes.counts[0];
    if (n_union == 0) return;
    if (n_union > plan.max_union) n_union = plan.max_union;

    unsigned char* at = smem + u64(kGroups) * plan.stages * plan.stage_bytes;
    float* s_gu = reinterpret_cast<float*>(at);  // [group][buffer][gate | up][entry][32]
    if (!DOWN) at += kGroups * 2 * 2 * kKE * 32 * 4;
    VExpert* table = reinterpret_cast<VExpert*>(at);
    at += u64(plan.vmax) * sizeof(VExpert);
    u64* full = reinterpret_cast<u64*>(at);
    u64* empty = full + kGroups * plan.stages;
    u64* gu_bar = empty + kGroups * plan.stages;
    at += (2 * kGroups * plan.stages + kGroups) * 8;
    u32* slot_item = reinterpret_cast<u32*>(at);
    at += kGroups * plan.stages * 4;
    u32* ctl = reinterpret_cast<u32*>(at);  // [0] abort flag, [1] next local item, [2] first item, [3] items of this CTA
    volatile u32* abort_flag = ctl;

    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid < kGroups * plan.stages) { mbar_init(&full[tid], 1); mbar_init(&empty[tid], kGroupWarps); }
    if (tid < kGroups) mbar_init(&gu_bar[tid], kGroupWarps);
    if (tid < 4) ctl[tid] = 0;
    if (tid < kGroups * plan.stages + kGroups) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");

    // ---- the virtual expert list (the stage area is free until the first copy is issued: it holds the copied routes)
    u32* t_beg = reinterpret_cast<u32*>(smem);
    u32* t_exp = t_beg + plan.max_union + 1;
    for (u32 j = tid; j <= n_union; j += kThreads) {
        t_beg[j] = __ldg(a.routes.begins + j);
        if (j < n_union) t_exp[j] = __ldg(a.routes.experts + j);
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
            for (u32 k = 0; k < nv && pos < plan.vmax; ++k, ++pos) {
                const u32 part = min(kKE, ne - k * kKE);
                table[pos] = VExpert{t_exp[j], eb + k * kKE, part, cum};
                cum += virtual_cost(part);
            }
            n_virtual += __shfl_sync(0xffffffffu, iv, 31);
            total += __shfl_sync(0xffffffffu, ic, 31);
        }
        if (n_virtual > plan.vmax) n_virtual = plan.vmax;
        __syncwarp();
        if (lane == 0) {
            const u64 all = u64(total) * plan.n_chunks;
            const u32 lo = item_at(table, n_virtual, plan.n_chunks, all, all * blockIdx.x / gridDim.x);
            const u32 hi = item_at(table, n_virtual, plan.n_chunks, all, all * (blockIdx.x + 1) / gridDim.x);
            ctl[2] = lo;
            ctl[3] = hi - lo;
        }
    }
    __syncthreads();
    const u32 first_item = ctl[2], n_local = ctl[3];
    if (n_local == 0) return;

    // ------------------------------------------------------------------------------------------ producer warps
    if (warp >= kConsumerWarps) {
        const u32 g = warp - kConsumerWarps;
        u64* g_full = full + g * plan.stages;
        u64* g_empty = empty + g * plan.stages;
        u32* g_item = slot_item + g * plan.stages;
        unsigned char* g_stage = smem + u64(g) * plan.stages * plan.stage_bytes;
        const u32 e = lane / 3u, part = lane - 3u * e;  // lanes 0 .. 3 * ne - 1 copy one piece of one entry each
        const u32 in_stride = a.in.stride ? a.in.stride : a.in.width, in_gs = in_stride / 32;
        u32 t = 0;
        bool ok = true;
        for (;;) {
            u32 k = 0;
            if (lane == 0) k = atomicAdd(&ctl[1], 1u);
            k = __shfl_sync(0xffffffffu, k, 0);
            const bool end = k >= n_local;
            const u32 item = first_item + k;
            VExpert ve{0, 0, 0, 0};
            u32 chunk = 0;
            if (!end) {
                const u32 jv = item / plan.n_chunks;
                chunk = item - jv * plan.n_chunks;
                ve = table[jv];
            }
            u32 r = 0;
            if (e < ve.ne) r = __ldg((DOWN ? a.routes.slots : a.routes.rows) + ve.begin + e);
            const u32 nsegs = end ? 1u : plan.nseg;
            for (u32 s = 0; s < nsegs; ++s, ++t) {
                const u32 slot = t % plan.stages, use = t / plan.stages;
                if (use) ok = mbar_wait(&g_empty[slot], (use - 1u) & 1u, plan.wait_limit, abort_flag);  // the slot's previous use is done
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (g == 0 && t == plan.stall_stage) { ok = false; break; }  // test hook: stop feeding, raise nothing
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the consumers' reads precede the copies below
                if (end) {
                    if (lane == 0) { g_item[slot] = kEndItem; mbar_arrive(&g_full[slot]); }
                    continue;
                }
                const u32 nbk = min(plan.S, plan.nb - s * plan.S);
                unsigned char* dst = g_stage + u64(slot) * plan.stage_bytes;
                if (lane == 0) {
                    g_item[slot] = item;
                    mbar_expect_tx(&g_full[slot], plan.w_bytes + ve.ne * nbk * 320u);
                }
                __syncwarp();
                if (lane == 0) {
                    const u32 x = s * plan.S * (kQ4KBlock / 4);  // 32-bit elements: a multiple of 36, i.e. of 144 bytes
                    if (DOWN) {
                        tma_2d(dst, &tm0, x, ve.expert * a.rows_per_expert + kItemRows * chunk, &g_full[slot]);
                    } else {
                        const u32 y = ve.expert * a.rows_per_expert + 32u * chunk;
                        tma_2d(dst, &tm0, x, y, &g_full[slot]);
                        tma_2d(dst + 32u * plan.row_seg_bytes, &tm1, x, y, &g_full[slot]);
                    }
                }
                if (e < ve.ne) {
                    unsigned char* xd = dst + plan.w_bytes + e * plan.x_entry_bytes;
                    if (part == 0) bulk_g2s(xd, a.in.codes + u64(r) * in_stride + u64(s) * plan.S * 256u, nbk * 256u, &g_full[slot]);
                    else if (part == 1) bulk_g2s(xd + 256u * plan.S, a.in.deltas + u64(r) * in_gs + u64(s) * plan.S * 8u, nbk * 32u, &g_full[slot]);
                    else bulk_g2s(xd + 288u * plan.S, a.in.sums + u64(r) * in_gs + u64(s) * plan.S * 8u, nbk * 32u, &g_full[slot]);
                }
            }
            if (!ok || end) break;
        }
        if (!ok && lane == 0) {  // wait (bounded) for the copies still in flight before the CTA retires
            for (u32 n = t > plan.stages ? t - plan.stages : 0u; n < t; ++n)
                for (u32 i = 0; i < (plan.wait_limit >> 4) + 64u; ++i)
                    if (mbar_try_wait(&g_full[n % plan.stages], (n / plan.stages) & 1u)) break;
        }
        return;
    }

    // ------------------------------------------------------------------------------------------ consumer warps
    const u32 g = warp / kGroupWarps, w = warp % kGroupWarps;
    const u32 p = lane >> 3, rr = lane & 7u;
    u64* g_full = full + g * plan.stages;
    u64* g_empty = empty + g * plan.stages;
    const u32* g_item = slot_item + g * plan.stages;
    const unsigned char* g_stage = smem + u64(g) * plan.stages * plan.stage_bytes;
    const u32 act_stride = DOWN ? 0u : (a.act.stride ? a.act.stride : a.act.width);
    u32 t = 0, kl = 0;
    bool ok = true;
    for (;;) {
        u32 slot = t % plan.stages;
        ok = mbar_wait(&g_full[slot], (t / plan.stages) & 1u, plan.wait_limit, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const u32 item = g_item[slot];
        if (item == kEndItem) break;
        const u32 jv = item / plan.n_chunks, chunk = item - jv * plan.n_chunks;
        const VExpert ve = table[jv];
        const u32 n1 = min(ve.ne, 4u), n2 = ve.ne - n1;
        float acc[kKE];
#pragma unroll
        for (int r = 0; r < (int)kKE; ++r) acc[r] = 0.0f;
        for (u32 s = 0; s < plan.nseg; ++s, ++t) {
            if (s) {
                slot = t % plan.stages;
                ok = mbar_wait(&g_full[slot], (t / plan.stages) & 1u, plan.wait_limit, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            const unsigned char* st = g_stage + u64(slot) * plan.stage_bytes;
            const uint4* blk = reinterpret_cast<const uint4*>(st + (8u * w + rr) * plan.row_seg_bytes);
            const unsigned char* xs = st + plan.w_bytes;
            const u32 nbk = min(plan.S, plan.nb - s * plan.S);
            stage_rows_n(n1, blk, nbk, p, xs, plan.x_entry_bytes, plan.S, acc);
            if (n2) stage_rows_n(n2, blk, nbk, p, xs + 4u * plan.x_entry_bytes, plan.x_entry_bytes, plan.S, acc + 4);
            __syncwarp();
            if (lane == 0) mbar_arrive(&g_empty[slot]);  // the stage is free for the producer
        }
        if (!ok) break;
        if (DOWN) {
#pragma unroll
            for (int r = 0; r < (int)kKE; ++r) {
                if (r < (int)ve.ne) {
                    const float val = tree4(acc[r]);
                    if (p == 0) a.raw[u64(__ldg(a.routes.slots + ve.begin + r)) * a.out_width + kItemRows * chunk + 8u * w + rr] = val;
                }
            }
        } else {
            // the item's 2 x 32 outputs of every entry meet in shared memory; then one warp per entry runs the epilogue
            float* gu = s_gu + u64((g * 2 + (kl & 1u)) * 2) * kKE * 32;
            float* mine = gu + (w >> 2) * kKE * 32 + 8u * (w & 3u) + rr;
#pragma unroll
            for (int r = 0; r < (int)kKE; ++r) {
                if (r < (int)ve.ne) {
                    const float val = tree4(acc[r]);
                    if (p == 0) mine[r * 32] = val;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&gu_bar[g]);
            ok = mbar_wait(&gu_bar[g], kl & 1u, plan.wait_limit, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (w < ve.ne) {  // SwiGLU + the A8 rule over the 32 outputs of entry w
                const float gv = gu[w * 32 + lane], uv = gu[kKE * 32 + w * 32 + lane];
                const u32 slot_id = __ldg(a.routes.slots + ve.begin + w), o_col = 32u * chunk + lane;
                if (a.gate_out) { a.gate_out[u64(slot_id) * a.out_width + o_col] = gv; a.up_out[u64(slot_id) * a.out_width + o_col] = uv; }
                const float h = swiglu_qwen(gv, uv);
                const bool bad = __any_sync(0xffffffffu, !finite_f(gv) || !finite_f(uv) || !finite_f(h));
                if (bad) {  // fail closed: nothing of the group is written (routed_expert.cpp:147-156)
                    if (lane == 0) {
                        if (a.row_status) atomicOr(&a.row_status[__ldg(a.routes.rows + ve.begin + w)], B200MOE_ROW_PROJECTION_NONFINITE);
                        if (a.summary) atomicOr(a.summary, B200MOE_ROW_PROJECTION_NONFINITE);
                    }
                } else {
                    float delta;
                    int sum;
                    const int code = a8_quantize_lane(h, &delta, &sum);
                    a.act.codes[u64(slot_id) * act_stride + o_col] = static_cast<i8>(code);
                    if (lane == 0) {
                        a.act.deltas[u64(slot_id) * (act_stride / 32) + chunk] = delta;
                        if (a.act.sums) a.act.sums[u64(slot_id) * (act_stride / 32) + chunk] = sum;
                    }
                }
            }
        }
        ++kl;
    }
    if (!ok && lane == 0 && a.summary) atomicOr(a.summary, kAbortBit);
}

int sm_count() {
    int dev = 0, v = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v;
}

// Tensor map of a [rows][row_bytes] tensor seen as 32-bit elements, boxes of (36 * S elements = S super-blocks) x box_rows
// rows, no swizzle. The encoder is the driver's cuTensorMapEncodeTiled, looked up through the runtime (no link against
// the driver library). Encoded maps are kept per (device, tensor, geometry): encoding is host work of a few microseconds
// that a decode step would otherwise pay on every call.
int rows_map(const u8* base, u64 row_bytes, u64 rows, u32 S, u32 box_rows, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    if (!fn) return fail(B200MOE_ERR_CUDA, "wide form: cuTensorMapEncodeTiled is not available from this driver");
    static std::mutex m;
    static std::map<std::tuple<int, const u8*, u64, u64, u32, u32>, CUtensorMap> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    const auto key = std::make_tuple(dev, base, row_bytes, rows, S, box_rows);
    std::lock_guard<std::mutex> lock(m);
    const auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return B200MOE_OK; }
    const cuuint64_t dims[2] = {row_bytes / 4, rows};
    const cuuint64_t strides[1] = {row_bytes};  // bytes between rows: a multiple of 16 (144 per super-block)
    const cuuint32_t box[2] = {S * (kQ4KBlock / 4), box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<u8*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200MOE_ERR_CUDA, "wide form: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    if (cache.size() >= 1024) cache.clear();
    cache.emplace(key, *out);
    return B200MOE_OK;
}

u32 round_up(u32 v, u32 a) { return (v + a - 1) / a * a; }

u32 fixed_smem(const WidePlan& p, bool down) {
    return (down ? 0u : kGroups * 2 * 2 * kKE * 32 * 4) + p.vmax * static_cast<u32>(sizeof(VExpert)) + (2 * kGroups * p.stages + kGroups) * 8 +
           kGroups * p.stages * 4 + 64;
}
u32 plan_smem(const WidePlan& p, bool down) { return kGroups * p.stages * p.stage_bytes + fixed_smem(p, down); }

// K: the row length; n_chunks: items per expert; slots: rows * top_k of the window. False when the form does not apply.
bool make_plan(u32 K, u32 n_chunks, u32 max_union, u64 slots, bool down, WidePlan* p) {
    if (K == 0 || K % 256 || max_union == 0 || slots == 0 || slots > 8192) return false;
    p->nb = K / 256;
    p->S = p->nb >= 3 ? 3u : 1u;  // odd: rows S * 144 bytes apart stay conflict free
    p->nseg = (p->nb + p->S - 1) / p->S;
    p->row_seg_bytes = p->S * kQ4KBlock;
    p->w_bytes = kItemRows * p->row_seg_bytes;
    p->x_entry_bytes = p->S * 320u;
    p->stage_bytes = round_up(p->w_bytes + kKE * p->x_entry_bytes, 128);
    p->n_chunks = n_chunks;
    p->max_union = max_union;
    p->vmax = max_union + static_cast<u32>(slots / kKE) + 1;
    if (u64(p->vmax) * n_chunks >= (1ull << 31)) return false;
    for (p->stages = 4; p->stages >= 2; --p->stages)
        if (plan_smem(*p, down) <= kSmemBudget) break;
    if (p->stages < 2) return false;
    if ((2 * max_union + 2) * 4 > kGroups * p->stages * p->stage_bytes) return false;  // the copied routes borrow the stage area
    p->wait_limit = kDefaultWaitLimit;
    p->stall_stage = 0xffffffffu;
    return true;
}

// The entries' A8 rows are moved by bulk copies: 16-byte aligned sources at every (row, stage) offset.
bool a8_bulk_ok(const b200moe_a8_rows& x) {
    const u32 stride = x.stride ? x.stride : x.width;
    return x.sums && aligned(x.codes, 16) && aligned(x.deltas, 16) && aligned(x.sums, 16) && stride % 128 == 0;
}

void apply_hooks(WidePlan* p) {
    const u32 limit = debug_value(B200MOE_DEBUG_WAIT_LIMIT), stall = debug_value(B200MOE_DEBUG_STALL_STAGE);
    if (limit) p->wait_limit = limit;
    if (stall) p->stall_stage = stall - 1u;
}

}  // namespace

bool wide_gate_up_fits(const b200moe_gate_up_view& v, u32 rows) {
    WidePlan p{};
    return v.shape.gate_type == B200MOE_TYPE_Q4_K && rows && a8_bulk_ok(v.x) && v.shape.inter % 32 == 0 &&
           make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p);
}
bool wide_down_fits(const b200moe_down_view& v, u32 rows) {
    WidePlan p{};
    return v.shape.down_type == B200MOE_TYPE_Q4_K && rows && a8_bulk_ok(v.act) && v.shape.hidden % 64 == 0 &&
           make_plan(v.shape.inter, v.shape.hidden / 64, v.max_union, u64(rows) * v.shape.top_k, true, &p);
}

int launch_gate_up_q4k_wide(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    WidePlan p{};
    if (!make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "gate_up: the segment-streaming form does not apply to this shape");
    apply_hooks(&p);
    WideArgs a{};
    a.routes = v.routes; a.in = v.x; a.act = v.act; a.gate_out = v.gate_out; a.up_out = v.up_out;
    a.row_status = v.row_status; a.summary = v.summary; a.rows_per_expert = v.shape.inter; a.out_width = v.shape.inter;
    CUtensorMap tm0, tm1;
    const u64 rb = u64(p.nb) * kQ4KBlock, total_rows = u64(v.shape.experts) * v.shape.inter;
    if (int rc = rows_map(v.weights.gate, rb, total_rows, p.S, 32, &tm0)) return rc;
    if (int rc = rows_map(v.weights.up, rb, total_rows, p.S, 32, &tm1)) return rc;
    const u32 smem = plan_smem(p, false);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<false>), smem)) return rc;
    q4k_wide_kernel<false><<<sm_count(), kThreads, smem, stream>>>(tm0, tm1, a, p);
    return after_launch("gate_up_q4k_wide");
}

int launch_down_q4k_wide(const b200moe_down_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    WidePlan p{};
    if (!make_plan(v.shape.inter, v.shape.hidden / 64, v.max_union, u64(rows) * v.shape.top_k, true, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "down: the segment-streaming form does not apply to this shape");
    apply_hooks(&p);
    WideArgs a{};
    a.routes = v.routes; a.in = v.act; a.raw = v.raw; a.summary = const_cast<u32*>(v.summary);
    a.rows_per_expert = v.shape.hidden; a.out_width = v.shape.hidden;
    CUtensorMap tm0;
    if (int rc = rows_map(v.weights.down, u64(p.nb) * kQ4KBlock, u64(v.shape.experts) * v.shape.hidden, p.S, 64, &tm0)) return rc;
    const u32 smem = plan_smem(p, true);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<true>), smem)) return rc;
    q4k_wide_kernel<true><<<sm_count(), kThreads, smem, stream>>>(tm0, tm0, a, p);
    return after_launch("down_q4k_wide");
}

}  // namespace b200moe
