// Routed experts, Qwen A8 family, decode form for ANY row length: a persistent kernel that streams SEGMENTS of the
// weight rows - and of the activations they meet - through shared memory with the TMA engine.
//
// Same arithmetic as gemv_q4k.cu (the contract of src/cpu/core/routed_expert.hpp:9-15, bit for bit). What this form adds
// over gemv_q4k_stream.cu is that nothing is sized by the row length or by the window: hidden 7168 (4032-byte gate rows),
// inter 17408 (9792-byte down rows) and 64-row windows stream exactly like the small layers.
//
//  * Work item = (virtual expert, 64 weight rows): 32 gate + 32 up rows of one output group, or 64 down rows. A virtual
//    expert is an expert of the window's union with at most kKE = 8 of its entries; an expert with more entries appears
//    several times (its rows are then streamed again, out of L2). Every CTA builds the same virtual list in shared memory
//    from the routes, ordered by entry count (longest items first); the items are dealt out over the whole grid through a
//    claim word in device memory (wide_common.cuh).
//  * A stage = S = 3 super-blocks of the item's 64 rows (one or two tiled TMA copies of 432 bytes x 32 / 64 rows: the rows
//    lie 432 bytes apart in shared memory, an odd count of 16-byte units, which keeps the 128-bit reads of eight rows
//    conflict free) PLUS the same K range of the A8 rows of the item's entries (codes, deltas, sums: three bulk copies per
//    entry), all counted on one mbarrier. The consumers therefore find everything a stage needs in shared memory.
//  * Two groups of eight consumer warps share a CTA, each with its own ring of stages and its own producer warp; a group's
//    producer claims the next item of the grid while its consumers still work on the stages in the ring. Lane =
//    (pair p, row): a lane walks its row's super-blocks in ascending order across the item's stages, the serial chains
//    acc_p += pair_p never leave their lane, and (a0 + a1) + (a2 + a3) is two xor-shuffles at the end of the item.
//  * gate/up: the group meets on an mbarrier once per item and eight warps run SwiGLU + the A8 rule of one entry each.
//  * Two forms of the integer dots, chosen per item by its entry count. Up to kMmaMinEntries - 1 entries: dp4a, lane =
//    (pair, row), 16 dp4a per (super-block, pair, entry). From kMmaMinEntries entries: the warp's 8 rows x up to 8 entries
//    x 32 weights of a group are ONE mma.sync.m16n8k32 (A = the entries' codes, signed; B = the rows' nibbles as unsigned
//    bytes, high nibbles left in place as 16 q; the k order inside a group is permuted the same way on both sides, which
//    an exact integer sum does not see). The accumulator fragment gives lane (entry, t) the dots of rows 2t and 2t + 1,
//    and the lane runs the same FP32 operation sequence on them with the rows' factors fetched from a per-warp scratch:
//    the kernel is bound by issue slots (ncu: three quarters of them busy at config 4), and this form needs about half
//    the instructions of the dp4a form at 8 entries; from 3 or 4 entries on it was measured slower than dp4a. Both forms produce the contract's bits.
//
// Every wait is bounded (plan.wait_limit polls): a waiter that runs out raises the CTA's abort flag, every role leaves
// its loops, the producers wait (bounded) for the copies they still have in flight, B200MOE_JOB_WAIT_ABORTED is set in the
// job summary and the kernel returns - the host reads a status, the GPU never hangs.
//
// Roofline: HBM. Algorithmic bytes per item = 64 rows x K / 256 x 144 (+ the entries' A8 bytes).
#include <algorithm>
#include <type_traits>

#include "wide_common.cuh"

namespace b200moe {

namespace {
using namespace q4k;
using namespace wide;

constexpr u32 kItemRows = 64;
constexpr u32 kMmaMinEntries = 5;                       // items with at least this many entries take the mma form
constexpr u32 kFacFloats = 128;                         // per-warp scratch of the mma form: [D, DM, D', DM'][pair][row]

struct WidePlan {
    u32 S;              // super-blocks per stage
    u32 nb;             // super-blocks per row
    u32 nseg;           // stages per item
    u32 stages;         // ring depth per group
    u32 row_seg_bytes;  // S * 144
    u32 w_bytes;        // 64 * row_seg_bytes
    u32 x_entry_bytes;  // >= S * 320: codes, deltas, sums of one entry over the stage's K range (+ padding)
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

// Stage geometry for S super-blocks per stage, as compile-time constants: the kernels are bound by issue slots, and
// address arithmetic on run-time strides was a measurable part of them.
constexpr u32 x_entry_bytes_of(u32 S) {  // codes, deltas, sums of one entry over a stage, padded so that entries lie 8 or 24
    u32 b = S * 320u;                     // (mod 32) words apart: the mma form reads 8 bytes per lane at (entry, k slice) and
    while ((b / 4) % 32 != 8 && (b / 4) % 32 != 24) b += 16;  // four entries then cover all banks once
    return b;
}
template <u32 S_>
struct Geo {
    static constexpr u32 S = S_;
    static constexpr u32 row_seg_bytes = S * kQ4KBlock;
    static constexpr u32 w_bytes = kItemRows * row_seg_bytes;
    static constexpr u32 x_entry_bytes = x_entry_bytes_of(S);
};

// (a0 + a1) + (a2 + a3) over the four pair lanes of a row (lane = 8 * p + row); every lane of the row gets the value.
__device__ __forceinline__ float tree4(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 8));
    return __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 16));
}

// One stage of one weight row (this lane's pair p of nbk super-blocks, ascending) against NR staged A8 rows. blk: the
// row's first super-block of the stage; xs: entry 0's area of the stage ({codes[S * 256], deltas[S * 8], sums[S * 8]},
// the next entry x_entry_bytes further). acc[r] is the lane's chain acc_p of entry r.
template <int NR, class G>
__device__ __forceinline__ void stage_rows(const uint4* blk, u32 nbk, u32 p, const unsigned char* xs, float* acc) {
    constexpr u32 x_entry_bytes = G::x_entry_bytes, S = G::S;
#pragma unroll
    for (u32 b = 0; b < S; ++b, blk += kQ4KBlock / 16) {
        if (b >= nbk) break;
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
// ---- the mma form of one stage ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_s8u8(int& c0, int& c1, u32 a0, u32 a2, u32 b0, u32 b1) {
    // D (16 x 8, s32) = A (16 x 32, s8, row) * B (32 x 8, u8, col); rows 8 .. 15 of A are zero (at most 8 entries).
    int c2, c3;
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
                 : "r"(a0), "r"(0), "r"(a2), "r"(0), "r"(b0), "r"(b1), "r"(0));
}
// x_2p + x_2p+1 of one (row, entry, super-block, pair) from the two exact group dots; hi16 = 16 * dot of the odd group.
__device__ __forceinline__ float pair_from_dots(float Dl, float DMl, float Dh, float DMh, int lo, int hi16, float El, float Eh, float Sl, float Sh) {
    const float xl = __fmul_rn(El, __fsub_rn(__fmul_rn(Dl, static_cast<float>(lo)), __fmul_rn(DMl, Sl)));
    const float xh = __fmul_rn(Eh, __fsub_rn(__fmul_rn(Dh, static_cast<float>(hi16 >> 4)), __fmul_rn(DMh, Sh)));
    return __fadd_rn(xl, xh);
}
// One stage of the warp's 8 weight rows against up to 8 staged A8 rows with tensor-core dots. w8: the warp's first row of
// the stage (rows row_seg_bytes apart); fac: the warp's scratch. Lane = (e = lane >> 2, t = lane & 3): acc[4 * i + p] is the
// chain acc_p of (row 2t + i, entry e). Lanes of absent entries compute on stale shared memory and are never stored.
template <class G>
__device__ __forceinline__ void stage_rows_mma(const unsigned char* w8, u32 nbk, u32 lane, const unsigned char* xs, float* fac, float* acc) {
    constexpr u32 row_seg_bytes = G::row_seg_bytes, x_entry_bytes = G::x_entry_bytes, S = G::S;
    const u32 p = lane >> 3, rr = lane & 7u;   // factor decode: lane = (pair, row), as in the dp4a form
    const u32 e = lane >> 2, t = lane & 3u;    // mma fragments: lane = (entry or weight row, k slice)
    const unsigned char* xe = xs + e * x_entry_bytes;
    const unsigned char* wdec = w8 + rr * row_seg_bytes;
    const unsigned char* wfrag = w8 + e * row_seg_bytes + 16u + 8u * t;   // B fragment: weight row n = lane >> 2
#pragma unroll 1
    for (u32 b = 0; b < nbk; ++b) {  // rolled: the body is long, and the form runs where the instruction cache matters
        const uint4 hdr = *reinterpret_cast<const uint4*>(wdec + kQ4KBlock * b);
        const Factors f = q4k_factors(hdr, p);
        __syncwarp();   // the previous block's readers are done with the scratch
        fac[(0 * 4 + p) * 8 + rr] = f.Dl; fac[(1 * 4 + p) * 8 + rr] = f.DMl; fac[(2 * 4 + p) * 8 + rr] = f.Dh; fac[(3 * 4 + p) * 8 + rr] = f.DMh;  // bank = lane
        __syncwarp();
        const float4 e0 = *reinterpret_cast<const float4*>(xe + 256u * S + 32u * b), e1 = *reinterpret_cast<const float4*>(xe + 256u * S + 32u * b + 16u);
        const int4 s0 = *reinterpret_cast<const int4*>(xe + 288u * S + 32u * b), s1 = *reinterpret_cast<const int4*>(xe + 288u * S + 32u * b + 16u);
        const float E[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
        const int Sg[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
            const uint2 w = *reinterpret_cast<const uint2*>(wfrag + kQ4KBlock * b + 32u * pp);   // 8 bytes = 16 nibbles: k slice t of groups 2pp, 2pp + 1
            const uint2 al = *reinterpret_cast<const uint2*>(xe + 256u * b + 64u * pp + 8u * t);          // the entry's codes, group 2pp, same k slice
            const uint2 ah = *reinterpret_cast<const uint2*>(xe + 256u * b + 64u * pp + 32u + 8u * t);    // group 2pp + 1
            int l0, l1, h0, h1;
            mma_s8u8(l0, l1, al.x, al.y, w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu);
            mma_s8u8(h0, h1, ah.x, ah.y, w.x & 0xf0f0f0f0u, w.y & 0xf0f0f0f0u);
            const float El = E[2 * pp], Eh = E[2 * pp + 1];
            const float Sl = small_int_to_float(Sg[2 * pp]), Sh = small_int_to_float(Sg[2 * pp + 1]);
            const float2 Dl = *reinterpret_cast<const float2*>(fac + (0 * 4 + pp) * 8 + 2 * t), DMl = *reinterpret_cast<const float2*>(fac + (1 * 4 + pp) * 8 + 2 * t);
            const float2 Dh = *reinterpret_cast<const float2*>(fac + (2 * 4 + pp) * 8 + 2 * t), DMh = *reinterpret_cast<const float2*>(fac + (3 * 4 + pp) * 8 + 2 * t);
            acc[pp] = __fadd_rn(acc[pp], pair_from_dots(Dl.x, DMl.x, Dh.x, DMh.x, l0, h0, El, Eh, Sl, Sh));
            acc[4 + pp] = __fadd_rn(acc[4 + pp], pair_from_dots(Dl.y, DMl.y, Dh.y, DMh.y, l1, h1, El, Eh, Sl, Sh));
        }
    }
}

// 18 warps: two of the SM's four register partitions (16 K registers each) hold five warps, which caps a thread at
// 16384 / (5 x 32) = 102 registers, 96 after rounding - what this launch bound gives (112 was tried: the launch is refused).
template <bool DOWN, u32 S_>
__global__ void __launch_bounds__(kThreads, 1)
q4k_wide_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, WideArgs a, WidePlan plan) {
    using G = Geo<S_>;
    extern __shared__ __align__(128) unsigned char smem[];
    if (DOWN && a.summary && *a.summary) return;  // a failed or aborted projection skips the whole stage (routed_expert.hpp:17-19)
    u32 n_union = a.routes.counts[0];
    if (n_union == 0) return;
    if (n_union > plan.max_union) n_union = plan.max_union;
    u32* claim = a.routes.counts + 3;  // the grid's claim word (wide_common.cuh)

    unsigned char* at = smem + kGroups * plan.stages * plan.stage_bytes;
    float* s_gu = reinterpret_cast<float*>(at);  // [group][buffer][gate | up][entry][32]
    if (!DOWN) at += kGroups * 2 * 2 * kKE * 32 * 4;
    VExpert* table = reinterpret_cast<VExpert*>(at);
    at += (u64(plan.vmax) * sizeof(VExpert) + 15) & ~u64(15);  // what follows holds 8- and 16-byte objects
    float* s_fac = reinterpret_cast<float*>(at);  // [consumer warp][kFacFloats]
    at += kConsumerWarps * kFacFloats * 4;
    u64* full = reinterpret_cast<u64*>(at);
    u64* empty = full + kGroups * plan.stages;
    u64* gu_bar = empty + kGroups * plan.stages;
    at += (2 * kGroups * plan.stages + kGroups) * 8;
    u32* slot_item = reinterpret_cast<u32*>(at);
    at += kGroups * plan.stages * 4;
    u32* ctl = reinterpret_cast<u32*>(at);  // [0] abort flag, [1] producers that have retired, [2] virtual experts, [3] items
    volatile u32* abort_flag = ctl;

    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid < kGroups * plan.stages) { mbar_init(&full[tid], 1); mbar_init(&empty[tid], kGroupWarps); }
    if (tid < kGroups) mbar_init(&gu_bar[tid], kGroupWarps);
    if (tid < 4) ctl[tid] = 0;
    if (tid < kGroups * plan.stages + kGroups) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");

    // ---- the virtual expert list (the stage area is free until the first copy is issued: it holds the copied routes)
    build_work_list(a.routes, n_union, plan.max_union, plan.vmax, plan.n_chunks, reinterpret_cast<u32*>(smem), table, ctl);
    const u32 n_items = ctl[3];
    if (n_items == 0) return;  // every CTA alike: nobody claims, the claim word stays zero

    // ------------------------------------------------------------------------------------------ producer warps
    if (warp >= kConsumerWarps) {
        const u32 g = warp - kConsumerWarps;
        u64* g_full = full + g * plan.stages;
        u64* g_empty = empty + g * plan.stages;
        u32* g_item = slot_item + g * plan.stages;
        unsigned char* g_stage = smem + g * plan.stages * plan.stage_bytes;
        const u32 e = lane / 3u, part = lane - 3u * e;  // lanes 0 .. 3 * ne - 1 copy one piece of one entry each
        const u32 in_stride = a.in.stride ? a.in.stride : a.in.width, in_gs = in_stride / 32;
        u32 t = 0, slot = 0, use = 0;  // stage count, ring position, lap
        bool ok = true, first = true;
        for (;;) {
            // A group's first item needs no round trip: group 0 of CTA b takes item b, group 1 item gridDim.x + b - so a
            // launch with fewer items than groups runs one group per SM, which has the SM's issue slots to itself.
            u32 k = g * gridDim.x + blockIdx.x;
            if (!first) {
                if (lane == 0) k = gridDim.x * kGroups + claim_item(claim);
                k = __shfl_sync(0xffffffffu, k, 0);
            }
            first = false;
            const bool end = k >= n_items;
            const u32 item = k;
            VExpert ve{0};
            u32 chunk = 0;
            if (!end) {
                const u32 jv = item / plan.n_chunks;
                chunk = item - jv * plan.n_chunks;
                ve = table[jv];
            }
            const u32 ve_ne = ve.ne();
            u32 r = 0;
            if (e < ve_ne) r = __ldg((DOWN ? a.routes.slots : a.routes.rows) + ve.begin() + e);
            const u32 nsegs = end ? 1u : plan.nseg;
            for (u32 s = 0; s < nsegs; ++s, ++t, ++slot) {
                if (slot == plan.stages) { slot = 0; ++use; }
                if (use) ok = mbar_wait(&g_empty[slot], (use - 1u) & 1u, plan.wait_limit, abort_flag);  // the slot's previous use is done
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (g == 0 && t == plan.stall_stage) { ok = false; break; }  // test hook: stop feeding, raise nothing
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the consumers' reads precede the copies below
                if (end) {
                    if (lane == 0) { g_item[slot] = kEndItem; mbar_arrive(&g_full[slot]); }
                    continue;
                }
                const u32 nbk = min(G::S, plan.nb - s * G::S);
                unsigned char* dst = g_stage + slot * plan.stage_bytes;
                if (lane == 0) {
                    g_item[slot] = item;
                    mbar_expect_tx(&g_full[slot], G::w_bytes + ve_ne * nbk * 320u);
                }
                __syncwarp();
                if (lane == 0) {
                    const u32 x = s * G::S * (kQ4KBlock / 8);  // 64-bit elements: a multiple of 18, i.e. of 144 bytes
                    if (DOWN) {
                        tma_2d(dst, &tm0, x, ve.expert() * a.rows_per_expert + kItemRows * chunk, &g_full[slot]);
                    } else {
                        const u32 y = ve.expert() * a.rows_per_expert + 32u * chunk;
                        tma_2d(dst, &tm0, x, y, &g_full[slot]);
                        tma_2d(dst + 32u * G::row_seg_bytes, &tm1, x, y, &g_full[slot]);
                    }
                }
                if (e < ve_ne) {
                    unsigned char* xd = dst + G::w_bytes + e * G::x_entry_bytes;
                    if (part == 0) bulk_g2s(xd, a.in.codes + u64(r) * in_stride + u64(s) * G::S * 256u, nbk * 256u, &g_full[slot]);
                    else if (part == 1) bulk_g2s(xd + 256u * G::S, a.in.deltas + u64(r) * in_gs + u64(s) * G::S * 8u, nbk * 32u, &g_full[slot]);
                    else bulk_g2s(xd + 288u * G::S, a.in.sums + u64(r) * in_gs + u64(s) * G::S * 8u, nbk * 32u, &g_full[slot]);
                }
            }
            if (!ok || end) break;
        }
        if (!ok && lane == 0) {  // wait (bounded) for the copies still in flight before the CTA retires
            for (u32 n = t > plan.stages ? t - plan.stages : 0u; n < t; ++n)
                for (u32 i = 0; i < (plan.wait_limit >> 4) + 64u; ++i)
                    if (mbar_try_wait(&g_full[n % plan.stages], (n / plan.stages) & 1u)) break;
        }
        if (lane == 0) retire_claims(claim, ctl);
        return;
    }

    // ------------------------------------------------------------------------------------------ consumer warps
    const u32 g = warp / kGroupWarps, w = warp % kGroupWarps;
    const u32 p = lane >> 3, rr = lane & 7u;
    float* fac = s_fac + warp * kFacFloats;
    u64* g_full = full + g * plan.stages;
    u64* g_empty = empty + g * plan.stages;
    const u32* g_item = slot_item + g * plan.stages;
    const unsigned char* g_stage = smem + g * plan.stages * plan.stage_bytes;
    const u32 act_stride = DOWN ? 0u : (a.act.stride ? a.act.stride : a.act.width);
    u32 slot = 0, phase = 0, kl = 0;  // ring position of the group's next stage, kept incrementally (no divisions in the loop)
    bool ok = true;
    for (;;) {
        ok = mbar_wait(&g_full[slot], phase, plan.wait_limit, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const u32 item = g_item[slot];
        if (item == kEndItem) break;
        const u32 jv = item / plan.n_chunks, chunk = item - jv * plan.n_chunks;
        const VExpert ve = table[jv];
        const u32 ne = ve.ne(), vbegin = ve.begin();
        const bool mma = ne >= kMmaMinEntries;
        float acc[kKE];
#pragma unroll
        for (int r = 0; r < (int)kKE; ++r) acc[r] = 0.0f;
        // the item's stages, with the form and the entry count fixed at compile time inside the loop (NR = 0: the mma form)
        auto run = [&](auto tag) {
            constexpr int NR = decltype(tag)::value;
            for (u32 s = 0; s < plan.nseg; ++s) {
                if (s) {
                    ok = mbar_wait(&g_full[slot], phase, plan.wait_limit, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) return;
                }
                const unsigned char* st = g_stage + slot * plan.stage_bytes;
                const u32 nbk = min(G::S, plan.nb - s * G::S);
                if constexpr (NR == 0) stage_rows_mma<G>(st + 8u * w * G::row_seg_bytes, nbk, lane, st + G::w_bytes, fac, acc);
                else stage_rows<NR, G>(reinterpret_cast<const uint4*>(st + (8u * w + rr) * G::row_seg_bytes), nbk, p, st + G::w_bytes, acc);
                __syncwarp();
                if (lane == 0) mbar_arrive(&g_empty[slot]);  // the stage is free for the producer
                if (++slot == plan.stages) { slot = 0; phase ^= 1u; }
            }
        };
        switch (mma ? 0u : ne) {
            case 0: run(std::integral_constant<int, 0>{}); break;
            case 1: run(std::integral_constant<int, 1>{}); break;
            case 2: run(std::integral_constant<int, 2>{}); break;
            case 3: run(std::integral_constant<int, 3>{}); break;
            default: run(std::integral_constant<int, 4>{}); break;
        }
        if (!ok) break;
        // mma form: lane (e = lane >> 2, t = lane & 3) holds the four chains of rows 2t and 2t + 1 of entry e
        const float m0 = __fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3]));
        const float m1 = __fadd_rn(__fadd_rn(acc[4], acc[5]), __fadd_rn(acc[6], acc[7]));
        const u32 me = lane >> 2, mt = lane & 3u;
        if (DOWN) {
            if (mma) {
                if (me < ne) {
                    float* dst = a.raw + u64(__ldg(a.routes.slots + vbegin + me)) * a.out_width + kItemRows * chunk + 8u * w + 2u * mt;
                    *reinterpret_cast<float2*>(dst) = make_float2(m0, m1);
                }
            } else {
#pragma unroll
                for (int r = 0; r < (int)kMmaMinEntries - 1; ++r) {
                    if (r < (int)ne) {
                        const float val = tree4(acc[r]);
                        if (p == 0) a.raw[u64(__ldg(a.routes.slots + vbegin + r)) * a.out_width + kItemRows * chunk + 8u * w + rr] = val;
                    }
                }
            }
        } else {
            // the item's 2 x 32 outputs of every entry meet in shared memory; then one warp per entry runs the epilogue
            float* gu = s_gu + u64((g * 2 + (kl & 1u)) * 2) * kKE * 32;
            if (mma) {
                if (me < ne) *reinterpret_cast<float2*>(gu + (w >> 2) * kKE * 32 + me * 32 + 8u * (w & 3u) + 2u * mt) = make_float2(m0, m1);
            } else {
                float* mine = gu + (w >> 2) * kKE * 32 + 8u * (w & 3u) + rr;
#pragma unroll
                for (int r = 0; r < (int)kMmaMinEntries - 1; ++r) {
                    if (r < (int)ne) {
                        const float val = tree4(acc[r]);
                        if (p == 0) mine[r * 32] = val;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&gu_bar[g]);
            ok = mbar_wait(&gu_bar[g], kl & 1u, plan.wait_limit, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (w < ne) {  // SwiGLU + the A8 rule over the 32 outputs of entry w
                const float gv = gu[w * 32 + lane], uv = gu[kKE * 32 + w * 32 + lane];
                const u32 slot_id = __ldg(a.routes.slots + vbegin + w), o_col = 32u * chunk + lane;
                if (a.gate_out) { a.gate_out[u64(slot_id) * a.out_width + o_col] = gv; a.up_out[u64(slot_id) * a.out_width + o_col] = uv; }
                const float h = swiglu_qwen(gv, uv);
                const bool bad = __any_sync(0xffffffffu, !finite_f(gv) || !finite_f(uv) || !finite_f(h));
                if (bad) {  // fail closed: nothing of the group is written (routed_expert.cpp:147-156)
                    if (lane == 0) {
                        if (a.row_status) atomicOr(&a.row_status[__ldg(a.routes.rows + vbegin + w)], B200MOE_ROW_PROJECTION_NONFINITE);
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

u32 round_up(u32 v, u32 a) { return (v + a - 1) / a * a; }

u32 fixed_smem(const WidePlan& p, bool down) {
    return (down ? 0u : kGroups * 2 * 2 * kKE * 32 * 4) + round_up(p.vmax * static_cast<u32>(sizeof(VExpert)), 16) + kConsumerWarps * kFacFloats * 4 +
           (2 * kGroups * p.stages + kGroups) * 8 + kGroups * p.stages * 4 + 64;
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
    p->x_entry_bytes = x_entry_bytes_of(p->S);
    // a stage holds the A8 segments of as many entries as a virtual expert of this window can have: windows of fewer than
    // kKE slots get smaller stages and with them a deeper ring
    p->stage_bytes = round_up(p->w_bytes + static_cast<u32>(std::min<u64>(kKE, slots)) * p->x_entry_bytes, 128);
    p->n_chunks = n_chunks;
    p->max_union = max_union;
    p->vmax = max_union + static_cast<u32>(slots / kKE) + 1;
    if (u64(p->vmax) * n_chunks + 4096 >= kClaimMask) return false;  // items and the groups' closing claims fit the claim word's count
    for (p->stages = 5; p->stages >= 2; --p->stages)
        if (plan_smem(*p, down) <= kSmemBudget) break;
    if (p->stages < 2) return false;
    if (work_list_scratch_words(max_union, p->vmax) * 4 > kGroups * p->stages * p->stage_bytes) return false;  // the work list is built in the stage area
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
    if (int rc = rows_map(v.weights.gate, rb, total_rows, p.S * kQ4KBlock, 32, &tm0)) return rc;
    if (int rc = rows_map(v.weights.up, rb, total_rows, p.S * kQ4KBlock, 32, &tm1)) return rc;
    const u32 smem = plan_smem(p, false);
    if (p.S == 3) {
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<false, 3>), smem)) return rc;
        q4k_wide_kernel<false, 3><<<sm_count(), kThreads, smem, stream>>>(tm0, tm1, a, p);
    } else {
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<false, 1>), smem)) return rc;
        q4k_wide_kernel<false, 1><<<sm_count(), kThreads, smem, stream>>>(tm0, tm1, a, p);
    }
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
    if (int rc = rows_map(v.weights.down, u64(p.nb) * kQ4KBlock, u64(v.shape.experts) * v.shape.hidden, p.S * kQ4KBlock, 64, &tm0)) return rc;
    const u32 smem = plan_smem(p, true);
    if (p.S == 3) {
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<true, 3>), smem)) return rc;
        q4k_wide_kernel<true, 3><<<sm_count(), kThreads, smem, stream>>>(tm0, tm0, a, p);
    } else {
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q4k_wide_kernel<true, 1>), smem)) return rc;
        q4k_wide_kernel<true, 1><<<sm_count(), kThreads, smem, stream>>>(tm0, tm0, a, p);
    }
    return after_launch("down_q4k_wide");
}

}  // namespace b200moe
