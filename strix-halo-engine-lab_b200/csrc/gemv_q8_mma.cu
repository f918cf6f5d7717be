// Q8_0 x A8 experts over windows of 8 rows and more, integer dots on the tensor cores: the lane-class contract of
// src/ds41_formats.cpp:188-197 (product_q8_0) with one mma.sync.m16n8k32 (s8 x s8 -> s32) per (16 weight rows, 8 entries,
// block) instead of 16 x 8 dp4a chains of eight.
//
// The contract adds the terms float(dot_g) * (scale_g * delta_g) of a row into 32 lane classes (group g -> class g % 32) in
// ascending g, then folds the classes with the butterfly v[l] += v[l ^ d], d = 16 .. 1. A class is an independent chain, so
// the CLASSES are what the warps of a CTA share out: consumer warp w owns classes 2w and 2w + 1 of all 16 rows x 8 entries
// of a tile, i.e. blocks 2w and 2w + 1 of every run of 32 blocks, and walks the runs in ascending order - eight FP32
// accumulators per lane, each product and each add the contract's own, in its order. When the tile's last run is done the
// 16 x 8 x 32 class sums meet in shared memory and warp w runs the butterfly of row w (lane = class), bit for bit.
//
//  * Item = (virtual expert of at most 8 entries, 32 outputs); tiles of 16 weight rows: gate rows, gate rows + 16, up rows,
//    up rows + 16 (gate/up) or the two halves of 32 down rows. A CTA takes a contiguous range of items (items of a dense
//    block cost the same), so consecutive items mostly share their entries, whose A8 rows stay in shared memory.
//  * A stage = 16 rows x up to 4 runs, one tiled TMA copy per run (box 138 x 64-bit = 1104 bytes per row: the run's 1088
//    bytes and 16 more, which puts consecutive rows 20 words apart - the eight rows and four k slices of an A fragment load
//    then fall into 32 different banks). Two stages in flight. The entries' codes lie 4 (mod 32) words apart for the same reason.
//  * Q8_0 blocks are 34 bytes: the quants of an even block of a run start 2 (mod 4) bytes in (two words and a byte permute
//    per fragment register), those of an odd block on a word. Which is which is fixed per warp at compile time.
//  * gate/up: after the fourth tile eight warps run swiglu_clamped (declared_exp) + the A8 rule of one entry each
//    (src/ds41_moe.cpp:134-146).
// Waits on mbarriers are bounded (B200MOE_JOB_WAIT_ABORTED); the consumer warps also meet at a hardware barrier, so they
// leave the item loop together, on a decision one thread publishes between two barriers.
#include <algorithm>

#include "wide_common.cuh"

namespace b200moe {
namespace {
using namespace q4k;   // the mbarrier / copy wrappers
using namespace wide;

constexpr u32 kTileRows = 16;
constexpr u32 kRunBlocks = 32, kRunBytes = kRunBlocks * kQ8Block;  // 1088
constexpr u32 kRowPitch = kRunBytes + 16;                          // bytes between the rows of a run in shared memory
constexpr u32 kRunBox = kTileRows * kRowPitch;                     // 17,664
constexpr u32 kStageRuns = 4, kStageBytes = kStageRuns * kRunBox, kStages = 2;
constexpr u32 kMmaWarps = 16;                                      // consumer warps; one producer warp after them
constexpr u32 kMmaThreads = (kMmaWarps + 1) * 32;
constexpr u32 kClsFloats = kTileRows * kKE * 32;                   // class sums of a tile
constexpr u32 kGuFloats = 2 * 2 * kKE * 32;                        // [item parity][gate | up][entry][32]
constexpr u32 kMaxK = 7168;                                        // the entries' A8 rows of a whole item stay in shared memory

struct MmaPlan {
    u32 K, groups, nruns, nst;  // nst: stages per tile
    u32 xc_pitch, xd_pitch;     // bytes between the entries' codes / deltas in shared memory
    u32 n_chunks, max_union, vmax, wait_limit;
};

struct MmaArgs {
    b200moe_routes routes;
    b200moe_a8_rows in, act;
    float* gate_out;
    float* up_out;
    float* raw;
    u32* summary;
    u32 rows_per_expert, out_width;
    float limit;
};

__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kMmaWarps * 32) : "memory"); }

__device__ __forceinline__ void mma_s8s8(int (&c)[4], u32 a0, u32 a1, u32 a2, u32 a3, u32 b0, u32 b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// One block of one run: rows gid and gid + 8 of the tile (A), the 8 entries (B), this lane's four (row, entry) cells.
// ODD: the block's position in its run is odd (quants on a word). box: the run in shared memory; blk: byte offset of the
// block in a row; codes / deltas: the entries' A8 rows at this block, for this lane's fragment cells.
template <bool ODD>
__device__ __forceinline__ void block_step(const unsigned char* rowA, const unsigned char* rowB, u32 blk, u32 t4, const unsigned char* codes,
                                           const unsigned char* d0p, const unsigned char* d1p, float (&acc)[4]) {
    u32 a0, a1, a2, a3;
    float sA, sB;
    if (ODD) {  // block at 2 (mod 4): the scale is the high half of the word before the quants
        const u32* pa = reinterpret_cast<const u32*>(rowA + blk + 2u + 4u * t4);
        const u32* pb = reinterpret_cast<const u32*>(rowB + blk + 2u + 4u * t4);
        a0 = pa[0]; a2 = pa[4]; a1 = pb[0]; a3 = pb[4];
        sA = half_bits_to_float(*reinterpret_cast<const unsigned short*>(rowA + blk));
        sB = half_bits_to_float(*reinterpret_cast<const unsigned short*>(rowB + blk));
    } else {    // block on a word: the quants start in its upper half
        const u32* pa = reinterpret_cast<const u32*>(rowA + blk + 4u * t4);
        const u32* pb = reinterpret_cast<const u32*>(rowB + blk + 4u * t4);
        a0 = __byte_perm(pa[0], pa[1], 0x5432u); a2 = __byte_perm(pa[4], pa[5], 0x5432u);
        a1 = __byte_perm(pb[0], pb[1], 0x5432u); a3 = __byte_perm(pb[4], pb[5], 0x5432u);
        sA = half_bits_to_float(*reinterpret_cast<const unsigned short*>(rowA + blk));
        sB = half_bits_to_float(*reinterpret_cast<const unsigned short*>(rowB + blk));
    }
    const u32* pc = reinterpret_cast<const u32*>(codes);
    const float d0 = *reinterpret_cast<const float*>(d0p), d1 = *reinterpret_cast<const float*>(d1p);
    int c[4];
    mma_s8s8(c, a0, a1, a2, a3, pc[0], pc[4]);
    // c[0]: (row gid, entry 2 t4), c[1]: (gid, 2 t4 + 1), c[2]: (gid + 8, 2 t4), c[3]: (gid + 8, 2 t4 + 1)
    acc[0] = __fadd_rn(acc[0], __fmul_rn(static_cast<float>(c[0]), __fmul_rn(sA, d0)));
    acc[1] = __fadd_rn(acc[1], __fmul_rn(static_cast<float>(c[1]), __fmul_rn(sA, d1)));
    acc[2] = __fadd_rn(acc[2], __fmul_rn(static_cast<float>(c[2]), __fmul_rn(sB, d0)));
    acc[3] = __fadd_rn(acc[3], __fmul_rn(static_cast<float>(c[3]), __fmul_rn(sB, d1)));
}

template <bool DOWN>
__global__ void __launch_bounds__(kMmaThreads, 1)
q8_mma_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, MmaArgs a, MmaPlan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    if (DOWN && a.summary && *a.summary) return;
    u32 n_union = a.routes.counts[0];
    if (n_union == 0) return;
    if (n_union > plan.max_union) n_union = plan.max_union;

    unsigned char* ring = smem;
    unsigned char* xc = ring + kStages * kStageBytes;
    unsigned char* xd = xc + kKE * plan.xc_pitch;
    float* cls = reinterpret_cast<float*>(xd + kKE * plan.xd_pitch);
    float* s_gu = cls + kClsFloats;
    unsigned char* at = reinterpret_cast<unsigned char*>(s_gu + (DOWN ? 0u : kGuFloats));
    VExpert* table = reinterpret_cast<VExpert*>(at);
    at += (u64(plan.vmax) * sizeof(VExpert) + 15) & ~u64(15);
    u64* full = reinterpret_cast<u64*>(at);
    u64* empty = full + kStages;
    u64* x_full = empty + kStages;
    u64* x_empty = x_full + 1;
    at += (2 * kStages + 2) * 8;
    u32* ctl = reinterpret_cast<u32*>(at);  // [0] abort flag, [2] virtual experts, [3] items, [4] the consumers' decision to stop
    volatile u32* abort_flag = ctl;

    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    if (tid < kStages) { mbar_init(&full[tid], 1); mbar_init(&empty[tid], kMmaWarps); }
    if (tid == kStages) { mbar_init(x_full, 1); mbar_init(x_empty, kMmaWarps); }
    if (tid < 8) ctl[tid] = 0;
    if (tid <= kStages) asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    build_work_list(a.routes, n_union, plan.max_union, plan.vmax, plan.n_chunks, reinterpret_cast<u32*>(smem), table, ctl);
    const u32 n_items = ctl[3];
    const u32 k0 = static_cast<u32>(u64(n_items) * blockIdx.x / gridDim.x), k1 = static_cast<u32>(u64(n_items) * (blockIdx.x + 1) / gridDim.x);
    if (k0 == k1) return;
    constexpr u32 kTiles = DOWN ? 2u : 4u;

    // ------------------------------------------------------------------------------------------ the producer warp
    if (warp == kMmaWarps) {
        const u32 e = lane >> 1, part = lane & 1u;  // lanes 0 .. 2 ne - 1 copy the codes or the deltas of one entry
        const u32 in_stride = a.in.stride ? a.in.stride : a.in.width;
        u32 t = 0, xl = 0, last_jv = 0xffffffffu;
        bool ok = true;
        for (u32 k = k0; k < k1 && ok; ++k) {
            const u32 jv = k / plan.n_chunks, chunk = k - jv * plan.n_chunks;
            const VExpert ve = table[jv];
            const u32 ne = ve.ne();
            const bool new_x = jv != last_jv;
            last_jv = jv;
            u32 r = 0;
            if (new_x && e < ne) r = __ldg((DOWN ? a.routes.slots : a.routes.rows) + ve.begin() + e);
            for (u32 si = 0; si < kTiles * plan.nst && ok; ++si, ++t) {
                const u32 tile = si / plan.nst, s = si - tile * plan.nst;
                const u32 slot = t & 1u, use = t >> 1;
                if (use) ok = mbar_wait(&empty[slot], (use - 1u) & 1u, plan.wait_limit, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the consumers' reads precede the copies below
                const u32 run0 = s * kStageRuns, nr = min(kStageRuns, plan.nruns - run0);
                if (lane == 0) mbar_expect_tx(&full[slot], nr * kRunBox);
                __syncwarp();
                if (lane < nr) {
                    const u32 y = ve.expert() * a.rows_per_expert + 32u * chunk + kTileRows * (DOWN ? tile : (tile & 1u));
                    tma_2d(ring + slot * kStageBytes + lane * kRunBox, (DOWN || tile < 2u) ? &tm0 : &tm1, (run0 + lane) * (kRunBytes / 8), y, &full[slot]);
                }
                if (si == 0 && new_x) {  // the entries' A8 rows, requested right after the item's first stage
                    if (xl) ok = mbar_wait(x_empty, (xl - 1u) & 1u, plan.wait_limit, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) { ++t; break; }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    if (lane == 0) mbar_expect_tx(x_full, ne * (plan.K + plan.K / 8));
                    __syncwarp();
                    if (e < ne) {
                        if (part == 0) bulk_g2s(xc + e * plan.xc_pitch, a.in.codes + u64(r) * in_stride, plan.K, x_full);
                        else bulk_g2s(xd + e * plan.xd_pitch, a.in.deltas + u64(r) * (in_stride / 32), plan.K / 8, x_full);
                    }
                    ++xl;
                }
            }
        }
        if (!ok && lane == 0) {  // wait (bounded) for the copies still in flight before the CTA retires
            for (u32 n = t > kStages ? t - kStages : 0u; n < t; ++n)
                for (u32 i = 0; i < (plan.wait_limit >> 4) + 64u; ++i)
                    if (mbar_try_wait(&full[n & 1u], (n >> 1) & 1u)) break;
            if (xl)
                for (u32 i = 0; i < (plan.wait_limit >> 4) + 64u; ++i)
                    if (mbar_try_wait(x_full, (xl - 1u) & 1u)) break;
        }
        return;
    }

    // ------------------------------------------------------------------------------------------ consumer warps
    const u32 gid = lane >> 2, t4 = lane & 3u;
    const u32 blk_even = kQ8Block * (2u * warp), blk_odd = blk_even + kQ8Block;  // this warp's blocks of a run = its lane classes
    const unsigned char* my_codes = xc + gid * plan.xc_pitch + 4u * t4;          // B fragment: entry gid, k slice t4
    const unsigned char* my_d0 = xd + (2u * t4) * plan.xd_pitch;                 // accumulator cells: entries 2 t4 and 2 t4 + 1
    const unsigned char* my_d1 = my_d0 + plan.xd_pitch;
    const u32 act_stride = DOWN ? 0u : (a.act.stride ? a.act.stride : a.act.width);
    u32 t = 0, xl = 0, last_jv = 0xffffffffu, kl = 0;
    bool ok = true;
    for (u32 k = k0; k < k1; ++k, ++kl) {
        const u32 jv = k / plan.n_chunks, chunk = k - jv * plan.n_chunks;
        const VExpert ve = table[jv];
        const u32 ne = ve.ne(), vbegin = ve.begin();
        if (jv != last_jv) {
            if (ok) ok = mbar_wait(x_full, xl & 1u, plan.wait_limit, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            ++xl;
            last_jv = jv;
        }
        u32 my_slot = 0;
        if (DOWN && lane < ne) my_slot = __ldg(a.routes.slots + vbegin + lane);
        float* gu = s_gu + (kl & 1u) * (kGuFloats / 2);
        bool stop = false;
        for (u32 tile = 0; tile < kTiles; ++tile) {
            float acc[2][4];
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[c][i] = 0.0f;
            for (u32 s = 0; s < plan.nst; ++s, ++t) {
                const u32 slot = t & 1u;
                if (ok) ok = mbar_wait(&full[slot], (t >> 1) & 1u, plan.wait_limit, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) continue;  // a wait ran out somewhere: no more work, but every warp still meets the barriers below
                const u32 run0 = s * kStageRuns, nr = min(kStageRuns, plan.nruns - run0);
                const unsigned char* box = ring + slot * kStageBytes;
                for (u32 r = 0; r < nr; ++r, box += kRunBox) {
                    const u32 b = (run0 + r) * kRunBlocks + 2u * warp;  // even block of this warp in the run
                    const unsigned char* rowA = box + gid * kRowPitch;
                    const unsigned char* rowB = rowA + 8u * kRowPitch;
                    if (b < plan.groups) block_step<false>(rowA, rowB, blk_even, t4, my_codes + 32u * b, my_d0 + 4u * b, my_d1 + 4u * b, acc[0]);
                    if (b + 1u < plan.groups) block_step<true>(rowA, rowB, blk_odd, t4, my_codes + 32u * (b + 1u), my_d0 + 4u * (b + 1u), my_d1 + 4u * (b + 1u), acc[1]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);  // the stage is free for the producer
            }
            if (tile == kTiles - 1u && ok && k + 1u < k1 && (k + 1u) / plan.n_chunks != jv) {
                __syncwarp();
                if (lane == 0) mbar_arrive(x_empty);  // the next item brings other entries
            }
            // the class sums meet: cell (row, entry) = pair, class c at word pair * 32 + (c + pair) % 32
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const u32 pair = (gid + 8u * (i >> 1)) * kKE + 2u * t4 + (i & 1u);
                    cls[pair * 32u + ((2u * warp + c + pair) & 31u)] = acc[c][i];
                }
            consumers_sync();
            float mine = 0.0f;  // warp w folds row w of the tile: lane = class; lane i keeps the product of entry i
#pragma unroll
            for (u32 i = 0; i < kKE; ++i) {
                const u32 pair = warp * kKE + i;
                const float tot = butterfly32(cls[pair * 32u + ((lane + pair) & 31u)]);
                if (lane == i) mine = tot;
            }
            if (lane < ne && ok) {
                if (DOWN) a.raw[u64(my_slot) * a.out_width + 32u * chunk + kTileRows * tile + warp] = mine;
                else gu[(tile >> 1) * kKE * 32u + lane * 32u + kTileRows * (tile & 1u) + warp] = mine;
            }
            if (tid == 0) ctl[4] = *abort_flag;  // one thread publishes the decision between the two barriers: every warp reads the same
            consumers_sync();
            if (ctl[4]) { stop = true; break; }
        }
        if (stop) break;
        if (!DOWN && warp < ne) {  // swiglu_clamped + the A8 rule over the 32 outputs of entry `warp` (src/ds41_moe.cpp:134-146)
            const float gv = gu[warp * 32u + lane], uv = gu[kKE * 32u + warp * 32u + lane];
            const u32 slot_id = __ldg(a.routes.slots + vbegin + warp), o_col = 32u * chunk + lane;
            if (a.gate_out) { a.gate_out[u64(slot_id) * a.out_width + o_col] = gv; a.up_out[u64(slot_id) * a.out_width + o_col] = uv; }
            const float h = swiglu_ds41(gv, uv, a.limit);  // NaN propagates: this family has no status rule
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
    if (*abort_flag && lane == 0 && a.summary) atomicOr(a.summary, kAbortBit);
}

u32 round_up(u32 v, u32 a) { return (v + a - 1) / a * a; }
u32 plan_smem(const MmaPlan& p, bool down) {
    return kStages * kStageBytes + kKE * (p.xc_pitch + p.xd_pitch) + kClsFloats * 4 + (down ? 0u : kGuFloats * 4) +
           round_up(p.vmax * static_cast<u32>(sizeof(VExpert)), 16) + (2 * kStages + 2) * 8 + 64;
}

bool make_plan(u32 K, u32 n_chunks, u32 max_union, u64 slots, bool down, MmaPlan* p) {
    // whole runs of 32 blocks exist, rows of K / 32 * 34 bytes are multiples of 16, the staged A8 rows fit beside the ring
    if (K < 1024 || K > kMaxK || K % 256 || max_union == 0 || slots == 0 || slots > 8192) return false;
    p->K = K;
    p->groups = K / 32;
    p->nruns = (p->groups + kRunBlocks - 1) / kRunBlocks;
    p->nst = (p->nruns + kStageRuns - 1) / kStageRuns;
    p->xc_pitch = K + 16;      // K is a multiple of 128 bytes: entries lie 4 (mod 32) words apart
    p->xd_pitch = K / 8 + 16;
    p->n_chunks = n_chunks;
    p->max_union = max_union;
    p->vmax = max_union + static_cast<u32>(slots / kKE) + 1;
    if (u64(p->vmax) * n_chunks >= (1ull << 31)) return false;
    if (plan_smem(*p, down) > kSmemBudget) return false;
    if (work_list_scratch_words(max_union, p->vmax) * 4 > kStages * kStageBytes) return false;  // the work list is built in the ring
    p->wait_limit = debug_value(B200MOE_DEBUG_WAIT_LIMIT) ? debug_value(B200MOE_DEBUG_WAIT_LIMIT) : kDefaultWaitLimit;
    return true;
}
bool a8_ok(const b200moe_a8_rows& x) {
    const u32 stride = x.stride ? x.stride : x.width;
    return aligned(x.codes, 16) && aligned(x.deltas, 16) && stride % 128 == 0;
}

}  // namespace

bool q8_mma_gate_up_fits(const b200moe_gate_up_view& v, u32 rows) {
    MmaPlan p{};
    return v.shape.gate_type == B200MOE_TYPE_Q8_0 && v.shape.down_type == B200MOE_TYPE_Q8_0 && rows && a8_ok(v.x) && v.shape.inter % 32 == 0 &&
           aligned(v.weights.gate, 16) && aligned(v.weights.up, 16) && make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p);
}
bool q8_mma_down_fits(const b200moe_down_view& v, u32 rows) {
    MmaPlan p{};
    return v.shape.gate_type == B200MOE_TYPE_Q8_0 && v.shape.down_type == B200MOE_TYPE_Q8_0 && rows && a8_ok(v.act) && v.shape.hidden % 32 == 0 &&
           aligned(v.weights.down, 16) && make_plan(v.shape.inter, v.shape.hidden / 32, v.max_union, u64(rows) * v.shape.top_k, true, &p);
}

int launch_gate_up_q8_mma(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    MmaPlan p{};
    if (!make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "gate_up: the Q8_0 tensor-core form does not apply to this shape");
    MmaArgs a{};
    a.routes = v.routes; a.in = v.x; a.act = v.act; a.gate_out = v.gate_out; a.up_out = v.up_out; a.summary = v.summary;
    a.rows_per_expert = v.shape.inter; a.out_width = v.shape.inter; a.limit = v.shape.limit;
    CUtensorMap tm0, tm1;
    const u64 rb = u64(p.groups) * kQ8Block, total_rows = u64(v.shape.experts) * v.shape.inter;
    if (int rc = rows_map(v.weights.gate, rb, total_rows, kRowPitch, kTileRows, &tm0)) return rc;
    if (int rc = rows_map(v.weights.up, rb, total_rows, kRowPitch, kTileRows, &tm1)) return rc;
    const u32 smem = plan_smem(p, false);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q8_mma_kernel<false>), smem)) return rc;
    q8_mma_kernel<false><<<sm_count(), kMmaThreads, smem, stream>>>(tm0, tm1, a, p);
    return after_launch("gate_up_q8_mma");
}

int launch_down_q8_mma(const b200moe_down_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    MmaPlan p{};
    if (!make_plan(v.shape.inter, v.shape.hidden / 32, v.max_union, u64(rows) * v.shape.top_k, true, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "down: the Q8_0 tensor-core form does not apply to this shape");
    MmaArgs a{};
    a.routes = v.routes; a.in = v.act; a.raw = v.raw; a.summary = const_cast<u32*>(v.summary);
    a.rows_per_expert = v.shape.hidden; a.out_width = v.shape.hidden; a.limit = v.shape.limit;
    CUtensorMap tm0;
    if (int rc = rows_map(v.weights.down, u64(p.groups) * kQ8Block, u64(v.shape.experts) * v.shape.hidden, kRowPitch, kTileRows, &tm0)) return rc;
    const u32 smem = plan_smem(p, true);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q8_mma_kernel<true>), smem)) return rc;
    q8_mma_kernel<true><<<sm_count(), kMmaThreads, smem, stream>>>(tm0, tm0, a, p);
    return after_launch("down_q8_mma");
}

}  // namespace b200moe
