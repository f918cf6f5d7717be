// Routed / dense experts of the DS41 family (Q8_0 gate, up and down) over MANY rows: the segment-streaming skeleton of
// gemv_q4k_wide.cu with the 32-lane-class contract of src/ds41_formats.cpp:188-197 (product_q8_0) inside.
//
// Why a second form: the decode kernels of gemv_q8.cu take one weight row per warp and re-read the activations' codes for
// every weight row (32 bytes per (row, token, group) through the load pipe) - fine for 1 to 8 rows, but a 64-row window or
// a token block over the shared expert then costs passes of 8 rows each. Here a warp keeps the codes of FOUR entries in
// registers and walks four weight rows against them, so a byte of codes is loaded once per four rows and a weight block
// once per eight entries.
//
//  * Work item = (virtual expert of at most 8 entries, 32 outputs): for gate/up the stages of the 32 gate rows followed by
//    the stages of the 32 up rows, for down the stages of 32 down rows. A stage = one RUN of 32 blocks (1088 bytes) of 32
//    rows, one tiled TMA copy, plus the entries' codes and deltas of the same 1024 columns (bulk copies), on one mbarrier.
//  * Lane = block of the run = lane class (group g of the row goes to class g % 32, and a run starts at a multiple of 32):
//    class sums accumulate in ascending g from +0 across the runs, the butterfly v[l] += v[l ^ d], d = 16 .. 1, closes a
//    row - the contract's order, bit for bit. Q8_0 blocks are 34 bytes: even lanes start on a word, odd lanes on a
//    halfword, as in gemv_q8.cu.
//  * gate/up: after the up rows the group meets on an mbarrier and eight warps run swiglu_clamped (declared_exp) + the A8
//    rule of one entry each (src/ds41_moe.cpp:134-146).
// Items are dealt out through the grid's claim word and waits are bounded, both as in gemv_q4k_wide.cu
// (B200MOE_JOB_WAIT_ABORTED). gemv_q8_mma.cu takes the same windows with the integer dots on the tensor cores and is the
// library's choice where it applies (rows of 1024 to 7168 weights); this form is what is left: other row lengths.
//
// Roofline: the FP32 tail of the contract (convert, scale * delta, product, add per (row, entry, group)) bounds it, not
// HBM: a 64-row window re-reads the shared expert's 46.8 MB out of L2.
#include <algorithm>

#include "wide_common.cuh"

namespace b200moe {
namespace {
using namespace q4k;   // the mbarrier / copy wrappers
using namespace wide;

constexpr u32 kRunBlocks = 32, kRunBytes = kRunBlocks * kQ8Block;  // 1088
constexpr u32 kRows = 32;                                          // weight rows of a stage: four per consumer warp
constexpr u32 kWBytes = kRows * kRunBytes;                         // 34,816
constexpr u32 kXEntry = kRunBlocks * 32 + kRunBlocks * 4;          // codes + deltas of one entry over a run: 1152
constexpr u32 kPass = 4;                                           // entries whose codes a lane holds at a time

struct Q8Plan {
    u32 groups;       // K / 32
    u32 nruns;        // stages per matrix of an item
    u32 stages;       // ring depth per group
    u32 stage_bytes;
    u32 n_chunks, max_union, vmax, wait_limit;
};

struct Q8Args {
    b200moe_routes routes;
    b200moe_a8_rows in, act;
    float* gate_out;
    float* up_out;
    float* raw;
    u32* summary;
    u32 rows_per_expert, out_width;
    float limit;
};

// One stage: the warp's four weight rows (blocks of this run) against the item's entries. cls[r][t]: lane class sums.
__device__ __forceinline__ void q8_stage(const unsigned char* w4, u32 nb, u32 ne, u32 lane, const unsigned char* xs, float (*cls)[kKE]) {
    if (lane >= nb) return;
    const u32 w0 = (kQ8Block * lane) >> 2;
    const u32 sel_scale = (lane & 1u) ? 0x4432u : 0x4410u, sel_quant = (lane & 1u) ? 0x7654u : 0x5432u;
#pragma unroll 1
    for (u32 t0 = 0; t0 < ne; t0 += kPass) {
        uint4 c0[kPass], c1[kPass];
        float dl[kPass];
#pragma unroll
        for (int t = 0; t < (int)kPass; ++t) {
            const unsigned char* xe = xs + min(t0 + t, ne - 1u) * kXEntry;
            const uint4* c = reinterpret_cast<const uint4*>(xe + 32u * lane);
            c0[t] = c[0]; c1[t] = c[1];
            dl[t] = *reinterpret_cast<const float*>(xe + kRunBlocks * 32 + 4u * lane);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const u32* row = reinterpret_cast<const u32*>(w4 + r * kRunBytes);
            // The block lies at byte 34 * lane: on a word for even lanes, on a halfword for odd ones. Nine words cover it
            // either way; a byte permute with a per-lane selector picks scale and quants without a divergent branch.
            u32 w[9], q[8];
#pragma unroll
            for (int i = 0; i < 9; ++i) w[i] = row[w0 + i];
            const float scale = half_bits_to_float(__byte_perm(w[0], 0u, sel_scale));
#pragma unroll
            for (int i = 0; i < 8; ++i) q[i] = __byte_perm(w[i], w[i + 1], sel_quant);
#pragma unroll
            for (int t = 0; t < (int)kPass; ++t) {
                int da = __dp4a((int)q[0], (int)c0[t].x, 0), db = __dp4a((int)q[1], (int)c0[t].y, 0);
                da = __dp4a((int)q[2], (int)c0[t].z, da); db = __dp4a((int)q[3], (int)c0[t].w, db);
                da = __dp4a((int)q[4], (int)c1[t].x, da); db = __dp4a((int)q[5], (int)c1[t].y, db);
                da = __dp4a((int)q[6], (int)c1[t].z, da); db = __dp4a((int)q[7], (int)c1[t].w, db);
                const float term = __fmul_rn(small_int_to_float(da + db), __fmul_rn(scale, dl[t]));
                // entries beyond ne are computed on entry ne - 1's data and dropped here (no branch in the dot chain)
                if (t0 + t < ne) {
                    if (t0 == 0) cls[r][t] = __fadd_rn(cls[r][t], term);
                    else cls[r][kPass + t] = __fadd_rn(cls[r][kPass + t], term);
                }
            }
        }
    }
}

template <bool DOWN>
__global__ void __launch_bounds__(kThreads, 1)
q8_wide_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1, Q8Args a, Q8Plan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    if (DOWN && a.summary && *a.summary) return;
    u32 n_union = a.routes.counts[0];
    if (n_union == 0) return;
    if (n_union > plan.max_union) n_union = plan.max_union;
    u32* claim = a.routes.counts + 3;  // the grid's claim word (wide_common.cuh)

    unsigned char* at = smem + kGroups * plan.stages * plan.stage_bytes;
    float* s_gu = reinterpret_cast<float*>(at);  // [group][buffer][gate | up][entry][32]
    if (!DOWN) at += kGroups * 2 * 2 * kKE * 32 * 4;
    VExpert* table = reinterpret_cast<VExpert*>(at);
    at += (u64(plan.vmax) * sizeof(VExpert) + 15) & ~u64(15);
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
    build_work_list(a.routes, n_union, plan.max_union, plan.vmax, plan.n_chunks, reinterpret_cast<u32*>(smem), table, ctl);
    const u32 n_items = ctl[3];
    if (n_items == 0) return;  // every CTA alike: nobody claims, the claim word stays zero
    const u32 item_stages = (DOWN ? 1u : 2u) * plan.nruns;

    // ------------------------------------------------------------------------------------------ producer warps
    if (warp >= kConsumerWarps) {
        const u32 g = warp - kConsumerWarps;
        u64* g_full = full + g * plan.stages;
        u64* g_empty = empty + g * plan.stages;
        u32* g_item = slot_item + g * plan.stages;
        unsigned char* g_stage = smem + g * plan.stages * plan.stage_bytes;
        const u32 e = lane >> 1, part = lane & 1u;  // lanes 0 .. 2 * ne - 1 copy the codes or the deltas of one entry
        const u32 in_stride = a.in.stride ? a.in.stride : a.in.width, in_gs = in_stride / 32;
        u32 t = 0, slot = 0, use = 0;
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
            const u32 n = end ? 1u : item_stages;
            for (u32 s = 0; s < n; ++s, ++t, ++slot) {
                if (slot == plan.stages) { slot = 0; ++use; }
                if (use) ok = mbar_wait(&g_empty[slot], (use - 1u) & 1u, plan.wait_limit, abort_flag);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                if (end) {
                    if (lane == 0) { g_item[slot] = kEndItem; mbar_arrive(&g_full[slot]); }
                    continue;
                }
                const u32 run = s < plan.nruns ? s : s - plan.nruns;
                const u32 nb = min(kRunBlocks, plan.groups - run * kRunBlocks);
                unsigned char* dst = g_stage + slot * plan.stage_bytes;
                if (lane == 0) {
                    g_item[slot] = item;
                    mbar_expect_tx(&g_full[slot], kWBytes + ve_ne * nb * 36u);
                }
                __syncwarp();
                if (lane == 0)
                    tma_2d(dst, (DOWN || s < plan.nruns) ? &tm0 : &tm1, run * (kRunBytes / 8), ve.expert() * a.rows_per_expert + kRows * chunk, &g_full[slot]);
                if (e < ve_ne) {
                    unsigned char* xd = dst + kWBytes + e * kXEntry;
                    if (part == 0) bulk_g2s(xd, a.in.codes + u64(r) * in_stride + u64(run) * (kRunBlocks * 32), nb * 32u, &g_full[slot]);
                    else bulk_g2s(xd + kRunBlocks * 32, a.in.deltas + u64(r) * in_gs + u64(run) * kRunBlocks, nb * 4u, &g_full[slot]);
                }
            }
            if (!ok || end) break;
        }
        if (!ok && lane == 0) {
            for (u32 n = t > plan.stages ? t - plan.stages : 0u; n < t; ++n)
                for (u32 i = 0; i < (plan.wait_limit >> 4) + 64u; ++i)
                    if (mbar_try_wait(&g_full[n % plan.stages], (n / plan.stages) & 1u)) break;
        }
        if (lane == 0) retire_claims(claim, ctl);
        return;
    }

    // ------------------------------------------------------------------------------------------ consumer warps
    const u32 g = warp / kGroupWarps, w = warp % kGroupWarps;
    u64* g_full = full + g * plan.stages;
    u64* g_empty = empty + g * plan.stages;
    const u32* g_item = slot_item + g * plan.stages;
    const unsigned char* g_stage = smem + g * plan.stages * plan.stage_bytes;
    const u32 act_stride = DOWN ? 0u : (a.act.stride ? a.act.stride : a.act.width);
    u32 slot = 0, phase = 0, kl = 0;
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
        float* gu = s_gu + u64((g * 2 + (kl & 1u)) * 2) * kKE * 32;
        for (u32 mat = 0; mat < (DOWN ? 1u : 2u); ++mat) {
            float cls[4][kKE];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int t = 0; t < (int)kKE; ++t) cls[r][t] = 0.0f;
            for (u32 run = 0; run < plan.nruns; ++run) {
                if (mat | run) {
                    ok = mbar_wait(&g_full[slot], phase, plan.wait_limit, abort_flag);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                const unsigned char* st = g_stage + slot * plan.stage_bytes;
                q8_stage(st + 4u * w * kRunBytes, min(kRunBlocks, plan.groups - run * kRunBlocks), ne, lane, st + kWBytes, cls);
                __syncwarp();
                if (lane == 0) mbar_arrive(&g_empty[slot]);
                if (++slot == plan.stages) { slot = 0; phase ^= 1u; }
            }
            if (!ok) break;
            // the butterfly closes the four rows of every entry; lane 0 holds (and stores) the products
#pragma unroll
            for (int t = 0; t < (int)kKE; ++t) {
                if (t < (int)ne) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const float val = butterfly32(cls[r][t]);
                        if (lane == 0) {
                            if (DOWN) a.raw[u64(__ldg(a.routes.slots + vbegin + t)) * a.out_width + kRows * chunk + 4u * w + r] = val;
                            else gu[mat * kKE * 32 + t * 32 + 4u * w + r] = val;
                        }
                    }
                }
            }
        }
        if (!ok) break;
        if (!DOWN) {
            __syncwarp();
            if (lane == 0) mbar_arrive(&gu_bar[g]);
            ok = mbar_wait(&gu_bar[g], kl & 1u, plan.wait_limit, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (w < ne) {  // swiglu_clamped + the A8 rule over the 32 outputs of entry w (src/ds41_moe.cpp:134-146)
                const float gv = gu[w * 32 + lane], uv = gu[kKE * 32 + w * 32 + lane];
                const u32 slot_id = __ldg(a.routes.slots + vbegin + w), o_col = 32u * chunk + lane;
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
        ++kl;
    }
    if (!ok && lane == 0 && a.summary) atomicOr(a.summary, kAbortBit);
}

u32 round_up(u32 v, u32 a) { return (v + a - 1) / a * a; }
u32 fixed_smem(const Q8Plan& p, bool down) {
    return (down ? 0u : kGroups * 2 * 2 * kKE * 32 * 4) + round_up(p.vmax * static_cast<u32>(sizeof(VExpert)), 16) + (2 * kGroups * p.stages + kGroups) * 8 +
           kGroups * p.stages * 4 + 64;
}
u32 plan_smem(const Q8Plan& p, bool down) { return kGroups * p.stages * p.stage_bytes + fixed_smem(p, down); }

bool make_plan(u32 K, u32 n_chunks, u32 max_union, u64 slots, bool down, Q8Plan* p) {
    if (K == 0 || K % 256 || max_union == 0 || slots == 0 || slots > 8192) return false;  // rows of K / 32 * 34 bytes are then multiples of 16
    p->groups = K / 32;
    p->nruns = (p->groups + kRunBlocks - 1) / kRunBlocks;
    p->stage_bytes = round_up(kWBytes + static_cast<u32>(std::min<u64>(kKE, slots)) * kXEntry, 128);
    p->n_chunks = n_chunks;
    p->max_union = max_union;
    p->vmax = max_union + static_cast<u32>(slots / kKE) + 1;
    if (u64(p->vmax) * n_chunks + 4096 >= kClaimMask) return false;  // items and the groups' closing claims fit the claim word's count
    for (p->stages = 4; p->stages >= 2; --p->stages)
        if (plan_smem(*p, down) <= kSmemBudget) break;
    if (p->stages < 2) return false;
    if (work_list_scratch_words(max_union, p->vmax) * 4 > kGroups * p->stages * p->stage_bytes) return false;  // the work list is built in the stage area
    p->wait_limit = debug_value(B200MOE_DEBUG_WAIT_LIMIT) ? debug_value(B200MOE_DEBUG_WAIT_LIMIT) : kDefaultWaitLimit;
    return true;
}
bool a8_ok(const b200moe_a8_rows& x) {
    const u32 stride = x.stride ? x.stride : x.width;
    return aligned(x.codes, 16) && aligned(x.deltas, 16) && stride % 128 == 0;
}

}  // namespace

bool q8_wide_gate_up_fits(const b200moe_gate_up_view& v, u32 rows) {
    Q8Plan p{};
    return v.shape.gate_type == B200MOE_TYPE_Q8_0 && v.shape.down_type == B200MOE_TYPE_Q8_0 && rows && a8_ok(v.x) && v.shape.inter % 32 == 0 &&
           aligned(v.weights.gate, 16) && aligned(v.weights.up, 16) && make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p);
}
bool q8_wide_down_fits(const b200moe_down_view& v, u32 rows) {
    Q8Plan p{};
    return v.shape.gate_type == B200MOE_TYPE_Q8_0 && v.shape.down_type == B200MOE_TYPE_Q8_0 && rows && a8_ok(v.act) && v.shape.hidden % 32 == 0 &&
           aligned(v.weights.down, 16) && make_plan(v.shape.inter, v.shape.hidden / 32, v.max_union, u64(rows) * v.shape.top_k, true, &p);
}

int launch_gate_up_q8_wide(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    Q8Plan p{};
    if (!make_plan(v.shape.hidden, v.shape.inter / 32, v.max_union, u64(rows) * v.shape.top_k, false, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "gate_up: the Q8_0 token-block form does not apply to this shape");
    Q8Args a{};
    a.routes = v.routes; a.in = v.x; a.act = v.act; a.gate_out = v.gate_out; a.up_out = v.up_out; a.summary = v.summary;
    a.rows_per_expert = v.shape.inter; a.out_width = v.shape.inter; a.limit = v.shape.limit;
    CUtensorMap tm0, tm1;
    const u64 rb = u64(p.groups) * kQ8Block, total_rows = u64(v.shape.experts) * v.shape.inter;
    if (int rc = rows_map(v.weights.gate, rb, total_rows, kRunBytes, kRows, &tm0)) return rc;
    if (int rc = rows_map(v.weights.up, rb, total_rows, kRunBytes, kRows, &tm1)) return rc;
    const u32 smem = plan_smem(p, false);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q8_wide_kernel<false>), smem)) return rc;
    q8_wide_kernel<false><<<sm_count(), kThreads, smem, stream>>>(tm0, tm1, a, p);
    return after_launch("gate_up_q8_wide");
}

int launch_down_q8_wide(const b200moe_down_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    Q8Plan p{};
    if (!make_plan(v.shape.inter, v.shape.hidden / 32, v.max_union, u64(rows) * v.shape.top_k, true, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "down: the Q8_0 token-block form does not apply to this shape");
    Q8Args a{};
    a.routes = v.routes; a.in = v.act; a.raw = v.raw; a.summary = const_cast<u32*>(v.summary);
    a.rows_per_expert = v.shape.hidden; a.out_width = v.shape.hidden; a.limit = v.shape.limit;
    CUtensorMap tm0;
    if (int rc = rows_map(v.weights.down, u64(p.groups) * kQ8Block, u64(v.shape.experts) * v.shape.hidden, kRunBytes, kRows, &tm0)) return rc;
    const u32 smem = plan_smem(p, true);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(q8_wide_kernel<true>), smem)) return rc;
    q8_wide_kernel<true><<<sm_count(), kThreads, smem, stream>>>(tm0, tm0, a, p);
    return after_launch("down_q8_wide");
}

}  // namespace b200moe
