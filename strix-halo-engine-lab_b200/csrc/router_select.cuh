// Score transform, k-pass top-k selection and weights of one router row by one warp: device code shared by the
// stand-alone select kernel (router.cu) and the fused select + routes kernel of decode windows (routes.cu).
// Contracts: include/strix/moe/route_policy.hpp:80-156 (see router.cu).
#pragma once
#include "declared_math.cuh"

namespace b200moe {
namespace select_detail {

__device__ __forceinline__ u32 ordered_key(float v) {  // route_policy.hpp:84-88
    u32 u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
// True when candidate (a, ai) beats the current pick (b, bi) in a reduction over disjoint ascending scans: the
// serial scan keeps the lower id on equal keys, so the parallel form orders by (key desc, id asc).
__device__ __forceinline__ bool beats(u32 key, float a, u32 ai, float b, u32 bi) {
    if (key == B200MOE_KEY_FLOAT_SERIAL) return a > b || (a == b && ai < bi);
    const u32 ka = ordered_key(a), kb = ordered_key(b);
    return ka > kb || (ka == kb && ai < bi);
}

constexpr u32 kNone = 0xffffffffu;

// The serial scan of one selection pass (route_policy.hpp:104-114) over a short candidate list, skipping `skip`.
__device__ __forceinline__ u32 serial_pick(u32 key, const float* c, u32 n, u32 skip) {
    u32 pick = kNone;
    float best = 0.0f;
    for (u32 e = 0; e < n; ++e) {
        if (e == skip) continue;
        const bool better = key == B200MOE_KEY_FLOAT_SERIAL ? c[e] > best : ordered_key(c[e]) > ordered_key(best);
        if (pick == kNone || better) { pick = e; best = c[e]; }
    }
    return pick;
}

// One k-pass over `n` candidates c[] (shared memory), lane-strided; `taken` holds this lane's taken candidates (bit j
// = candidate lane + 32 j), `allowed_groups` masks candidates by group (per = candidates per group; all ones = no
// mask). Returns the pick (kNone when nothing is left) to every lane and marks it taken.
__device__ __forceinline__ u32 k_pass(u32 key, const float* c, u32 n, u32 lane, u32& taken, u32 allowed_groups, u32 per) {
    // the serial scan's first candidate: lowest untaken allowed id
    u32 first = kNone, pick = kNone;
    float best = 0.0f;
    for (u32 j = 0, e = lane; e < n; ++j, e += 32) {
        if ((taken >> j) & 1u) continue;
        if (!((allowed_groups >> (e / per)) & 1u)) continue;
        if (first == kNone) first = e;
        const float v = c[e];
        if (key == B200MOE_KEY_FLOAT_SERIAL && v != v) continue;  // a NaN never replaces a pick
        if (pick == kNone || beats(key, v, e, best, pick)) { pick = e; best = v; }
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        const u32 of = __shfl_xor_sync(0xffffffffu, first, d);
        first = min(first, of);
        const u32 op = __shfl_xor_sync(0xffffffffu, pick, d);
        const float ob = __shfl_xor_sync(0xffffffffu, best, d);
        if (op != kNone && (pick == kNone || beats(key, ob, op, best, pick))) { pick = op; best = ob; }
    }
    if (first == kNone) return kNone;
    if (key == B200MOE_KEY_FLOAT_SERIAL) {
        const float fv = c[first];
        if (fv != fv) pick = first;  // a NaN taken as the first candidate stays (route_policy.hpp:11-12)
    }
    if (pick != kNone && (pick & 31u) == lane) taken |= 1u << (pick >> 5);
    return pick;
}

// Warp arg-max of (value, id) pairs under the order of beats(); kNone = no candidate. Rolled: these selections run once
// per step in one warp per row on cold instruction caches, where a fetched line costs more than the instructions in it.
__device__ __forceinline__ void warp_best(u32 key, u32& pick, float& best) {
#pragma unroll 1
    for (int d = 16; d; d >>= 1) {
        const u32 op = __shfl_xor_sync(0xffffffffu, pick, d);
        const float ob = __shfl_xor_sync(0xffffffffu, best, d);
        if (op != kNone && (pick == kNone || beats(key, ob, op, best, pick))) { pick = op; best = ob; }
    }
}

// Fast path of one row, one warp: the row's choices live in registers (EPL per lane), no group limit, and no NaN among
// the choices (then the serial scan of the contract is plain "largest choice, lowest id on ties", so a warp arg-max
// per pass gives the same picks). Returns false - having written nothing - when the row needs the general path.
// `s` = this warp's scratch of at least `experts` floats (shared memory).
template <int EPL>
__device__ __forceinline__ bool select_row_fast(const float* logits, float* scores_out, const float* __restrict__ bias,
                                                const b200moe_route_policy& p, u32 row, u32 lane, float* s,
                                                u32* __restrict__ ids, float* __restrict__ weights) {
    const u32 E = p.experts;
    const float* z = logits + u64(row) * E;
    float sc[EPL], c[EPL];
    const float ninf = -__uint_as_float(0x7f800000u);
    if (p.score == B200MOE_SCORE_SOFTMAX) {  // route_policy.hpp:135-144
        float zz[EPL];
        float m = ninf;
#pragma unroll
        for (int j = 0; j < EPL; ++j) { const u32 e = lane + 32u * j; zz[j] = e < E ? z[e] : ninf; m = zz[j] > m ? zz[j] : m; }
#pragma unroll
        for (int d = 16; d; d >>= 1) { const float o = __shfl_xor_sync(0xffffffffu, m, d); m = o > m ? o : m; }
#pragma unroll
        for (int j = 0; j < EPL; ++j) { const u32 e = lane + 32u * j; sc[j] = declared_exp(__fsub_rn(zz[j], m)); if (e < E) s[e] = sc[j]; }
        __syncwarp();
        float sum = 0.0f;
#pragma unroll 8
        for (u32 e = 0; e < E; ++e) sum = __fadd_rn(sum, s[e]);  // ascending serial sum (the declared order), every lane alike
#pragma unroll
        for (int j = 0; j < EPL; ++j) sc[j] = __fdiv_rn(sc[j], sum);
        __syncwarp();
    } else {
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const u32 e = lane + 32u * j;
            const float zj = e < E ? z[e] : 0.0f;
            sc[j] = p.score == B200MOE_SCORE_SIGMOID ? sigmoid_score(zj) : sqrt_softplus_score(zj);
        }
    }
    bool has_nan = false;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const u32 e = lane + 32u * j;
        c[j] = (p.selection_bias && e < E) ? __fadd_rn(sc[j], bias[e]) : sc[j];
        has_nan |= e < E && c[j] != c[j];
    }
    if (__any_sync(0xffffffffu, has_nan)) return false;
#pragma unroll
    for (int j = 0; j < EPL; ++j) { const u32 e = lane + 32u * j; if (e < E) s[e] = sc[j]; }  // scores for the weight step
    if (scores_out) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) { const u32 e = lane + 32u * j; if (e < E) scores_out[u64(row) * E + e] = sc[j]; }
    }
    __syncwarp();
    u32 taken = 0, my_id = kNone;
    for (u32 k = 0; k < p.top_k; ++k) {
        u32 pick = kNone;
        float best = 0.0f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const u32 e = lane + 32u * j;
            if (e < E && !((taken >> j) & 1u) && (pick == kNone || beats(p.key, c[j], e, best, pick))) { pick = e; best = c[j]; }
        }
        warp_best(p.key, pick, best);
        if (pick != kNone && (pick & 31u) == lane) taken |= 1u << (pick >> 5);
        if (lane == k) my_id = pick;
    }
    if (p.order == B200MOE_ORDER_ASCENDING_ID) {
        u32 rank = 0;
        for (u32 k = 0; k < p.top_k; ++k) { const u32 o = __shfl_sync(0xffffffffu, my_id, k); rank += (o < my_id) ? 1u : 0u; }
        u32 sorted = kNone;
        for (u32 k = 0; k < p.top_k; ++k) {
            const u32 o = __shfl_sync(0xffffffffu, my_id, k), orank = __shfl_sync(0xffffffffu, rank, k);
            if (orank == lane) sorted = o;
        }
        my_id = sorted;
    }
    const float my_s = (lane < p.top_k && my_id != kNone) ? s[my_id] : 0.0f;
    float sum = 0.0f;  // ((0 + s0) + s1) + ... in output order (route_policy.hpp:121-123)
    for (u32 k = 0; k < p.top_k; ++k) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_s, k));
    const bool renorm = p.renormalize && (p.top_k > 1 || p.renorm_single);
    const float den = __fadd_rn(sum, p.renorm_eps);
    if (lane < p.top_k) {
        ids[u64(row) * p.top_k + lane] = my_id;
        weights[u64(row) * p.top_k + lane] = __fmul_rn(renorm ? __fdiv_rn(my_s, den) : my_s, p.scale);
    }
    return true;
}

// Output order, weights and the stores of one row; lane k holds pick k in `my_id`, s[] the scores.
__device__ __forceinline__ void finish_row(const b200moe_route_policy& p, u32 row, u32 lane, const float* s, u32 my_id,
                                        u32* __restrict__ ids, float* __restrict__ weights) {
    if (p.order == B200MOE_ORDER_ASCENDING_ID) {  // rank sort of the (distinct) ids held one per lane
        u32 rank = 0;
        for (u32 k = 0; k < p.top_k; ++k) { const u32 o = __shfl_sync(0xffffffffu, my_id, k); rank += (o < my_id) ? 1u : 0u; }
        u32 sorted = kNone;
        for (u32 k = 0; k < p.top_k; ++k) {
            const u32 o = __shfl_sync(0xffffffffu, my_id, k), orank = __shfl_sync(0xffffffffu, rank, k);
            if (orank == lane) sorted = o;
        }
        my_id = sorted;
    }
    const float my_s = (lane < p.top_k && my_id != kNone) ? s[my_id] : 0.0f;
    float sum = 0.0f;  // ((0 + s0) + s1) + ... in output order (route_policy.hpp:121-123)
    for (u32 k = 0; k < p.top_k; ++k) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, my_s, k));
    const bool renorm = p.renormalize && (p.top_k > 1 || p.renorm_single);
    const float den = __fadd_rn(sum, p.renorm_eps);
    if (lane < p.top_k) {
        ids[u64(row) * p.top_k + lane] = my_id;
        weights[u64(row) * p.top_k + lane] = __fmul_rn(renorm ? __fdiv_rn(my_s, den) : my_s, p.scale);
    }
}

// One warp selects one row. `s` points to this warp's scratch of 2 * experts + 32 floats (shared memory).
__device__ __forceinline__ void select_row(const float* logits, float* scores_out, const float* __restrict__ bias,
                                           const b200moe_route_policy& p, u32 row, u32 lane, float* s,
                                           u32* __restrict__ ids, float* __restrict__ weights) {
    const u32 E = p.experts;
    if (p.n_group == 1 && E <= 256) {  // registers hold the row: the fast path unless a NaN choice needs the serial rule
        const bool done = E <= 128 ? select_row_fast<4>(logits, scores_out, bias, p, row, lane, s, ids, weights)
                                   : select_row_fast<8>(logits, scores_out, bias, p, row, lane, s, ids, weights);
        if (done) return;
    }
    float* c = s + E;
    float* gs = c + E;
    const float* z = logits + u64(row) * E;

    if (p.score == B200MOE_SCORE_SOFTMAX) {  // route_policy.hpp:135-144
        float m = -__uint_as_float(0x7f800000u);
        for (u32 e = lane; e < E; e += 32) { const float v = z[e]; m = v > m ? v : m; }
#pragma unroll
        for (int d = 16; d; d >>= 1) { const float o = __shfl_xor_sync(0xffffffffu, m, d); m = o > m ? o : m; }
        for (u32 e = lane; e < E; e += 32) s[e] = declared_exp(__fsub_rn(z[e], m));
        __syncwarp();
        float sum = 0.0f;
#pragma unroll 8
        for (u32 e = 0; e < E; ++e) sum = __fadd_rn(sum, s[e]);  // ascending serial sum (the declared order), every lane alike
        for (u32 e = lane; e < E; e += 32) s[e] = __fdiv_rn(s[e], sum);
    } else if (p.score == B200MOE_SCORE_SIGMOID) {
        for (u32 e = lane; e < E; e += 32) s[e] = sigmoid_score(z[e]);
    } else {
        for (u32 e = lane; e < E; e += 32) s[e] = sqrt_softplus_score(z[e]);
    }
    for (u32 e = lane; e < E; e += 32) c[e] = p.selection_bias ? __fadd_rn(s[e], bias[e]) : s[e];
    __syncwarp();
    if (scores_out) for (u32 e = lane; e < E; e += 32) scores_out[u64(row) * E + e] = s[e];

    u32 allowed = 0xffffffffu, per = E;
    if (p.n_group > 1 && (E / p.n_group) % 32 == 0 && p.n_group <= 32) {
        // Groups of whole 32-expert runs and no NaN among the choices: every serial scan of the contract is then "largest
        // choice, lowest id on ties", which a warp arg-max reproduces; bit j of `live` = this lane's candidate lane + 32 j
        // is still to be had. Short rolled loops over shared memory keep the code small (see warp_best).
        per = E / p.n_group;
        bool bad = false;
        for (u32 e = lane; e < E; e += 32) bad |= c[e] != c[e];
        float my_gs = 0.0f;
        if (!__any_sync(0xffffffffu, bad)) {
#pragma unroll 1
            for (u32 g = 0; g < p.n_group; ++g) {
                u32 i0 = kNone, i1 = kNone;
                float b0 = 0.0f, b1 = 0.0f;
#pragma unroll 1
                for (u32 e = g * per + lane; e < (g + 1) * per; e += 32) { const float v = c[e]; if (i0 == kNone || beats(p.key, v, e, b0, i0)) { i0 = e; b0 = v; } }
                warp_best(p.key, i0, b0);
#pragma unroll 1
                for (u32 e = g * per + lane; e < (g + 1) * per; e += 32) { const float v = c[e]; if (e != i0 && (i1 == kNone || beats(p.key, v, e, b1, i1))) { i1 = e; b1 = v; } }
                warp_best(p.key, i1, b1);
                const float v = __fadd_rn(b0, b1);
                bad |= v != v;
                if (lane == g) my_gs = v;
            }
        }
        if (!__any_sync(0xffffffffu, bad)) {
            u32 gmask = 0;
#pragma unroll 1
            for (u32 k = 0; k < p.topk_group; ++k) {
                u32 pick = (lane < p.n_group && !((gmask >> lane) & 1u)) ? lane : kNone;
                float best = my_gs;
                warp_best(p.key, pick, best);
                if (pick != kNone) gmask |= 1u << pick;
            }
            const u32 m = per >> 5;
            u32 live = 0;
            for (u32 j = 0, g = 0, i = 0; lane + 32u * j < E; ++j) {  // register j belongs to group j / m
                if ((gmask >> g) & 1u) live |= 1u << j;
                if (++i == m) { i = 0; ++g; }
            }
            u32 my_id = kNone;
#pragma unroll 1
            for (u32 k = 0; k < p.top_k; ++k) {
                u32 pick = kNone;
                float best = 0.0f;
#pragma unroll 1
                for (u32 rest = live; rest; rest &= rest - 1u) {
                    const u32 e = lane + 32u * (__ffs(rest) - 1u);
                    const float v = c[e];
                    if (pick == kNone || beats(p.key, v, e, best, pick)) { pick = e; best = v; }
                }
                warp_best(p.key, pick, best);
                if (pick != kNone && (pick & 31u) == lane) live &= ~(1u << (pick >> 5));
                if (lane == k) my_id = pick;
            }
            finish_row(p, row, lane, s, my_id, ids, weights);
            return;
        }
        per = E;  // a NaN: the serial rules below decide
    }
    if (p.n_group > 1) {  // group-limited extension (include/b200moe.h): group score = its two best choices summed
        per = E / p.n_group;
        if (lane < p.n_group) {
            const float* cg = c + lane * per;
            const u32 i0 = serial_pick(p.key, cg, per, kNone);
            const u32 i1 = serial_pick(p.key, cg, per, i0);
            const float b0 = cg[i0], b1 = cg[i1];
            gs[lane] = __fadd_rn(b0, b1);
        }
        __syncwarp();
        u32 gtaken = 0;
        allowed = 0;
        for (u32 k = 0; k < p.topk_group; ++k) {
            const u32 g = k_pass(p.key, gs, p.n_group, lane, gtaken, 0xffffffffu, p.n_group);
            if (g != kNone) allowed |= 1u << g;
        }
    }

    u32 taken = 0, my_id = kNone;
    for (u32 k = 0; k < p.top_k; ++k) {
        const u32 pick = k_pass(p.key, c, E, lane, taken, allowed, per);
        if (lane == k) my_id = pick;
    }
    finish_row(p, row, lane, s, my_id, ids, weights);
}


}  // namespace select_detail
}  // namespace b200moe
