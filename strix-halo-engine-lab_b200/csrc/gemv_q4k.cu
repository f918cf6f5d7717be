// Routed experts, Qwen A8 family, decode form: dequant-fused GEMVs over Q4_K super-blocks kept in their GGUF bytes.
//
// Contract (src/cpu/core/routed_expert.hpp:9-15, routed_expert.cpp:73-170): per super-block b of 256 weights and
// group j of 32 (g = 8b + j):  x_j = E_g * ((d * sc_j) * float(dot_j) - (dmin * m_j) * float(S_g)),
// pair_p = x_2p + x_2p+1, acc_p += pair_p over ascending b, value = (acc0 + acc1) + (acc2 + acc3); then
// h = (g / (1 + exp(-g))) * u and the A8 rule per 32 outputs. Q4_K down = the same row rule over K = inter
// (src/moe_a8_down_contract.cpp:141-146); Q8_0 down = four chains by g % 4 (routed_expert.cpp:110-144).
// Integer dots are exact (dp4a), every FP32 step is one IEEE operation, so results equal the host's bit for bit.
// The same kernels read the executor's other stored formats (routed_expert.hpp:27-28): Q5_K gate / up (176-byte
// super-blocks, the Q4_K rule with a fifth bit per weight) and Q5_1 down (24-byte blocks on the four chains,
// d * float(dot) + m * float(S_g)).
//
// Mapping: 4 lanes per super-block (lane = pair p: 32 B of nibbles serve groups 2p (low) and 2p+1 (high)), LPR lanes
// per weight row (8 / 16 / 32 by row length), so a warp streams 32 / LPR rows at once with 16-byte loads: per
// super-block one 16 B header (broadcast to its 4 lanes) + 4 x 32 B = 144 B, fully coalesced. The serial chain over b
// is rebuilt with shuffles. Up to 8 entries (tokens routed to the expert) share one pass over the weights.
//
// Roofline: HBM. Algorithmic bytes per (expert, call) = 2 * inter * hidden / 256 * 144 (gate, up) and
// hidden * inter / 256 * 144 (down), read once however many of the <= 8 staged rows use the expert.
#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr int kR = 8;  // entries staged per pass

struct A8Smem {
    const i8* codes;    // [kR][width]
    const float* deltas;  // [kR][width / 32]
    const i32* sums;    // [kR][width / 32]
    u32 width;
};

__device__ __forceinline__ void q4k_factor(const uint4& hdr, u32 j, float d, float dm, float* D, float* DM) {
    const u32 shift = 8u * (j & 3u);
    const u32 a = (hdr.y >> shift) & 255u, b = (hdr.z >> shift) & 255u, c = (hdr.w >> shift) & 255u;
    const u32 sc = j < 4u ? (a & 63u) : ((c & 15u) | ((a >> 6) << 4));
    const u32 mn = j < 4u ? (b & 63u) : ((c >> 4) | ((b >> 6) << 4));
    *D = __fmul_rn(d, static_cast<float>(sc));
    *DM = __fmul_rn(dm, static_cast<float>(mn));
}

// 32 weights of one group against 32 codes: nibbles at `shift` (0 = low, 4 = high) of the 32 bytes wa | wb. Q5_K adds
// bit j of the 32 high-bit bytes ha | hb as bit 4 of each weight (routed_expert.cpp:88-95).
template <bool Q5K>
__device__ __forceinline__ int dot8(const uint4& wa, const uint4& wb, const uint4& ha, const uint4& hb, u32 j, const uint4& ca, const uint4& cb, u32 shift) {
    auto w = [&](u32 q, u32 h) -> int {
        u32 v = (q >> shift) & 0x0f0f0f0fu;
        if (Q5K) v |= ((h >> j) & 0x01010101u) << 4;
        return static_cast<int>(v);
    };
    int s = 0;
    s = __dp4a(w(wa.x, ha.x), static_cast<int>(ca.x), s);
    s = __dp4a(w(wa.y, ha.y), static_cast<int>(ca.y), s);
    s = __dp4a(w(wa.z, ha.z), static_cast<int>(ca.z), s);
    s = __dp4a(w(wa.w, ha.w), static_cast<int>(ca.w), s);
    s = __dp4a(w(wb.x, hb.x), static_cast<int>(cb.x), s);
    s = __dp4a(w(wb.y, hb.y), static_cast<int>(cb.y), s);
    s = __dp4a(w(wb.z, hb.z), static_cast<int>(cb.z), s);
    s = __dp4a(w(wb.w, hb.w), static_cast<int>(cb.w), s);
    return s;
}

// One Q4_K weight row (nblocks super-blocks at wrow) against nr <= kR staged A8 rows. LPR lanes cooperate on the row
// (lane-in-row li: super-block li / 4 of each step, pair li % 4); `base` is the first lane of the row's lane group.
// Every lane of the group returns the row values in out[].
template <int LPR, bool Q5K = false>
__device__ __forceinline__ void q4k_row(const u8* __restrict__ wrow, u32 nblocks, const A8Smem& x, int nr, u32 li, u32 base, float* out) {
    constexpr u32 BPI = LPR / 4;
    const u32 p = li & 3u, bsub = li >> 2;
    float acc[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) acc[r] = 0.0f;
    // The loads of step b0 + BPI are issued before the arithmetic of step b0 (one step of register prefetch): the row walk
    // is otherwise a chain of load -> dot -> shuffle with nothing in flight.
    struct Blk { uint4 hdr, q0, q1, h0, h1; };
    auto load_blk = [&](u32 b) {
        Blk k;
        k.hdr = make_uint4(0, 0, 0, 0); k.q0 = k.hdr; k.q1 = k.hdr; k.h0 = k.hdr; k.h1 = k.hdr;
        if (b < nblocks) {
            const uint4* blk = reinterpret_cast<const uint4*>(wrow + u64(b) * (Q5K ? kQ5KBlock : kQ4KBlock));
            k.hdr = __ldg(blk);
            if (Q5K) { k.h0 = __ldg(blk + 1); k.h1 = __ldg(blk + 2); }  // Q5_K: 32 bytes of high bits between header and nibbles
            k.q0 = __ldg(blk + (Q5K ? 3 : 1) + 2 * p);
            k.q1 = __ldg(blk + (Q5K ? 4 : 2) + 2 * p);
        }
        return k;
    };
    Blk nxt = load_blk(bsub);
    for (u32 b0 = 0; b0 < nblocks; b0 += BPI) {
        const u32 b = b0 + bsub;
        const bool valid = b < nblocks;
        const Blk cur = nxt;
        nxt = load_blk(b + BPI);
        const uint4 hdr = cur.hdr, q0 = cur.q0, q1 = cur.q1, h0 = cur.h0, h1 = cur.h1;
        const float d = half_bits_to_float(hdr.x & 0xffffu), dm = half_bits_to_float(hdr.x >> 16);
        float Dl, DMl, Dh, DMh;
        q4k_factor(hdr, 2 * p, d, dm, &Dl, &DMl);
        q4k_factor(hdr, 2 * p + 1, d, dm, &Dh, &DMh);
        const u32 nb = min(BPI, nblocks - b0);
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            if (r < nr) {
                float pair = 0.0f;
                if (valid) {
                    const uint4* c = reinterpret_cast<const uint4*>(x.codes + u64(r) * x.width + 256u * b + 64u * p);
                    const uint4 c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3];
                    const int dl = dot8<Q5K>(q0, q1, h0, h1, 2 * p, c0, c1, 0), dh = dot8<Q5K>(q0, q1, h0, h1, 2 * p + 1, c2, c3, 4);
                    const u32 g = r * (x.width / 32) + 8u * b + 2u * p;
                    const float2 e = *reinterpret_cast<const float2*>(x.deltas + g);
                    const int2 s = *reinterpret_cast<const int2*>(x.sums + g);
                    const float xl = __fmul_rn(e.x, __fsub_rn(__fmul_rn(Dl, static_cast<float>(dl)), __fmul_rn(DMl, static_cast<float>(s.x))));
                    const float xh = __fmul_rn(e.y, __fsub_rn(__fmul_rn(Dh, static_cast<float>(dh)), __fmul_rn(DMh, static_cast<float>(s.y))));
                    pair = __fadd_rn(xl, xh);
                }
                // acc_p += pair_p over ascending super-blocks: the serial chain, rebuilt across the row's lanes
#pragma unroll
                for (u32 bb = 0; bb < BPI; ++bb) {
                    const float t = __shfl_sync(0xffffffffu, pair, base + 4u * bb + p);
                    if (bb < nb) acc[r] = __fadd_rn(acc[r], t);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kR; ++r) {
        const float a0 = __shfl_sync(0xffffffffu, acc[r], base + 0), a1 = __shfl_sync(0xffffffffu, acc[r], base + 1);
        const float a2 = __shfl_sync(0xffffffffu, acc[r], base + 2), a3 = __shfl_sync(0xffffffffu, acc[r], base + 3);
        out[r] = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
    }
}

// Stage nr A8 rows (row ids from idx[]) of `width` into shared memory. All threads of the block take part.
__device__ __forceinline__ void stage_a8(const b200moe_a8_rows& src, const u32* idx, int nr, u32 width, i8* s_codes, float* s_deltas, i32* s_sums) {
    const u32 stride = src.stride ? src.stride : src.width, groups = width / 32;
    for (int r = 0; r < nr; ++r) {
        const u64 row = idx[r];
        const uint4* c = reinterpret_cast<const uint4*>(src.codes + row * stride);
        uint4* dc = reinterpret_cast<uint4*>(s_codes + u64(r) * width);
        for (u32 i = threadIdx.x; i < width / 16; i += blockDim.x) dc[i] = c[i];
        for (u32 i = threadIdx.x; i < groups; i += blockDim.x) {
            s_deltas[r * groups + i] = src.deltas[row * (stride / 32) + i];
            s_sums[r * groups + i] = src.sums ? src.sums[row * (stride / 32) + i] : 0;
        }
    }
}

// grid (inter / 32, max_union); 256 threads. One CTA = one expert x one 32-output group (= one A8 group of h).
template <int LPR, bool Q5K>
__global__ void __launch_bounds__(256) gate_up_q4k_kernel(b200moe_gate_up_view v) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const u32 j = blockIdx.y;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = H / 32, nblocks = H / 256;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * H);
    i32* s_sums = reinterpret_cast<i32*>(s_deltas + kR * groups);
    float* s_g = reinterpret_cast<float*>(s_sums + kR * groups);  // [kR][32]
    float* s_u = s_g + kR * 32;
    __shared__ u32 s_rows[kR], s_slots[kR];

    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    constexpr u32 RPW = 32 / LPR;
    const u32 sub = lane / LPR, li = lane % LPR, base = sub * LPR;
    const u64 row_bytes = u64(nblocks) * (Q5K ? kQ5KBlock : kQ4KBlock);
    const u8* gate = v.weights.gate + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const u8* up = v.weights.up + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const A8Smem xs{s_codes, s_deltas, s_sums, H};
    const u32 act_stride = v.act.stride ? v.act.stride : v.act.width;

    for (u32 p0 = eb; p0 < ee; p0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < (u32)nr) { s_rows[threadIdx.x] = v.routes.rows[p0 + threadIdx.x]; s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x]; }
        __syncthreads();
        stage_a8(v.x, s_rows, nr, H, s_codes, s_deltas, s_sums);
        __syncthreads();
        // 64 weight rows (gate 0..31, up 32..63): 8 warps x RPW rows per step
        for (u32 t0 = warp * RPW; t0 < 64; t0 += 8 * RPW) {
            const u32 t = t0 + sub;
            const u8* wrow = (t < 32 ? gate : up) + u64(t & 31u) * row_bytes;
            float val[kR];
            q4k_row<LPR, Q5K>(wrow, nblocks, xs, nr, li, base, val);
            if (li == 0) {
                float* dst = t < 32 ? s_g : s_u;
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) dst[r * 32 + (t & 31u)] = val[r];
            }
        }
        __syncthreads();
        // epilogue: one warp per entry: SwiGLU, then the A8 rule over the 32 outputs
        for (int r = warp; r < nr; r += 8) {
            const float g = s_g[r * 32 + lane], u = s_u[r * 32 + lane];
            const u32 slot = s_slots[r];
            const u32 o = 32u * blockIdx.x + lane;
            if (v.gate_out) { v.gate_out[u64(slot) * I + o] = g; v.up_out[u64(slot) * I + o] = u; }
            const float h = swiglu_qwen(g, u);
            const bool bad = __any_sync(0xffffffffu, !finite_f(g) || !finite_f(u) || !finite_f(h));
            if (bad) {  // fail closed: nothing of the group is written (routed_expert.cpp:147-156)
                if (lane == 0) {
                    if (v.row_status) atomicOr(&v.row_status[s_rows[r]], B200MOE_ROW_PROJECTION_NONFINITE);
                    if (v.summary) atomicOr(v.summary, B200MOE_ROW_PROJECTION_NONFINITE);
                }
                continue;
            }
            float delta;
            int sum;
            const int code = a8_quantize_lane(h, &delta, &sum);
            v.act.codes[u64(slot) * act_stride + o] = static_cast<i8>(code);
            if (lane == 0) {
                v.act.deltas[u64(slot) * (act_stride / 32) + blockIdx.x] = delta;
                if (v.act.sums) v.act.sums[u64(slot) * (act_stride / 32) + blockIdx.x] = sum;
            }
        }
    }
}

// grid (hidden / rows_per_cta, max_union); 256 threads: rows_per_cta (64, or fewer when that grid would leave SMs idle:
// the dense block has one "expert") down rows per CTA, Q4_K rows over K = inter.
template <int LPR>
__global__ void __launch_bounds__(256) down_q4k_kernel(b200moe_down_view v, u32 rows_per_cta) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (v.summary && *v.summary) return;  // a failed projection skips the whole down stage (routed_expert.hpp:17-19)
    const u32 j = blockIdx.y;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = I / 32, nblocks = I / 256;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * I);
    i32* s_sums = reinterpret_cast<i32*>(s_deltas + kR * groups);
    __shared__ u32 s_slots[kR];
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    constexpr u32 RPW = 32 / LPR;
    const u32 sub = lane / LPR, li = lane % LPR, base = sub * LPR;
    const u64 row_bytes = u64(nblocks) * kQ4KBlock;
    const u32 o0 = rows_per_cta * blockIdx.x;
    const u8* down = v.weights.down + (u64(expert) * H + o0) * row_bytes;
    const A8Smem xs{s_codes, s_deltas, s_sums, I};

    for (u32 p0 = eb; p0 < ee; p0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < (u32)nr) s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x];
        __syncthreads();
        stage_a8(v.act, s_slots, nr, I, s_codes, s_deltas, s_sums);
        __syncthreads();
        for (u32 t0 = warp * RPW; t0 < rows_per_cta; t0 += 8 * RPW) {
            const u32 t = t0 + sub;
            float val[kR];
            q4k_row<LPR>(down + u64(t) * row_bytes, nblocks, xs, nr, li, base, val);
            if (li == 0) {
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) v.raw[u64(s_slots[r]) * H + o0 + t] = val[r];
            }
        }
    }
}

// Q8_0 down in the four-chain rule (routed_expert.cpp:110-144): chain c = g % 4 adds E_g * (d * float(dot)) in
// ascending g; value = (acc0 + acc1) + (acc2 + acc3). One warp per down row, lane = group within a run of 32.
// grid (hidden / 32, max_union); 256 threads.
template <bool Q51>
__global__ void __launch_bounds__(256) down_q8_chain4_kernel(b200moe_down_view v) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (v.summary && *v.summary) return;
    const u32 j = blockIdx.y;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = I / 32;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * I);
    i32* s_sums = reinterpret_cast<i32*>(s_deltas + kR * groups);
    __shared__ u32 s_slots[kR];
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const u64 row_bytes = u64(groups) * (Q51 ? kQ51Block : kQ8Block);
    const u32 o0 = 32u * blockIdx.x;
    const u8* down = v.weights.down + (u64(expert) * H + o0) * row_bytes;
    const u32 chain = lane & 3u;

    for (u32 p0 = eb; p0 < ee; p0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < (u32)nr) s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x];
        __syncthreads();
        stage_a8(v.act, s_slots, nr, I, s_codes, s_deltas, s_sums);
        __syncthreads();
        for (u32 t = warp; t < 32; t += 8) {
            const u8* wrow = down + u64(t) * row_bytes;
            float acc[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r) acc[r] = 0.0f;
            for (u32 g0 = 0; g0 < groups; g0 += 32) {
                const u32 g = g0 + lane;
                const bool valid = g < groups;
                u32 q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                float d = 0.0f, mn = 0.0f;
                if (valid && Q51) {
                    // Q5_1 (routed_expert.cpp:124-133): 24-byte blocks, 8-byte aligned. Weight k < 16 = low nibble of byte
                    // k, k >= 16 = high nibble of byte k - 16, bit k of the 32 high bits on top: unsigned 0..31.
                    const uint2* b8 = reinterpret_cast<const uint2*>(wrow + u64(g) * kQ51Block);
                    const uint2 hd = __ldg(b8), qa = __ldg(b8 + 1), qb = __ldg(b8 + 2);
                    d = half_bits_to_float(hd.x & 0xffffu);
                    mn = half_bits_to_float(hd.x >> 16);
                    const u32 qs[4] = {qa.x, qa.y, qb.x, qb.y};
                    auto spread = [](u32 x) { return ((x & 1u) | ((x & 2u) << 7) | ((x & 4u) << 14) | ((x & 8u) << 21)) << 4; };
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        q[i] = (qs[i] & 0x0f0f0f0fu) | spread(hd.y >> (4 * i));
                        q[4 + i] = ((qs[i] >> 4) & 0x0f0f0f0fu) | spread(hd.y >> (16 + 4 * i));
                    }
                } else if (valid) {  // 34-byte blocks are only 2-byte aligned: halfword loads
                    const u16* b16 = reinterpret_cast<const u16*>(wrow + u64(g) * kQ8Block);
                    d = half_bits_to_float(b16[0]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[i] = u32(b16[1 + 2 * i]) | (u32(b16[2 + 2 * i]) << 16);
                }
                const u32 ng = min(32u, groups - g0);
#pragma unroll
                for (int r = 0; r < kR; ++r) {
                    if (r < nr) {
                        float term = 0.0f;
                        if (valid) {
                            const uint4* c = reinterpret_cast<const uint4*>(s_codes + u64(r) * I + 32u * g);
                            const uint4 c0 = c[0], c1 = c[1];
                            int dot = 0;
                            dot = __dp4a((int)q[0], (int)c0.x, dot); dot = __dp4a((int)q[1], (int)c0.y, dot);
                            dot = __dp4a((int)q[2], (int)c0.z, dot); dot = __dp4a((int)q[3], (int)c0.w, dot);
                            dot = __dp4a((int)q[4], (int)c1.x, dot); dot = __dp4a((int)q[5], (int)c1.y, dot);
                            dot = __dp4a((int)q[6], (int)c1.z, dot); dot = __dp4a((int)q[7], (int)c1.w, dot);
                            float combined = __fmul_rn(d, static_cast<float>(dot));
                            if (Q51) combined = __fadd_rn(combined, __fmul_rn(mn, static_cast<float>(s_sums[r * groups + g])));
                            term = __fmul_rn(s_deltas[r * groups + g], combined);
                        }
#pragma unroll
                        for (u32 k = 0; k < 8; ++k) {  // chain c takes groups c, c + 4, ... ascending
                            const float tv = __shfl_sync(0xffffffffu, term, chain + 4u * k);
                            if (chain + 4u * k < ng) acc[r] = __fadd_rn(acc[r], tv);
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                const float a0 = __shfl_sync(0xffffffffu, acc[r], 0), a1 = __shfl_sync(0xffffffffu, acc[r], 1);
                const float a2 = __shfl_sync(0xffffffffu, acc[r], 2), a3 = __shfl_sync(0xffffffffu, acc[r], 3);
                if (lane == 0 && r < nr) v.raw[u64(s_slots[r]) * H + o0 + t] = __fadd_rn(__fadd_rn(a0, a1), __fadd_rn(a2, a3));
            }
        }
    }
}

template <class K>
int set_smem(K kernel, u32 bytes) {
    return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}
inline int lanes_per_row(u32 nblocks) { return nblocks > 4 ? 32 : (nblocks > 2 ? 16 : 8); }

}  // namespace

int launch_gate_up_q4k(const b200moe_gate_up_view& v, cudaStream_t stream) {
    const u32 H = v.shape.hidden, I = v.shape.inter;
    if (v.max_union == 0) return B200MOE_OK;
    const u32 smem = kR * (H + H / 32 * 8) + 2 * kR * 32 * 4;
    const dim3 grid(I / 32, v.max_union);
#define B200_GU(L)                                                                   \
    {                                                                                \
        if (v.shape.gate_type == B200MOE_TYPE_Q5_K) {                                \
            if (int rc = set_smem(gate_up_q4k_kernel<L, true>, smem)) return rc;     \
            gate_up_q4k_kernel<L, true><<<grid, 256, smem, stream>>>(v);             \
        } else {                                                                     \
            if (int rc = set_smem(gate_up_q4k_kernel<L, false>, smem)) return rc;    \
            gate_up_q4k_kernel<L, false><<<grid, 256, smem, stream>>>(v);            \
        }                                                                            \
    }
    switch (lanes_per_row(H / 256)) {
        case 32: B200_GU(32) break;
        case 16: B200_GU(16) break;
        default: B200_GU(8) break;
    }
#undef B200_GU
    return after_launch("gate_up_q4k");
}

int launch_down_q4k(const b200moe_down_view& v, cudaStream_t stream) {
    const u32 H = v.shape.hidden, I = v.shape.inter;
    if (v.max_union == 0) return B200MOE_OK;
    const u32 smem = kR * (I + I / 32 * 8);
    u32 rpc = 64;  // rows per CTA: halved while the grid would not give every SM two CTAs (H is a multiple of 256)
    while (rpc > 8 && u64(H / rpc) * v.max_union < 2u * static_cast<u32>(device_sm_count())) rpc /= 2;  // at least two CTAs per SM
    const dim3 grid(H / rpc, v.max_union);
#define B200_DN(L)                                                     \
    {                                                                  \
        if (int rc = set_smem(down_q4k_kernel<L>, smem)) return rc;    \
        down_q4k_kernel<L><<<grid, 256, smem, stream>>>(v, rpc);       \
    }
    switch (lanes_per_row(I / 256)) {
        case 32: B200_DN(32) break;
        case 16: B200_DN(16) break;
        default: B200_DN(8) break;
    }
#undef B200_DN
    return after_launch("down_q4k");
}

int launch_down_q8_chain4(const b200moe_down_view& v, cudaStream_t stream) {
    const u32 H = v.shape.hidden, I = v.shape.inter;
    if (v.max_union == 0) return B200MOE_OK;
    const u32 smem = kR * (I + I / 32 * 8);
    if (v.shape.down_type == B200MOE_TYPE_Q5_1) {
        if (int rc = set_smem(down_q8_chain4_kernel<true>, smem)) return rc;
        down_q8_chain4_kernel<true><<<dim3(H / 32, v.max_union), 256, smem, stream>>>(v);
    } else {
        if (int rc = set_smem(down_q8_chain4_kernel<false>, smem)) return rc;
        down_q8_chain4_kernel<false><<<dim3(H / 32, v.max_union), 256, smem, stream>>>(v);
    }
    return after_launch("down_q8_chain4");
}

}  // namespace b200moe
