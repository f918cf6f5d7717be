// Routed experts, Qwen A8 family, GROUPED form for token blocks (prefill): the integer dots run on the 5th-generation
// tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), everything after the dots is the same declared
// FP32 arithmetic as the decode kernels, so the results are bit for bit those of gemv_q4k.cu / gemv_q4k_stream.cu
// (contract: src/cpu/core/routed_expert.hpp:9-15, row rule routed_expert.cpp:73-108; the reference's own tensor-core
// form is project_kernel / down_kernel over IMMA tiles, src/cuda/moe_a8.cuh:76-206, :225-341).
//
// Why one MMA per 32-wide group: the contract scales every group's EXACT integer dot by its own FP32 factors and adds
// the terms in a fixed order, so the tensor core may only produce dot_g, never a sum over groups. kind::i8 has K = 32:
// one instruction = one Q4_K group for a 128 x 64 tile (weight rows x tokens).
//
// Tile = (expert, 128 weight rows, 64 of the expert's tokens). gate/up: rows 0..63 are gate rows [64c, 64c + 64), rows
// 64..127 the up rows of the same outputs, so SwiGLU + the A8 rule of h finish inside the tile. down: 128 rows of H.
// A persistent CTA per SM walks tiles round-robin; three roles:
//   * loader warps (4): per stage = half a super-block (4 groups): unpack the rows' nibbles to bytes into the MMA's
//     canonical K-major layout (8-row x 16-byte core matrices), gather the tokens' A8 codes into the same layout, and
//     stage the tokens' {E_g, S_g} and the rows' 16-byte block headers. Its first thread then issues the 4 MMAs
//     (M 128, N 64, K 32, s8 x s8 -> s32) into one half of tensor memory and commits them to an mbarrier.
//   * drain warps (8): thread = (weight row = TMEM lane, 32 of the 64 tokens). tcgen05.ld brings 8 dots at a time;
//     x_g = E_g * ((d * sc_g) * float(dot_g) - (dmin * m_g) * float(S_g)), pair sums, the four chains acc_p over
//     ascending super-blocks, (a0 + a1) + (a2 + a3) at the end - exactly the decode kernels' order.
//   * tensor memory: 512 columns = 2 buffers x 4 groups x 64 tokens; smem stages follow the same two buffers.
// Every wait is bounded (kWaitLimit polls); on a timeout the roles stop working, the launch sets bit 30 of the job
// summary, frees tensor memory and returns.
//
// Roofline: CUDA-core FP32 issue, not the tensor pipe and not HBM - about 8 instructions per (row, token, group),
// against 1/32 of a tensor instruction. Weights are re-read from L2 once per token tile.
#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kGM = 128, kGN = 64;           // tile: weight rows x tokens
constexpr u32 kDrainWarps = 8, kLoadWarps = 4, kGThreads = (kDrainWarps + kLoadWarps) * 32;
constexpr u32 kStageGroups = 4;              // half a super-block per stage
constexpr u32 kTPT = kGN / (kDrainWarps / 4);   // tokens per drain thread (16)
constexpr u32 kTmemCols = 512;
constexpr u32 kABytes = kStageGroups * kGM * 32, kBBytes = kStageGroups * kGN * 32, kEsBytes = kStageGroups * kGN * 8, kHdrBytes = kGM * 16;
constexpr u32 kStageBytes = kABytes + kBBytes + kEsBytes + kHdrBytes;  // 28672
constexpr u32 kOutBytes = kGN * kGM * 4;     // epilogue tile (gate/up)
constexpr u32 kMaxUnion = 1024;
constexpr u32 kGroupedSmem = 120u * 1024u;   // above half an SM's shared memory: never two CTAs (and two TMEM allocations) per SM
constexpr u32 kWaitLimit = 1u << 22;
constexpr u32 kAbortBit = 1u << 30;
// instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = 64, M = 128
constexpr u32 kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((kGN >> 3) << 17) | ((kGM >> 4) << 24);

__device__ __forceinline__ u32 saddr(const void* p) { return static_cast<u32>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64* bar, u32 parity) {
    u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(saddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(u64* bar, u32 parity, volatile u32* abort_flag) {
    for (u32 i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 127u) == 127u) {
            if (*abort_flag) return false;
            __nanosleep(64);
        }
    }
    *abort_flag = 1;
    return false;
}
// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; LBO = bytes between the two
// 16-byte K chunks of a row group, SBO = bytes between 8-row groups; bits 46-47 = 1 (Blackwell descriptor version).
__device__ __forceinline__ u64 smem_desc(u32 addr, u32 lbo, u32 sbo) {
    return u64((addr >> 4) & 0x3fffu) | (u64((lbo >> 4) & 0x3fffu) << 16) | (u64((sbo >> 4) & 0x3fffu) << 32) | (u64(1) << 46);
}
__device__ __forceinline__ void mma_i8(u32 d_tmem, u64 a_desc, u64 b_desc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(u64* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(u32 taddr, u32* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
// Ties registers to the point after tcgen05.wait::ld, so that no use of a loaded value is scheduled before the wait.
__device__ __forceinline__ void tie8(u32* v) {
    asm volatile("" : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ float small_int_to_float(int v) { return __fsub_rn(__int_as_float(0x4b400000 + v), 12582912.0f); }
// Two FP32 lanes per instruction (Blackwell packed FP32): each lane is one IEEE round-to-nearest multiplication, the
// same result as two scalar instructions at half the issue slots. Only the multiplications are packed: a packed add
// fed by a packed multiply did not reproduce the scalar bits on B200 (it behaves as contracted), so the adds stay scalar.
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 c;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(reinterpret_cast<u64&>(c)) : "l"(reinterpret_cast<const u64&>(a)), "l"(reinterpret_cast<const u64&>(b)));
    return c;
}

struct Factors { float Dl, DMl, Dh, DMh; };
__device__ __forceinline__ Factors q4k_factors(const uint4& hdr, u32 p) {  // routed_expert.cpp:65-71, as in gemv_q4k_stream.cu
    const float d = half_bits_to_float(hdr.x & 0xffffu), dm = half_bits_to_float(hdr.x >> 16);
    const u32 sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
    const u32 sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
    const u32 mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
    const u32 scw = p < 2u ? sc_lo : sc_hi, mnw = p < 2u ? mn_lo : mn_hi;
    const u32 sh = 16u * (p & 1u);
    Factors f;
    f.Dl = __fmul_rn(d, small_int_to_float((scw >> sh) & 0xffu));
    f.Dh = __fmul_rn(d, small_int_to_float((scw >> (sh + 8u)) & 0xffu));
    f.DMl = __fmul_rn(dm, small_int_to_float((mnw >> sh) & 0xffu));
    f.DMh = __fmul_rn(dm, small_int_to_float((mnw >> (sh + 8u)) & 0xffu));
    return f;
}

struct GroupedArgs {
    b200moe_shape shape;
    b200moe_routes routes;
    const u8* w0;            // gate (gate/up mode) or down tensor
    const u8* w1;            // up
    b200moe_a8_rows in;      // x (gate/up: indexed by row) or act (down: indexed by slot)
    b200moe_a8_rows act;     // gate/up output
    float* gate_out;
    float* up_out;
    float* raw;              // down output [slots][hidden]
    u32* row_status;
    u32* summary;
    u32 n_row_tiles;         // inter / 64 (gate/up) or hidden / 128 (down)
    u32 K;                   // hidden (gate/up) or inter (down)
};

struct Tile { u32 expert, eb, nt, c, tt; };

// Tile id -> (union expert, token tile, row tile): row tiles fastest, then the expert's token tiles, experts ascending.
__device__ __forceinline__ Tile find_tile(const GroupedArgs& a, const u32* cum, u32 n_union, u32 id) {
    const u32 q = id / a.n_row_tiles;
    Tile t;
    t.c = id - q * a.n_row_tiles;
    u32 lo = 0, hi = n_union;  // largest j with cum[j] <= q
    while (hi - lo > 1) {
        const u32 mid = (lo + hi) >> 1;
        if (cum[mid] <= q) lo = mid; else hi = mid;
    }
    t.tt = q - cum[lo];
    t.expert = a.routes.experts[lo];
    const u32 b0 = a.routes.begins[lo], b1 = a.routes.begins[lo + 1];
    t.eb = b0 + kGN * t.tt;
    t.nt = min(kGN, b1 - t.eb);
    return t;
}

template <bool kDown>
__global__ void __launch_bounds__(kGThreads, 1) grouped_q4k_kernel(GroupedArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stage0 = smem;                                       // 2 x kStageBytes
    float* s_out = reinterpret_cast<float*>(smem + 2 * kStageBytes);    // [kGN][kGM]
    u32* cum = reinterpret_cast<u32*>(smem + 2 * kStageBytes + kOutBytes);  // [kMaxUnion + 1]
    u64* bars = reinterpret_cast<u64*>(cum + kMaxUnion + 2);            // full[2], empty[2]
    u32* s_tmem = reinterpret_cast<u32*>(bars + 4);
    volatile u32* s_abort = s_tmem + 1;

    if (kDown && a.summary && (*a.summary & ~kAbortBit)) return;  // a failed projection skips the stage (routed_expert.hpp:17-19)

    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const u32 n_union = min(a.routes.counts[0], kMaxUnion);
    for (u32 j = tid; j < n_union; j += kGThreads) cum[j + 1] = (a.routes.begins[j + 1] - a.routes.begins[j] + kGN - 1) / kGN;
    if (tid == 0) {
        cum[0] = 0;
        mbar_init(&bars[0], 1); mbar_init(&bars[1], 1);
        mbar_init(&bars[2], kDrainWarps * 32); mbar_init(&bars[3], kDrainWarps * 32);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 0) {  // inclusive scan of the token-tile counts, 32 at a time
        u32 carry = 0;
        for (u32 j0 = 0; j0 < n_union; j0 += 32) {
            u32 v = j0 + lane < n_union ? cum[j0 + lane + 1] : 0u;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, v, d); if (lane >= (u32)d) v += o; }
            if (j0 + lane < n_union) cum[j0 + lane + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(s_tmem)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const u32 tmem = *s_tmem;
    const u32 n_tiles = cum[n_union] * a.n_row_tiles;
    const u32 K = a.K, I = a.shape.inter, H = a.shape.hidden;
    const u32 nblocks = K / 256, row_bytes = nblocks * kQ4KBlock;
    const u32 in_stride = a.in.stride ? a.in.stride : a.in.width, in_gs = in_stride / 32;
    u64* full = bars;
    u64* empty = bars + 2;
    bool ok = true;
    u32 n = 0;  // stage counter of this role (both roles count alike)

    if (warp >= kDrainWarps) {
        // ===================================================================================== loader + MMA issue
        // Register split (the CTA holds 384 x 168): the loaders give registers up, the drain threads - 128 accumulators
        // each - take them: 128 x 72 + 256 x 216 = 384 x 168.
        static_assert(kLoadWarps * 32 * 72 + kDrainWarps * 32 * 216 <= kGThreads * 168, "setmaxnreg split exceeds the register file share");
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        const u32 lt = tid - kDrainWarps * 32;            // 0..127 = weight row of the tile
        for (u32 id = blockIdx.x; id < n_tiles; id += gridDim.x) {
            const Tile t = find_tile(a, cum, n_union, id);
            const u8* wrow;
            if (kDown) wrow = a.w0 + (u64(t.expert) * H + kGM * t.c + lt) * row_bytes;
            else wrow = (lt < 64 ? a.w0 : a.w1) + (u64(t.expert) * I + 64u * t.c + (lt & 63u)) * row_bytes;
            // the token this thread gathers codes for (two threads per token), and the one it stages {E, S} for
            const u32 tok_b = lt >> 1, half = lt & 1u, tok_e = lt & 63u, ge = lt >> 6;
            const u32 ent_b = t.eb + min(tok_b, t.nt - 1), ent_e = t.eb + min(tok_e, t.nt - 1);
            const u32 src_b = kDown ? a.routes.slots[ent_b] : a.routes.rows[ent_b];
            const u32 src_e = kDown ? a.routes.slots[ent_e] : a.routes.rows[ent_e];
            const i8* codes = a.in.codes + u64(src_b) * in_stride;
            const float* deltas = a.in.deltas + u64(src_e) * in_gs;
            const i32* sums = a.in.sums + u64(src_e) * in_gs;
            for (u32 s = 0; s < 2 * nblocks; ++s, ++n) {
                const u32 buf = n & 1u, use = n >> 1, b = s >> 1, hf = s & 1u;
                // global loads first: they do not depend on the buffer
                const uint4* wq = reinterpret_cast<const uint4*>(wrow + u64(b) * kQ4KBlock);
                const uint4 hdr = __ldg(wq);
                uint4 q[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) q[c] = __ldg(wq + 1 + 4 * hf + c);
                const uint4* cq = reinterpret_cast<const uint4*>(codes + 32u * (8u * b + 4u * hf)) + 4 * half;
                uint4 cc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) cc[c] = __ldg(cq + c);
                const u32 g0 = 8u * b + 4u * hf + 2u * ge;   // this thread stages pair ge of the stage for token tok_e
                const float e0 = __ldg(deltas + g0), e1 = __ldg(deltas + g0 + 1);
                const i32 s0 = __ldg(sums + g0), s1 = __ldg(sums + g0 + 1);
                if (ok) ok = mbar_wait(&empty[buf], (use & 1u) ^ 1u, s_abort);  // the drain is done with this buffer
                unsigned char* st = stage0 + buf * kStageBytes;
                if (ok) {
                    // A: row lt, chunk c = (pair pp, 16-byte half kc): low nibbles -> group 2pp, high nibbles -> group 2pp + 1
                    const u32 core = (lt >> 3) * 256u + (lt & 7u) * 16u;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const u32 pp = c >> 1, kc = c & 1;
                        uint4 lo, hi;
                        lo.x = q[c].x & 0x0f0f0f0fu; lo.y = q[c].y & 0x0f0f0f0fu; lo.z = q[c].z & 0x0f0f0f0fu; lo.w = q[c].w & 0x0f0f0f0fu;
                        hi.x = (q[c].x >> 4) & 0x0f0f0f0fu; hi.y = (q[c].y >> 4) & 0x0f0f0f0fu; hi.z = (q[c].z >> 4) & 0x0f0f0f0fu; hi.w = (q[c].w >> 4) & 0x0f0f0f0fu;
                        *reinterpret_cast<uint4*>(st + (2 * pp) * (kGM * 32) + core + kc * 128u) = lo;
                        *reinterpret_cast<uint4*>(st + (2 * pp + 1) * (kGM * 32) + core + kc * 128u) = hi;
                    }
                    // B: token tok_b, chunks 4 * half .. + 3 of the stage's 128 code bytes: chunk = (group gi, half kc)
                    unsigned char* sb = st + kABytes + (tok_b >> 3) * 256u + (tok_b & 7u) * 16u;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const u32 ch = 4 * half + c, gi = ch >> 1, kc = ch & 1u;
                        *reinterpret_cast<uint4*>(sb + gi * (kGN * 32) + kc * 128u) = cc[c];
                    }
                    reinterpret_cast<float4*>(st + kABytes + kBBytes)[ge * kGN + tok_e] =
                        make_float4(e0, e1, static_cast<float>(s0), static_cast<float>(s1));
                    reinterpret_cast<uint4*>(st + kABytes + kBBytes + kEsBytes)[lt] = hdr;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> the tensor core's reads
                asm volatile("bar.sync 2, %0;" ::"r"(kLoadWarps * 32) : "memory");
                if (lt == 0 && ok && !*s_abort) {
                    tc_fence_after();
                    const u32 abase = saddr(st), bbase = abase + kABytes;
#pragma unroll
                    for (u32 gi = 0; gi < kStageGroups; ++gi)
                        mma_i8(tmem + buf * (kStageGroups * kGN) + gi * kGN, smem_desc(abase + gi * (kGM * 32), 128, 256),
                               smem_desc(bbase + gi * (kGN * 32), 128, 256));
                    mma_commit(&full[buf]);
                }
            }
        }
    } else {
        // ================================================================================================ drain
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const u32 quarter = warp & 3u, w = warp >> 2;   // TMEM lane quarter, token half
        const u32 o = 32u * quarter + lane;             // weight row of the tile = TMEM lane
        const u32 lane_addr = (32u * quarter) << 16;
        const u32 act_stride = a.act.stride ? a.act.stride : a.act.width;
        for (u32 id = blockIdx.x; id < n_tiles; id += gridDim.x) {
            const Tile t = find_tile(a, cum, n_union, id);
            float acc[kTPT][4];
#pragma unroll
            for (int i = 0; i < (int)kTPT; ++i) { acc[i][0] = 0.0f; acc[i][1] = 0.0f; acc[i][2] = 0.0f; acc[i][3] = 0.0f; }
            for (u32 b = 0; b < nblocks; ++b) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf, ++n) {
                    const u32 buf = n & 1u, use = n >> 1;
                    if (ok) ok = mbar_wait(&full[buf], use & 1u, s_abort);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) continue;
                    tc_fence_after();
                    const unsigned char* st = stage0 + buf * kStageBytes;
                    const float4* es = reinterpret_cast<const float4*>(st + kABytes + kBBytes);  // [pair][token] {E_l, E_h, S_l, S_h}
                    const uint4 hdr = reinterpret_cast<const uint4*>(st + kABytes + kBBytes + kEsBytes)[o];
                    const u32 tbase = tmem + lane_addr + buf * (kStageGroups * kGN) + kTPT * w;
#pragma unroll
                    for (int pp = 0; pp < 2; ++pp) {
                        const Factors f = q4k_factors(hdr, 2 * hf + pp);
                        const float2 D = make_float2(f.Dl, f.Dh), DMn = make_float2(-f.DMl, -f.DMh);
#pragma unroll
                        for (int tq = 0; tq < (int)kTPT / 8; ++tq) {
                            if (kTPT * w + 8u * tq >= t.nt) continue;  // no valid token in these 8 columns (warp-uniform)
                            u32 dl[8], dh[8];
                            tmem_ld8(tbase + (2 * pp) * kGN + 8 * tq, dl);
                            tmem_ld8(tbase + (2 * pp + 1) * kGN + 8 * tq, dh);
                            tmem_wait_ld();
                            tie8(dl); tie8(dh);
                            const float4* e4 = es + pp * kGN + kTPT * w + 8 * tq;
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float4 e = e4[i];
                                const float2 fd = make_float2(__int2float_rn(static_cast<int>(dl[i])), __int2float_rn(static_cast<int>(dh[i])));
                                // x = E * ((D * float(dot)) - (DM * S)) for the pair's two groups; (-DM) * S = -(DM * S) exactly
                                const float2 pa = mul2(D, fd), pb = mul2(DMn, make_float2(e.z, e.w));
                                const float2 x = mul2(make_float2(e.x, e.y), make_float2(__fadd_rn(pa.x, pb.x), __fadd_rn(pa.y, pb.y)));
                                acc[8 * tq + i][2 * hf + pp] = __fadd_rn(acc[8 * tq + i][2 * hf + pp], __fadd_rn(x.x, x.y));
                            }
                        }
                    }
                    tc_fence_before();
                    mbar_arrive(&empty[buf]);  // every drain thread arrives: the buffer (TMEM half + stage) is free
                }
            }
            // (a0 + a1) + (a2 + a3)
            if (kDown) {
                if (ok) {
#pragma unroll
                    for (int i = 0; i < (int)kTPT; ++i) {
                        const u32 tok = kTPT * w + i;
                        if (tok < t.nt) {
                            const u32 slot = a.routes.slots[t.eb + tok];
                            a.raw[u64(slot) * H + kGM * t.c + o] = __fadd_rn(__fadd_rn(acc[i][0], acc[i][1]), __fadd_rn(acc[i][2], acc[i][3]));
                        }
                    }
                }
            } else {
                asm volatile("bar.sync 3, %0;" ::"r"(kDrainWarps * 32) : "memory");  // the previous tile's epilogue has read s_out
#pragma unroll
                for (int i = 0; i < (int)kTPT; ++i)
                    s_out[(kTPT * w + i) * kGM + o] = __fadd_rn(__fadd_rn(acc[i][0], acc[i][1]), __fadd_rn(acc[i][2], acc[i][3]));
                asm volatile("bar.sync 3, %0;" ::"r"(kDrainWarps * 32) : "memory");
                // SwiGLU + the A8 rule: one warp per (token, 32 outputs); the tile holds 2 groups of 32 per token
                for (u32 task = warp; ok && task < 2 * t.nt; task += kDrainWarps) {
                    const u32 tok = task >> 1, q32 = task & 1u;
                    const float g = s_out[tok * kGM + 32u * q32 + lane], u = s_out[tok * kGM + 64u + 32u * q32 + lane];
                    const u32 slot = a.routes.slots[t.eb + tok], group = 2u * t.c + q32, o_col = 32u * group + lane;
                    if (a.gate_out) { a.gate_out[u64(slot) * I + o_col] = g; a.up_out[u64(slot) * I + o_col] = u; }
                    const float h = swiglu_qwen(g, u);
                    const bool bad = __any_sync(0xffffffffu, !finite_f(g) || !finite_f(u) || !finite_f(h));
                    if (bad) {  // fail closed: nothing of the group is written (routed_expert.cpp:147-156)
                        if (lane == 0) {
                            if (a.row_status) atomicOr(&a.row_status[a.routes.rows[t.eb + tok]], B200MOE_ROW_PROJECTION_NONFINITE);
                            if (a.summary) atomicOr(a.summary, B200MOE_ROW_PROJECTION_NONFINITE);
                        }
                        continue;
                    }
                    float delta;
                    int sum;
                    const int code = a8_quantize_lane(h, &delta, &sum);
                    a.act.codes[u64(slot) * act_stride + o_col] = static_cast<i8>(code);
                    if (lane == 0) {
                        a.act.deltas[u64(slot) * (act_stride / 32) + group] = delta;
                        if (a.act.sums) a.act.sums[u64(slot) * (act_stride / 32) + group] = sum;
                    }
                }
            }
        }
    }
    if (!ok && lane == 0 && a.summary) atomicOr(a.summary, kAbortBit);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

bool grouped_shape_ok(const b200moe_shape& s) {
    return s.gate_type == B200MOE_TYPE_Q4_K && s.down_type == B200MOE_TYPE_Q4_K && s.hidden % 256 == 0 && s.inter % 256 == 0 &&
           s.hidden % kGM == 0 && s.inter % 64 == 0 && s.experts <= kMaxUnion;
}

int grid_size() {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

}  // namespace

bool grouped_fits(const b200moe_shape& s, bool have_sums) { return have_sums && grouped_shape_ok(s); }

int launch_gate_up_q4k_grouped(const b200moe_gate_up_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    GroupedArgs a{};
    a.shape = v.shape; a.routes = v.routes; a.w0 = v.weights.gate; a.w1 = v.weights.up; a.in = v.x; a.act = v.act;
    a.gate_out = v.gate_out; a.up_out = v.up_out; a.row_status = v.row_status; a.summary = v.summary;
    a.n_row_tiles = v.shape.inter / 64; a.K = v.shape.hidden;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_q4k_kernel<false>), kGroupedSmem)) return rc;
    grouped_q4k_kernel<false><<<grid_size(), kGThreads, kGroupedSmem, stream>>>(a);
    return after_launch("gate_up_q4k_grouped");
}

int launch_down_q4k_grouped(const b200moe_down_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    GroupedArgs a{};
    a.shape = v.shape; a.routes = v.routes; a.w0 = v.weights.down; a.in = v.act; a.raw = v.raw;
    a.summary = const_cast<u32*>(v.summary);
    a.n_row_tiles = v.shape.hidden / kGM; a.K = v.shape.inter;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_q4k_kernel<true>), kGroupedSmem)) return rc;
    grouped_q4k_kernel<true><<<grid_size(), kGThreads, kGroupedSmem, stream>>>(a);
    return after_launch("down_q4k_grouped");
}

}  // namespace b200moe
