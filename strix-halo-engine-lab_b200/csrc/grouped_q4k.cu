// Routed experts, Qwen A8 family, GROUPED form for token blocks (prefill): the integer dots run on the 5th-generation
// tensor cores (tcgen05.mma kind::i8, accumulators in tensor memory), everything after the dots is the same declared
// FP32 arithmetic as the decode kernels, so the results are bit for bit those of gemv_q4k.cu / gemv_q4k_stream.cu
// (contract: src/cpu/core/routed_expert.hpp:9-15, row rule routed_expert.cpp:73-108; the reference's own tensor-core
// form is project_kernel / down_kernel over IMMA tiles, src/cuda/core/moe_a8.cuh:76-206, :225-341).
//
// Why one MMA per 32-wide group: the contract scales every group's EXACT integer dot by its own FP32 factors and adds
// the terms in a fixed order, so the tensor core may only produce dot_g, never a sum over groups. kind::i8 has K = 32:
// one instruction = one Q4_K group for a 128 x 64 tile (weight rows x tokens).
//
// Tile = (expert, 128 weight rows, 64 of the expert's tokens). gate/up: rows 0..63 are gate rows [64c, 64c + 64), rows
// 64..127 the up rows of the same outputs, so SwiGLU + the A8 rule of h finish inside the tile. down: 128 rows of H.
// A persistent CTA per SM walks tiles round-robin; four roles:
//   * issuer (1 warp, one thread): drives both asynchronous engines. The weight rows of a super-block arrive by two tiled
//     TMA copies (cp.async.bulk.tensor.2d: 144 bytes x 64 rows, the tile's gate rows and up rows, or two halves of its
//     down rows) into a raw ring, four super-blocks ahead of their use; the 4 MMAs of a stage (M 128, N 64, K 32,
//     s8 x s8 -> s32) go into one half of tensor memory as soon as the stage's operands are published, and are
//     committed to an mbarrier.
//   * unpacker warps (4): per stage = half a super-block (4 groups): unpack the rows' nibbles (from the raw ring) to
//     bytes into the MMA's canonical K-major layout (8-row x 16-byte core matrices), gather the tokens' A8 codes into
//     the same layout (ordinary loads, one stage ahead), stage the tokens' {E_g, S_g} and the rows' 16-byte block headers.
//   * drain warps (8): thread = (weight row = TMEM lane, 32 of the 64 tokens: the 8-token chunks alternate between the
//     two warp groups, so a tile with few tokens still uses every warp). tcgen05.ld brings 8 dots at a time;
//     x_g = E_g * ((d * sc_g) * float(dot_g) - (dmin * m_g) * float(S_g)), pair sums, the four chains acc_p over
//     ascending super-blocks, (a0 + a1) + (a2 + a3) at the end - exactly the decode kernels' order.
//   * tensor memory: 512 columns = 2 buffers x 4 groups x 64 tokens; smem stages follow the same two buffers.
// Every wait is bounded (kWaitLimit polls); on a timeout the roles stop working, the launch sets bit 30 of the job
// summary, frees tensor memory and returns.
//
// Roofline: CUDA-core FP32 issue, not the tensor pipe and not HBM - about 8 instructions per (row, token, group),
// against 1/32 of a tensor instruction. Weights are re-read from L2 once per token tile.
#include <cuda.h>

#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kGM = 128, kGN = 64;           // tile: weight rows x tokens
constexpr u32 kDrainWarps = 8, kLoadWarps = 4, kIssueWarps = 4;  // of the last group only warp 0 works (whole warp groups trade registers)
constexpr u32 kGThreads = (kDrainWarps + kLoadWarps + kIssueWarps) * 32;
constexpr u32 kStageGroups = 4;              // half a super-block per stage
constexpr u32 kTPT = kGN / (kDrainWarps / 4);   // tokens per drain thread (32)
constexpr u32 kDrainGroups = kDrainWarps / 4;    // warp groups sharing a tile's tokens: the 8-token chunks alternate between them
constexpr u32 kTmemCols = 512;
constexpr u32 kABytes = kStageGroups * kGM * 32, kBBytes = kStageGroups * kGN * 32, kEsBytes = kStageGroups * kGN * 8, kHdrBytes = kGM * 16;
constexpr u32 kStageBytes = kABytes + kBBytes + kEsBytes + kHdrBytes;  // 28672
constexpr u32 kOutBytes = kGN * kGM * 4;     // epilogue tile (gate/up)
constexpr u32 kMaxUnion = 1024;
constexpr u32 kRawDepth = 4, kRawBlock = kGM * kQ4KBlock;  // ring of raw super-blocks (128 rows x 144 B) fed by bulk copies
constexpr u32 kBarBytes = (6 + 2 * kRawDepth) * 8 + 16;  // full[2], empty[2], ready[2], raw_full[], raw_free[]
// above half an SM's shared memory: never two CTAs (and two TMEM allocations) per SM
constexpr u32 kGroupedSmem = 2 * kStageBytes + kOutBytes + (kMaxUnion + 2) * 4 + kBarBytes + kRawDepth * kRawBlock + 256;
static_assert(kGroupedSmem > 114u * 1024u && kGroupedSmem <= 227u * 1024u, "one CTA per SM, within the shared memory of an SM");
constexpr u32 kWaitLimit = 1u << 22;
constexpr u32 kAbortBit = B200MOE_JOB_WAIT_ABORTED;
// instruction descriptor: D = s32, A = B = signed 8-bit, both K-major, N = 64, M = 128
constexpr u32 kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((kGN >> 3) << 17) | ((kGM >> 4) << 24);

__device__ __forceinline__ u32 saddr(const void* p) { return static_cast<u32>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u64* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
}
// One tiled TMA copy: a box of 144 bytes x 64 rows of a [rows][row_bytes] byte tensor into shared memory (rows end up
// contiguous, 144 bytes each). x is a multiple of 16 bytes (a super-block boundary).
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, u32 x, u32 y, u64* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(saddr(dst)),
                 "l"(reinterpret_cast<u64>(map)), "r"(x), "r"(y), "r"(saddr(bar))
                 : "memory");
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
__global__ void __launch_bounds__(kGThreads, 1) grouped_q4k_kernel(const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1,
                                                                   GroupedArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stage0 = smem;                                       // 2 x kStageBytes
    float* s_out = reinterpret_cast<float*>(smem + 2 * kStageBytes);    // [kGN][kGM]
    u32* cum = reinterpret_cast<u32*>(smem + 2 * kStageBytes + kOutBytes);  // [kMaxUnion + 1]
    u64* bars = reinterpret_cast<u64*>(cum + kMaxUnion + 2);            // full[2], empty[2], ready[2], raw_full[], raw_free[]
    u32* s_tmem = reinterpret_cast<u32*>(bars + 6 + 2 * kRawDepth);
    volatile u32* s_abort = s_tmem + 1;
    unsigned char* raw = smem + ((2 * kStageBytes + kOutBytes + (kMaxUnion + 2) * 4 + kBarBytes + 127u) & ~127u);  // [kRawDepth][kRawBlock]

    if (kDown && a.summary && *a.summary) return;  // a failed or aborted projection skips the stage (routed_expert.hpp:17-19)

    const u32 tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const u32 n_union = min(a.routes.counts[0], kMaxUnion);
    for (u32 j = tid; j < n_union; j += kGThreads) cum[j + 1] = (a.routes.begins[j + 1] - a.routes.begins[j] + kGN - 1) / kGN;
    if (tid == 0) {
        cum[0] = 0;
        mbar_init(&bars[0], 1); mbar_init(&bars[1], 1);
        mbar_init(&bars[2], kDrainWarps * 32); mbar_init(&bars[3], kDrainWarps * 32);
        mbar_init(&bars[4], kLoadWarps * 32); mbar_init(&bars[5], kLoadWarps * 32);
        for (u32 i = 0; i < kRawDepth; ++i) { mbar_init(&bars[6 + i], 1); mbar_init(&bars[6 + kRawDepth + i], kLoadWarps * 32); }
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
    const u32 nblocks = K / 256;
    const u32 in_stride = a.in.stride ? a.in.stride : a.in.width, in_gs = in_stride / 32;
    u64* full = bars;
    u64* empty = bars + 2;
    u64* ready = bars + 4;
    u64* raw_full = bars + 6;
    u64* raw_free = bars + 6 + kRawDepth;
    bool ok = true;
    u32 n = 0;  // stage counter of this role (all roles count alike)
    const u32 my_tiles = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
    const u32 total_sb = my_tiles * nblocks;
    // Register split between whole warp groups (the CTA holds 512 x 128): the drain threads - 128 accumulators each - take
    // what the unpackers and the issuer group give up: 256 x 192 + 128 x 96 + 128 x 24 <= 512 x 128.
    static_assert(kDrainWarps * 32 * 192 + kLoadWarps * 32 * 96 + kIssueWarps * 32 * 24 <= kGThreads * 128, "setmaxnreg split exceeds the register file share");

    if (warp >= kDrainWarps + kLoadWarps) {
        // ============================================================================ issuer: TMA copies + MMA issue
        // One thread drives both asynchronous engines. The weight rows of super-block m of the CTA's sequence (tiles in
        // order, blocks in order) arrive by two tiled TMA copies (144 bytes x 64 rows each: the gate rows and the up rows
        // of the tile, or two halves of the down rows) into ring slot m % kRawDepth, kRawDepth super-blocks ahead of
        // their use; the four MMAs of a stage are issued as soon as the unpackers have published its operands.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
        if (warp == kDrainWarps + kLoadWarps) {
            u32 ck = 0xffffffffu, cy = 0;
            auto tma_block = [&](u32 mm) {  // lane 0 only
                const u32 k = mm / nblocks, b = mm - k * nblocks;
                if (k != ck) {
                    ck = k;
                    const Tile t = find_tile(a, cum, n_union, blockIdx.x + k * gridDim.x);
                    cy = kDown ? t.expert * H + kGM * t.c : t.expert * I + 64u * t.c;
                }
                const u32 slot = mm % kRawDepth;
                unsigned char* dst = raw + slot * kRawBlock;
                mbar_expect_tx(&raw_full[slot], kRawBlock);
                tma_2d(dst, &tm0, b * kQ4KBlock, cy, &raw_full[slot]);
                tma_2d(dst + 64u * kQ4KBlock, kDown ? &tm0 : &tm1, b * kQ4KBlock, kDown ? cy + 64u : cy, &raw_full[slot]);
            };
            if (lane == 0) for (u32 mm = 0; mm < min(kRawDepth, total_sb); ++mm) tma_block(mm);
            u32 m = 0;
            for (u32 k = 0; k < my_tiles; ++k) {
                for (u32 s = 0; s < 2 * nblocks; ++s, ++n) {
                    const u32 buf = n & 1u, use = n >> 1, hf = s & 1u;
                    if (ok) ok = mbar_wait(&ready[buf], use & 1u, s_abort);  // the stage's operands are in shared memory
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok && lane == 0) {
                        tc_fence_after();
                        const u32 abase = saddr(stage0 + buf * kStageBytes), bbase = abase + kABytes;
#pragma unroll
                        for (u32 gi = 0; gi < kStageGroups; ++gi)
                            mma_i8(tmem + buf * (kStageGroups * kGN) + gi * kGN, smem_desc(abase + gi * (kGM * 32), 128, 256),
                                   smem_desc(bbase + gi * (kGN * 32), 128, 256));
                        mma_commit(&full[buf]);
                    }
                    if (hf == 1) {
                        if (m + kRawDepth < total_sb) {  // the slot has been read out: the block kRawDepth ahead takes it
                            if (ok) ok = mbar_wait(&raw_free[m % kRawDepth], (m / kRawDepth) & 1u, s_abort);
                            ok = __all_sync(0xffffffffu, ok);
                            if (ok && lane == 0) tma_block(m + kRawDepth);
                        }
                        ++m;
                    }
                }
            }
            if (!ok) for (u32 i = 0; i < 400; ++i) __nanosleep(100);  // an aborted launch: let the copies in flight land before the CTA retires
        }
    } else if (warp >= kDrainWarps) {
        // ================================================================================================= unpackers
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        const u32 lt = tid - kDrainWarps * 32;            // 0..127 = weight row of the tile
        // The tokens' bytes (A8 codes, deltas, sums) come by ordinary loads - L2 hits - one stage AHEAD: the registers
        // filled here are stored in the next iteration, so their latency hides behind this stage's work.
        const u32 tok_b = lt >> 1, half = lt & 1u, tok_e = lt & 63u, ge = lt >> 6;
        struct Tok { uint4 cc[4]; float e0, e1; i32 s0, s1; };
        u32 tk = 0xffffffffu;
        const i8* t_codes = nullptr;
        const float* t_deltas = nullptr;
        const i32* t_sums = nullptr;
        const u32 stages_per_tile = 2 * nblocks, total_stages = my_tiles * stages_per_tile;
        auto load_tok = [&](u32 sn, Tok& r) {  // stage sn of the CTA's sequence
            const u32 k = sn / stages_per_tile, s = sn - k * stages_per_tile, b = s >> 1, hf = s & 1u;
            if (k != tk) {
                tk = k;
                const Tile t = find_tile(a, cum, n_union, blockIdx.x + k * gridDim.x);
                // the token this thread gathers codes for (two threads per token), and the one it stages {E, S} for
                const u32 ent_b = t.eb + min(tok_b, t.nt - 1), ent_e = t.eb + min(tok_e, t.nt - 1);
                const u32 src_b = kDown ? a.routes.slots[ent_b] : a.routes.rows[ent_b];
                const u32 src_e = kDown ? a.routes.slots[ent_e] : a.routes.rows[ent_e];
                t_codes = a.in.codes + u64(src_b) * in_stride;
                t_deltas = a.in.deltas + u64(src_e) * in_gs;
                t_sums = a.in.sums + u64(src_e) * in_gs;
            }
            const uint4* cq = reinterpret_cast<const uint4*>(t_codes + 32u * (8u * b + 4u * hf)) + 4 * half;
#pragma unroll
            for (int c = 0; c < 4; ++c) r.cc[c] = __ldg(cq + c);
            const u32 g0 = 8u * b + 4u * hf + 2u * ge;   // this thread stages pair ge of the stage for token tok_e
            r.e0 = __ldg(t_deltas + g0); r.e1 = __ldg(t_deltas + g0 + 1);
            r.s0 = __ldg(t_sums + g0); r.s1 = __ldg(t_sums + g0 + 1);
        };
        Tok tok{};
        if (total_stages) load_tok(0, tok);
        u32 m = 0;  // super-block counter of the sequence
        for (; n < total_stages; ++n) {
            const u32 buf = n & 1u, use = n >> 1, hf = n & 1u;  // a tile has an even number of stages
            const u32 rslot = m % kRawDepth;
            const Tok cur = tok;
            if (n + 1 < total_stages) load_tok(n + 1, tok);
            if (ok && hf == 0) ok = mbar_wait(&raw_full[rslot], (m / kRawDepth) & 1u, s_abort);  // the super-block's rows have landed
            if (ok) ok = mbar_wait(&empty[buf], (use & 1u) ^ 1u, s_abort);  // the drain is done with this buffer
            unsigned char* st = stage0 + buf * kStageBytes;
            if (ok) {
                const uint4* wq = reinterpret_cast<const uint4*>(raw + rslot * kRawBlock + lt * kQ4KBlock);
                const uint4 hdr = wq[0];
                // A: row lt, chunk c = (pair pp, 16-byte half kc): low nibbles -> group 2pp, high nibbles -> group 2pp + 1
                const u32 core = (lt >> 3) * 256u + (lt & 7u) * 16u;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const u32 pp = c >> 1, kc = c & 1;
                    const uint4 q = wq[1 + 4 * hf + c];
                    uint4 lo, hi;
                    lo.x = q.x & 0x0f0f0f0fu; lo.y = q.y & 0x0f0f0f0fu; lo.z = q.z & 0x0f0f0f0fu; lo.w = q.w & 0x0f0f0f0fu;
                    hi.x = (q.x >> 4) & 0x0f0f0f0fu; hi.y = (q.y >> 4) & 0x0f0f0f0fu; hi.z = (q.z >> 4) & 0x0f0f0f0fu; hi.w = (q.w >> 4) & 0x0f0f0f0fu;
                    *reinterpret_cast<uint4*>(st + (2 * pp) * (kGM * 32) + core + kc * 128u) = lo;
                    *reinterpret_cast<uint4*>(st + (2 * pp + 1) * (kGM * 32) + core + kc * 128u) = hi;
                }
                // B: token tok_b, chunks 4 * half .. + 3 of the stage's 128 code bytes: chunk = (group gi, half kc)
                unsigned char* sb = st + kABytes + (tok_b >> 3) * 256u + (tok_b & 7u) * 16u;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const u32 ch = 4 * half + c, gi = ch >> 1, kc = ch & 1u;
                    *reinterpret_cast<uint4*>(sb + gi * (kGN * 32) + kc * 128u) = cur.cc[c];
                }
                reinterpret_cast<float4*>(st + kABytes + kBBytes)[ge * kGN + tok_e] =
                    make_float4(cur.e0, cur.e1, static_cast<float>(cur.s0), static_cast<float>(cur.s1));
                reinterpret_cast<uint4*>(st + kABytes + kBBytes + kEsBytes)[lt] = hdr;
                // generic-proxy accesses (the stores above, the reads of the raw slot) before the async proxy's:
                // the tensor core reading the operands, the next TMA copy overwriting the slot
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&ready[buf]);
                if (hf == 1) mbar_arrive(&raw_free[rslot]);
            }
            if (hf == 1) ++m;
        }
    } else {
        // ================================================================================================ drain
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
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
                    const u32 tbase = tmem + lane_addr + buf * (kStageGroups * kGN) + 8u * w;
#pragma unroll
                    for (int pp = 0; pp < 2; ++pp) {
                        const Factors f = q4k_factors(hdr, 2 * hf + pp);
                        const float2 D = make_float2(f.Dl, f.Dh), DMn = make_float2(-f.DMl, -f.DMh);
#pragma unroll
                        for (int tq = 0; tq < (int)kTPT / 8; ++tq) {  // chunk 2 * tq + w of the tile: a short tile still uses every warp
                            if (8u * (kDrainGroups * tq + w) >= t.nt) continue;  // no valid token in these 8 columns (warp-uniform)
                            u32 dl[8], dh[8];
                            tmem_ld8(tbase + (2 * pp) * kGN + 8 * kDrainGroups * tq, dl);
                            tmem_ld8(tbase + (2 * pp + 1) * kGN + 8 * kDrainGroups * tq, dh);
                            tmem_wait_ld();
                            tie8(dl); tie8(dh);
                            const float4* e4 = es + pp * kGN + 8u * (kDrainGroups * tq + w);
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
                        const u32 tok = 8u * (kDrainGroups * (i >> 3) + w) + (i & 7);
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
                    s_out[(8u * (kDrainGroups * (i >> 3) + w) + (i & 7)) * kGM + o] = __fadd_rn(__fadd_rn(acc[i][0], acc[i][1]), __fadd_rn(acc[i][2], acc[i][3]));
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

// Tensor map of a [rows][row_bytes] byte tensor with boxes of 144 bytes x 64 rows (no swizzle, no interleave). The
// encoder is the driver's cuTensorMapEncodeTiled, looked up through the runtime (no link against the driver library).
int encode_rows_map(const u8* base, u64 row_bytes, u64 rows, CUtensorMap* out) {
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    if (!fn) return fail(B200MOE_ERR_CUDA, "grouped: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};       // bytes between rows: a multiple of 16 (144 per super-block)
    const cuuint32_t box[2] = {kQ4KBlock, 64};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<u8*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(B200MOE_ERR_CUDA, "grouped: cuTensorMapEncodeTiled failed (%d)", static_cast<int>(r));
    return B200MOE_OK;
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
    CUtensorMap tm0, tm1;
    const u64 rb = u64(v.shape.hidden / 256) * kQ4KBlock, rows = u64(v.shape.experts) * v.shape.inter;
    if (int rc = encode_rows_map(v.weights.gate, rb, rows, &tm0)) return rc;
    if (int rc = encode_rows_map(v.weights.up, rb, rows, &tm1)) return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_q4k_kernel<false>), kGroupedSmem)) return rc;
    grouped_q4k_kernel<false><<<grid_size(), kGThreads, kGroupedSmem, stream>>>(tm0, tm1, a);
    return after_launch("gate_up_q4k_grouped");
}

int launch_down_q4k_grouped(const b200moe_down_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    GroupedArgs a{};
    a.shape = v.shape; a.routes = v.routes; a.w0 = v.weights.down; a.in = v.act; a.raw = v.raw;
    a.summary = const_cast<u32*>(v.summary);
    a.n_row_tiles = v.shape.hidden / kGM; a.K = v.shape.inter;
    CUtensorMap tm0;
    if (int rc = encode_rows_map(v.weights.down, u64(v.shape.inter / 256) * kQ4KBlock, u64(v.shape.experts) * v.shape.hidden, &tm0)) return rc;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(grouped_q4k_kernel<true>), kGroupedSmem)) return rc;
    grouped_q4k_kernel<true><<<grid_size(), kGThreads, kGroupedSmem, stream>>>(tm0, tm0, a);
    return after_launch("down_q4k_grouped");
}

}  // namespace b200moe
