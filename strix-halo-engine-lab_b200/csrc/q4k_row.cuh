// Device pieces of the segment-streaming form of the Q4_K x A8 row rule (gemv_q4k_wide.cu): mbarrier / bulk-copy / TMA
// wrappers whose waits are bounded, and the arithmetic of one (super-block, pair) of the contract of
// src/cpu/core/routed_expert.hpp:9-15 - the same operation sequence as gemv_q4k.cu and gemv_q4k_stream.cu, so every
// form produces the same bits.
#pragma once
#include <cuda.h>

#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace q4k {

constexpr u32 kAbortBit = B200MOE_JOB_WAIT_ABORTED;

// ---- PTX: mbarrier, bulk copy, tiled TMA copy ------------------------------------------------------------------------
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
// One poll. The instruction may suspend the warp until the phase completes or `hint_ns` nanoseconds have passed: a waiting
// warp then issues nothing, instead of spinning in the issue slots that the working warps of its scheduler need.
__device__ __forceinline__ bool mbar_try_wait(u64* bar, u32 parity, u32 hint_ns = 0) {
    u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(saddr(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: false when `limit` polls ran out (the abort flag is then raised) or another role has raised it.
constexpr u32 kWaitHintNs = 1000;
__device__ __forceinline__ bool mbar_wait(u64* bar, u32 parity, u32 limit, volatile u32* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;  // the common case: the phase is already complete
    for (u32 i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity, kWaitHintNs)) return true;
        if ((i & 7u) == 7u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// Untiled bulk copy global -> shared: both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(saddr(dst)),
                 "l"(src), "r"(bytes), "r"(saddr(bar))
                 : "memory");
}
// Tiled copy of one box of a 2-D tensor map (this GPU's own memory, no multicast). x counts elements of the map's type;
// x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_2d(void* dst, const CUtensorMap* map, u32 x, u32 y, u64* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(saddr(dst)),
                 "l"(reinterpret_cast<u64>(map)), "r"(x), "r"(y), "r"(saddr(bar))
                 : "memory");
}
__device__ __forceinline__ int dp4a_us(u32 a, u32 b, int c) {  // unsigned bytes of a times signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Exact int -> float for |v| < 2^22 without the conversion pipe: (1.5 * 2^23 + v) - 1.5 * 2^23.
__device__ __forceinline__ float small_int_to_float(int v) { return __fsub_rn(__int_as_float(0x4b400000 + v), 12582912.0f); }

// ---- one (super-block, pair) of the row rule -------------------------------------------------------------------------
// Decoded factors of one super-block for pair p: D / DM of groups 2p (l) and 2p + 1 (h).
struct Factors { float Dl, DMl, Dh, DMh; };
__device__ __forceinline__ Factors q4k_factors(const uint4& hdr, u32 p) {
    const float d = half_bits_to_float(hdr.x & 0xffffu), dm = half_bits_to_float(hdr.x >> 16);
    // the eight 6-bit scales / mins, four per word (routed_expert.cpp:65-71, vectorised over the four bytes)
    const u32 sc_lo = hdr.y & 0x3f3f3f3fu, mn_lo = hdr.z & 0x3f3f3f3fu;
    const u32 sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
    const u32 mn_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
    const u32 scw = p < 2u ? sc_lo : sc_hi, mnw = p < 2u ? mn_lo : mn_hi;
    const u32 sh = 16u * (p & 1u);
    const int s0 = (scw >> sh) & 0xffu, s1 = (scw >> (sh + 8u)) & 0xffu;
    const int m0 = (mnw >> sh) & 0xffu, m1 = (mnw >> (sh + 8u)) & 0xffu;
    Factors f;
    f.Dl = __fmul_rn(d, small_int_to_float(s0));
    f.Dh = __fmul_rn(d, small_int_to_float(s1));
    f.DMl = __fmul_rn(dm, small_int_to_float(m0));
    f.DMh = __fmul_rn(dm, small_int_to_float(m1));
    return f;
}
// The 64 nibbles of one (super-block, pair): low nibbles (group 2p) as bytes, high nibbles (group 2p + 1) left in
// place as 16 * q. Split once per block, used by every entry.
struct Nibbles { u32 lo[8], hi[8]; };
__device__ __forceinline__ Nibbles split_nibbles(const uint4& q0, const uint4& q1) {
    Nibbles n;
    const u32 w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) { n.lo[i] = w[i] & 0x0f0f0f0fu; n.hi[i] = w[i] & 0xf0f0f0f0u; }
    return n;
}
// Exact group dots: two interleaved chains of four for each group (integer sums are order free). c0, c1: the 32 codes of
// group 2p; c2, c3: those of group 2p + 1.
__device__ __forceinline__ void dots(const Nibbles& n, const uint4& c0, const uint4& c1, const uint4& c2, const uint4& c3, int* lo, int* hi) {
    int la = __dp4a(static_cast<int>(n.lo[0]), static_cast<int>(c0.x), 0), lb = __dp4a(static_cast<int>(n.lo[1]), static_cast<int>(c0.y), 0);
    la = __dp4a(static_cast<int>(n.lo[2]), static_cast<int>(c0.z), la); lb = __dp4a(static_cast<int>(n.lo[3]), static_cast<int>(c0.w), lb);
    la = __dp4a(static_cast<int>(n.lo[4]), static_cast<int>(c1.x), la); lb = __dp4a(static_cast<int>(n.lo[5]), static_cast<int>(c1.y), lb);
    la = __dp4a(static_cast<int>(n.lo[6]), static_cast<int>(c1.z), la); lb = __dp4a(static_cast<int>(n.lo[7]), static_cast<int>(c1.w), lb);
    // bytes 16 * q (unsigned) times signed codes = 16 * dot, an exact shift away
    int ha = dp4a_us(n.hi[0], c2.x, 0), hb = dp4a_us(n.hi[1], c2.y, 0);
    ha = dp4a_us(n.hi[2], c2.z, ha); hb = dp4a_us(n.hi[3], c2.w, hb);
    ha = dp4a_us(n.hi[4], c3.x, ha); hb = dp4a_us(n.hi[5], c3.y, hb);
    ha = dp4a_us(n.hi[6], c3.z, ha); hb = dp4a_us(n.hi[7], c3.w, hb);
    *lo = la + lb;
    *hi = (ha + hb) >> 4;
}
// x_2p + x_2p+1 with x_j = E_g * (D_j * float(dot_j) - DM_j * float(S_g)).
__device__ __forceinline__ float pair_value(const Factors& f, int lo, int hi, float El, float Eh, float Sl, float Sh) {
    const float xl = __fmul_rn(El, __fsub_rn(__fmul_rn(f.Dl, small_int_to_float(lo)), __fmul_rn(f.DMl, Sl)));
    const float xh = __fmul_rn(Eh, __fsub_rn(__fmul_rn(f.Dh, small_int_to_float(hi)), __fmul_rn(f.DMh, Sh)));
    return __fadd_rn(xl, xh);
}

}  // namespace q4k
}  // namespace b200moe
