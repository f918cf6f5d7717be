// Routed experts, Qwen A8 family, decode form on Blackwell: persistent GEMVs fed by the bulk-copy engine.
//
// Same arithmetic as gemv_q4k.cu (the contract of src/cpu/core/routed_expert.hpp:9-15, bit for bit); what changes is how
// the bytes reach the SM and how few instructions touch each byte.
//
//  * One persistent CTA per SM walks a contiguous run of work items (expert, 32-output group | 64 hidden outputs); the
//    runs are cut by estimated cost (entries per expert), not by count, so the CTAs finish together.
//  * Four producer warps stream weight rows - contiguous, 16-byte aligned GGUF bytes - into a ring of shared-memory
//    stages with cp.async.bulk (global -> shared, completion counted on an mbarrier; eight lanes of a producer issue the
//    eight row copies of its octet). A stage holds one OCTET = 8 weight rows, laid down with a stride whose 16-byte count
//    is odd, which makes the consumers' 128-bit reads conflict free. The A8 rows the consumers read (x for gate/up, h of
//    the run's entries for down) are staged in shared memory with cp.async.
//  * Each consumer warp owns whole octets (octet n goes to warp n mod W): lane = (row of the octet, pair p). A lane walks
//    its row's super-blocks in ascending order, so the serial chain acc_p += pair_p needs no shuffle at all; the final
//    (a0 + a1) + (a2 + a3) is two xor-shuffles. Integer -> float conversions use the exact 2^23 magic-number form.
//  * gate/up: the last warp to finish an item's eight octets (a shared-memory counter) runs SwiGLU + the A8 rule.
//
// Every wait on an mbarrier is bounded: after kWaitLimit polls the waiter raises an abort flag, all roles stop waiting
// (they still walk their loops, doing no work), the producers drain the copies they have in flight (bounded), bit 30 of the
// job summary is set and the kernel returns: the host reads a status, the GPU never hangs.
//
// Roofline: HBM. Algorithmic bytes per item = 64 rows x K / 256 x 144.

#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr int kR = 4;             // entries per pass over an octet
constexpr u32 kMaxWarps = 16;     // consumer warps at most
constexpr u32 kWaitLimit = 1u << 22;
constexpr u32 kAbortBit = B200MOE_JOB_WAIT_ABORTED;
constexpr u32 kOctetsPerItem = 8;
constexpr u32 kProducers = 4;       // producer warps

// ---- PTX: mbarrier + bulk copy ---------------------------------------------------------------------------------------
__device__ __forceinline__ u32 saddr(const void* p) { return static_cast<u32>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(u64* bar, u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(saddr(bar)), "r"(bytes) : "memory");
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
// Bounded wait; false when the limit ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(u64* bar, u32 parity, volatile u32* abort_flag) {
    for (u32 i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 127u) == 127u) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, u32 bytes, u64* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(saddr(dst)),
                 "l"(src), "r"(bytes), "r"(saddr(bar))
                 : "memory");
}
__device__ __forceinline__ int dp4a_us(u32 a, u32 b, int c) {  // unsigned bytes of a times signed bytes of b
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Exact int -> float for |v| < 2^22 without the conversion pipe: (1.5 * 2^23 + v) - 1.5 * 2^23.
__device__ __forceinline__ float small_int_to_float(int v) { return __fsub_rn(__int_as_float(0x4b400000 + v), 12582912.0f); }

// ---- shared plan -----------------------------------------------------------------------------------------------------
struct StreamPlan {
    u32 stages;        // ring depth (octets)
    u32 warps;         // consumer warps
    u32 row_bytes;     // bytes of one weight row
    u32 row_stride;    // stride of a row inside a stage (odd count of 16-byte units)
    u32 stage_bytes;   // 8 * row_stride
    u32 n_chunks;      // items per expert
    u32 chunk_magic;   // floor(2^32 / n_chunks) + 1: item / n_chunks = umulhi(item, magic) for item < 2^20
    u32 item_slots;    // power of two: item state ring (gate/up)
    u32 max_entries;   // bound of the entries of one expert (the window's rows)
    u32 x_rows;        // rows of the A8 input copied to shared memory (gate/up)
    u32 stage_entries; // entries of the CTA's run whose activations are copied to shared memory (down)
};

// Ring of stages. An mbarrier's phase test only tells odd from even uses of a slot, and here the successive uses of a
// slot belong to different warps (producers and consumers alike), which may drift a whole lap apart. So every slot also
// carries two generation words: gen = octet index + 1 written by the producer before it arms the barrier, rel = octet
// index + 1 written by the consumer when it is done. A consumer first waits for ITS generation to be armed and only then
// for the phase; a producer waits for the previous use's release by exact match. No wait can be satisfied by another lap.
struct Ring {
    unsigned char* data;
    u64* full;
    volatile u32* gen;
    volatile u32* rel;
    volatile u32* abort_flag;
};

__device__ __forceinline__ void ring_init(const Ring& r, u32 stages) {
    if (threadIdx.x < stages) {
        mbar_init(&r.full[threadIdx.x], 1);
        r.gen[threadIdx.x] = 0;
        r.rel[threadIdx.x] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x == 0) *r.abort_flag = 0;
    __syncthreads();
}
// Bounded spin until *word == want; false when the limit ran out or another role aborted.
__device__ __forceinline__ bool flag_wait(volatile u32* word, u32 want, volatile u32* abort_flag) {
    for (u32 i = 0; i < kWaitLimit; ++i) {
        if (*word == want) return true;
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = 1;
    return false;
}
// Consumer side: the octet's generation is armed, then its bytes have landed.
__device__ __forceinline__ bool stage_wait(const Ring& ring, u32 slot, u32 q, u32 phase) {
    if (!flag_wait(&ring.gen[slot], q + 1u, ring.abort_flag)) return false;
    return mbar_wait(&ring.full[slot], phase, ring.abort_flag);
}
// Consumer side: done reading the stage.
__device__ __forceinline__ void stage_release(const Ring& ring, u32 slot, u32 q) {
    __threadfence_block();
    ring.rel[slot] = q + 1u;
}

// The producer warps: kProducers warps share the octet stream (octet q goes to producer q mod kProducers); lanes 0..7
// of a producer issue the eight row copies of its octet. A bulk copy costs its issuing thread a few hundred cycles
// whatever its size, so one thread - or one warp - issuing 1 KB row copies tops out near half of HBM bandwidth;
// four warps of eight lanes reach it (measured on B200: 1 warp 3.0 TB/s, 2 warps 5.8, 4 warps 6.5).
// `row_of(item, octet)` gives the first of the octet's 8 consecutive weight rows.
template <class RowOf>
__device__ __forceinline__ void produce(const Ring& ring, const StreamPlan& plan, u32 first_item, u32 n_local, u32 pw, RowOf row_of) {
    const u32 lane = threadIdx.x & 31u;
    const bool one_copy = plan.row_stride == plan.row_bytes;  // rows already conflict free: one copy per octet
    const u32 local_octets = n_local * kOctetsPerItem;
    u32 slot = pw % plan.stages, phase = (pw / plan.stages) & 1u, q = pw;
    bool ok = true;
    for (; q < local_octets; q += kProducers) {
        if (q >= plan.stages) ok = flag_wait(&ring.rel[slot], q - plan.stages + 1u, ring.abort_flag);  // the slot's previous use is done
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the consumers' reads precede the copies below
        const unsigned char* src = row_of(first_item + (q >> 3), q & 7u);
        unsigned char* dst = ring.data + u64(slot) * plan.stage_bytes;
        if (lane == 0) {
            ring.gen[slot] = q + 1u;
            __threadfence_block();
            mbar_expect_tx(&ring.full[slot], 8u * plan.row_bytes);
        }
        __syncwarp();
        if (one_copy) {
            if (lane == 0) bulk_g2s(dst, src, 8u * plan.row_bytes, &ring.full[slot]);
        } else if (lane < 8) {
            bulk_g2s(dst + lane * plan.row_stride, src + u64(lane) * plan.row_bytes, plan.row_bytes, &ring.full[slot]);
        }
        slot += kProducers;
        while (slot >= plan.stages) { slot -= plan.stages; phase ^= 1u; }
    }
    if (!ok && lane == 0) {  // wait (bounded) for this producer's copies still in flight before the CTA retires
        const u32 back = (plan.stages + kProducers - 1) / kProducers * kProducers;  // keeps n on this producer's octets
        for (u32 n = q > back ? q - back : pw; n < q; n += kProducers)
            for (u32 i = 0; i < (kWaitLimit >> 6); ++i)
                if (mbar_try_wait(&ring.full[n % plan.stages], (n / plan.stages) & 1u)) break;
    }
}

// Work split: every CTA takes a contiguous run of items (expert-major, chunks ascending) of about equal COST, not
// equal count: an item of an expert with ne entries costs the fixed per-block decode once per pass of up to kR entries
// plus the per-entry dots, roughly 3 * ceil(ne / kR) + 2 * ne. Item i belongs to CTA b when its cumulative cost start
// lies in [total * b / G, total * (b + 1) / G). Every warp computes the run itself (two short warp scans over the
// union's counts), so no barrier is involved. Returns the first item and the count.
__device__ __forceinline__ u32 item_cost(u32 ne) { return 3u * ((ne + kR - 1) / kR) + 2u * ne; }
__device__ __forceinline__ u32 warp_inclusive_scan(u32 v, u32 lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) { const u32 o = __shfl_up_sync(0xffffffffu, v, d); if (lane >= (u32)d) v += o; }
    return v;
}
__device__ __forceinline__ void item_range(const StreamPlan& plan, const b200moe_routes& routes, u32 n_union, u32* first_item, u32* n_local) {
    const u32 lane = threadIdx.x & 31u, G = gridDim.x, b = blockIdx.x, nc = plan.n_chunks;
    u32 total = 0;
    for (u32 j0 = 0; j0 < n_union; j0 += 32) {
        const u32 j = j0 + lane;
        const u32 c = j < n_union ? item_cost(__ldg(routes.begins + j + 1) - __ldg(routes.begins + j)) * nc : 0u;
        total += __shfl_sync(0xffffffffu, warp_inclusive_scan(c, lane), 31);
    }
    const u32 n_items = n_union * nc;
    const u32 B0 = static_cast<u32>(u64(total) * b / G), B1 = static_cast<u32>(u64(total) * (b + 1) / G);
    u32 lo = n_items, hi = n_items, cum = 0;  // a boundary at `total` means "past the last item"
    for (u32 j0 = 0; j0 < n_union; j0 += 32) {
        const u32 j = j0 + lane;
        const u32 ci = j < n_union ? item_cost(__ldg(routes.begins + j + 1) - __ldg(routes.begins + j)) : 0u;
        const u32 c = ci * nc, incl = warp_inclusive_scan(c, lane), excl = cum + incl - c;
        const bool h0 = c && B0 >= excl && B0 < excl + c, h1 = c && B1 >= excl && B1 < excl + c;
        const u32 c0 = h0 ? j * nc + (B0 - excl + ci - 1) / ci : 0u, c1 = h1 ? j * nc + (B1 - excl + ci - 1) / ci : 0u;
        const u32 m0 = __ballot_sync(0xffffffffu, h0), m1 = __ballot_sync(0xffffffffu, h1);
        if (m0) lo = __shfl_sync(0xffffffffu, c0, __ffs(m0) - 1);
        if (m1) hi = __shfl_sync(0xffffffffu, c1, __ffs(m1) - 1);
        cum += __shfl_sync(0xffffffffu, incl, 31);
    }
    *first_item = lo;
    *n_local = hi - lo;
}

// item -> (union expert j, chunk) without a hardware division.
__device__ __forceinline__ void split_item(const StreamPlan& plan, u32 item, u32* j, u32* chunk) {
    *j = plan.n_chunks == 1 ? item : __umulhi(item, plan.chunk_magic);
    *chunk = item - *j * plan.n_chunks;
}
// A consumer warp's walk over its octets q = warp, warp + W, ...: ring slot and phase kept incrementally.
struct Cursor {
    u32 q, slot, phase;
    __device__ __forceinline__ void advance(const StreamPlan& plan) {
        q += plan.warps;
        slot += plan.warps;
        while (slot >= plan.stages) { slot -= plan.stages; phase ^= 1u; }
    }
};

// Entry metadata of the item an octet belongs to, fetched one octet ahead so that its two dependent global loads
// (begins[j], then the first entries' ids) hide behind the current octet's arithmetic.
struct Meta { u32 chunk, eb, ne; };
__device__ __forceinline__ Meta load_meta(const StreamPlan& plan, const b200moe_routes& routes, u32 item) {
    u32 j;
    Meta m;
    split_item(plan, item, &j, &m.chunk);
    m.eb = __ldg(routes.begins + j);
    m.ne = __ldg(routes.begins + j + 1) - m.eb;
    return m;
}
__device__ __forceinline__ void load_first(const u32* __restrict__ ids, const Meta& m, u32* first) {
#pragma unroll
    for (int r = 0; r < kR; ++r) first[r] = __ldg(ids + m.eb + min(u32(r), m.ne - 1u));
}

// ---- the row rule over one octet -----------------------------------------------------------------------------------
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
// Exact group dots: two interleaved chains of four for each group (integer sums are order free).
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
__device__ __forceinline__ float pair_value(const Factors& f, int lo, int hi, float El, float Eh, float Sl, float Sh) {
    const float xl = __fmul_rn(El, __fsub_rn(__fmul_rn(f.Dl, small_int_to_float(lo)), __fmul_rn(f.DMl, Sl)));
    const float xh = __fmul_rn(Eh, __fsub_rn(__fmul_rn(f.Dh, small_int_to_float(hi)), __fmul_rn(f.DMh, Sh)));
    return __fadd_rn(xl, xh);
}
// (a0 + a1) + (a2 + a3) over the four pair lanes of a row; every lane of the row gets the value.
__device__ __forceinline__ float tree4(float a) {
    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 1));
    return __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, 2));
}

// One weight row (this lane's pair p of every super-block, ascending) against NR staged A8 rows (gate/up form: codes
// chunk-swapped and {E, E, S, S} packs in shared memory). acc[r] is the lane's chain acc_p of row r.
template <int NR>
__device__ __forceinline__ void row_gate_up(const uint4* blk, u32 nblocks, u32 p, u32 swz, u32 H, const unsigned char* const* xr, float* acc) {
#pragma unroll(NR == 1 ? 4 : (NR == 2 ? 2 : 1))
    for (u32 b = 0; b < nblocks; ++b, blk += kQ4KBlock / 16) {
        const uint4 hdr = blk[0], q0 = blk[1 + 2 * p], q1 = blk[2 + 2 * p];
        const Factors f = q4k_factors(hdr, p);
        const Nibbles n = split_nibbles(q0, q1);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint4* c = reinterpret_cast<const uint4*>(xr[r] + 256u * b);
            const uint4 c0 = c[swz], c1 = c[1 - swz], c2 = c[2 + swz], c3 = c[3 - swz];
            const float4 es = *reinterpret_cast<const float4*>(xr[r] + (H - 48u * p) + 64u * b);
            int lo, hi;
            dots(n, c0, c1, c2, c3, &lo, &hi);
            acc[r] = __fadd_rn(acc[r], pair_value(f, lo, hi, es.x, es.y, es.z, es.w));
        }
    }
}
// The same against NR A8 rows given by generic pointers (down form: codes / deltas / sums of the slots' activations,
// staged in shared memory for the first entries of the CTA's run, in global memory beyond).
template <int NR>
__device__ __forceinline__ void row_down(const uint4* blk, u32 nblocks, u32 p, const i8* const* cr, const float* const* dr, const i32* const* sr,
                                         float* acc) {
#pragma unroll(NR == 1 ? 3 : 1)
    for (u32 b = 0; b < nblocks; ++b, blk += kQ4KBlock / 16) {
        const uint4 hdr = blk[0], q0 = blk[1 + 2 * p], q1 = blk[2 + 2 * p];
        const Factors f = q4k_factors(hdr, p);
        const Nibbles n = split_nibbles(q0, q1);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint4* c = reinterpret_cast<const uint4*>(cr[r] + 256u * b);
            const uint4 c0 = c[0], c1 = c[1], c2 = c[2], c3 = c[3];
            const float2 e = *reinterpret_cast<const float2*>(dr[r] + 8u * b);
            const int2 sm = *reinterpret_cast<const int2*>(sr[r] + 8u * b);
            int lo, hi;
            dots(n, c0, c1, c2, c3, &lo, &hi);
            acc[r] = __fadd_rn(acc[r], pair_value(f, lo, hi, e.x, e.y, small_int_to_float(sm.x), small_int_to_float(sm.y)));
        }
    }
}

// ---- gate/up ---------------------------------------------------------------------------------------------------------
// A8 input rows in shared memory, per row: codes[H] with the two 16-byte chunks of every 32-byte half swapped for
// pairs 2 and 3 (bank spread), then per (super-block, pair) 16 bytes {E_2p, E_2p+1, float(S_2p), float(S_2p+1)}.
// Issued as asynchronous copies from short loops, so that every request is in flight at once; the sums arrive as
// integers in the pack's last two words and are converted in place by finish_x_rows once the copies have landed.
__device__ __forceinline__ void cp_async(u32 dst, const void* src, int bytes) {
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
    else if (bytes == 8) asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void copy_x_rows_async(const b200moe_a8_rows& x, u32 rows, u32 H, unsigned char* dst, u32 nthreads) {
    const u32 stride = x.stride ? x.stride : x.width, row_bytes = H + H / 4, gs = stride / 32;
    const bool al8 = (reinterpret_cast<uintptr_t>(x.deltas) % 8 == 0) && (reinterpret_cast<uintptr_t>(x.sums) % 8 == 0) && gs % 2 == 0;
    for (u32 r = 0; r < rows; ++r) {
        const i8* src = x.codes + u64(r) * stride;  // 16-byte aligned rows (checked by the caller)
        const u32 d = saddr(dst + u64(r) * row_bytes);
        for (u32 c = threadIdx.x; c < H / 16; c += nthreads) cp_async(d + 16u * (c ^ ((c >> 3) & 1u)), src + 16u * c, 16);
        const u32 es = d + H;
        const float* dl = x.deltas + u64(r) * gs;
        const i32* sm = x.sums + u64(r) * gs;
        if (al8) {
            for (u32 g2 = threadIdx.x; g2 < H / 64; g2 += nthreads) { cp_async(es + 16u * g2, dl + 2 * g2, 8); cp_async(es + 16u * g2 + 8u, sm + 2 * g2, 8); }
        } else {
            for (u32 g = threadIdx.x; g < H / 32; g += nthreads) {
                cp_async(es + 16u * (g >> 1) + 4u * (g & 1u), dl + g, 4);
                cp_async(es + 16u * (g >> 1) + 8u + 4u * (g & 1u), sm + g, 4);
            }
        }
    }
}
__device__ __forceinline__ void finish_x_rows(u32 rows, u32 H, unsigned char* dst, u32 nthreads) {
    const u32 row_bytes = H + H / 4;
    for (u32 i = threadIdx.x; i < rows * (H / 64); i += nthreads) {
        const u32 r = i / (H / 64), g2 = i - r * (H / 64);
        int2* s = reinterpret_cast<int2*>(dst + u64(r) * row_bytes + H + 16u * g2 + 8u);
        const int2 v = *s;
        *reinterpret_cast<float2*>(s) = make_float2(static_cast<float>(v.x), static_cast<float>(v.y));
    }
}

__global__ void __launch_bounds__((kMaxWarps + kProducers) * 32, 1) gate_up_q4k_stream_kernel(b200moe_gate_up_view v, StreamPlan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    const u32 H = v.shape.hidden, I = v.shape.inter, nblocks = H / 256;
    const u32 ME = plan.max_entries;
    unsigned char* at = smem + u64(plan.stages) * plan.stage_bytes;
    float* s_gu = reinterpret_cast<float*>(at);                       // [item_slots][2][ME][32]
    at += u64(plan.item_slots) * 2 * ME * 32 * 4;
    u64* bars = reinterpret_cast<u64*>(at);
    at += 2 * plan.stages * 8;
    u32* s_done = reinterpret_cast<u32*>(at);                         // [item_slots] octets finished
    at += plan.item_slots * 4;
    u32* s_flag = reinterpret_cast<u32*>(at);
    at += 16;
    at = smem + ((at - smem + 15) & ~size_t(15));
    unsigned char* x_copy = at;
    const Ring ring{smem, bars, reinterpret_cast<volatile u32*>(bars + plan.stages), reinterpret_cast<volatile u32*>(bars + plan.stages) + plan.stages, s_flag};
    for (u32 i = threadIdx.x; i < plan.item_slots; i += blockDim.x) s_done[i] = 0;
    ring_init(ring, plan.stages);

    const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const u32 n_union = v.routes.counts[0];
    const u64 row_bytes = plan.row_bytes;
    u32 first_item, n_local;

    if (warp >= plan.warps) {  // ------------------------------------------------------------- producer warps
        item_range(plan, v.routes, n_union, &first_item, &n_local);
        produce(ring, plan, first_item, n_local, warp - plan.warps, [&](u32 item, u32 o) {
            u32 j, gx;
            split_item(plan, item, &j, &gx);
            const u64 row = u64(v.routes.experts[j]) * I + 32u * gx + 8u * (o & 3u);
            return (o < 4 ? v.weights.gate : v.weights.up) + row * row_bytes;
        });
        return;
    }

    // ------------------------------------------------------------------------------------------ consumer warps
    copy_x_rows_async(v.x, plan.x_rows, H, x_copy, plan.warps * 32);  // in flight while the item run is worked out
    item_range(plan, v.routes, n_union, &first_item, &n_local);
    const u32 x_row_bytes = H + H / 4;
    const u32 rsub = lane >> 2, p = lane & 3u;
    const u32 swz = p >> 1;  // chunk swap of the staged codes
    const u32 act_stride = v.act.stride ? v.act.stride : v.act.width;
    const u32 local_octets = n_local * kOctetsPerItem;
    bool ok = true;
    Meta m{};
    u32 first[kR];
    if (warp < local_octets) m = load_meta(plan, v.routes, first_item + (warp >> 3));
    asm volatile("cp.async.wait_all;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"r"(plan.warps * 32) : "memory");
    finish_x_rows(plan.x_rows, H, x_copy, plan.warps * 32);
    asm volatile("bar.sync 1, %0;" ::"r"(plan.warps * 32) : "memory");
    if (warp < local_octets) load_first(v.routes.rows, m, first);
    for (Cursor cur{warp, warp % plan.stages, (warp / plan.stages) & 1u}; cur.q < local_octets; cur.advance(plan)) {
        const u32 slot = cur.slot, local_item = cur.q >> 3, o = cur.q & 7u;
        const bool has_next = cur.q + plan.warps < local_octets;
        Meta nm{};
        if (has_next) nm = load_meta(plan, v.routes, first_item + ((cur.q + plan.warps) >> 3));
        const u32 gx = m.chunk, eb = m.eb, ne = min(m.ne, ME);
        const u32 islot = local_item & (plan.item_slots - 1);
        float* s_g = s_gu + u64(islot) * 2 * ME * 32;
        float* s_u = s_g + ME * 32;
        if (ok) ok = stage_wait(ring, slot, cur.q, cur.phase);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { m = nm; if (has_next) load_first(v.routes.rows, m, first); continue; }
        const unsigned char* wrow = ring.data + u64(slot) * plan.stage_bytes + rsub * plan.row_stride;
        float* dst = (o < 4 ? s_g : s_u) + 8u * (o & 3u) + rsub;
        for (u32 e0 = 0; e0 < ne; e0 += kR) {
            const int nr = static_cast<int>(min(u32(kR), ne - e0));
            const unsigned char* xr[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r)
                xr[r] = x_copy + (e0 == 0 ? first[r] : v.routes.rows[eb + e0 + min(r, nr - 1)]) * x_row_bytes + 64u * p;
            float acc[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r) acc[r] = 0.0f;
            const uint4* blk = reinterpret_cast<const uint4*>(wrow);
            switch (nr) {  // no per-entry branches inside the block loop
                case 1: row_gate_up<1>(blk, nblocks, p, swz, H, xr, acc); break;
                case 2: row_gate_up<2>(blk, nblocks, p, swz, H, xr, acc); break;
                case 3: row_gate_up<3>(blk, nblocks, p, swz, H, xr, acc); break;
                default: row_gate_up<4>(blk, nblocks, p, swz, H, xr, acc); break;
            }
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                if (r < nr) {
                    const float val = tree4(acc[r]);
                    if (p == 0) dst[(e0 + r) * 32] = val;
                }
            }
        }
        __syncwarp();
        if (lane == 0) stage_release(ring, slot, cur.q);  // the stage is free for the producers
        // item completion: the warp that brings the count to eight runs the epilogue
        __threadfence_block();
        u32 done = 0;
        if (lane == 0) done = atomicAdd(&s_done[islot], 1u) + 1u;
        done = __shfl_sync(0xffffffffu, done, 0);
        m = nm;  // the next octet's entries: second hop of the prefetch
        if (has_next) load_first(v.routes.rows, m, first);
        if (done != kOctetsPerItem) continue;
        __threadfence_block();
        if (lane == 0) s_done[islot] = 0;
        for (u32 r = 0; r < ne; ++r) {  // SwiGLU + the A8 rule over the item's 32 outputs
            const float g = s_g[r * 32 + lane], u = s_u[r * 32 + lane];
            const u32 slot_id = v.routes.slots[eb + r], o_col = 32u * gx + lane;
            if (v.gate_out) { v.gate_out[u64(slot_id) * I + o_col] = g; v.up_out[u64(slot_id) * I + o_col] = u; }
            const float h = swiglu_qwen(g, u);
            const bool bad = __any_sync(0xffffffffu, !finite_f(g) || !finite_f(u) || !finite_f(h));
            if (bad) {  // fail closed: nothing of the group is written (routed_expert.cpp:147-156)
                if (lane == 0) {
                    if (v.row_status) atomicOr(&v.row_status[v.routes.rows[eb + r]], B200MOE_ROW_PROJECTION_NONFINITE);
                    if (v.summary) atomicOr(v.summary, B200MOE_ROW_PROJECTION_NONFINITE);
                }
                continue;
            }
            float delta;
            int sum;
            const int code = a8_quantize_lane(h, &delta, &sum);
            v.act.codes[u64(slot_id) * act_stride + o_col] = static_cast<i8>(code);
            if (lane == 0) {
                v.act.deltas[u64(slot_id) * (act_stride / 32) + gx] = delta;
                if (v.act.sums) v.act.sums[u64(slot_id) * (act_stride / 32) + gx] = sum;
            }
        }
    }
    if (!ok && lane == 0 && v.summary) atomicOr(v.summary, kAbortBit);
}

// ---- down ------------------------------------------------------------------------------------------------------------
// Item = (expert, 64 hidden outputs) = 8 octets. Activations (the A8 of h) are read from global memory: every lane of a
// row group reads the same addresses, so the loads are broadcasts served by L1 / L2.
__global__ void __launch_bounds__((kMaxWarps + kProducers) * 32, 1) down_q4k_stream_kernel(b200moe_down_view v, StreamPlan plan) {
    extern __shared__ __align__(128) unsigned char smem[];
    const u32 H = v.shape.hidden, I = v.shape.inter, nblocks = I / 256;
    u64* bars = reinterpret_cast<u64*>(smem + u64(plan.stages) * plan.stage_bytes);
    u32* s_flag = reinterpret_cast<u32*>(bars + 2 * plan.stages);
    const Ring ring{smem, bars, reinterpret_cast<volatile u32*>(bars + plan.stages), reinterpret_cast<volatile u32*>(bars + plan.stages) + plan.stages, s_flag};
    ring_init(ring, plan.stages);
    if (v.summary && *v.summary) return;  // a failed or aborted projection skips the whole stage (routed_expert.hpp:17-19)

    const u32 warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const u32 n_union = v.routes.counts[0];
    const u64 row_bytes = plan.row_bytes;
    u32 first_item, n_local;
    item_range(plan, v.routes, n_union, &first_item, &n_local);
    if (warp >= plan.warps) {
        produce(ring, plan, first_item, n_local, warp - plan.warps, [&](u32 item, u32 o) {
            u32 j, cx;
            split_item(plan, item, &j, &cx);
            const u64 row = u64(v.routes.experts[j]) * H + 64u * cx + 8u * o;
            return v.weights.down + row * row_bytes;
        });
        return;
    }

    const u32 act_stride = v.act.stride ? v.act.stride : v.act.width;
    const u32 rsub = lane >> 2, p = lane & 3u;
    const u32 local_octets = n_local * kOctetsPerItem;
    bool ok = true;
    Meta m{};
    u32 first[kR];
    if (warp < local_octets) { m = load_meta(plan, v.routes, first_item + (warp >> 3)); load_first(v.routes.slots, m, first); }
    // The run's entries are contiguous in the routes; the activations of its first stage_entries entries are staged in
    // shared memory (asynchronous copies, all in flight at once), the rest - rare - is read from global memory.
    const u32 a_row = I + I / 4;  // codes, deltas, sums of one entry
    unsigned char* a_copy = reinterpret_cast<unsigned char*>(s_flag + 4);
    u32 eb_lo = 0, n_stage = 0;
    if (n_local) {
        u32 j_lo, j_hi, unused;
        split_item(plan, first_item, &j_lo, &unused);
        split_item(plan, first_item + n_local - 1u, &j_hi, &unused);
        eb_lo = __ldg(v.routes.begins + j_lo);
        n_stage = min(__ldg(v.routes.begins + j_hi + 1) - eb_lo, plan.stage_entries);
        const u32 gs = act_stride / 32, nthreads = plan.warps * 32;
        const bool al16 = (reinterpret_cast<uintptr_t>(v.act.deltas) % 16 == 0) && (reinterpret_cast<uintptr_t>(v.act.sums) % 16 == 0) && gs % 4 == 0 && I % 128 == 0;
        for (u32 e = 0; e < n_stage; ++e) {
            const u32 sl = __ldg(v.routes.slots + eb_lo + e);
            const u32 d = saddr(a_copy + u64(e) * a_row);
            const i8* src = v.act.codes + u64(sl) * act_stride;
            for (u32 c = threadIdx.x; c < I / 16; c += nthreads) cp_async(d + 16u * c, src + 16u * c, 16);
            const float* dl = v.act.deltas + u64(sl) * gs;
            const i32* sm = v.act.sums + u64(sl) * gs;
            if (al16) {
                for (u32 c = threadIdx.x; c < I / 128; c += nthreads) { cp_async(d + I + 16u * c, dl + 4 * c, 16); cp_async(d + I + I / 8 + 16u * c, sm + 4 * c, 16); }
            } else {
                for (u32 g = threadIdx.x; g < I / 32; g += nthreads) { cp_async(d + I + 4u * g, dl + g, 4); cp_async(d + I + I / 8 + 4u * g, sm + g, 4); }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"r"(plan.warps * 32) : "memory");
    for (Cursor cur{warp, warp % plan.stages, (warp / plan.stages) & 1u}; cur.q < local_octets; cur.advance(plan)) {
        const u32 slot = cur.slot, o = cur.q & 7u;
        const bool has_next = cur.q + plan.warps < local_octets;
        Meta nm{};
        if (has_next) nm = load_meta(plan, v.routes, first_item + ((cur.q + plan.warps) >> 3));
        const u32 cx = m.chunk, eb = m.eb, ne = m.ne;
        if (ok) ok = stage_wait(ring, slot, cur.q, cur.phase);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) { m = nm; if (has_next) load_first(v.routes.slots, m, first); continue; }
        const unsigned char* wrow = ring.data + u64(slot) * plan.stage_bytes + rsub * plan.row_stride;
        const u32 out_col = 64u * cx + 8u * o + rsub;
        for (u32 e0 = 0; e0 < ne; e0 += kR) {
            const int nr = static_cast<int>(min(u32(kR), ne - e0));
            u32 sl[kR];
            const i8* cr[kR];
            const float* dr[kR];
            const i32* sr[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                const u32 ent = eb + e0 + min(r, nr - 1);
                sl[r] = e0 == 0 ? first[r] : v.routes.slots[ent];
                if (ent - eb_lo < n_stage) {
                    const unsigned char* a = a_copy + u64(ent - eb_lo) * a_row;
                    cr[r] = reinterpret_cast<const i8*>(a) + 64u * p;
                    dr[r] = reinterpret_cast<const float*>(a + I) + 2u * p;
                    sr[r] = reinterpret_cast<const i32*>(a + I + I / 8) + 2u * p;
                } else {
                    cr[r] = v.act.codes + u64(sl[r]) * act_stride + 64u * p;
                    dr[r] = v.act.deltas + u64(sl[r]) * (act_stride / 32) + 2u * p;
                    sr[r] = v.act.sums + u64(sl[r]) * (act_stride / 32) + 2u * p;
                }
            }
            float acc[kR];
#pragma unroll
            for (int r = 0; r < kR; ++r) acc[r] = 0.0f;
            const uint4* blk = reinterpret_cast<const uint4*>(wrow);
            switch (nr) {
                case 1: row_down<1>(blk, nblocks, p, cr, dr, sr, acc); break;
                case 2: row_down<2>(blk, nblocks, p, cr, dr, sr, acc); break;
                case 3: row_down<3>(blk, nblocks, p, cr, dr, sr, acc); break;
                default: row_down<4>(blk, nblocks, p, cr, dr, sr, acc); break;
            }
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                if (r < nr) {
                    const float val = tree4(acc[r]);
                    if (p == 0) v.raw[u64(sl[r]) * H + out_col] = val;
                }
            }
        }
        __syncwarp();
        if (lane == 0) stage_release(ring, slot, cur.q);
        m = nm;  // the next octet's entries: second hop of the prefetch
        if (has_next) load_first(v.routes.slots, m, first);
    }
    // an aborted launch leaves raw partly unwritten: flag it in the job summary (held read-only here for the skip test)
    if (!ok && lane == 0 && v.summary) atomicOr(const_cast<u32*>(v.summary), kAbortBit);
}

int sm_count() {
    static int n = [] {
        int dev = 0, v = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v;
    }();
    return n;
}

constexpr u32 kSmemBudget = 224u * 1024u;

u32 padded_stride(u32 row_bytes) { return ((row_bytes / 16) & 1u) ? row_bytes : row_bytes + 16; }
u32 pow2_at_least(u32 v) { u32 p = 1; while (p < v) p <<= 1; return p; }

u32 plan_smem(const StreamPlan& p, u32 fixed_bytes, u32 per_item_slot_bytes) {
    return p.stages * p.stage_bytes + p.item_slots * per_item_slot_bytes + fixed_bytes + 2 * p.stages * 8 + p.item_slots * 4 + 64;
}
// Ring depth, consumer warps and item slots for a row length. Items in flight inside a CTA never exceed
// (stages + warps) / 8 + 2, so item_slots covers that with room. False when fewer than 4 stages fit.
bool make_plan(u32 row_bytes, u32 fixed_bytes, u32 per_item_slot_bytes, StreamPlan* p) {
    p->row_bytes = row_bytes;
    p->row_stride = padded_stride(row_bytes);
    p->stage_bytes = 8 * p->row_stride;
    // The warps hold one octet each while they compute; what the ring holds beyond that is the prefetch depth. Measured
    // on B200 (config 2, batch 8): time falls with every added consumer warp up to 16 as long as a few stages stay ahead.
    for (u32 stages = 40; stages >= 4; --stages) {
        p->stages = stages;
        p->warps = std::max(2u, std::min(kMaxWarps, stages > 6 ? stages - 3 : stages / 2));
        p->item_slots = pow2_at_least((stages + p->warps) / kOctetsPerItem + 3);
        if (plan_smem(*p, fixed_bytes, per_item_slot_bytes) <= kSmemBudget) return true;
    }
    return false;
}

u32 gate_up_x_bytes(const b200moe_gate_up_view& v, u32 rows) { return rows * (v.shape.hidden + v.shape.hidden / 4); }

}  // namespace
bool stream_gate_up_fits(const b200moe_gate_up_view& v, u32 rows) {
    if (!v.x.sums || rows == 0 || rows > 64 || u64(v.shape.experts) * (v.shape.inter / 32) >= (1u << 20)) return false;
    StreamPlan p{};
    return gate_up_x_bytes(v, rows) <= 80u * 1024u && make_plan(v.shape.hidden / 256 * kQ4KBlock, gate_up_x_bytes(v, rows), 2 * rows * 32 * 4, &p);
}
namespace {
// Entries staged per CTA by the down kernel: up to 32, within 48 KB.
u32 down_stage_entries(const b200moe_down_view& v) { return std::min<u32>(32u, 48u * 1024u / (v.shape.inter + v.shape.inter / 4)); }
u32 down_fixed_bytes(const b200moe_down_view& v) { return down_stage_entries(v) * (v.shape.inter + v.shape.inter / 4) + 16; }

}  // namespace

bool stream_down_fits(const b200moe_down_view& v, u32 rows) {
    if (!v.act.sums || rows == 0 || rows > 64 || u64(v.shape.experts) * (v.shape.hidden / 64) >= (1u << 20)) return false;
    StreamPlan p{};
    return make_plan(v.shape.inter / 256 * kQ4KBlock, down_fixed_bytes(v), 0, &p);
}

int launch_gate_up_q4k_stream(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    StreamPlan p{};
    const u32 x_bytes = gate_up_x_bytes(v, rows), slot_bytes = 2 * rows * 32 * 4;
    if (!make_plan(v.shape.hidden / 256 * kQ4KBlock, x_bytes, slot_bytes, &p))
        return fail(B200MOE_ERR_UNSUPPORTED, "gate_up stream form does not fit shared memory");
    p.n_chunks = v.shape.inter / 32;
    p.chunk_magic = static_cast<u32>((u64(1) << 32) / p.n_chunks) + 1;
    p.max_entries = rows;
    p.x_rows = rows;
    const u32 smem = plan_smem(p, x_bytes, slot_bytes);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(gate_up_q4k_stream_kernel), smem)) return rc;
    gate_up_q4k_stream_kernel<<<sm_count(), (p.warps + kProducers) * 32, smem, stream>>>(v, p);
    return after_launch("gate_up_q4k_stream");
}

int launch_down_q4k_stream(const b200moe_down_view& v, u32 rows, cudaStream_t stream) {
    (void)rows;
    if (v.max_union == 0) return B200MOE_OK;
    StreamPlan p{};
    if (!make_plan(v.shape.inter / 256 * kQ4KBlock, down_fixed_bytes(v), 0, &p)) return fail(B200MOE_ERR_UNSUPPORTED, "down stream form does not fit shared memory");
    p.n_chunks = v.shape.hidden / 64;
    p.chunk_magic = static_cast<u32>((u64(1) << 32) / p.n_chunks) + 1;
    p.stage_entries = down_stage_entries(v);
    const u32 smem = plan_smem(p, down_fixed_bytes(v), 0);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(down_q4k_stream_kernel), smem)) return rc;
    down_q4k_stream_kernel<<<sm_count(), (p.warps + kProducers) * 32, smem, stream>>>(v, p);
    return after_launch("down_q4k_stream");
}

}  // namespace b200moe
