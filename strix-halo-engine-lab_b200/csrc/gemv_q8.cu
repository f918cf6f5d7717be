// Q8_0 x A8 products in the 32-lane-class contract: the dense GEMV site and the routed experts of the DS41 family.
//
// Contract (src/cpu/core/backend.hpp:8-12; src/ds41_formats.cpp:45-50, :188-197; src/cpu/core/reference.cpp:57-84):
// per 32-weight group float(int32 dot) * (scale * delta); group g goes to lane class g % 32, classes accumulate in
// ascending g from +0, the classes are combined by the butterfly v[l] += v[l ^ d], d = 16 .. 1. One warp per weight
// row with lane = lane class reproduces it directly; the gate/up epilogue is swiglu_clamped (declared_exp) followed by
// the A8 rule per 32 outputs (src/ds41_moe.cpp:134-146).
//
// Q8_0 blocks are 34 bytes, so only 2-byte aligned inside a row. A warp therefore stages each run of 32 blocks
// (1088 B = 68 x 16 B) into shared memory with 16-byte coalesced loads and every lane picks its block from there; rows
// whose runs are not 16-byte aligned fall back to halfword loads. Up to 8 A8 rows share one pass over the weights.
//
// Roofline: HBM; algorithmic bytes per weight row = K / 32 * 34.
#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr int kR = 8;
constexpr u32 kStageBytes = 1088 + 16;
// Warps per CTA. The kernels are latency bound, not instruction bound: what counts is how many weight rows are in flight,
// so the routed kernels give every row of a 32-output group its own warp.
constexpr u32 kRoutedWarps = 32, kDenseWarps = 16;

struct A8View {
    const i8* codes;      // row r at codes + r * stride
    const float* deltas;  // row r at deltas + r * (stride / 32)
    u32 stride;
};

// A run of up to 32 blocks (1088 B = 68 x 16 B) held in registers between its global load and its store to the
// warp's stage: the load of the NEXT run (of this row or of the warp's next row) is issued before the current run is
// computed, so a warp always has a run in flight.
struct RunRegs { uint4 v[3]; };
__device__ __forceinline__ bool run_is_fast(u32 align, u32 nb) { return align >= 16 && (nb & 7u) == 0; }
__device__ __forceinline__ void run_load(const u8* src, u32 nb, u32 lane, RunRegs& r) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    const u32 n16 = nb * kQ8Block / 16;
#pragma unroll
    for (int k = 0; k < 3; ++k) if (lane + 32u * k < n16) r.v[k] = __ldg(s4 + lane + 32u * k);
}
__device__ __forceinline__ void run_store(u32* stage, u32 nb, u32 lane, const RunRegs& r) {
    uint4* d4 = reinterpret_cast<uint4*>(stage);
    const u32 n16 = nb * kQ8Block / 16;
#pragma unroll
    for (int k = 0; k < 3; ++k) if (lane + 32u * k < n16) d4[lane + 32u * k] = r.v[k];
}

// One Q8_0 weight row against nr <= kR A8 rows; lane = lane class. `stage` is this warp's 1104-byte scratch.
// `pre` carries the row's first run when `have_pre` (loaded by the previous call); `next_row` (nullable) is the row the
// warp takes next: its first run is loaded into `pre` during this row's last run. Returns whether `pre` holds it.
// Every lane returns the products in out[].
__device__ __forceinline__ bool q8_row(const u8* __restrict__ wrow, u32 groups, u32 align, u32* stage, const A8View& x, int nr,
                                       u32 lane, float* out, RunRegs& pre, bool have_pre, const u8* next_row) {
    float cls[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) cls[r] = 0.0f;
    bool next_loaded = false;
    for (u32 g0 = 0; g0 < groups; g0 += 32) {
        const u32 nb = min(32u, groups - g0);
        const u8* src = wrow + u64(g0) * kQ8Block;
        __syncwarp();
        if (run_is_fast(align, nb)) {
            if (!have_pre) run_load(src, nb, lane, pre);
            run_store(stage, nb, lane, pre);
            have_pre = false;
            const u32 g1 = g0 + 32;
            if (g1 < groups) {  // this row's next run
                const u32 nb1 = min(32u, groups - g1);
                if (run_is_fast(align, nb1)) { run_load(wrow + u64(g1) * kQ8Block, nb1, lane, pre); have_pre = true; }
            } else if (next_row && run_is_fast(align, min(32u, groups))) {  // the next row's first run
                run_load(next_row, min(32u, groups), lane, pre);
                next_loaded = true;
            }
        } else if (align >= 2) {
            const u16* s2 = reinterpret_cast<const u16*>(src);
            u16* d2 = reinterpret_cast<u16*>(stage);
            for (u32 i = lane; i < nb * (kQ8Block / 2); i += 32) d2[i] = s2[i];
        } else {  // odd row strides: rows are only byte aligned
            u8* d1 = reinterpret_cast<u8*>(stage);
            for (u32 i = lane; i < nb * kQ8Block; i += 32) d1[i] = src[i];
        }
        __syncwarp();
        if (lane < nb) {
            // block at byte 34 * lane: even lanes start on a word, odd lanes on a halfword
            const u32 w0 = (kQ8Block * lane) >> 2;
            u32 q[8];
            float scale;
            if (lane & 1u) {
                scale = half_bits_to_float(stage[w0] >> 16);
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = stage[w0 + 1 + i];
            } else {
                u32 w[9];
#pragma unroll
                for (int i = 0; i < 9; ++i) w[i] = stage[w0 + i];
                scale = half_bits_to_float(w[0] & 0xffffu);
#pragma unroll
                for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i], w[i + 1], 16);
            }
            const u32 g = g0 + lane;
#pragma unroll
            for (int r = 0; r < kR; ++r) {
                if (r < nr) {
                    const uint4* c = reinterpret_cast<const uint4*>(x.codes + u64(r) * x.stride + 32u * g);
                    const uint4 c0 = c[0], c1 = c[1];
                    int dot = 0;
                    dot = __dp4a((int)q[0], (int)c0.x, dot); dot = __dp4a((int)q[1], (int)c0.y, dot);
                    dot = __dp4a((int)q[2], (int)c0.z, dot); dot = __dp4a((int)q[3], (int)c0.w, dot);
                    dot = __dp4a((int)q[4], (int)c1.x, dot); dot = __dp4a((int)q[5], (int)c1.y, dot);
                    dot = __dp4a((int)q[6], (int)c1.z, dot); dot = __dp4a((int)q[7], (int)c1.w, dot);
                    const float sd = __fmul_rn(scale, x.deltas[u64(r) * (x.stride / 32) + g]);
                    cls[r] = __fadd_rn(cls[r], __fmul_rn(static_cast<float>(dot), sd));
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kR; ++r) out[r] = butterfly32(cls[r]);
    return next_loaded;
}

__device__ __forceinline__ void stage_rows(const b200moe_a8_rows& src, const u32* idx, u32 first_row, int nr, u32 width, i8* s_codes,
                                           float* s_deltas) {
    const u32 stride = src.stride ? src.stride : src.width, groups = width / 32;
    for (int r = 0; r < nr; ++r) {
        const u64 row = idx ? idx[r] : first_row + r;
        const uint4* c = reinterpret_cast<const uint4*>(src.codes + row * stride);
        uint4* dc = reinterpret_cast<uint4*>(s_codes + u64(r) * width);
        for (u32 i = threadIdx.x; i < width / 16; i += blockDim.x) dc[i] = c[i];
        for (u32 i = threadIdx.x; i < groups; i += blockDim.x) s_deltas[r * groups + i] = src.deltas[row * (stride / 32) + i];
    }
}

// Dense site: out[r][o] for o in [first, first + count). grid (ceil(count / 32)); 256 threads; rows in passes of 8.
__global__ void __launch_bounds__(1024) q8_0_a8_kernel(b200moe_q8a8_view v, u32 align) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const u32 K = v.width, groups = K / 32, nw = blockDim.x >> 5;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * K);
    u32* s_stage = reinterpret_cast<u32*>(s_deltas + kR * groups);
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    u32* stage = s_stage + warp * (kStageBytes / 4);
    const u32 out_stride = v.out_stride ? v.out_stride : v.count;
    const A8View xs{s_codes, s_deltas, K};
    for (u32 r0 = 0; r0 < v.x.rows; r0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), v.x.rows - r0));
        __syncthreads();
        stage_rows(v.x, nullptr, r0, nr, K, s_codes, s_deltas);
        __syncthreads();
        RunRegs pre;
        bool have_pre = false;
        for (u32 t = warp; t < 32; t += nw) {
            const u32 o = 32u * blockIdx.x + t;
            if (o >= v.count) break;
            float val[kR];
            const bool more = t + nw < 32 && o + nw < v.count;
            have_pre = q8_row(v.weight + u64(v.first + o) * v.row_bytes, groups, align, stage, xs, nr, lane, val, pre, have_pre,
                              more ? v.weight + u64(v.first + o + nw) * v.row_bytes : nullptr);
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < kR; ++r)
                    if (r < nr) {
                        float* y = v.out + u64(r0 + r) * out_stride + o;
                        *y = v.accumulate ? __fadd_rn(*y, val[r]) : val[r];
                    }
            }
        }
    }
}

// Routed gate/up: grid (inter / 32, max_union); 256 threads; one CTA = one expert x one 32-output group.
__global__ void __launch_bounds__(1024) gate_up_q8_kernel(b200moe_gate_up_view v, u32 align) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const u32 j = blockIdx.y, nw = blockDim.x >> 5;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = H / 32;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * H);
    float* s_g = s_deltas + kR * groups;
    float* s_u = s_g + kR * 32;
    u32* s_stage = reinterpret_cast<u32*>(s_u + kR * 32);
    __shared__ u32 s_rows[kR], s_slots[kR];
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    u32* stage = s_stage + warp * (kStageBytes / 4);
    const u64 row_bytes = u64(groups) * kQ8Block;
    const u8* gate = v.weights.gate + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const u8* up = v.weights.up + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const A8View xs{s_codes, s_deltas, H};
    const u32 act_stride = v.act.stride ? v.act.stride : v.act.width;
    // the warp's first weight run is requested before the activations are staged: its latency hides behind the staging
    RunRegs pre;
    bool have_pre = false;
    if (warp < 64 && run_is_fast(align, min(32u, groups))) {
        run_load((warp < 32 ? gate : up) + u64(warp & 31u) * row_bytes, min(32u, groups), lane, pre);
        have_pre = true;
    }
    for (u32 p0 = eb + kR * blockIdx.z; p0 < ee; p0 += kR * gridDim.z) {  // grid.z shares an expert's passes of kR entries
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < (u32)nr) { s_rows[threadIdx.x] = v.routes.rows[p0 + threadIdx.x]; s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x]; }
        __syncthreads();
        stage_rows(v.x, s_rows, 0, nr, H, s_codes, s_deltas);
        __syncthreads();
        for (u32 t = warp; t < 64; t += nw) {
            const u8* wrow = (t < 32 ? gate : up) + u64(t & 31u) * row_bytes;
            const u32 tn = t + nw;
            float val[kR];
            have_pre = q8_row(wrow, groups, align, stage, xs, nr, lane, val, pre, have_pre,
                              tn < 64 ? (tn < 32 ? gate : up) + u64(tn & 31u) * row_bytes : nullptr);
            if (lane == 0) {
                float* dst = t < 32 ? s_g : s_u;
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) dst[r * 32 + (t & 31u)] = val[r];
            }
        }
        __syncthreads();
        for (int r = warp; r < nr; r += nw) {
            const float g = s_g[r * 32 + lane], u = s_u[r * 32 + lane];
            const u32 slot = s_slots[r], o = 32u * blockIdx.x + lane;
            if (v.gate_out) { v.gate_out[u64(slot) * I + o] = g; v.up_out[u64(slot) * I + o] = u; }
            const float h = swiglu_ds41(g, u, v.shape.limit);  // NaN propagates: this family has no status rule
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

// Routed down: grid (hidden / 32, max_union); 256 threads.
__global__ void __launch_bounds__(1024) down_q8_kernel(b200moe_down_view v, u32 align) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (v.summary && *v.summary) return;
    const u32 j = blockIdx.y, nw = blockDim.x >> 5;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = I / 32;
    i8* s_codes = reinterpret_cast<i8*>(smem_raw);
    float* s_deltas = reinterpret_cast<float*>(smem_raw + u64(kR) * I);
    u32* s_stage = reinterpret_cast<u32*>(s_deltas + kR * groups);
    __shared__ u32 s_slots[kR];
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    u32* stage = s_stage + warp * (kStageBytes / 4);
    const u64 row_bytes = u64(groups) * kQ8Block;
    const u32 o0 = 32u * blockIdx.x;
    const u8* down = v.weights.down + (u64(expert) * H + o0) * row_bytes;
    const A8View xs{s_codes, s_deltas, I};
    RunRegs pre;  // the first weight run is requested before the activations are staged
    bool have_pre = false;
    if (warp < 32 && run_is_fast(align, min(32u, groups))) {
        run_load(down + u64(warp) * row_bytes, min(32u, groups), lane, pre);
        have_pre = true;
    }
    for (u32 p0 = eb + kR * blockIdx.z; p0 < ee; p0 += kR * gridDim.z) {  // grid.z shares an expert's passes of kR entries
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < (u32)nr) s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x];
        __syncthreads();
        stage_rows(v.act, s_slots, 0, nr, I, s_codes, s_deltas);
        __syncthreads();
        for (u32 t = warp; t < 32; t += nw) {
            float val[kR];
            have_pre = q8_row(down + u64(t) * row_bytes, groups, align, stage, xs, nr, lane, val, pre, have_pre,
                              t + nw < 32 ? down + u64(t + nw) * row_bytes : nullptr);
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) v.raw[u64(s_slots[r]) * H + o0 + t] = val[r];
            }
        }
    }
}

template <class K>
int set_smem(K kernel, u32 bytes) {
    return ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), bytes);
}

}  // namespace

int launch_q8_0_a8(const b200moe_q8a8_view& v, cudaStream_t stream) {
    if (v.count == 0 || v.x.rows == 0) return B200MOE_OK;
    const u32 K = v.width;
    const u32 align = (aligned(v.weight, 16) && v.row_bytes % 16 == 0) ? 16u : ((aligned(v.weight, 2) && v.row_bytes % 2 == 0) ? 2u : 1u);
    const u32 nw = kDenseWarps;
    const u32 smem = kR * (K + K / 32 * 4) + nw * kStageBytes;
    if (int rc = set_smem(q8_0_a8_kernel, smem)) return rc;
    q8_0_a8_kernel<<<(v.count + 31) / 32, nw * 32, smem, stream>>>(v, align);
    return after_launch("q8_0_a8");
}

// An expert with many entries (the dense shared expert over a token block) is walked in passes of kR entries; when the
// grid of (output groups x experts) would leave SMs idle, grid.z shares the passes: up to 16 ways, never more than the
// passes `entries_bound` entries can need, until there are two CTAs per SM.
static u32 pass_split(u32 ctas, u32 entries_bound) {
    const u32 passes = std::max(1u, (entries_bound + kR - 1) / kR), want = (2u * 148u + ctas - 1) / std::max(1u, ctas);
    return std::max(1u, std::min(std::min(passes, want), 16u));
}

int launch_gate_up_q8(const b200moe_gate_up_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    const u32 H = v.shape.hidden, I = v.shape.inter;
    const u32 align = (aligned(v.weights.gate, 16) && aligned(v.weights.up, 16) && (H / 32 * kQ8Block) % 16 == 0) ? 16u : 2u;
    const u32 nw = kRoutedWarps;   // 64 weight rows per CTA: two per warp, the second one prefetched
    const u32 smem = kR * (H + H / 32 * 4) + 2 * kR * 32 * 4 + nw * kStageBytes;
    if (int rc = set_smem(gate_up_q8_kernel, smem)) return rc;
    gate_up_q8_kernel<<<dim3(I / 32, v.max_union, pass_split(I / 32 * v.max_union, v.x.rows)), nw * 32, smem, stream>>>(v, align);
    return after_launch("gate_up_q8");
}

int launch_down_q8(const b200moe_down_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    const u32 H = v.shape.hidden, I = v.shape.inter;
    const u32 align = (aligned(v.weights.down, 16) && (I / 32 * kQ8Block) % 16 == 0) ? 16u : 2u;
    const u32 nw = kRoutedWarps;   // 32 weight rows per CTA: one per warp, every row of the expert in flight at once
    const u32 smem = kR * (I + I / 32 * 4) + nw * kStageBytes;
    if (int rc = set_smem(down_q8_kernel, smem)) return rc;
    down_q8_kernel<<<dim3(H / 32, v.max_union, pass_split(H / 32 * v.max_union, v.act.rows)), nw * 32, smem, stream>>>(v, align);
    return after_launch("down_q8");
}

}  // namespace b200moe
