// Routed experts of the DS41 family over ANY of its block types - Q8_0 and Q2_K, the same or different for gate / up and
// down - in the family's one contract: a term per 32-weight group, group g into lane class g % 32, classes accumulated in
// ascending g from +0 and folded by the butterfly v[l] += v[l ^ d], d = 16 .. 1 (lane_product, src/ds41_formats.cpp:37-50).
// Terms:
//   Q8_0 (product_q8_0, :188-197):  float(dot) * (scale * delta)
//   Q2_K (product_q2_k, :198-218):  per half h of the group (16 weights): qx_h = sum q * x, sx_h = sum x;
//                                   a = sum_h (scale_h & 15) * qx_h, b = sum_h (scale_h >> 4) * sx_h (integers);
//                                   (d * float(a) - dmin * float(b)) * delta
// One warp per weight row, lane = lane class, weights read where they lie (a lane's group is 32 quants = eight words of the
// super-block, aligned to 4 bytes since a row is a multiple of 84 bytes); up to eight entries of an expert share a pass.
// This is the plain form: the layers made of Q8_0 alone take the streaming forms of gemv_q8*.cu. The gate/up epilogue
// is swiglu_clamped (declared_exp) + the A8 rule per 32 outputs (src/ds41_moe.cpp:134-146).
//
// Roofline: HBM; algorithmic bytes per weight row = K / 256 * 84 (Q2_K) or K / 32 * 34 (Q8_0).
#include "declared_math.cuh"
#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr int kR = 8;      // entries per pass
constexpr u32 kWarps = 8;  // weight rows in flight per CTA

// The term of group g of a Q2_K row for one A8 row (codes: the 32 codes of the group, 4-byte aligned).
__device__ __forceinline__ float term_q2_k(const u8* __restrict__ wrow, u32 g, const i8* __restrict__ codes, float delta) {
    const u8* blk = wrow + u64(g >> 3) * kQ2KBlock;
    const u32 within = g & 7u, half = within >> 2, shift = 2u * (within & 3u);
    const u32* q = reinterpret_cast<const u32*>(blk + 16u + 32u * half);
    const u32* x = reinterpret_cast<const u32*>(codes);
    int qx[2] = {0, 0}, sx[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const u32 qw = (__ldg(q + i) >> shift) & 0x03030303u, xw = x[i];
        qx[i >> 2] = __dp4a(static_cast<int>(qw), static_cast<int>(xw), qx[i >> 2]);
        sx[i >> 2] = __dp4a(0x01010101, static_cast<int>(xw), sx[i >> 2]);
    }
    const u32 s0 = blk[8u * half + 2u * (within & 3u)], s1 = blk[8u * half + 2u * (within & 3u) + 1u];
    const int a = static_cast<int>(s0 & 15u) * qx[0] + static_cast<int>(s1 & 15u) * qx[1];
    const int b = static_cast<int>(s0 >> 4) * sx[0] + static_cast<int>(s1 >> 4) * sx[1];
    const float d = half_bits_to_float(*reinterpret_cast<const unsigned short*>(blk + 80u));
    const float dmin = half_bits_to_float(*reinterpret_cast<const unsigned short*>(blk + 82u));
    return __fmul_rn(__fsub_rn(__fmul_rn(d, static_cast<float>(a)), __fmul_rn(dmin, static_cast<float>(b))), delta);
}
// The term of group g of a Q8_0 row (blocks are 2-byte aligned only: halfword loads).
__device__ __forceinline__ float term_q8_0(const u8* __restrict__ wrow, u32 g, const i8* __restrict__ codes, float delta) {
    const unsigned short* blk = reinterpret_cast<const unsigned short*>(wrow + u64(g) * kQ8Block);
    const unsigned short* x = reinterpret_cast<const unsigned short*>(codes);
    const float scale = half_bits_to_float(__ldg(blk));
    int dot = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const u32 w = __ldg(blk + 1 + i), c = x[i];
        dot += static_cast<int>(static_cast<signed char>(w & 0xffu)) * static_cast<int>(static_cast<signed char>(c & 0xffu));
        dot += static_cast<int>(static_cast<signed char>(w >> 8)) * static_cast<int>(static_cast<signed char>(c >> 8));
    }
    return __fmul_rn(static_cast<float>(dot), __fmul_rn(scale, delta));
}

// One weight row against nr <= kR A8 rows (row r: codes[r], deltas[r]); every lane returns the products.
template <u32 TYPE>
__device__ __forceinline__ void ds41_row(const u8* __restrict__ wrow, u32 groups, const i8* const* codes, const float* const* deltas, int nr,
                                         u32 lane, float* out) {
    float cls[kR];
#pragma unroll
    for (int r = 0; r < kR; ++r) cls[r] = 0.0f;
    for (u32 g = lane; g < groups; g += 32) {  // ascending g within the lane's class
#pragma unroll
        for (int r = 0; r < kR; ++r) {
            if (r < nr) {
                const float t = TYPE == B200MOE_TYPE_Q2_K ? term_q2_k(wrow, g, codes[r] + 32u * g, deltas[r][g]) : term_q8_0(wrow, g, codes[r] + 32u * g, deltas[r][g]);
                cls[r] = __fadd_rn(cls[r], t);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kR; ++r) out[r] = butterfly32(cls[r]);
}

// grid (inter / 32, max_union): one CTA = one expert x one 32-output group; 8 warps walk the 64 rows (32 gate, 32 up).
template <u32 TYPE>
__global__ void __launch_bounds__(kWarps * 32) gate_up_ds41_any_kernel(b200moe_gate_up_view v) {
    __shared__ float s_g[kR * 32], s_u[kR * 32];
    __shared__ u32 s_slots[kR];
    __shared__ const i8* s_codes[kR];
    __shared__ const float* s_deltas[kR];
    const u32 j = blockIdx.y;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = H / 32;
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const u64 row_bytes = TYPE == B200MOE_TYPE_Q2_K ? u64(H / 256) * kQ2KBlock : u64(groups) * kQ8Block;
    const u8* gate = v.weights.gate + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const u8* up = v.weights.up + (u64(expert) * I + 32u * blockIdx.x) * row_bytes;
    const u32 x_stride = v.x.stride ? v.x.stride : v.x.width, act_stride = v.act.stride ? v.act.stride : v.act.width;
    for (u32 p0 = eb; p0 < ee; p0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < static_cast<u32>(nr)) {
            const u32 row = v.routes.rows[p0 + threadIdx.x];
            s_slots[threadIdx.x] = v.routes.slots[p0 + threadIdx.x];
            s_codes[threadIdx.x] = v.x.codes + u64(row) * x_stride;
            s_deltas[threadIdx.x] = v.x.deltas + u64(row) * (x_stride / 32);
        }
        __syncthreads();
        for (u32 t = warp; t < 64; t += kWarps) {
            float val[kR];
            ds41_row<TYPE>((t < 32 ? gate : up) + u64(t & 31u) * row_bytes, groups, s_codes, s_deltas, nr, lane, val);
            if (lane == 0) {
                float* dst = t < 32 ? s_g : s_u;
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) dst[r * 32 + (t & 31u)] = val[r];
            }
        }
        __syncthreads();
        for (int r = warp; r < nr; r += kWarps) {
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

// grid (hidden / 32, max_union): 8 warps walk 32 down rows.
template <u32 TYPE>
__global__ void __launch_bounds__(kWarps * 32) down_ds41_any_kernel(b200moe_down_view v) {
    __shared__ u32 s_slots[kR];
    __shared__ const i8* s_codes[kR];
    __shared__ const float* s_deltas[kR];
    if (v.summary && *v.summary) return;
    const u32 j = blockIdx.y;
    if (j >= v.routes.counts[0]) return;
    const u32 H = v.shape.hidden, I = v.shape.inter, groups = I / 32;
    const u32 expert = v.routes.experts[j], eb = v.routes.begins[j], ee = v.routes.begins[j + 1];
    const u32 lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const u64 row_bytes = TYPE == B200MOE_TYPE_Q2_K ? u64(I / 256) * kQ2KBlock : u64(groups) * kQ8Block;
    const u32 o0 = 32u * blockIdx.x;
    const u8* down = v.weights.down + (u64(expert) * H + o0) * row_bytes;
    const u32 act_stride = v.act.stride ? v.act.stride : v.act.width;
    for (u32 p0 = eb; p0 < ee; p0 += kR) {
        const int nr = static_cast<int>(min(u32(kR), ee - p0));
        __syncthreads();
        if (threadIdx.x < static_cast<u32>(nr)) {
            const u32 slot = v.routes.slots[p0 + threadIdx.x];
            s_slots[threadIdx.x] = slot;
            s_codes[threadIdx.x] = v.act.codes + u64(slot) * act_stride;
            s_deltas[threadIdx.x] = v.act.deltas + u64(slot) * (act_stride / 32);
        }
        __syncthreads();
        for (u32 t = warp; t < 32; t += kWarps) {
            float val[kR];
            ds41_row<TYPE>(down + u64(t) * row_bytes, groups, s_codes, s_deltas, nr, lane, val);
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < kR; ++r) if (r < nr) v.raw[u64(s_slots[r]) * H + o0 + t] = val[r];
            }
        }
    }
}

}  // namespace

int launch_gate_up_ds41_any(const b200moe_gate_up_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    const dim3 grid(v.shape.inter / 32, v.max_union);
    if (v.shape.gate_type == B200MOE_TYPE_Q2_K) gate_up_ds41_any_kernel<B200MOE_TYPE_Q2_K><<<grid, kWarps * 32, 0, stream>>>(v);
    else gate_up_ds41_any_kernel<B200MOE_TYPE_Q8_0><<<grid, kWarps * 32, 0, stream>>>(v);
    return after_launch("gate_up_ds41_any");
}

int launch_down_ds41_any(const b200moe_down_view& v, cudaStream_t stream) {
    if (v.max_union == 0) return B200MOE_OK;
    const dim3 grid(v.shape.hidden / 32, v.max_union);
    if (v.shape.down_type == B200MOE_TYPE_Q2_K) down_ds41_any_kernel<B200MOE_TYPE_Q2_K><<<grid, kWarps * 32, 0, stream>>>(v);
    else down_ds41_any_kernel<B200MOE_TYPE_Q8_0><<<grid, kWarps * 32, 0, stream>>>(v);
    return after_launch("down_ds41_any");
}

}  // namespace b200moe
