// Weighted combine of the raw slot vectors, plus the small elementwise helpers of the layer.
//
// Forms (include/b200moe.h):
//   PARTS     y = ((shared + S_0) + S_1) + ...; S_p over the row's slots of expert range p in ascending expert id from
//             +0, one product then one add per step (src/ds41_moe.cpp:99-115, :152-163; device twin
//             include/strix/cuda/ds41_moe.hpp:109-134).
//   FMA_SLOTS acc = fma(w[k], raw[k], acc) in slot order (src/cuda/models/qwen/qwen_moe.cu:298-306;
//             include/strix/moe/combine.hpp:36-59), y = acc (+ shared), optional bfloat16 RNE commit (:330-335).
// HBM: rows * top_k * hidden * 4 B read, rows * hidden * 4 B written; elementwise over hidden, coalesced.
#include <algorithm>

#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kMaxTopK = 32;

// grid (ceil(hidden / 256), min(rows, 65535)); 256 threads; a block walks rows blockIdx.y, blockIdx.y + gridDim.y, ...
__global__ void __launch_bounds__(256) combine_kernel(b200moe_combine_view v) {
    const u32 o = blockIdx.x * blockDim.x + threadIdx.x;
    if (v.summary && (*v.summary & B200MOE_JOB_WAIT_ABORTED)) return;  // an aborted stage left raw partly unwritten
    __shared__ float s_w[kMaxTopK];
    __shared__ u32 s_slot[kMaxTopK], s_part[kMaxTopK];
    for (u32 row = blockIdx.y; row < v.rows; row += gridDim.y) {
        __syncthreads();  // the previous row's readers are done with the shared arrays
        if (v.row_status && v.row_status[row]) continue;  // fail closed (qwen_moe.cu:291); uniform over the block
        if (threadIdx.x < v.top_k) {
            const u32 k = threadIdx.x;
            if (v.form == B200MOE_COMBINE_PARTS) {
                const u32 slot = v.order[row * v.top_k + k];
                s_slot[k] = slot;
                s_w[k] = v.weights[slot];
                s_part[k] = v.low_counts ? (k < v.low_counts[row] ? 0u : 1u) : min(v.ids[slot] / v.part_experts, v.parts - 1);
            } else {
                s_slot[k] = row * v.top_k + k;
                s_w[k] = v.weights[row * v.top_k + k];
            }
        }
        __syncthreads();
        if (o >= v.hidden) continue;
        float out;
        if (v.form == B200MOE_COMBINE_FMA_SLOTS) {
            float acc = 0.0f;
            for (u32 k = 0; k < v.top_k; ++k) acc = __fmaf_rn(s_w[k], v.raw[u64(s_slot[k]) * v.hidden + o], acc);
            out = v.shared ? __fadd_rn(acc, v.shared[u64(row) * v.hidden + o]) : acc;
        } else {
            float total = v.shared ? v.shared[u64(row) * v.hidden + o] : 0.0f, single = 0.0f;
            const u32 first_part = v.only_part >= 0 ? static_cast<u32>(v.only_part) : 0u, n_parts = v.only_part_count > 1 ? v.only_part_count : 1u;
            u32 k = 0;
            for (u32 p = 0; p < v.parts; ++p) {  // the slots are sorted by expert id, so each part is one run
                float sum = 0.0f;
                while (k < v.top_k && s_part[k] == p) {
                    sum = __fadd_rn(sum, __fmul_rn(s_w[k], v.raw[u64(s_slot[k]) * v.hidden + o]));
                    ++k;
                }
                if (static_cast<int>(p) == v.only_part) single = sum;
                else if (v.only_part >= 0 && p > first_part && p < first_part + n_parts) {  // the further sums of a rank that owns several ranges
                    const u64 at = u64(p - first_part) * v.part_stride;
                    if (v.y_blocks) { const u32 blk = row / v.y_block_rows; v.y_blocks[blk][at + u64(row - blk * v.y_block_rows) * v.hidden + o] = sum; }
                    else v.y[at + u64(row) * v.hidden + o] = sum;
                }
                total = __fadd_rn(total, sum);
            }
            out = v.only_part >= 0 ? single : total;
        }
        if (v.y_blocks) {  // the row's home rank's buffer: a peer store
            const u32 blk = row / v.y_block_rows;
            v.y_blocks[blk][u64(row - blk * v.y_block_rows) * v.hidden + o] = out;
            continue;
        }
        v.y[u64(row) * v.hidden + o] = out;
        if (v.y_bf16) v.y_bf16[u64(row) * v.hidden + o] = bf16_rne_bits(out);
    }
}

__global__ void __launch_bounds__(256) canonical_sum_kernel(const float* a, const float* b, const float* c, u64 count, float* y) {
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float ab = __fadd_rn(a[i], b[i]);
    y[i] = c ? __fadd_rn(ab, c[i]) : ab;
}

__global__ void __launch_bounds__(256) fill_u32_kernel(u32* p, u32 value, u64 count) {
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < count) p[i] = value;
}

__global__ void __launch_bounds__(256) row_order_kernel(const u32* ids, u32 rows, u32 top_k, u32* order) {
    const u32 row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    u32 key[kMaxTopK], slot[kMaxTopK];
    for (u32 k = 0; k < top_k; ++k) {
        const u32 s = row * top_k + k, e = ids[s];
        u32 j = k;
        while (j > 0 && key[j - 1] > e) { key[j] = key[j - 1]; slot[j] = slot[j - 1]; --j; }
        key[j] = e; slot[j] = s;
    }
    for (u32 k = 0; k < top_k; ++k) order[row * top_k + k] = slot[k];
}

// The complete first non-zero summary stays (include/strix/deferred_moe_status.hpp:19-28); one thread, stream ordered.
__global__ void merge_first_error_kernel(b200moe_first_error* record, const u32* summary, u32 domain) {
    const u32 bits = *summary;
    if (bits != 0u && record->domain == 0u) {
        record->bits = bits;
        record->domain = domain;
    }
}

}  // namespace

int launch_merge_first_error(b200moe_first_error* record, const u32* summary, u32 domain, cudaStream_t stream) {
    merge_first_error_kernel<<<1, 1, 0, stream>>>(record, summary, domain);
    return after_launch("merge_first_error");
}
int launch_combine(const b200moe_combine_view& v, cudaStream_t stream) {
    if (v.rows == 0) return B200MOE_OK;
    if (int rc = prefer_max_shared(reinterpret_cast<const void*>(combine_kernel))) return rc;
    combine_kernel<<<dim3((v.hidden + 255) / 256, std::min<u32>(v.rows, 65535u)), 256, 0, stream>>>(v);
    return after_launch("combine");
}
int launch_canonical_sum(const float* a, const float* b, const float* c, u64 count, float* y, cudaStream_t stream) {
    if (count == 0) return B200MOE_OK;
    canonical_sum_kernel<<<static_cast<u32>((count + 255) / 256), 256, 0, stream>>>(a, b, c, count, y);
    return after_launch("canonical_sum");
}
int launch_fill_u32(u32* p, u32 value, u64 count, cudaStream_t stream) {
    if (count == 0) return B200MOE_OK;
    fill_u32_kernel<<<static_cast<u32>((count + 255) / 256), 256, 0, stream>>>(p, value, count);
    return after_launch("fill_u32");
}
int launch_row_order(const u32* ids, u32 rows, u32 top_k, u32* order, cudaStream_t stream) {
    if (rows == 0) return B200MOE_OK;
    row_order_kernel<<<(rows + 255) / 256, 256, 0, stream>>>(ids, rows, top_k, order);
    return after_launch("row_order");
}

}  // namespace b200moe
