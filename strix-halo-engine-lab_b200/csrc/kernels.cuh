// Internal launch interface between the C ABI layer (api.cu) and the kernel translation units. Every function
// validates nothing (api.cu has done it), enqueues on `stream` and returns after_launch()'s status.
#pragma once
#include "common.cuh"

namespace b200moe {

// a8.cu
int launch_quantize_a8(const b200moe_quantize_a8_view& v, cudaStream_t stream);
int launch_rmsnorm_a8(const b200moe_rmsnorm_view& v, cudaStream_t stream);
// out[i] = float(bfloat16 bits in[i]) (exact widening)
int launch_widen_bf16(const u16* in, float* out, u64 count, cudaStream_t stream);

// router.cu
// fused_quantize (optional): the A8 quantiser of the same activations is enqueued first
int launch_router_logits(const b200moe_router_view& v, cudaStream_t stream, const b200moe_quantize_a8_view* fused_quantize = nullptr);
int launch_router_select(const b200moe_router_view& v, cudaStream_t stream);

// routes.cu
u64 routes_scratch_words(u32 rows, u32 top_k, u32 experts);
int launch_routes(const b200moe_routes_view& v, cudaStream_t stream);
int launch_dense_routes(const b200moe_routes& out, u32 rows, u32* row_status, u32* summary4, cudaStream_t stream);
// grouped (token-block) form of the Q4_K experts on the tensor cores (grouped_q4k.cu)
bool grouped_fits(const b200moe_shape& s, bool have_sums);
int launch_gate_up_q4k_grouped(const b200moe_gate_up_view& v, cudaStream_t stream);
int launch_down_q4k_grouped(const b200moe_down_view& v, cudaStream_t stream);
// decode windows: selection of r (logits already present) and the routes of the selected ids in one launch
bool select_routes_fusable(const b200moe_router_view& r, u32 top_k);
int launch_select_routes(const b200moe_router_view& r, const b200moe_routes_view& v, cudaStream_t stream);

// gemv_q8.cu: Q8_0 x A8 products in the 32-lane-class contract (dense rows and the routed DS41-family experts)
int launch_q8_0_a8(const b200moe_q8a8_view& v, cudaStream_t stream);
int launch_gate_up_q8(const b200moe_gate_up_view& v, cudaStream_t stream);
int launch_down_q8(const b200moe_down_view& v, cudaStream_t stream);

// gemv_q4k.cu: Q4_K x A8 rows in the four-chain contract (routed Qwen-family experts; Q8_0 four-chain down)
int launch_gate_up_q4k(const b200moe_gate_up_view& v, cudaStream_t stream);
int launch_down_q4k(const b200moe_down_view& v, cudaStream_t stream);
// gemv_ds41_any.cu: the DS41 family over any of its block types (Q8_0, Q2_K), one weight row per warp, weights read in place.
int launch_gate_up_ds41_any(const b200moe_gate_up_view& v, cudaStream_t stream);
int launch_down_ds41_any(const b200moe_down_view& v, cudaStream_t stream);
int launch_down_q8_chain4(const b200moe_down_view& v, cudaStream_t stream);

// gemv_q4k_stream.cu: the same Q4_K contracts as persistent kernels fed by bulk copies (decode windows up to 64 rows)
bool stream_gate_up_fits(const b200moe_gate_up_view& v, u32 rows);
bool stream_down_fits(const b200moe_down_view& v, u32 rows);
int launch_gate_up_q4k_stream(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream);
int launch_down_q4k_stream(const b200moe_down_view& v, u32 rows, cudaStream_t stream);

// gemv_q4k_wide.cu: the same contracts with SEGMENTS of the rows (and of the entries' A8 rows) streamed by TMA: any row
// length, windows of any size whose routes fit shared memory
bool wide_gate_up_fits(const b200moe_gate_up_view& v, u32 rows);
bool wide_down_fits(const b200moe_down_view& v, u32 rows);
int launch_gate_up_q4k_wide(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream);
int launch_down_q4k_wide(const b200moe_down_view& v, u32 rows, cudaStream_t stream);
// gemv_q8_wide.cu: the Q8_0 x A8 lane-class contract in the same streaming skeleton, for windows of many rows.
bool q8_wide_gate_up_fits(const b200moe_gate_up_view& v, u32 rows);
bool q8_wide_down_fits(const b200moe_down_view& v, u32 rows);
int launch_gate_up_q8_wide(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream);
int launch_down_q8_wide(const b200moe_down_view& v, u32 rows, cudaStream_t stream);
// gemv_q8_mma.cu: the same contract with the integer dots on the tensor cores (mma.sync s8 x s8), lane classes shared out over the warps.
bool q8_mma_gate_up_fits(const b200moe_gate_up_view& v, u32 rows);
bool q8_mma_down_fits(const b200moe_down_view& v, u32 rows);
int launch_gate_up_q8_mma(const b200moe_gate_up_view& v, u32 rows, cudaStream_t stream);
int launch_down_q8_mma(const b200moe_down_view& v, u32 rows, cudaStream_t stream);
// value of a B200MOE_DEBUG_* hook (api.cu)
u32 debug_value(u32 key);

// prologue.cu: A8 + router + routes of a decode window (rows <= 8) in one launch; ticket: a zeroed workspace word
bool prologue_fusable(const b200moe_router_view& r, u32 top_k);
int launch_prologue(const b200moe_router_view& r, const b200moe_quantize_a8_view& q, const b200moe_routes_view& routes, u32* ticket,
                    cudaStream_t stream);

// combine.cu
int launch_merge_first_error(b200moe_first_error* record, const u32* summary, u32 domain, cudaStream_t stream);
int launch_combine(const b200moe_combine_view& v, cudaStream_t stream);
int launch_canonical_sum(const float* a, const float* b, const float* c, u64 count, float* y, cudaStream_t stream);
int launch_fill_u32(u32* p, u32 value, u64 count, cudaStream_t stream);
// order[row][k] (slots in ascending expert id) for the PARTS combine when no routes were built
int launch_row_order(const u32* ids, u32 rows, u32 top_k, u32* order, cudaStream_t stream);

}  // namespace b200moe
