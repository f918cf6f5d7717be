// Reference-side adapter: the routed-expert operator layer of the reference's CUDA backend
// (include/strix/cuda/ds41_moe.hpp, include/strix/cuda/ds41_core.hpp) implemented on top of the C ABI of b200moe.h.
//
// A maintainer adds this file to the backend library in place of the sm_120 kernels' translation units
// (cmake/StrixCudaBackend.cmake:14-21) and links libb200moe.so; callers such as LayerCore::ffn_core
// (src/cuda/models/ds41/ds41_core_layer.cu:314-341) compile unchanged. Every function is a field-for-field copy of a
// reference view into the matching C view, the reference's error behaviour included: an argument error leaves the C
// ABI as a status and becomes the std::invalid_argument the reference throws before anything is enqueued
// (include/strix/cuda/ds41_common.hpp:33-35), every other failure a std::runtime_error.
//
// The stored formats are chosen by the two constants below: the reference header documents IQ2_XXS / Q2_K tensors for
// this family, the B200 library binds the Q8_0 and Q4_K families (ggml type ids 8 and 12), so a build that links this
// adapter loads those tensors.
//
// tests/test_abi.py compiles this file against the reference checkout's headers (syntax and types only).
#include <stdexcept>

#include "b200moe.h"
#include "strix/cuda/ds41_core.hpp"
#include "strix/cuda/ds41_moe.hpp"

namespace strix::ds41::cuda {
namespace {

constexpr std::uint32_t kGateType = B200MOE_TYPE_Q8_0, kDownType = B200MOE_TYPE_Q8_0;

void b200_check(int rc) {
    if (rc == B200MOE_OK) return;
    if (rc == B200MOE_ERR_INVALID_ARGUMENT || rc == B200MOE_ERR_WORKSPACE) throw std::invalid_argument(b200moe_last_error());
    throw std::runtime_error(b200moe_last_error());
}
b200moe_shape shape_of(const MoeShape& s) { return b200moe_shape{s.hidden, s.inter, s.experts, s.top_k, kGateType, kDownType, s.limit}; }
b200moe_a8_rows rows_of(const A8Rows& a) { return b200moe_a8_rows{a.codes, a.deltas, a.sums, a.rows, a.width, a.stride}; }
b200moe_expert_weights weights_of(const ExpertWeights& w) { return b200moe_expert_weights{w.gate, w.up, w.down}; }
b200moe_routes routes_of(const MoeRoutes& r) { return b200moe_routes{r.experts, r.begins, r.rows, r.slots, r.order, r.low_counts, r.counts}; }

}  // namespace

void enqueue_quantize_a8(const QuantizeA8View& v, cudaStream_t stream) {
    b200moe_quantize_a8_view b{};
    b.x = v.x; b.rows = v.rows; b.width = v.width; b.x_stride = v.x_stride; b.x_is_bf16 = 0; b.out = rows_of(v.out);
    b200_check(b200moe_quantize_a8(&b, stream));
}

void enqueue_moe_routes(const MoeRoutesView& v, cudaStream_t stream) {
    b200moe_routes_view b{};
    b.ids = v.ids; b.rows = v.rows; b.top_k = v.top_k; b.experts = v.experts; b.split = v.split;
    b.first = v.first; b.end = v.end; b.base = v.base; b.scratch = v.scratch; b.out = routes_of(v.out);
    b200_check(b200moe_build_routes(&b, stream));
}

void enqueue_routed_gate_up(const RoutedGateUpView& v, cudaStream_t stream) {
    b200moe_gate_up_view b{};
    b.shape = shape_of(v.shape); b.weights = weights_of(v.weights); b.routes = routes_of(v.routes); b.max_union = v.max_union;
    b.x = rows_of(v.x); b.act = rows_of(v.act); b.gate_out = v.gate_out; b.up_out = v.up_out;
    b200_check(b200moe_gate_up(&b, stream));
}

void enqueue_routed_down(const RoutedDownView& v, cudaStream_t stream) {
    if (v.raw1) throw std::invalid_argument("b200 adapter: the two-rank K-half split of the down projection (raw1) is not bound; use b200moe_tp_dense / b200moe_ep_ffn");
    b200moe_down_view b{};
    b.shape = shape_of(v.shape); b.weights = weights_of(v.weights); b.routes = routes_of(v.routes); b.max_union = v.max_union;
    b.act = rows_of(v.act); b.raw = v.raw;
    b200_check(b200moe_down(&b, stream));
}

void enqueue_moe_combine(const MoeCombineView& v, cudaStream_t stream) {
    if (v.raw1 || v.hc_out) throw std::invalid_argument("b200 adapter: the K-half combine (raw1) and the fused hc_expand are outside the bound path");
    b200moe_combine_view b{};
    b.raw = v.raw; b.shared = v.shared; b.weights = v.weights; b.order = v.order; b.low_counts = v.low_counts;
    b.rows = v.rows; b.top_k = v.top_k; b.hidden = v.hidden;
    b.form = B200MOE_COMBINE_PARTS; b.parts = 2; b.part_experts = 0; b.only_part = v.half;   // half 0 / 1 = the low / high sum alone
    b.y = v.out;
    b200_check(b200moe_combine(&b, stream));
}

void enqueue_moe_canonical_sum(const float* shared, const float* low, const float* high, std::size_t count, float* out, cudaStream_t stream) {
    b200_check(b200moe_canonical_sum(shared, low, high, count, out, stream));
}

std::size_t moe_layer_workspace_bytes(std::uint32_t capacity, const MoeShape& shape) noexcept {
    const b200moe_shape b = shape_of(shape);
    return static_cast<std::size_t>(b200moe_layer_workspace_bytes(&b, capacity));
}

void enqueue_moe_layer(const MoeLayerView& v, cudaStream_t stream) {
    if (v.raw1) throw std::invalid_argument("b200 adapter: expert TP parts (raw1) are not bound");
    b200moe_layer_view b{};
    b.shape = shape_of(v.shape); b.weights = weights_of(v.weights); b.rows = v.rows; b.x = rows_of(v.x);
    b.ids = v.ids; b.route_weights = v.route_weights; b.shared = v.shared;
    b.combine_form = B200MOE_COMBINE_PARTS; b.parts = 2; b.part_experts = v.split; b.only_part = -1;   // y = (shared + low) + high
    b.raw = v.raw; b.y = v.y;
    b.workspace = v.workspace; b.workspace_bytes = moe_layer_workspace_bytes(v.capacity, v.shape);
    b.capacity = v.capacity; b.grouped_min_rows = v.grouped_min_rows;
    b200_check(b200moe_layer(&b, stream));
}

void enqueue_router(const RouterView& v, cudaStream_t stream) {
    if (v.bias_image) throw std::invalid_argument("b200 adapter: the per-row bias image of the router is not bound");
    b200moe_router_view b{};
    b.x = v.x; b.x_stride = v.x_stride; b.rows = v.rows; b.hidden = v.weight.width; b.weight = v.weight.data; b.bias = v.bias;
    // the family's preset (include/strix/moe/route_policy.hpp:62-71): sqrt-softplus scores, biased selection, float key,
    // selection order, renormalised weights times route_scale
    b.policy = b200moe_route_policy{B200MOE_SCORE_SQRT_SOFTPLUS, v.bias != nullptr, B200MOE_KEY_FLOAT_SERIAL, B200MOE_ORDER_SELECTION,
                                    v.weight.rows, v.top_k, 1, 1, 1, 0, 1e-20F, v.route_scale};
    b.logits = v.scores; b.scores = v.scores; b.ids = v.ids; b.weights = v.weights;
    b200_check(b200moe_router(&b, stream));
}

}  // namespace strix::ds41::cuda
