// Reference-side adapter: the Qwen routed-MoE operator layer (include/strix/cuda/qwen_moe.hpp:96-109) on top of the C
// ABI of b200moe.h. The reference's Rows are per-row strided views in bytes; the C ABI takes dense row-major arrays, so
// the adapter admits the layouts whose strides are exactly the dense ones (what prepare_known_moe_prefill produces for a
// contiguous block) and says so otherwise - before anything is enqueued, as the reference's own argument checks do.
//
// enqueue_routed + enqueue_combine map onto b200moe_layer (routes, gate/up + SwiGLU + A8 of h, down, the slot-order fma
// merge, the bfloat16 commit); the prologue (A8 of the bfloat16 input) is b200moe_quantize_a8 with x_is_bf16.
// The gfx1151 correction tables (amdmath::Tables) are not an input: the library evaluates the exp twin at zero tables,
// the form the reference's own bench uses (scripts/bench/residency/cpu_expert_bench.cpp:78-89).
//
// tests/test_abi.py compiles this file against the reference checkout's headers (syntax and types only).
#include <stdexcept>

#include "b200moe.h"
#include "strix/cuda/qwen_moe.hpp"

namespace strix::cuda::qwen_moe {
namespace {

void b200_check(int rc) {
    if (rc == B200MOE_OK) return;
    if (rc == B200MOE_ERR_INVALID_ARGUMENT || rc == B200MOE_ERR_WORKSPACE) throw std::invalid_argument(b200moe_last_error());
    throw std::runtime_error(b200moe_last_error());
}
template <class T>
T* dense(const Strided<T>& v, std::uint64_t row_bytes, const char* what) {
    if (v.base && v.stride != row_bytes) throw std::invalid_argument(std::string("b200 adapter: ") + what + " must be a dense row-major array");
    return v.base;
}
b200moe_shape shape_of(const Weights& w) { return b200moe_shape{hidden, ffn, experts, top_k, w.gate_type, w.down_type, 0.0F}; }

// Caller-owned scratch of the layer call: the adapter keeps the reference's rule that entry points allocate nothing, so
// the engine passes it in through Rows::intermediates (sized >= b200moe_layer_workspace_bytes, checked by the library).
b200moe_layer_view layer_view(const Rows& r, std::uint32_t rows, const Weights& w) {
    b200moe_layer_view b{};
    b.shape = shape_of(w);
    b.weights = b200moe_expert_weights{w.gate, w.up, w.down};
    b.rows = rows;
    b.x = b200moe_a8_rows{dense(r.codes, hidden, "codes"), dense(r.deltas, hidden / 32 * 4, "deltas"), dense(r.sums, hidden / 32 * 4, "sums"), rows, hidden, hidden};
    b.ids = dense(r.routes, top_k * 4, "routes");
    b.route_weights = dense(r.route_weights, top_k * 4, "route_weights");
    b.combine_form = B200MOE_COMBINE_FMA_SLOTS;
    b.only_part = -1;
    b.raw = dense(r.rawdots, std::uint64_t{top_k} * hidden * 4, "rawdots");
    b.y = dense(r.accumulation, hidden * 4, "accumulation");
    b.y_bf16 = dense(r.output, hidden * 2, "output");
    b.row_status = dense(r.status, 4, "status");
    b.summary = r.csr.summary;
    b.workspace = r.intermediates.base;
    b.workspace_bytes = r.intermediates.stride * rows;
    b.capacity = rows;
    return b;
}

}  // namespace

void enqueue_prologue(const Rows& r, std::uint32_t rows, std::uint32_t, cudaStream_t stream) {
    b200moe_quantize_a8_view b{};
    b.x = dense(r.input, hidden * 2, "input"); b.rows = rows; b.width = hidden; b.x_stride = hidden; b.x_is_bf16 = 1;
    b.out = b200moe_a8_rows{dense(r.codes, hidden, "codes"), dense(r.deltas, hidden / 32 * 4, "deltas"), dense(r.sums, hidden / 32 * 4, "sums"), rows, hidden, hidden};
    b.status = dense(r.status, 4, "status");
    b200_check(b200moe_quantize_a8(&b, stream));
}

bool enqueue(const Rows& r, std::uint32_t rows, std::uint32_t clear_words, const Weights& w, const amdmath::Tables&, std::uint32_t*, cudaStream_t stream, bool moe_mma) {
    if (moe_mma || native_types(w) || gsq_types(w)) throw std::invalid_argument("b200 adapter: only the exact A8 profile (Q4_K / Q5_K gate, Q5_1 / Q8_0 / Q4_K down) is bound");
    enqueue_prologue(r, rows, clear_words, stream);
    const b200moe_layer_view b = layer_view(r, rows, w);
    b200_check(b200moe_layer(&b, stream));
    return false;
}

}  // namespace strix::cuda::qwen_moe
