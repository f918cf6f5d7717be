// TEST INFRASTRUCTURE - not part of the shipped library.
//
// C entry points around the reference engine's OWN CPU code for the MoE FFN path. This file holds no arithmetic of
// its own (apart from the clearly marked threaded driver at the end, used only to time the reference's row kernels):
// it includes the reference's headers and is linked with object files compiled from the reference's source files
// where they lie (see oracle/Makefile); nothing of the reference is copied into this repository. The result,
// oracle/_ref/libstrixref.so, validates the restatement in oracle/moe_oracle.cpp, generates the vectors under
// tests/golden/, and is the "reference" CPU baseline of the benchmark.
#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <mutex>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <functional>
#include <limits>
#include <unistd.h>
#include <memory>
#include <optional>
#include <span>
#include <stdexcept>
#include <string>
#include <thread>
#include <vector>

#include "cpu/arch/avx2/routed_expert_avx2.hpp"
#include "cpu/core/backend.hpp"
#include "cpu/core/routed_expert.hpp"
#include "cpu/core/routed_expert_kernels.hpp"
#include "strix/ds41_formats.hpp"
#include "strix/ds41_moe.hpp"
#include "strix/gguf_reader.hpp"
#include "strix/moe/combine.hpp"
#include "strix/moe/route_policy.hpp"
#include "strix/moe_a8_down_contract.hpp"
#include "strix/moe_plan.hpp"
#include "strix/moe_q4k_a8_contract.hpp"
#include "strix/residency/expert_residency.hpp"

// src/moe_plan.cpp references this symbol from the GGUF reader (storage planning only, never on the routing path);
// the reader itself drags in the whole weight library, so the link is closed with an empty answer.
namespace strix::gguf {
std::optional<TensorTypeGeometry> tensor_type_geometry(std::uint32_t) noexcept { return std::nullopt; }
}

namespace {
using u8 = std::uint8_t;
using u32 = std::uint32_t;
using i8 = std::int8_t;
using i32 = std::int32_t;
namespace ex = strix::cpu::expert;

struct Ds41Math {
    static float exp(float x) { return strix::ds41::declared_exp(x); }
    static float log1p(float x) { return strix::ds41::declared_log1p(x); }
    static float sqrt(float x) { return strix::ds41::declared_sqrt(x); }
};

const ex::Gfx1151Exp& zero_exp() {
    static const std::unique_ptr<ex::Gfx1151Exp> exp = [] {
        const auto dir = std::filesystem::temp_directory_path() / ("b200moe_exp_tables_" + std::to_string(::getpid()));
        std::filesystem::create_directories(dir);
        const u32 zero[2] = {0, 0};  // the bench's zero tables (scripts/bench/residency/cpu_expert_bench.cpp:78-89)
        for (const char* n : {"tbl_exp_pm.bin", "hard_v_exp_f32.bin"}) {
            FILE* f = std::fopen((dir / n).c_str(), "wb");
            std::fwrite(zero, 4, 2, f);
            std::fclose(f);
        }
        return std::make_unique<ex::Gfx1151Exp>(dir.string());
    }();
    return *exp;
}

strix::moe::RoutePolicy to_policy(const u32* p, float eps, float scale) {
    strix::moe::RoutePolicy r;
    r.score = static_cast<strix::moe::RouteScore>(p[0]);
    r.selection_bias = p[1] != 0;
    r.key = static_cast<strix::moe::RouteKey>(p[2]);
    r.order = static_cast<strix::moe::RouteOrder>(p[3]);
    r.experts = p[4]; r.top_k = p[5]; r.n_group = p[6]; r.topk_group = p[7];
    r.renormalize = p[8] != 0; r.renorm_single = p[9] != 0;
    r.renorm_eps = eps; r.scale = scale;
    return r;
}
}  // namespace

extern "C" {

float ref_half_to_float(std::uint16_t h) { return strix::cpu::half_to_float(h); }
float ref_declared_exp(float x) { return strix::ds41::declared_exp(x); }
float ref_router_score(float z) { return strix::ds41::router_score(z); }
float ref_swiglu_clamped(float g, float u, float limit) { return strix::ds41::swiglu_clamped(g, u, limit); }
float ref_gfx1151_expf(float x) { return zero_exp().expf(x); }
const char* ref_cpu_isa() { return strix::cpu::isa_name(strix::cpu::select(strix::cpu::caps()).isa); }
// Name of the routed-expert row-kernel table the executor binds on this host ("scalar", "avx2", "avx2+vnni").
const char* ref_expert_isa() {
    static const std::string name = [] { ex::Executor e(1, zero_exp(), true); return std::string(e.isa()); }();
    return name.c_str();
}

// strix::cpu reference table (src/cpu/core/reference.cpp). 1 = rejected (std::invalid_argument).
int ref_quantize_a8(const float* x, std::size_t width, i8* codes, float* deltas, i32* sums) {
    try { strix::cpu::reference_kernels().quantize_a8(x, width, codes, deltas, sums); } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
int ref_gemv_q8_0_a8(const u8* weight, u32 row_bytes, u32 in, u32 count, u32 rows, const i8* codes, const float* deltas,
                     u32 x_stride, float* out, u32 out_stride, u32 accumulate) {
    const strix::cpu::Q8a8View v{weight, codes, deltas, out, row_bytes, in, count, rows, x_stride, out_stride, accumulate};
    try { strix::cpu::reference_kernels().gemv_q8_0_a8(v, {}); } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
// strix::ds41 host references (src/ds41_formats.cpp).
void ref_rmsnorm_f32(const float* x, const float* w, u32 n, float eps, float* y, u32 rows) {
    strix::cpu::reference_kernels().rmsnorm_f32(x, w, n, eps, y, rows, strix::cpu::Stream{});
}

void ref_ds41_quantize_a8(const float* x, std::size_t width, i8* codes, float* deltas, i32* sums) {
    const auto a = strix::ds41::quantize_a8(std::span<const float>(x, width));
    std::memcpy(codes, a.codes.data(), width);
    std::memcpy(deltas, a.deltas.data(), width / 32 * 4);
    std::memcpy(sums, a.sums.data(), width / 32 * 4);
}
float ref_product_q8_0(const u8* row, const i8* codes, const float* deltas, std::size_t width) {
    strix::ds41::A8Activation a;
    a.codes.assign(codes, codes + width);
    a.deltas.assign(deltas, deltas + width / 32);
    a.sums.assign(width / 32, 0);
    return strix::ds41::product_q8_0(std::span<const u8>(row, width / 32 * 34), a, width);
}

// strix::ds41::reference_router (src/ds41_moe.cpp:63-97): sqrt-softplus scores, ds41 preset.
int ref_reference_router(const float* x, u32 rows, u32 hidden, const float* weight, u32 experts, const float* bias,
                         const float* bias_image, const u8* image_rows, u32 top_k, float scale, float* scores, u32* ids,
                         float* weights) {
    try {
        const auto out = strix::ds41::reference_router(
            std::span<const float>(x, (std::size_t)rows * hidden), rows, hidden,
            std::span<const float>(weight, (std::size_t)experts * hidden), experts, std::span<const float>(bias, experts),
            bias_image ? std::span<const float>(bias_image, experts) : std::span<const float>(),
            image_rows ? std::span<const u8>(image_rows, rows) : std::span<const u8>(), top_k, scale);
        if (scores) std::memcpy(scores, out.scores.data(), out.scores.size() * 4);
        std::memcpy(ids, out.ids.data(), out.ids.size() * 4);
        std::memcpy(weights, out.weights.data(), out.weights.size() * 4);
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
// strix::moe::route_scores_ref<Ds41Math> / route_select_ref (include/strix/moe/route_policy.hpp:99-156).
// policy words: score, selection_bias, key, order, experts, top_k, n_group, topk_group, renormalize, renorm_single.
int ref_route_scores(u32 score, const float* logits, u32 n, float* scores) {
    try {
        strix::moe::route_scores_ref<Ds41Math>(static_cast<strix::moe::RouteScore>(score), std::span<const float>(logits, n),
                                               std::span<float>(scores, n));
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
int ref_route_select(const u32* policy, float eps, float scale, const float* scores, const float* bias, u32* ids, float* weights) {
    const auto p = to_policy(policy, eps, scale);
    try {
        strix::moe::route_select_ref(p, std::span<const float>(scores, p.experts),
                                     bias ? std::span<const float>(bias, p.experts) : std::span<const float>(),
                                     std::span<u32>(ids, p.top_k), std::span<float>(weights, p.top_k));
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
// strix::select_moe_experts_deterministic (src/moe_plan.cpp:101-162): std::exp softmax cross-check.
int ref_select_softmax(const float* logits, u32 n, u32 top_k, int normalize, u32* ids, float* weights) {
    try {
        const auto s = strix::select_moe_experts_deterministic(std::span<const float>(logits, n), top_k, normalize != 0);
        std::memcpy(ids, s.experts.data(), top_k * 4);
        std::memcpy(weights, s.weights.data(), top_k * 4);
    } catch (const std::exception&) { return 1; }
    return 0;
}

// build_window_routes + restrict_routes (src/ds41_moe.cpp:11-61). Output arrays as include/b200moe.h; experts are NOT
// rebased here. Returns the union count or -1 (std::invalid_argument).
int ref_window_routes(const u32* ids, u32 rows, u32 top_k, u32 split, u32 first, u32 end, u32* experts, u32* begins, u32* out_rows,
                      u32* slots, u32* order, u32* low_counts, u32* max_rows) {
    try {
        auto r = strix::ds41::build_window_routes(std::span<const u32>(ids, (std::size_t)rows * top_k), rows, top_k, split);
        if (end) r = strix::ds41::restrict_routes(r, first, end);
        std::memcpy(experts, r.experts.data(), r.experts.size() * 4);
        std::memcpy(begins, r.begins.data(), r.begins.size() * 4);
        std::memcpy(out_rows, r.rows.data(), r.rows.size() * 4);
        std::memcpy(slots, r.slots.data(), r.slots.size() * 4);
        std::memcpy(order, r.order.data(), r.order.size() * 4);
        std::memcpy(low_counts, r.low_counts.data(), r.low_counts.size() * 4);
        *max_rows = r.max_rows;
        return (int)r.experts.size();
    } catch (const std::invalid_argument&) { return -1; }
}

// strix::ds41::reference_window with Q8_0 tensors (src/ds41_moe.cpp:124-165). x: FP32 rows quantised with
// ds41::quantize_a8. Outputs: gate / up [slot][inter], act codes [slot][inter] / deltas / sums, raw [slot][hidden], y.
// gate_type / down_type: ggml type ids 8 (Q8_0) or 10 (Q2_K), the two block types of the family that this build binds.
int ref_window_ds41(u32 gate_type, u32 down_type, const u8* gate, const u8* up, const u8* down, u32 experts, u32 hidden, u32 inter, float limit,
                    const float* x, u32 rows, const u32* ids, const float* weights, const float* shared, u32 top_k, u32 split, u32 first, u32 end,
                    float* gate_out, float* up_out, i8* act_codes, float* act_deltas, i32* act_sums, float* raw, float* y) {
    try {
        const auto format_of = [](u32 t) { return t == 10 ? strix::ds41::WeightFormat::q2_k : strix::ds41::WeightFormat::q8_0; };
        const auto row_bytes = [](u32 t, u32 width) { return t == 10 ? std::size_t(width / 256) * 84 : std::size_t(width / 32) * 34; };
        strix::ds41::ExpertTensors t;
        t.gate_up_format = format_of(gate_type);
        t.down_format = format_of(down_type);
        t.hidden = hidden; t.inter = inter; t.limit = limit;
        t.gate = std::span<const u8>(gate, (std::size_t)experts * inter * row_bytes(gate_type, hidden));
        t.up = std::span<const u8>(up, t.gate.size());
        t.down = std::span<const u8>(down, (std::size_t)experts * hidden * row_bytes(down_type, inter));
        std::vector<strix::ds41::A8Activation> xa;
        for (u32 r = 0; r < rows; ++r) xa.push_back(strix::ds41::quantize_a8(std::span<const float>(x + (std::size_t)r * hidden, hidden)));
        auto routes = strix::ds41::build_window_routes(std::span<const u32>(ids, (std::size_t)rows * top_k), rows, top_k, split);
        if (end) routes = strix::ds41::restrict_routes(routes, first, end);
        const auto out = strix::ds41::reference_window(t, xa, routes, std::span<const float>(weights, (std::size_t)rows * top_k),
                                                       std::span<const float>(shared, (std::size_t)rows * hidden), top_k);
        const std::size_t slots = (std::size_t)rows * top_k;
        if (gate_out) std::memcpy(gate_out, out.gate.data(), slots * inter * 4);
        if (up_out) std::memcpy(up_out, out.up.data(), slots * inter * 4);
        for (std::size_t s = 0; s < slots; ++s) {
            if (out.activation[s].codes.empty()) continue;
            if (act_codes) std::memcpy(act_codes + s * inter, out.activation[s].codes.data(), inter);
            if (act_deltas) std::memcpy(act_deltas + s * (inter / 32), out.activation[s].deltas.data(), inter / 32 * 4);
            if (act_sums) std::memcpy(act_sums + s * (inter / 32), out.activation[s].sums.data(), inter / 32 * 4);
        }
        if (raw) std::memcpy(raw, out.raw.data(), slots * hidden * 4);
        if (y) std::memcpy(y, out.y.data(), (std::size_t)rows * hidden * 4);
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}
int ref_window_q8_0(const u8* gate, const u8* up, const u8* down, u32 experts, u32 hidden, u32 inter, float limit, const float* x,
                    u32 rows, const u32* ids, const float* weights, const float* shared, u32 top_k, u32 split, u32 first, u32 end,
                    float* gate_out, float* up_out, i8* act_codes, float* act_deltas, i32* act_sums, float* raw, float* y) {
    return ref_window_ds41(8, 8, gate, up, down, experts, hidden, inter, limit, x, rows, ids, weights, shared, top_k, split, first, end, gate_out, up_out,
                           act_codes, act_deltas, act_sums, raw, y);
}
// reference_half_sum (src/ds41_moe.cpp:99-115).
int ref_half_sum(const u32* ids, u32 rows, u32 top_k, u32 split, const float* weights, const float* raw, u32 hidden, unsigned half, float* out) {
    try {
        const auto routes = strix::ds41::build_window_routes(std::span<const u32>(ids, (std::size_t)rows * top_k), rows, top_k, split);
        const auto v = strix::ds41::reference_half_sum(routes, std::span<const float>(weights, (std::size_t)rows * top_k),
                                                       std::span<const float>(raw, (std::size_t)rows * top_k * hidden), rows, top_k, hidden, half);
        std::memcpy(out, v.data(), v.size() * 4);
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}

// strix::cpu::expert (src/cpu/core/routed_expert.cpp): reference_run (threads == 0) or Executor(threads, simd).
// gate_format 0 q4_k / 1 q5_k; down_format 0 q5_1 / 1 q8_0. assignments: count x {row, slot, expert}.
// rawdots [rows][slots_per_row][hidden]; status [rows].
int ref_expert_run(const u8* gate, const u8* up, const u8* down, u32 gate_format, u32 down_format, u32 hidden, u32 ffn,
                   const i8* codes, const float* deltas, const i32* sums, u32 rows, const u32* assignments, u32 count,
                   u32 slots_per_row, float* rawdots, u32* status, u32 threads, int simd) {
    std::vector<ex::RowA8> ra(rows);
    for (u32 r = 0; r < rows; ++r)
        ra[r] = {codes + (std::size_t)r * hidden, deltas + (std::size_t)r * (hidden / 32), sums + (std::size_t)r * (hidden / 32)};
    std::vector<ex::Assignment> as(count);
    for (u32 a = 0; a < count; ++a) as[a] = {assignments[3 * a], assignments[3 * a + 1], assignments[3 * a + 2]};
    ex::Job job;
    job.weights.gate = gate; job.weights.up = up; job.weights.down = down;
    job.weights.gate_format = static_cast<ex::GateFormat>(gate_format);
    job.weights.down_format = static_cast<ex::DownFormat>(down_format);
    job.weights.shape = {hidden, ffn};
    job.rows = ra.data(); job.assignments = as.data(); job.count = count;
    job.rawdots = rawdots; job.rawdot_row_stride = (std::uint64_t)slots_per_row * hidden; job.status = status;
    if (threads == 0) ex::reference_run(job, zero_exp());
    else { ex::Executor e(threads, zero_exp(), simd != 0); e.run(job); }
    return 0;
}
// One gate/up row through the executor's kernel tables (scalar oracle table or the AVX2 table).
float ref_gate_row_q4k(const u8* wrow, u32 blocks, const i8* codes, const float* deltas, const i32* sums, int simd) {
    const ex::RowA8 row{codes, deltas, sums};
    const ex::RowA8* rp = &row;
    const ex::detail::Kernels* k = &ex::detail::scalar_kernels();
    if (simd) if (const auto* a = strix::cpu::arch::avx2::expert_kernels()) k = a;
    float out = 0.0f;
    k->gate[0](wrow, blocks, &rp, 1, &out);
    return out;
}
float ref_down_row_q8_0(const u8* wrow, u32 groups, const i8* codes, const float* deltas, const i32* sums) {
    float out = 0.0f;
    ex::detail::scalar_kernels().down[1](wrow, groups, &codes, &deltas, &sums, 1, &out);
    return out;
}
// Contract-level oracles (src/moe_q4k_a8_contract.cpp:126-141; src/moe_a8_down_contract.cpp:141-211). NaN on a
// rejected row (width limits: 2560 gate/up, 1536 K-quant down).
float ref_evaluate_row_q4k(const u8* w, const i8* codes, const float* deltas, const i32* sums, u32 width) {
    strix::moe_q4k_a8::QuantizedRow q;
    q.codes.assign(codes, codes + width); q.deltas.assign(deltas, deltas + width / 32); q.sums.assign(sums, sums + width / 32);
    try { return strix::moe_q4k_a8::evaluate_row(std::span<const std::byte>(reinterpret_cast<const std::byte*>(w), width / 256 * 144), q); }
    catch (const std::exception&) { return std::numeric_limits<float>::quiet_NaN(); }
}
float ref_evaluate_down_row(const u8* w, const i8* codes, const float* deltas, const i32* sums, u32 width, u32 type) {
    strix::moe_q4k_a8::QuantizedRow q;
    q.codes.assign(codes, codes + width); q.deltas.assign(deltas, deltas + width / 32); q.sums.assign(sums, sums + width / 32);
    try {
        const auto bytes = strix::moe_q4k_a8::down_row_bytes(type, width);
        return strix::moe_q4k_a8::evaluate_down_row(std::span<const std::byte>(reinterpret_cast<const std::byte*>(w), type == 12 ? width / 256 * 144 : bytes), q, type);
    } catch (const std::exception&) { return std::numeric_limits<float>::quiet_NaN(); }
}
// strix::moe::combine_ref (include/strix/moe/combine.hpp:36-59). form 0 fma_f32, 1 bf16_steps.
int ref_combine(u32 form, u32 rows, u32 top_k, u32 width, const float* w, const float* eo, const float* base, float* y) {
    const std::size_t n = (std::size_t)rows * width;
    try {
        strix::moe::combine_ref(static_cast<strix::moe::CombineForm>(form), rows, top_k, width,
                                w ? std::span<const float>(w, (std::size_t)rows * top_k) : std::span<const float>(),
                                std::span<const float>(eo, n * top_k), base ? std::span<const float>(base, n) : std::span<const float>(),
                                std::span<float>(y, n));
    } catch (const std::invalid_argument&) { return 1; }
    return 0;
}

// The reference's residency planner (include/strix/residency/expert_residency.hpp:102-147) driven over a scripted trace:
// optional seed + fill_from_seed, then per step observe(layer, ids) for every layer, end_step, plan (twice: it must not
// change the state), and commit of every planned move. Outputs: the moves of every step, the final tables and scores,
// the receipt counters.
int ref_planner_trace(u32 layers, u32 experts, u32 top_k, u32 slots, const std::uint64_t* expert_bytes, double decay, double margin,
                      std::uint64_t budget, const u32* seed_counts, int fill, u32 steps, const u32* ids, u32 n_ids, u32* moves_out, u32 max_moves,
                      u32* move_counts, i32* tables_out, double* scores_out, std::uint64_t* receipt_out) {
    try {
        strix::residency::ModelBytes m;
        m.layers = layers; m.experts = experts; m.top_k = top_k;
        m.expert_bytes.assign(expert_bytes, expert_bytes + layers);
        strix::residency::PlannerConfig cfg;
        cfg.decay = decay; cfg.margin_reuses = margin; cfg.upload_bytes_per_step = budget;
        strix::residency::Planner planner(m, slots, cfg);
        if (seed_counts)
            for (u32 l = 0; l < layers; ++l) planner.seed(l, seed_counts + std::size_t(l) * experts);
        if (fill) planner.fill_from_seed();
        for (u32 s = 0; s < steps; ++s) {
            for (u32 l = 0; l < layers; ++l) planner.observe(l, ids + (std::size_t(s) * layers + l) * n_ids, n_ids);
            planner.end_step();
            const auto first = planner.plan(), moves = planner.plan();
            if (first.size() != moves.size()) return 2;
            move_counts[s] = static_cast<u32>(moves.size());
            for (std::size_t i = 0; i < moves.size(); ++i) {
                if (i < max_moves) {
                    u32* o = moves_out + (std::size_t(s) * max_moves + i) * 4;
                    o[0] = moves[i].layer; o[1] = moves[i].slot; o[2] = moves[i].evict; o[3] = moves[i].expert;
                }
                planner.commit(moves[i]);
            }
        }
        for (u32 l = 0; l < layers; ++l) std::copy(planner.table(l).begin(), planner.table(l).end(), tables_out + std::size_t(l) * experts);
        (void)scores_out;  // the scores are private to the reference's class: the moves and tables are what they decide
        const auto r = planner.receipt();
        receipt_out[0] = r.active_bytes; receipt_out[1] = r.hit_bytes; receipt_out[2] = r.promoted_bytes;
        receipt_out[3] = r.promotions; receipt_out[4] = r.evictions; receipt_out[5] = r.steps;
        return 0;
    } catch (const std::exception&) {
        return 1;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Timing driver (the benchmark's reference arm). It runs the reference's own row kernels - the executor's table
// (AVX2 / AVX-VNNI when the host has it, else scalar) for Q4_K gate/up AND for the Q4_K down rows (the reference's
// Q4_K down contract is the gate/up row rule over K = inter, include/strix/moe_a8_down_contract.hpp:9-11; its executor
// itself only binds Q5_1 / Q8_0 down, src/cpu/core/routed_expert.hpp:27-28), its Gfx1151Exp and its A8 rule, its
// router (reference_router's dot order + route_scores_ref / route_select_ref) - over all host threads with the
// executor's item split ((expert, 32-output group), then (expert, 16 hidden outputs)). The worker threads are created
// once and kept (a pool, as Executor keeps its own), so that no thread start or join sits inside a timed call.
}  // extern "C"

namespace {

class Pool {
  public:
    explicit Pool(unsigned threads) : n_(std::max(1u, threads)) {
        for (unsigned t = 1; t < n_; ++t) workers_.emplace_back([this] { loop(); });
    }
    ~Pool() {
        { std::lock_guard<std::mutex> l(m_); stop_ = true; ++epoch_; }
        cv_.notify_all();
        for (auto& t : workers_) t.join();
    }
    unsigned size() const { return n_; }
    void run(u32 n, const std::function<void(u32)>& fn) {
        { std::lock_guard<std::mutex> l(m_); fn_ = &fn; count_ = n; next_.store(0); busy_ = n_ - 1; ++epoch_; }
        cv_.notify_all();
        work();
        std::unique_lock<std::mutex> l(m_);
        done_.wait(l, [this] { return busy_ == 0; });
    }

  private:
    void work() { for (;;) { const u32 i = next_.fetch_add(1, std::memory_order_relaxed); if (i >= count_) break; (*fn_)(i); } }
    void loop() {
        std::uint64_t seen = 0;
        for (;;) {
            { std::unique_lock<std::mutex> l(m_); cv_.wait(l, [&] { return epoch_ != seen; }); seen = epoch_; if (stop_) return; }
            work();
            { std::lock_guard<std::mutex> l(m_); if (--busy_ == 0) done_.notify_one(); }
        }
    }
    unsigned n_;
    std::vector<std::thread> workers_;
    std::mutex m_;
    std::condition_variable cv_, done_;
    const std::function<void(u32)>* fn_ = nullptr;
    u32 count_ = 0;
    std::atomic<u32> next_{0};
    unsigned busy_ = 0;
    std::uint64_t epoch_ = 0;
    bool stop_ = false;
};

Pool& pool_of(unsigned threads) {
    static std::mutex m;
    static std::unique_ptr<Pool> pool;
    std::lock_guard<std::mutex> l(m);
    if (!pool || pool->size() != std::max(1u, threads)) pool.reset(new Pool(threads));
    return *pool;
}

// The routed experts of one layer call on given routes: A8 of x, gate/up + SwiGLU + A8 of h, down -> raw slot vectors.
void experts_q4k(Pool& pool, const u8* gate, const u8* up, const u8* down, u32 hidden, u32 inter, u32 top_k, const float* x, u32 rows,
                 const u32* ids, std::vector<float>& raw) {
    const ex::detail::Kernels* k = &ex::detail::scalar_kernels();
    if (strix::cpu::caps().avx2) if (const auto* a = strix::cpu::arch::avx2::expert_kernels()) k = a;
    const u32 blocks = hidden / 256, groups = inter / 32, dblocks = inter / 256;
    const std::size_t grow = (std::size_t)blocks * 144, drow = (std::size_t)dblocks * 144;
    const auto& exp = zero_exp();
    // A8 of the input (strix::cpu reference table)
    std::vector<i8> xc((std::size_t)rows * hidden);
    std::vector<float> xd((std::size_t)rows * hidden / 32);
    std::vector<i32> xs(xd.size());
    for (u32 r = 0; r < rows; ++r)
        strix::cpu::reference_kernels().quantize_a8(x + (std::size_t)r * hidden, hidden, xc.data() + (std::size_t)r * hidden,
                                                   xd.data() + (std::size_t)r * hidden / 32, xs.data() + (std::size_t)r * hidden / 32);
    // group slots by expert (stable), as Executor::prepare
    const std::size_t slots = (std::size_t)rows * top_k;
    std::vector<u32> order(slots);
    for (u32 i = 0; i < order.size(); ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](u32 a, u32 b) { return ids[a] < ids[b]; });
    std::vector<u32> ex_begin, ex_id;
    for (u32 p = 0; p < order.size(); ++p)
        if (p == 0 || ids[order[p]] != ids[order[p - 1]]) { ex_id.push_back(ids[order[p]]); ex_begin.push_back(p); }
    ex_begin.push_back((u32)order.size());
    std::vector<ex::RowA8> rowa(rows);
    for (u32 r = 0; r < rows; ++r) rowa[r] = {xc.data() + (std::size_t)r * hidden, xd.data() + (std::size_t)r * hidden / 32, xs.data() + (std::size_t)r * hidden / 32};
    std::vector<i8> hc(slots * inter);
    std::vector<float> hd(slots * groups);
    std::vector<i32> hs(slots * groups);
    const u32 n_ex = (u32)ex_id.size();
    pool.run(n_ex * groups, [&](u32 item) {
        const u32 e = item / groups, grp = item % groups, expert = ex_id[e];
        for (u32 p = ex_begin[e]; p < ex_begin[e + 1]; p += ex::detail::kMaxAssign) {
            const u32 na = std::min(ex::detail::kMaxAssign, ex_begin[e + 1] - p);
            const ex::RowA8* rp[ex::detail::kMaxAssign];
            for (u32 a = 0; a < na; ++a) rp[a] = &rowa[order[p + a] / top_k];
            float g[ex::detail::kMaxAssign][32], u[ex::detail::kMaxAssign][32];
            for (u32 l = 0; l < 32; ++l) {
                float tg[ex::detail::kMaxAssign], tu[ex::detail::kMaxAssign];
                const std::size_t off = ((std::size_t)expert * inter + grp * 32 + l) * grow;
                k->gate[0](gate + off, blocks, rp, na, tg);
                k->gate[0](up + off, blocks, rp, na, tu);
                for (u32 a = 0; a < na; ++a) { g[a][l] = tg[a]; u[a][l] = tu[a]; }
            }
            for (u32 a = 0; a < na; ++a) {
                float hv[32];
                for (u32 l = 0; l < 32; ++l) hv[l] = (g[a][l] / (1.0F + exp.expf(-g[a][l]))) * u[a][l];
                const std::size_t s = order[p + a];
                strix::cpu::reference_kernels().quantize_a8(hv, 32, hc.data() + s * inter + grp * 32, &hd[s * groups + grp], &hs[s * groups + grp]);
            }
        }
    });
    raw.assign(slots * hidden, 0.0F);
    pool.run(n_ex * (hidden / 16), [&](u32 item) {
        const u32 per = hidden / 16, e = item / per, o0 = (item % per) * 16, expert = ex_id[e];
        for (u32 p = ex_begin[e]; p < ex_begin[e + 1]; p += ex::detail::kMaxAssign) {
            const u32 na = std::min(ex::detail::kMaxAssign, ex_begin[e + 1] - p);
            ex::RowA8 ha[ex::detail::kMaxAssign];
            const ex::RowA8* rp[ex::detail::kMaxAssign];
            for (u32 a = 0; a < na; ++a) {
                const std::size_t s = order[p + a];
                ha[a] = {hc.data() + s * inter, hd.data() + s * groups, hs.data() + s * groups};
                rp[a] = &ha[a];
            }
            for (u32 l = 0; l < 16; ++l) {
                float t[ex::detail::kMaxAssign];
                k->gate[0](down + ((std::size_t)expert * hidden + o0 + l) * drow, dblocks, rp, na, t);
                for (u32 a = 0; a < na; ++a) raw[(std::size_t)order[p + a] * hidden + o0 + l] = t[a];
            }
        }
    });
}

}  // namespace

extern "C" {

// Router (softmax policy) + routed experts + Qwen merge, `reps` times. Returns seconds; y receives the last call's output
// so the caller can check it.
double ref_time_layer_q4k(const u8* gate, const u8* up, const u8* down, u32 experts, u32 hidden, u32 inter, u32 top_k,
                          const float* router_w, const float* x, u32 rows, unsigned threads, u32 reps, float* y, u32* ids_out) {
    Pool& pool = pool_of(threads);
    const strix::moe::RoutePolicy policy{strix::moe::RouteScore::softmax, false, strix::moe::RouteKey::float_serial,
                                         strix::moe::RouteOrder::selection, experts, top_k, 1U, 1U, true, true, 1e-20F, 1.0F};
    const auto t0 = std::chrono::steady_clock::now();
    for (u32 rep = 0; rep < reps; ++rep) {
        // router: declared dot order (src/ds41_moe.cpp:72-82), softmax transform, k-pass selection
        std::vector<float> logits((std::size_t)rows * experts);
        pool.run(rows * experts, [&](u32 i) {
            const u32 r = i / experts, e = i % experts;
            float lanes[32] = {};
            for (u32 c = 0; c < hidden; ++c) lanes[c % 32] = lanes[c % 32] + router_w[(std::size_t)e * hidden + c] * x[(std::size_t)r * hidden + c];
            for (unsigned d = 16; d; d /= 2) { float n[32]; for (unsigned l = 0; l < 32; ++l) n[l] = lanes[l] + lanes[l ^ d]; std::memcpy(lanes, n, sizeof n); }
            logits[i] = lanes[0];
        });
        std::vector<u32> ids((std::size_t)rows * top_k);
        std::vector<float> rw(ids.size());
        for (u32 r = 0; r < rows; ++r) {
            std::vector<float> s(experts);
            strix::moe::route_scores_ref<Ds41Math>(policy.score, std::span<const float>(logits.data() + (std::size_t)r * experts, experts), s);
            strix::moe::route_select_ref(policy, s, {}, std::span<u32>(ids.data() + (std::size_t)r * top_k, top_k),
                                         std::span<float>(rw.data() + (std::size_t)r * top_k, top_k));
        }
        std::vector<float> raw;
        experts_q4k(pool, gate, up, down, hidden, inter, top_k, x, rows, ids.data(), raw);
        // Qwen merge (combine_ref fma_f32, base 0)
        std::vector<float> zero((std::size_t)rows * hidden, 0.0F);
        strix::moe::combine_ref(strix::moe::CombineForm::fma_f32, rows, top_k, hidden, rw, raw, zero, std::span<float>(y, (std::size_t)rows * hidden));
        if (ids_out) std::memcpy(ids_out, ids.data(), ids.size() * 4);
    }
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

// The routed experts alone on the caller's routes (ids [rows][top_k] into the given tensors), `reps` times: what the
// benchmark's CPU arm times for a layer whose router the reference does not have (group-limited selection). raw_out
// [rows * top_k][hidden] receives the last call's raw slot vectors.
double ref_time_experts_q4k(const u8* gate, const u8* up, const u8* down, u32 hidden, u32 inter, u32 top_k, const float* x, u32 rows,
                            const u32* ids, unsigned threads, u32 reps, float* raw_out) {
    Pool& pool = pool_of(threads);
    std::vector<float> raw;
    const auto t0 = std::chrono::steady_clock::now();
    for (u32 rep = 0; rep < reps; ++rep) experts_q4k(pool, gate, up, down, hidden, inter, top_k, x, rows, ids, raw);
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (raw_out) std::memcpy(raw_out, raw.data(), raw.size() * 4);
    return sec;
}

// The dense Q8_0 x A8 product of the CPU backend (strix::cpu::Kernels::gemv_q8_0_a8, scalar) with the output rows
// partitioned over the host threads, which docs/architecture/backends.md:94-98 allows a Stream to do. `reps` times.
double ref_time_gemv_q8_0_a8(const u8* weight, u32 row_bytes, u32 width, u32 count, u32 rows, const i8* codes, const float* deltas,
                             unsigned threads, u32 reps, float* out) {
    Pool& pool = pool_of(threads);
    const auto& kernels = strix::cpu::reference_kernels();
    const u32 chunk = 64, chunks = (count + chunk - 1) / chunk;
    const auto t0 = std::chrono::steady_clock::now();
    for (u32 rep = 0; rep < reps; ++rep)
        pool.run(chunks, [&](u32 item) {
            const u32 c0 = item * chunk, n = std::min(chunk, count - c0);
            const strix::cpu::Q8a8View v{weight + (std::size_t)c0 * row_bytes, codes, deltas, out + c0, row_bytes, width, n, rows, width, count, 0U};
            kernels.gemv_q8_0_a8(v, {});
        });
    return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

// Pure read of `bytes` bytes with all host threads (64-bit sums over 1 MiB pieces), `reps` times: the host's read-bandwidth
// ceiling that the timed CPU arm is quoted beside (the reference's own bench prints the same figure first,
// scripts/bench/residency/cpu_expert_bench.cpp:168-177). Returns seconds; *sink receives the sum so the reads are kept.
double ref_time_read(const u8* buf, std::size_t bytes, unsigned threads, u32 reps, std::uint64_t* sink) {
    Pool& pool = pool_of(threads);
    const std::size_t piece = std::size_t(1) << 20, pieces = (bytes + piece - 1) / piece;
    std::atomic<std::uint64_t> total{0};
    const auto t0 = std::chrono::steady_clock::now();
    for (u32 rep = 0; rep < reps; ++rep)
        pool.run(static_cast<u32>(pieces), [&](u32 item) {
            const std::size_t b = item * piece, e = std::min(bytes, b + piece);
            std::uint64_t s = 0;
            for (std::size_t i = b; i + 8 <= e; i += 8) { std::uint64_t v; std::memcpy(&v, buf + i, 8); s += v; }
            total.fetch_add(s, std::memory_order_relaxed);
        });
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (sink) *sink = total.load();
    return sec;
}

}  // extern "C"
