// Residency planner: which experts to bring into HBM slots ahead of need, under an upload budget per step. Host code only
// (no device work): the counterpart of strix::residency::Planner (include/strix/residency/expert_residency.hpp:102-147,
// src/residency/expert_residency.cpp:277-410), behind the C ABI, with the state in flat arrays.
//
// Rule (expert_residency.hpp:121-127): score = decayed count of steps that used the expert. Per layer the non-resident
// experts with a positive score, best first, take the free slots; the rest are paired in order with the resident experts
// the current step does not use, weakest first, for as long as score_candidate - score_victim > margin_reuses. All pairs
// of all layers are then ordered (free slots first, gain descending, layer, expert) and accepted while the step's upload
// budget lasts - a pair that does not fit is skipped, not the end of the list, and one expert larger than the whole budget
// may still move alone. plan() does not change the state; commit() records one move.
#include <algorithm>
#include <numeric>
#include <vector>

#include "kernels.cuh"

namespace b200moe {
namespace {

struct Planner {
    u32 layers = 0, experts = 0, slots = 0, top_k = 0;
    double decay = 0.97, margin = 1.5;
    u64 budget = 64ull << 20;
    std::vector<u64> bytes;        // [layers] one expert of the layer
    std::vector<double> score;     // [layers][experts]
    std::vector<i32> table;        // [layers][experts] expert -> slot or -1
    std::vector<i32> slot_expert;  // [layers][slots]   slot -> expert or -1
    std::vector<u8> used;          // [layers][experts] seen in the current (or the just ended) step
    bool step_ended = true;
    b200moe_planner_receipt receipt{};

    double& sc(u32 l, u32 e) { return score[size_t(l) * experts + e]; }
    double sc(u32 l, u32 e) const { return score[size_t(l) * experts + e]; }
    i32& tb(u32 l, u32 e) { return table[size_t(l) * experts + e]; }
    i32 tb(u32 l, u32 e) const { return table[size_t(l) * experts + e]; }
    i32& se(u32 l, u32 s) { return slot_expert[size_t(l) * slots + s]; }
    i32 se(u32 l, u32 s) const { return slot_expert[size_t(l) * slots + s]; }
    bool seen(u32 l, u32 e) const { return used[size_t(l) * experts + e] != 0; }
};

struct Pair {
    b200moe_move move;
    double gain;
    bool into_free_slot;
};

// The layer's pairs, appended to `out`.
void pairs_of_layer(const Planner& p, u32 l, std::vector<Pair>* out) {
    std::vector<u32> incoming, leaving, open;
    for (u32 e = 0; e < p.experts; ++e)
        if (p.tb(l, e) < 0 && p.sc(l, e) > 0.0) incoming.push_back(e);
    for (u32 s = 0; s < p.slots; ++s) {
        const i32 e = p.se(l, s);
        if (e < 0) open.push_back(s);
        else if (!p.seen(l, static_cast<u32>(e))) leaving.push_back(static_cast<u32>(e));
    }
    std::sort(incoming.begin(), incoming.end(), [&](u32 a, u32 b) { return p.sc(l, a) != p.sc(l, b) ? p.sc(l, a) > p.sc(l, b) : a < b; });
    std::sort(leaving.begin(), leaving.end(), [&](u32 a, u32 b) { return p.sc(l, a) != p.sc(l, b) ? p.sc(l, a) < p.sc(l, b) : a < b; });
    size_t next = 0;
    for (size_t i = 0; i < open.size() && next < incoming.size(); ++i, ++next)
        out->push_back({b200moe_move{l, open[i], B200MOE_MOVE_NO_EVICTION, incoming[next]}, p.sc(l, incoming[next]), true});
    for (size_t v = 0; v < leaving.size() && next < incoming.size(); ++v, ++next) {
        const double gain = p.sc(l, incoming[next]) - p.sc(l, leaving[v]);  // one layer's experts have one size
        if (!(gain > p.margin)) break;
        out->push_back({b200moe_move{l, static_cast<u32>(p.tb(l, leaving[v])), leaving[v], incoming[next]}, gain, false});
    }
}

Planner* as_planner(void* h) { return static_cast<Planner*>(h); }
const Planner* as_planner(const void* h) { return static_cast<const Planner*>(h); }

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_planner_create(const b200moe_planner_desc* d, void** out) {
    B200_REQUIRE(d && out, "planner_create: null argument");
    B200_REQUIRE(d->layers && d->experts && d->slots && d->expert_bytes, "planner_create: layers / experts / slots / expert_bytes must be set");
    B200_REQUIRE(!(d->decay < 0.0) && d->decay < 1.0, "planner_create: decay must lie in [0, 1)");
    auto* p = new Planner;
    p->layers = d->layers; p->experts = d->experts; p->slots = std::min(d->slots, d->experts); p->top_k = d->top_k;
    p->decay = d->decay > 0.0 ? d->decay : 0.97;
    p->margin = d->margin_reuses > 0.0 ? d->margin_reuses : 1.5;
    p->budget = d->upload_bytes_per_step ? d->upload_bytes_per_step : (64ull << 20);
    p->bytes.assign(d->expert_bytes, d->expert_bytes + d->layers);
    p->score.assign(size_t(p->layers) * p->experts, 0.0);
    p->table.assign(size_t(p->layers) * p->experts, -1);
    p->slot_expert.assign(size_t(p->layers) * p->slots, -1);
    p->used.assign(size_t(p->layers) * p->experts, 0);
    *out = p;
    return B200MOE_OK;
}

void b200moe_planner_destroy(void* planner) { delete as_planner(planner); }

// A prior: counts [experts] of how often each expert was used; turned into the steady-state score of that use rate.
int b200moe_planner_seed(void* planner, uint32_t layer, const uint32_t* counts) {
    Planner* p = as_planner(planner);
    B200_REQUIRE(p && counts && layer < p->layers, "planner_seed: null argument or layer out of range");
    double total = 0;
    for (u32 e = 0; e < p->experts; ++e) total += counts[e];
    if (total <= 0) return B200MOE_OK;
    const double steady = 1.0 / (1.0 - p->decay), k = p->top_k ? double(p->top_k) : 1.0;
    for (u32 e = 0; e < p->experts; ++e) p->sc(layer, e) = std::min(1.0, counts[e] / total * k) * steady;
    return B200MOE_OK;
}

int b200moe_planner_observe(void* planner, uint32_t layer, const uint32_t* ids, uint32_t n) {
    Planner* p = as_planner(planner);
    B200_REQUIRE(p && (ids || !n) && layer < p->layers, "planner_observe: null argument or layer out of range");
    if (p->step_ended) {  // the first observation of a new step forgets the last step's marks
        std::fill(p->used.begin(), p->used.end(), u8{0});
        p->step_ended = false;
    }
    for (u32 i = 0; i < n; ++i)
        if (ids[i] < p->experts) p->used[size_t(layer) * p->experts + ids[i]] = 1;
    return B200MOE_OK;
}

int b200moe_planner_end_step(void* planner) {
    Planner* p = as_planner(planner);
    B200_REQUIRE(p, "planner_end_step: null handle");
    for (u32 l = 0; l < p->layers; ++l)
        for (u32 e = 0; e < p->experts; ++e) {
            const bool hit = p->seen(l, e);
            p->sc(l, e) = p->sc(l, e) * p->decay + (hit ? 1.0 : 0.0);
            if (hit) {
                p->receipt.active_bytes += p->bytes[l];
                if (p->tb(l, e) >= 0) p->receipt.hit_bytes += p->bytes[l];
            }
        }
    p->receipt.steps += 1;
    p->step_ended = true;  // the marks stay readable for plan() until the next observation
    return B200MOE_OK;
}

int b200moe_planner_plan(const void* planner, b200moe_move* moves, uint32_t capacity, uint32_t* count) {
    const Planner* p = as_planner(planner);
    B200_REQUIRE(p && count && (moves || !capacity), "planner_plan: null argument");
    std::vector<Pair> all;
    for (u32 l = 0; l < p->layers; ++l) pairs_of_layer(*p, l, &all);
    std::sort(all.begin(), all.end(), [](const Pair& a, const Pair& b) {  // (layer, expert) is unique: a total order
        if (a.into_free_slot != b.into_free_slot) return a.into_free_slot;
        if (a.gain != b.gain) return a.gain > b.gain;
        if (a.move.layer != b.move.layer) return a.move.layer < b.move.layer;
        return a.move.expert < b.move.expert;
    });
    u64 spent = 0;
    u32 n = 0;
    for (const Pair& c : all) {
        const u64 b = p->bytes[c.move.layer];
        const bool alone_over_budget = n == 0 && b > p->budget;
        if (spent + b > p->budget && !alone_over_budget) continue;
        spent += b;
        if (n < capacity) moves[n] = c.move;
        ++n;
    }
    *count = n;  // more than `capacity`: the caller's array was too small, the first `capacity` moves are valid
    return B200MOE_OK;
}

int b200moe_planner_commit(void* planner, const b200moe_move* m) {
    Planner* p = as_planner(planner);
    B200_REQUIRE(p && m, "planner_commit: null argument");
    B200_REQUIRE(m->layer < p->layers && m->slot < p->slots && m->expert < p->experts && (m->evict == B200MOE_MOVE_NO_EVICTION || m->evict < p->experts),
                 "planner_commit: the move is out of range");
    if (m->evict != B200MOE_MOVE_NO_EVICTION) {
        p->tb(m->layer, m->evict) = -1;
        p->receipt.evictions += 1;
    }
    p->se(m->layer, m->slot) = static_cast<i32>(m->expert);
    p->tb(m->layer, m->expert) = static_cast<i32>(m->slot);
    p->receipt.promotions += 1;
    p->receipt.promoted_bytes += p->bytes[m->layer];
    return B200MOE_OK;
}

// Initial residency: the best seeded experts of every layer, in score order (ties: lower expert), at no receipt cost.
int b200moe_planner_fill_from_seed(void* planner) {
    Planner* p = as_planner(planner);
    B200_REQUIRE(p, "planner_fill_from_seed: null handle");
    std::vector<u32> order(p->experts);
    for (u32 l = 0; l < p->layers; ++l) {
        std::iota(order.begin(), order.end(), 0u);
        std::stable_sort(order.begin(), order.end(), [&](u32 a, u32 b) { return p->sc(l, a) > p->sc(l, b); });
        for (u32 e = 0; e < p->experts; ++e) p->tb(l, e) = -1;
        for (u32 s = 0; s < p->slots; ++s) {
            p->se(l, s) = static_cast<i32>(order[s]);
            p->tb(l, order[s]) = static_cast<i32>(s);
        }
    }
    return B200MOE_OK;
}

int b200moe_planner_table(const void* planner, uint32_t layer, int32_t* table) {
    const Planner* p = as_planner(planner);
    B200_REQUIRE(p && table && layer < p->layers, "planner_table: null argument or layer out of range");
    std::copy(p->table.begin() + size_t(layer) * p->experts, p->table.begin() + size_t(layer + 1) * p->experts, table);
    return B200MOE_OK;
}

int b200moe_planner_scores(const void* planner, uint32_t layer, double* scores) {
    const Planner* p = as_planner(planner);
    B200_REQUIRE(p && scores && layer < p->layers, "planner_scores: null argument or layer out of range");
    std::copy(p->score.begin() + size_t(layer) * p->experts, p->score.begin() + size_t(layer + 1) * p->experts, scores);
    return B200MOE_OK;
}

int b200moe_planner_get_receipt(const void* planner, b200moe_planner_receipt* out) {
    const Planner* p = as_planner(planner);
    B200_REQUIRE(p && out, "planner_get_receipt: null argument");
    *out = p->receipt;
    return B200MOE_OK;
}

}  // extern "C"
