// Expert residency: a layer with more experts than HBM slots. The expert ids of a window are mapped to slots through a
// device table; an expert that is not resident is copied from host memory into a victim slot on the caller's stream and
// then computed on the GPU like any other (the reference computes such an expert on the CPU and lets a device kernel spin
// on a host flag: include/strix/cuda/tiered_experts.hpp:1-17 - here no kernel waits on the host).
//
// Policy (after include/strix/residency/expert_residency.hpp:121-127): score = decayed count of windows that used the
// expert; free slots fill first; an expert the current window uses is never evicted; victims by (score, expert) ascending.
//
// Per window: memset(marks) -> mark kernel -> marks to pinned host memory -> ONE stream synchronisation -> host picks
// victims, enqueues the copies (gate, up, down of each missing expert) and the new table -> remap kernel writes the
// slot ids. No miss: the first kernel has already written the slot ids and nothing else is enqueued.
#include <algorithm>
#include <numeric>
#include <vector>

#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kNoSlot = 0xffffffffu;

// slot_ids[i] = table[ids[i]] (kNoSlot for an id out of range or a non-resident expert); marks[e] = 1 for every id seen.
__global__ void __launch_bounds__(256) residency_map_kernel(const u32* __restrict__ ids, u32 count, const i32* __restrict__ table, u32 experts,
                                                            u32* __restrict__ slot_ids, u32* __restrict__ marks) {
    const u32 i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const u32 e = ids[i];
    u32 slot = kNoSlot;
    if (e < experts) {
        const i32 s = table[e];
        if (s >= 0) slot = static_cast<u32>(s);
        if (marks) marks[e] = 1u;
    }
    slot_ids[i] = slot;
}

struct Residency {
    b200moe_residency_desc d{};
    u64 gate_bytes = 0, down_bytes = 0;    // per expert (up = gate)
    std::vector<i32> table;                // expert -> slot or -1
    std::vector<i32> slot_expert;          // slot -> expert or -1
    std::vector<double> score;
    i32* table_dev = nullptr;
    u32* marks_dev = nullptr;
    u32* marks_host = nullptr;             // pinned
    i32* table_host = nullptr;             // pinned staging of the table upload
    i32* promote_host = nullptr;           // pinned staging of the table upload of b200moe_residency_promote
    cudaEvent_t promote_done = nullptr;    // that upload has left promote_host
    int device = 0;
    double decay = 0.97;
    b200moe_residency_stats stats{};
};

int choose_victims(const i32* slot_expert, u32 slots, const double* score, const u8* used, u32 experts, const u32* missing, u32 n_missing,
                   u32* victims) {
    std::vector<u32> order;
    order.reserve(slots);
    for (u32 s = 0; s < slots; ++s)
        if (slot_expert[s] < 0) order.push_back(s);
    const size_t n_free = order.size();
    for (u32 s = 0; s < slots; ++s) {
        const i32 e = slot_expert[s];
        if (e >= 0 && static_cast<u32>(e) < experts && !used[e]) order.push_back(s);
    }
    std::stable_sort(order.begin() + static_cast<std::ptrdiff_t>(n_free), order.end(), [&](u32 a, u32 b) {
        const i32 ea = slot_expert[a], eb = slot_expert[b];
        if (score[ea] != score[eb]) return score[ea] < score[eb];
        return ea < eb;
    });
    if (order.size() < n_missing)
        return fail(B200MOE_ERR_WORKSPACE, "residency: the window needs %u more experts than the %zu slots that may be refilled", n_missing, order.size());
    for (u32 i = 0; i < n_missing; ++i) victims[i] = order[i];
    (void)missing;
    return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_residency_choose_victims(const int32_t* slot_expert, uint32_t slots, const double* score, const uint8_t* used, uint32_t experts,
                                     const uint32_t* missing, uint32_t n_missing, uint32_t* victims) {
    B200_REQUIRE(slot_expert && score && used && (missing || !n_missing) && (victims || !n_missing), "choose_victims: null argument");
    for (u32 s = 0; s < slots; ++s) B200_REQUIRE(slot_expert[s] < static_cast<i32>(experts), "choose_victims: slot %u holds expert %d of %u", s, slot_expert[s], experts);
    return choose_victims(slot_expert, slots, score, used, experts, missing, n_missing, victims);
}

int b200moe_residency_create(const b200moe_residency_desc* desc, void** out) {
    B200_REQUIRE(desc && out, "residency_create: null argument");
    const b200moe_shape& s = desc->shape;
    B200_REQUIRE(s.experts && s.hidden && s.inter, "residency_create: shape has a zero dimension");
    B200_REQUIRE(desc->slots >= 1 && desc->slots <= s.experts, "residency_create: slots %u outside 1 .. %u", desc->slots, s.experts);
    B200_REQUIRE(desc->gate_host && desc->up_host && desc->down_host, "residency_create: host tensors are null");
    B200_REQUIRE(desc->gate_slots && desc->up_slots && desc->down_slots, "residency_create: slot tensors are null");
    B200_REQUIRE(aligned(desc->gate_slots, 16) && aligned(desc->up_slots, 16) && aligned(desc->down_slots, 16), "residency_create: slot tensors must be 16-byte aligned");
    B200_REQUIRE(desc->decay >= 0.0f && desc->decay <= 1.0f, "residency_create: decay %g outside 0 .. 1", desc->decay);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    auto* r = new Residency();
    r->d = *desc;
    r->gate_bytes = row_bytes_of(s.gate_type, s.hidden) * s.inter;
    r->down_bytes = row_bytes_of(s.down_type, s.inter) * s.hidden;
    r->table.assign(s.experts, -1);
    r->slot_expert.assign(desc->slots, -1);
    r->score.assign(s.experts, 0.0);
    if (desc->decay > 0.0f) r->decay = desc->decay;
    cudaError_t e = cudaGetDevice(&r->device);
    if (e == cudaSuccess) e = cudaMalloc(&r->table_dev, sizeof(i32) * s.experts);
    if (e == cudaSuccess) e = cudaMalloc(&r->marks_dev, sizeof(u32) * s.experts);
    if (e == cudaSuccess) e = cudaHostAlloc(&r->marks_host, sizeof(u32) * s.experts, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaHostAlloc(&r->table_host, sizeof(i32) * s.experts, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaHostAlloc(&r->promote_host, sizeof(i32) * s.experts, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&r->promote_done, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaMemset(r->table_dev, 0xff, sizeof(i32) * s.experts);  // every expert absent (-1)
    if (e != cudaSuccess) {
        const int rc = fail(B200MOE_ERR_CUDA, "residency_create: %s", cudaGetErrorString(e));
        b200moe_residency_destroy(r);
        return rc;
    }
    *out = r;
    return B200MOE_OK;
}

void b200moe_residency_destroy(void* residency) {
    auto* r = static_cast<Residency*>(residency);
    if (!r) return;
    if (r->table_dev) cudaFree(r->table_dev);
    if (r->marks_dev) cudaFree(r->marks_dev);
    if (r->marks_host) cudaFreeHost(r->marks_host);
    if (r->table_host) cudaFreeHost(r->table_host);
    if (r->promote_host) cudaFreeHost(r->promote_host);
    if (r->promote_done) cudaEventDestroy(r->promote_done);
    delete r;
}

int b200moe_residency_get_stats(const void* residency, b200moe_residency_stats* out) {
    B200_REQUIRE(residency && out, "residency_get_stats: null argument");
    *out = static_cast<const Residency*>(residency)->stats;
    return B200MOE_OK;
}

int b200moe_residency_table(const void* residency, int32_t* table_host) {
    B200_REQUIRE(residency && table_host, "residency_table: null argument");
    const auto* r = static_cast<const Residency*>(residency);
    std::copy(r->table.begin(), r->table.end(), table_host);
    return B200MOE_OK;
}

int b200moe_residency_map(void* residency, const uint32_t* ids, uint32_t count, uint32_t* slot_ids, void* stream) {
    B200_REQUIRE(residency, "residency_map: null handle");
    if (count == 0) return B200MOE_OK;
    B200_REQUIRE(ids && slot_ids, "residency_map: ids / slot_ids are null");
    auto* r = static_cast<Residency*>(residency);
    const u32 E = r->d.shape.experts, S = r->d.slots;
    cudaStream_t st = as_stream(stream);
    const u32 blocks = (count + 255u) / 256u;
    cudaError_t e = cudaMemsetAsync(r->marks_dev, 0, sizeof(u32) * E, st);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "residency_map: cudaMemsetAsync: %s", cudaGetErrorString(e));
    residency_map_kernel<<<blocks, 256, 0, st>>>(ids, count, r->table_dev, E, slot_ids, r->marks_dev);
    if (int rc = after_launch("residency_map")) return rc;
    e = cudaMemcpyAsync(r->marks_host, r->marks_dev, sizeof(u32) * E, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);  // the one host wait of a window: which experts does it use?
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "residency_map: reading the marks: %s", cudaGetErrorString(e));

    std::vector<u8> used(E);
    std::vector<u32> missing;
    u32 n_used = 0;
    for (u32 x = 0; x < E; ++x) {
        used[x] = r->marks_host[x] != 0;
        n_used += used[x];
        if (used[x] && r->table[x] < 0) missing.push_back(x);
    }
    std::vector<u32> victims(missing.size());
    if (!missing.empty())  // refused before any state changes: the caller may split the window and try again
        if (int rc = choose_victims(r->slot_expert.data(), S, r->score.data(), used.data(), E, missing.data(), static_cast<u32>(missing.size()), victims.data()))
            return rc;
    // scores: decayed count of the windows that used the expert
    for (u32 x = 0; x < E; ++x) r->score[x] = r->score[x] * r->decay + (used[x] ? 1.0 : 0.0);
    r->stats.windows += 1;
    r->stats.hits += n_used - missing.size();
    r->stats.misses += missing.size();
    if (missing.empty()) return B200MOE_OK;

    for (size_t i = 0; i < missing.size(); ++i) {
        const u32 x = missing[i], s = victims[i];
        if (r->slot_expert[s] >= 0) { r->table[r->slot_expert[s]] = -1; r->stats.evictions += 1; }
        r->slot_expert[s] = static_cast<i32>(x);
        r->table[x] = static_cast<i32>(s);
        e = cudaMemcpyAsync(r->d.gate_slots + u64(s) * r->gate_bytes, r->d.gate_host + u64(x) * r->gate_bytes, r->gate_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(r->d.up_slots + u64(s) * r->gate_bytes, r->d.up_host + u64(x) * r->gate_bytes, r->gate_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(r->d.down_slots + u64(s) * r->down_bytes, r->d.down_host + u64(x) * r->down_bytes, r->down_bytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "residency_map: loading expert %u into slot %u: %s", x, s, cudaGetErrorString(e));
        r->stats.bytes_loaded += 2 * r->gate_bytes + r->down_bytes;
    }
    // the previous upload from table_host completed before the synchronisation above
    std::copy(r->table.begin(), r->table.end(), r->table_host);
    e = cudaMemcpyAsync(r->table_dev, r->table_host, sizeof(i32) * E, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "residency_map: table upload: %s", cudaGetErrorString(e));
    residency_map_kernel<<<blocks, 256, 0, st>>>(ids, count, r->table_dev, E, slot_ids, nullptr);
    return after_launch("residency_remap");
}

int b200moe_residency_promote(void* residency, const b200moe_move* moves, uint32_t count, void* stream) {
    B200_REQUIRE(residency && (moves || !count), "residency_promote: null argument");
    if (count == 0) return B200MOE_OK;
    auto* r = static_cast<Residency*>(residency);
    const u32 E = r->d.shape.experts, S = r->d.slots;
    // every move is checked against the state the earlier moves leave, before anything is copied
    std::vector<i32> slot_expert = r->slot_expert, table = r->table;
    for (u32 i = 0; i < count; ++i) {
        const b200moe_move& m = moves[i];
        B200_REQUIRE(m.slot < S && m.expert < E, "residency_promote: move %u names slot %u / expert %u outside %u / %u", i, m.slot, m.expert, S, E);
        B200_REQUIRE(table[m.expert] < 0, "residency_promote: move %u: expert %u is already resident", i, m.expert);
        const i32 cur = slot_expert[m.slot];
        B200_REQUIRE(cur < 0 ? m.evict == B200MOE_MOVE_NO_EVICTION : static_cast<u32>(cur) == m.evict,
                     "residency_promote: move %u: slot %u holds expert %d, the move expects %d", i, m.slot, cur, static_cast<int>(m.evict));
        if (cur >= 0) table[cur] = -1;
        slot_expert[m.slot] = static_cast<i32>(m.expert);
        table[m.expert] = static_cast<i32>(m.slot);
    }
    cudaStream_t st = as_stream(stream);
    cudaError_t e = cudaEventSynchronize(r->promote_done);  // the previous promotion's table has left the staging buffer
    for (u32 i = 0; i < count && e == cudaSuccess; ++i) {
        const u32 x = moves[i].expert, s = moves[i].slot;
        e = cudaMemcpyAsync(r->d.gate_slots + u64(s) * r->gate_bytes, r->d.gate_host + u64(x) * r->gate_bytes, r->gate_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(r->d.up_slots + u64(s) * r->gate_bytes, r->d.up_host + u64(x) * r->gate_bytes, r->gate_bytes, cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaMemcpyAsync(r->d.down_slots + u64(s) * r->down_bytes, r->d.down_host + u64(x) * r->down_bytes, r->down_bytes, cudaMemcpyHostToDevice, st);
        if (moves[i].evict != B200MOE_MOVE_NO_EVICTION) r->stats.evictions += 1;
        r->stats.bytes_loaded += 2 * r->gate_bytes + r->down_bytes;
    }
    if (e == cudaSuccess) {
        std::copy(table.begin(), table.end(), r->promote_host);
        e = cudaMemcpyAsync(r->table_dev, r->promote_host, sizeof(i32) * E, cudaMemcpyHostToDevice, st);
    }
    if (e == cudaSuccess) e = cudaEventRecord(r->promote_done, st);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "residency_promote: %s", cudaGetErrorString(e));
    r->slot_expert.swap(slot_expert);
    r->table.swap(table);
    return B200MOE_OK;
}

}  // extern "C"
