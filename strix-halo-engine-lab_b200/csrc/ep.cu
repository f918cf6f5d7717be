// Expert parallelism of one node behind the C ABI: the whole step of a rank - route its home rows, DISPATCH them to the
// ranks whose experts they selected, run the local experts over what arrived, RETURN the partial sums to the rows' home
// ranks, fold - is enqueued on the caller's stream by one call, b200moe_ep_ffn. No host synchronisation, no collective
// library on the path: both exchanges are this library's own kernels storing straight into the peers' memory over
// NVLink (CUDA IPC mappings, plain stores, no multicast), each followed by a per-source arrival flag, and the receiving
// rank's next kernel waits for those flags with a BOUNDED poll.
//
// The reference runs the same split on two ranks through Communicator::exchange (include/strix/dist/communicator.hpp:180;
// message shapes include/strix/ds41_moe.hpp:5-11): a rank that owns a subset of the experts restricts the window routes to
// its range (restrict_routes, src/ds41_moe.cpp:45-61), sends only what the peer's range needs and folds the partial sums
// in a fixed order (reference_half_sum, src/ds41_moe.cpp:99-115). Here: W <= 8 ranks, rank r owns experts
// [r * E / W, (r + 1) * E / W), y = (((shared + S_0) + S_1) + ...) + S_{W-1} - the bits of b200moe_ffn with parts = W.
//
// Window (one per rank, written by its peers; layout in EpLayout): per step parity p in {0, 1} the global window's A8
// rows, ids and route weights ([W * R] rows, a row lands at index home_rank * R + local row) and the returned partial
// sums ([W][R][hidden] FP32, block r from rank r), plus two flag arrays of W words (dispatch, return). A row's A8 record
// (codes + deltas + sums = 1.25 * hidden bytes) crosses NVLink only towards the ranks that own one of its experts - the
// all-to-all-v of the exchange, without counts: positions are fixed by the global row index, rows a rank does not need
// are simply not written there and its restricted routes never name them. Ids and weights (a few KB) go to every rank.
//
// Ordering. A sender's stores are followed by __threadfence_system() in every thread, a block barrier, and a ticket;
// the last block to finish fences again and stores the step number into its word of every peer's flag array. A
// receiver's wait kernel polls its own flag words (volatile loads) until each holds at least the current step, at most
// wait_polls times; after that it sets B200MOE_JOB_WAIT_ABORTED and the step's result is not written. Step numbers come
// from a device counter, so a captured graph replays correctly; the two parities separate a step's stores from the
// reads of the step before (a rank can be at most one step ahead of a peer: it needs every peer's return of step s
// before it can finish step s).
#include <cstring>

#include "kernels.cuh"

namespace b200moe {
namespace {

constexpr u32 kMaxWorld = 8;
constexpr u32 kDefaultWaitPolls = 1u << 22;  // x (a volatile load + 200 ns of sleep): about a second

struct EpLayout {
    u64 codes, deltas, sums, ids, wts, parts;  // offsets inside one parity half
    u64 half;                                  // bytes of one parity half
    u64 total;
};
constexpr u64 kFlagBytes = 256;                // dispatch flags at +0, return flags at +128 (kMaxWorld words each)

u64 up256(u64 v) { return (v + 255) & ~u64(255); }
EpLayout make_layout(const b200moe_shape& s, u32 world, u32 rows, u32 fold) {
    const u64 n = u64(world) * rows;
    EpLayout L{};
    u64 at = 0;
    L.codes = at; at = up256(at + n * s.hidden);
    L.deltas = at; at = up256(at + n * (s.hidden / 32) * 4);
    L.sums = at; at = up256(at + n * (s.hidden / 32) * 4);
    L.ids = at; at = up256(at + n * s.top_k * 4);
    L.wts = at; at = up256(at + n * s.top_k * 4);
    L.parts = at; at = up256(at + u64(fold) * rows * s.hidden * 4);  // [fold][rows][hidden]: sum p of every home row
    L.half = at;
    L.total = kFlagBytes + 2 * L.half;
    return L;
}

struct Ep {
    b200moe_shape shape;
    b200moe_route_policy policy;
    u32 world, rank, rows, per;
    u32 fold, ranges;   // expert ranges of the fold; ranges = fold / world of them belong to this rank
    unsigned char* win[kMaxWorld];
    EpLayout lay;
    float** yblocks[2];  // device arrays [world]: block `rank` of every home rank's parts, per parity
    u32* counters;       // device: [0] completed steps, [1] dispatch ticket, [2] the dispatch wait gave up, [3] fold ticket, [4] prologue ticket
    u32 calls;
    u32 wait_polls;
};

struct EpWorkspace {
    b200moe_a8_rows x;
    float* x_f32;
    float* logits;
    u32* ids;
    float* wts;
    u32* summary;
    void* layer;
    u64 layer_bytes;
    u64 bytes;
};
EpWorkspace carve(const Ep& ep, void* ws) {
    const b200moe_shape& s = ep.shape;
    unsigned char* base = static_cast<unsigned char*>(ws);
    u64 at = 0;
    auto take = [&](u64 bytes) { unsigned char* p = base ? base + at : nullptr; at = up256(at + bytes); return p; };
    EpWorkspace W{};
    W.x.codes = reinterpret_cast<i8*>(take(u64(ep.rows) * s.hidden));
    W.x.deltas = reinterpret_cast<float*>(take(u64(ep.rows) * (s.hidden / 32) * 4));
    W.x.sums = reinterpret_cast<i32*>(take(u64(ep.rows) * (s.hidden / 32) * 4));
    W.x.rows = ep.rows; W.x.width = s.hidden; W.x.stride = s.hidden;
    W.x_f32 = reinterpret_cast<float*>(take(u64(ep.rows) * s.hidden * 4));
    W.logits = reinterpret_cast<float*>(take(u64(ep.rows) * s.experts * 4));
    W.ids = reinterpret_cast<u32*>(take(u64(ep.rows) * s.top_k * 4));
    W.wts = reinterpret_cast<float*>(take(u64(ep.rows) * s.top_k * 4));
    W.summary = reinterpret_cast<u32*>(take(16));
    W.layer = take(0);
    W.layer_bytes = b200moe_layer_workspace_bytes(&s, ep.world * ep.rows);
    W.bytes = at + W.layer_bytes;
    return W;
}

struct EpDev {  // what the exchange kernels need, by value
    unsigned char* win[kMaxWorld];
    u32 world, rank, rows, per, experts, top_k, hidden;
    u64 half_base;  // kFlagBytes + parity * half
    u64 codes, deltas, sums, ids, wts;
};

// Step numbers: counters[0] holds the number of COMPLETED steps; every kernel of a step uses counters[0] + 1 and the
// step's last kernel (the fold) increments it, so a replayed graph keeps counting without a host-side argument.
__device__ __forceinline__ u32 current_step(const u32* counters) { return *reinterpret_cast<const volatile u32*>(&counters[0]) + 1u; }

// One block per home row: the row's A8 record to every rank that owns one of its experts, its ids and weights to all.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(EpDev d, b200moe_a8_rows x, const u32* __restrict__ ids, const float* __restrict__ wts,
                                                          u32* counters) {
    __shared__ u32 s_mask, s_last;
    const u32 i = blockIdx.x, tid = threadIdx.x;
    if (tid == 0) {
        u32 m = 0;
        for (u32 k = 0; k < d.top_k; ++k) {
            const u32 e = ids[i * d.top_k + k];
            if (e < d.experts) m |= 1u << min(e / d.per, d.world - 1u);
        }
        s_mask = m;
    }
    __syncthreads();
    const u32 mask = s_mask, stride = x.stride ? x.stride : x.width, gs = stride / 32;
    const u64 g = u64(d.rank) * d.rows + i;  // the row's index in the global window
    const uint4* src_c = reinterpret_cast<const uint4*>(x.codes + u64(i) * stride);
    const uint4* src_d = reinterpret_cast<const uint4*>(x.deltas + u64(i) * gs);
    const uint4* src_s = reinterpret_cast<const uint4*>(x.sums + u64(i) * gs);
    const u32 nc = d.hidden / 16, ng = d.hidden / 128;  // 16-byte pieces of the codes / of the deltas and of the sums
    for (u32 r = 0; r < d.world; ++r) {
        unsigned char* half = d.win[r] + d.half_base;
        if (tid < d.top_k) {
            reinterpret_cast<u32*>(half + d.ids)[g * d.top_k + tid] = ids[i * d.top_k + tid];
            reinterpret_cast<float*>(half + d.wts)[g * d.top_k + tid] = wts[i * d.top_k + tid];
        }
        if (!((mask >> r) & 1u)) continue;
        uint4* dst_c = reinterpret_cast<uint4*>(half + d.codes + g * d.hidden);
        uint4* dst_d = reinterpret_cast<uint4*>(half + d.deltas + g * (d.hidden / 32) * 4);
        uint4* dst_s = reinterpret_cast<uint4*>(half + d.sums + g * (d.hidden / 32) * 4);
        for (u32 v = tid; v < nc; v += blockDim.x) dst_c[v] = src_c[v];
        for (u32 v = tid; v < ng; v += blockDim.x) { dst_d[v] = src_d[v]; dst_s[v] = src_s[v]; }
    }
    // arrival: every store above is ordered before the flag stores of the block that finishes last
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&counters[1], 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    const u32 step = current_step(counters);
    if (tid < d.world) *reinterpret_cast<volatile u32*>(d.win[tid] + 4u * d.rank) = step;
}

// Waits until every source's dispatch flag holds at least the current step; bounded. On a timeout it notes it in
// counters[2] (the layer clears the job summary after this kernel, so the fold reports it). Also resets the dispatch ticket.
__global__ void ep_wait_dispatch_kernel(const unsigned char* flags, u32 world, u32* counters, u32 polls) {
    const u32 step = current_step(counters);
    if (threadIdx.x == 0) { counters[1] = 0; counters[2] = 0; }
    __syncthreads();
    if (threadIdx.x >= world) return;
    const volatile u32* f = reinterpret_cast<const volatile u32*>(flags) + threadIdx.x;
    for (u32 i = 0; i < polls; ++i) {
        if (static_cast<int>(*f - step) >= 0) { __threadfence_system(); return; }
        __nanosleep(200);
    }
    counters[2] = 1u;
}

// The last kernel of a step, after the combine kernel's peer stores (a launch boundary orders them before this kernel):
// block 0 raises this rank's return flag on every rank; every block then waits (bounded) for all W return flags and
// folds y = (((shared + S_0) + S_1) + ...) + S_{F-1}. Block 0 closes the step (counters[0] += 1), aborted or not.
__global__ void __launch_bounds__(256) ep_fold_kernel(EpDev d, const unsigned char* window, const float* __restrict__ parts, u32 n_parts, u64 part_stride,
                                                      const float* __restrict__ shared, u64 count, float* __restrict__ y, u16* __restrict__ y_bf16,
                                                      u32* counters, u32 polls, u32* summary) {
    __shared__ u32 s_ok;
    const u32 step = current_step(counters);
    if (threadIdx.x == 0) s_ok = 1;
    if (blockIdx.x == 0) {
        __threadfence_system();
        if (threadIdx.x < d.world) *reinterpret_cast<volatile u32*>(d.win[threadIdx.x] + 128u + 4u * d.rank) = step;
    }
    __syncthreads();
    if (threadIdx.x < d.world) {
        const volatile u32* f = reinterpret_cast<const volatile u32*>(window + 128) + threadIdx.x;
        bool seen = false;
        for (u32 i = 0; i < polls && !seen; ++i) {
            seen = static_cast<int>(*f - step) >= 0;
            if (!seen) __nanosleep(200);
        }
        if (!seen || counters[2]) s_ok = 0;  // a return never arrived, or the dispatch wait had given up
        __threadfence_system();
    }
    __syncthreads();
    const bool ok = s_ok != 0 && !(summary && (*summary & B200MOE_JOB_WAIT_ABORTED));
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        if (!s_ok && summary) atomicOr(summary, B200MOE_JOB_WAIT_ABORTED);
    }
    // the step is closed by the last block to get here (every block has read the step number by then)
    __shared__ u32 s_last;
    if (threadIdx.x == 0) s_last = atomicAdd(&counters[3], 1u) == gridDim.x - 1u ? 1u : 0u;
    __syncthreads();
    if (s_last && threadIdx.x == 0) { counters[3] = 0; __threadfence(); counters[0] = step; }
    if (!ok) return;  // fail closed: a piece never arrived
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float acc = shared ? shared[i] : 0.0f;
    for (u32 p = 0; p < n_parts; ++p) acc = __fadd_rn(acc, parts[u64(p) * part_stride + i]);
    y[i] = acc;
    if (y_bf16) y_bf16[i] = static_cast<u16>(bf16_rne_bits(acc));
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

uint64_t b200moe_ep_window_bytes(const b200moe_shape* shape, uint32_t world, uint32_t rows_per_rank, uint32_t fold_parts) {
    if (!shape || world == 0 || world > kMaxWorld || rows_per_rank == 0) return 0;
    const u32 fold = fold_parts ? fold_parts : world;
    if (fold % world || fold > 64) return 0;
    return make_layout(*shape, world, rows_per_rank, fold).total;
}

int b200moe_ep_create(const b200moe_ep_desc* desc, void** out) {
    B200_REQUIRE(desc && out, "ep_create: null descriptor / output");
    const b200moe_shape& s = desc->shape;
    B200_REQUIRE(desc->world >= 1 && desc->world <= kMaxWorld && desc->rank < desc->world, "ep_create: need 1 <= world <= 8 and rank < world");
    B200_REQUIRE(s.experts % desc->world == 0, "ep_create: %u experts do not split over %u ranks", s.experts, desc->world);
    B200_REQUIRE(desc->rows_per_rank >= 1 && u64(desc->rows_per_rank) * desc->world * s.top_k <= (1u << 20), "ep_create: rows_per_rank is 0 or the window is too large");
    B200_REQUIRE(s.hidden % 128 == 0, "ep_create: hidden %u must be a multiple of 128 (the A8 records move as 16-byte pieces)", s.hidden);
    B200_REQUIRE(desc->policy.experts == s.experts && desc->policy.top_k == s.top_k, "ep_create: the route policy and the shape disagree");
    B200_REQUIRE(desc->fold_parts == 0 || (desc->fold_parts % desc->world == 0 && desc->fold_parts <= 64 && s.experts % desc->fold_parts == 0),
                 "ep_create: fold_parts must be a multiple of world that divides experts (at most 64)");
    B200_REQUIRE(desc->windows, "ep_create: windows is null");
    for (u32 r = 0; r < desc->world; ++r) B200_REQUIRE(desc->windows[r] && aligned(desc->windows[r], 256), "ep_create: window %u is null or not 256-byte aligned", r);
    if (b200moe_layer_workspace_bytes(&s, desc->world * desc->rows_per_rank) == 0) return B200MOE_ERR_INVALID_ARGUMENT;  // the shape check's message stands
    if (!device_ready()) return B200MOE_ERR_CUDA;
    Ep* ep = new Ep{};
    ep->shape = s; ep->policy = desc->policy; ep->world = desc->world; ep->rank = desc->rank; ep->rows = desc->rows_per_rank;
    ep->per = s.experts / desc->world;
    ep->fold = desc->fold_parts ? desc->fold_parts : desc->world;
    ep->ranges = ep->fold / ep->world;
    ep->lay = make_layout(s, ep->world, ep->rows, ep->fold);
    ep->wait_polls = desc->wait_polls ? desc->wait_polls : kDefaultWaitPolls;
    for (u32 r = 0; r < ep->world; ++r) ep->win[r] = static_cast<unsigned char*>(desc->windows[r]);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&ep->counters), 256);
    if (e == cudaSuccess) e = cudaMemset(ep->counters, 0, 256);
    for (u32 p = 0; p < 2 && e == cudaSuccess; ++p) {
        float* host[kMaxWorld];
        for (u32 h = 0; h < ep->world; ++h)
            host[h] = reinterpret_cast<float*>(ep->win[h] + kFlagBytes + p * ep->lay.half + ep->lay.parts) + u64(ep->rank) * ep->ranges * ep->rows * s.hidden;
        e = cudaMalloc(reinterpret_cast<void**>(&ep->yblocks[p]), sizeof(float*) * kMaxWorld);
        if (e == cudaSuccess) e = cudaMemcpy(ep->yblocks[p], host, sizeof(float*) * ep->world, cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        const int rc = fail(B200MOE_ERR_CUDA, "ep_create: %s", cudaGetErrorString(e));
        b200moe_ep_destroy(ep);
        return rc;
    }
    *out = ep;
    return B200MOE_OK;
}

void b200moe_ep_destroy(void* handle) {
    Ep* ep = static_cast<Ep*>(handle);
    if (!ep) return;
    if (ep->counters) cudaFree(ep->counters);
    for (u32 p = 0; p < 2; ++p) if (ep->yblocks[p]) cudaFree(ep->yblocks[p]);
    delete ep;
}

uint64_t b200moe_ep_workspace_bytes(const void* handle) {
    const Ep* ep = static_cast<const Ep*>(handle);
    return ep ? carve(*ep, nullptr).bytes : 0;
}

int b200moe_ep_ffn(void* handle, const b200moe_ep_step_view* v, void* stream) {
    Ep* ep = static_cast<Ep*>(handle);
    B200_REQUIRE(ep && v, "ep_ffn: null handle / view");
    const b200moe_shape& s = ep->shape;
    B200_REQUIRE(v->rows == ep->rows, "ep_ffn: every rank passes rows_per_rank = %u rows, got %u", ep->rows, v->rows);
    B200_REQUIRE(v->x && v->y && v->router_weight, "ep_ffn: x / y / router_weight are null");
    B200_REQUIRE(v->weights.gate && v->weights.up && v->weights.down, "ep_ffn: the local expert tensors are null");
    B200_REQUIRE(!ep->policy.selection_bias || v->select_bias, "ep_ffn: the policy has a selection bias but select_bias is null");
    const EpWorkspace W = carve(*ep, v->workspace);
    if (!v->workspace || v->workspace_bytes < W.bytes)
        return fail(B200MOE_ERR_WORKSPACE, "ep_ffn: workspace of %llu bytes needed, %llu given", (unsigned long long)W.bytes, (unsigned long long)v->workspace_bytes);
    B200_REQUIRE(aligned(v->workspace, 256), "ep_ffn: workspace must be 256-byte aligned");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);
    const u32 parity = ep->calls++ & 1u;
    const u64 half_base = kFlagBytes + parity * ep->lay.half;
    unsigned char* mine = ep->win[ep->rank];

    // 1. route the home rows
    const float* x32 = static_cast<const float*>(v->x);
    if (v->x_is_bf16) {
        if (int rc = launch_widen_bf16(static_cast<const u16*>(v->x), W.x_f32, u64(v->rows) * s.hidden, st)) return rc;
        x32 = W.x_f32;
    }
    b200moe_quantize_a8_view q{};
    q.x = x32; q.rows = v->rows; q.width = s.hidden; q.x_stride = s.hidden; q.out = W.x;
    b200moe_router_view r{};
    r.x = x32; r.x_stride = s.hidden; r.rows = v->rows; r.hidden = s.hidden;
    r.weight = v->router_weight; r.logit_bias = v->logit_bias; r.bias = v->select_bias; r.policy = ep->policy;
    r.logits = W.logits; r.scores = W.logits; r.ids = W.ids; r.weights = W.wts;
    if (prologue_fusable(r, s.top_k)) {  // decode windows: A8 + logits + selection in one launch (no local routes: null outputs)
        b200moe_routes_view none{};
        none.rows = v->rows; none.top_k = s.top_k; none.experts = s.experts;
        if (int rc = launch_prologue(r, q, none, ep->counters + 4, st)) return rc;
    } else {
        if (int rc = launch_router_logits(r, st, &q)) return rc;
        if (int rc = launch_router_select(r, st)) return rc;
    }

    // 2. dispatch, then wait for every rank's rows
    EpDev d{};
    for (u32 k = 0; k < ep->world; ++k) d.win[k] = ep->win[k];
    d.world = ep->world; d.rank = ep->rank; d.rows = ep->rows; d.per = ep->per; d.experts = s.experts; d.top_k = s.top_k; d.hidden = s.hidden;
    d.half_base = half_base; d.codes = ep->lay.codes; d.deltas = ep->lay.deltas; d.sums = ep->lay.sums; d.ids = ep->lay.ids; d.wts = ep->lay.wts;
    ep_dispatch_kernel<<<v->rows, 256, 0, st>>>(d, W.x, W.ids, W.wts, ep->counters);
    if (int rc = after_launch("ep_dispatch")) return rc;
    ep_wait_dispatch_kernel<<<1, 32, 0, st>>>(mine, ep->world, ep->counters, ep->wait_polls);
    if (int rc = after_launch("ep_wait_dispatch")) return rc;

    // 3. the local experts over the global window; the combine stores S_rank of every row into its home rank's window
    u32* summary = v->summary ? v->summary : W.summary;
    unsigned char* half = mine + half_base;
    b200moe_layer_view lv{};
    lv.shape = s; lv.weights = v->weights; lv.rows = ep->world * ep->rows;
    lv.x.codes = reinterpret_cast<i8*>(half + ep->lay.codes);
    lv.x.deltas = reinterpret_cast<float*>(half + ep->lay.deltas);
    lv.x.sums = reinterpret_cast<i32*>(half + ep->lay.sums);
    lv.x.rows = lv.rows; lv.x.width = s.hidden; lv.x.stride = s.hidden;
    lv.ids = reinterpret_cast<const u32*>(half + ep->lay.ids);
    lv.route_weights = reinterpret_cast<const float*>(half + ep->lay.wts);
    lv.first = ep->rank * ep->per; lv.end = lv.first + ep->per; lv.base = lv.first;
    lv.combine_form = B200MOE_COMBINE_PARTS; lv.parts = ep->fold; lv.part_experts = s.experts / ep->fold; lv.only_part = static_cast<int>(ep->rank * ep->ranges);
    lv.only_part_count = ep->ranges; lv.part_stride = u64(ep->rows) * s.hidden;
    lv.y_blocks = ep->yblocks[parity]; lv.y_block_rows = ep->rows;
    lv.workspace = W.layer; lv.workspace_bytes = W.layer_bytes; lv.capacity = lv.rows; lv.grouped_min_rows = v->grouped_min_rows;
    lv.summary = summary; lv.stage_events = v->stage_events;
    if (int rc = b200moe_layer(&lv, stream)) return rc;

    // 4. return flags, the wait for every rank's partial sums and the fold: one launch
    const u64 count = u64(v->rows) * s.hidden;
    const float* parts = reinterpret_cast<const float*>(half + ep->lay.parts);
    ep_fold_kernel<<<static_cast<u32>((count + 255) / 256), 256, 0, st>>>(d, mine, parts, ep->fold, u64(ep->rows) * s.hidden, v->shared, count, v->y, v->y_bf16,
                                                                          ep->counters, ep->wait_polls, summary);
    return after_launch("ep_fold");
}

}  // extern "C"
