// The C ABI (include/b200moe.h): host-side validation and composition. Argument errors are reported before anything
// is enqueued; nothing here allocates, synchronises (except b200moe_ffn_host, which says so) or starts threads.
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>

#include "kernels.cuh"

namespace b200moe {

std::string& last_error_slot() {
    thread_local std::string text;
    return text;
}
int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error_slot() = buf;
    return code;
}
std::atomic<u64>& launch_counter() {
    static std::atomic<u64> n{0};
    return n;
}
int after_launch(const char* what) {
    launch_counter().fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return B200MOE_OK;
}
bool device_ready() {
    static std::once_flag once;
    static bool ok = false;
    static std::string why;
    std::call_once(once, [] {
        int n = 0;
        cudaError_t e = cudaGetDeviceCount(&n);
        if (e != cudaSuccess || n == 0) { why = std::string("no CUDA device: ") + cudaGetErrorString(e); cudaGetLastError(); return; }
        int dev = 0;
        cudaDeviceProp p{};
        if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&p, dev) != cudaSuccess) { why = "cannot query the CUDA device"; return; }
        if (p.major != 10) { why = "this library holds sm_100a code only; device is sm_" + std::to_string(p.major * 10 + p.minor); return; }
        ok = true;
    });
    if (!ok) fail(B200MOE_ERR_CUDA, "%s (there is no CPU fallback)", why.c_str());
    return ok;
}

int device_sm_count() {
    int dev = 0, n = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n;
}

int ensure_dynamic_smem(const void* kernel, u32 bytes) {
    // The 48 KiB a launch gets without opting in cover static AND dynamic shared memory: kernels here declare up to a few
    // KiB statically, so the opt-in starts below the limit.
    if (bytes <= 40u * 1024u) return B200MOE_OK;
    static std::mutex m;
    static std::map<std::pair<int, const void*>, u32> granted;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(m);
    u32& have = granted[{dev, kernel}];
    if (bytes <= have) return B200MOE_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "cudaFuncSetAttribute(dynamic smem %u): %s", bytes, cudaGetErrorString(e));
    have = bytes;
    return B200MOE_OK;
}

// The decode step alternates kernels that need almost all of an SM's shared memory with kernels that need little. Asking
// for the largest shared-memory carve-out on the small ones too keeps the SMs' L1 / shared split the same from one
// kernel of the step to the next (a change of the split has to wait for the SM to drain). Once per kernel and device.
int prefer_max_shared(const void* kernel) {
    static std::mutex m;
    static std::map<std::pair<int, const void*>, bool> done;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(m);
    bool& set = done[{dev, kernel}];
    if (set) return B200MOE_OK;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, static_cast<int>(cudaSharedmemCarveoutMaxShared));
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "cudaFuncSetAttribute(carve-out): %s", cudaGetErrorString(e));
    set = true;
    return B200MOE_OK;
}

namespace {
std::atomic<u32> g_debug[3] = {{0}, {0}, {0}};
}
u32 debug_value(u32 key) { return key < 3 ? g_debug[key].load(std::memory_order_relaxed) : 0u; }

namespace {

constexpr u32 kMaxExperts = 1024, kMaxTopK = 32;

struct Carver {  // caller-owned workspace, 256-byte aligned sections
    unsigned char* base;
    u64 used = 0;
    explicit Carver(void* p) : base(static_cast<unsigned char*>(p)) {}
    template <class T>
    T* take(u64 count) {
        used = (used + 255) & ~u64(255);
        T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
        used += count * sizeof(T);
        return p;
    }
};

int check_shape(const b200moe_shape& s) {
    B200_REQUIRE(is_ds41_type(s.gate_type) || is_kquant(s.gate_type), "gate/up type %u is not bound (Q8_0 = 8, Q2_K = 10, Q4_K = 12, Q5_K = 13)", s.gate_type);
    B200_REQUIRE(is_ds41_type(s.down_type) || s.down_type == B200MOE_TYPE_Q4_K || s.down_type == B200MOE_TYPE_Q5_1,
                 "down type %u is not bound (Q5_1 = 7, Q8_0 = 8, Q2_K = 10, Q4_K = 12)", s.down_type);
    B200_REQUIRE(!(is_ds41_type(s.gate_type) && !is_ds41_type(s.down_type)), "Q8_0 / Q2_K gate/up with a down type other than Q8_0 / Q2_K has no declared contract");
    B200_REQUIRE(!(is_kquant(s.gate_type) && s.down_type == B200MOE_TYPE_Q2_K), "Q2_K down tensors belong to the Q8_0 / Q2_K family");
    B200_REQUIRE(s.hidden && s.inter && s.experts && s.top_k, "shape has a zero dimension");
    B200_REQUIRE(s.experts <= kMaxExperts && s.top_k <= kMaxTopK && s.top_k <= s.experts, "need top_k <= 32, top_k <= experts <= 1024");
    B200_REQUIRE(s.hidden % ((is_kquant(s.gate_type) || s.gate_type == B200MOE_TYPE_Q2_K) ? 256u : 32u) == 0, "hidden %u is not a whole number of gate/up blocks", s.hidden);
    B200_REQUIRE(s.inter % ((s.down_type == B200MOE_TYPE_Q4_K || s.down_type == B200MOE_TYPE_Q2_K) ? 256u : 32u) == 0, "inter %u is not a whole number of down blocks", s.inter);
    B200_REQUIRE(s.hidden % 64 == 0, "hidden %u must be a multiple of 64", s.hidden);
    return B200MOE_OK;
}
int check_a8(const b200moe_a8_rows& a, u32 rows, u32 width, bool need_sums, const char* what) {
    const u32 stride = a.stride ? a.stride : a.width;
    B200_REQUIRE(a.codes && a.deltas, "%s: A8 codes / deltas are null", what);
    B200_REQUIRE(!need_sums || a.sums, "%s: A8 sums are required by this contract", what);
    B200_REQUIRE(a.width == width && stride >= width && stride % 32 == 0, "%s: A8 width %u / stride %u do not fit width %u", what, a.width, stride, width);
    B200_REQUIRE(a.rows >= rows, "%s: A8 view holds %u rows, %u needed", what, a.rows, rows);
    B200_REQUIRE(aligned(a.codes, 16) && aligned(a.deltas, 8) && (!a.sums || aligned(a.sums, 8)), "%s: A8 pointers must be 16 / 8-byte aligned", what);
    return B200MOE_OK;
}
int check_routes(const b200moe_routes& r) {
    B200_REQUIRE(r.experts && r.begins && r.rows && r.slots && r.counts, "routes arrays are null");
    return B200MOE_OK;
}
int check_policy(const b200moe_route_policy& p) {
    B200_REQUIRE(p.experts && p.top_k && p.top_k <= p.experts, "route policy: need 0 < top_k <= experts");
    B200_REQUIRE(p.experts <= kMaxExperts && p.top_k <= kMaxTopK, "route policy: experts <= 1024 and top_k <= 32");
    B200_REQUIRE(p.score <= B200MOE_SCORE_SQRT_SOFTPLUS && p.key <= B200MOE_KEY_ORDERED_BITS && p.order <= B200MOE_ORDER_ASCENDING_ID, "route policy: unknown enum value");
    B200_REQUIRE(p.n_group >= 1 && p.topk_group >= 1 && p.topk_group <= p.n_group, "route policy: need 1 <= topk_group <= n_group");
    if (p.n_group > 1) {
        B200_REQUIRE(p.n_group <= 32 && p.experts % p.n_group == 0, "route policy: n_group must divide experts and be <= 32");
        B200_REQUIRE(p.experts / p.n_group >= 2 && u64(p.topk_group) * (p.experts / p.n_group) >= p.top_k, "route policy: the kept groups hold fewer than top_k experts");
    }
    return B200MOE_OK;
}

struct LayerScratch {
    b200moe_routes routes;
    u32* routes_scratch;
    b200moe_a8_rows act;
    float* raw;
    u32* summary;
    u32* row_status;
    u32* aux;  // [capacity * top_k] words for callers of the layer pieces
    u64 bytes;
};
LayerScratch carve_layer(void* ws, const b200moe_shape& s, u32 capacity) {
    Carver c(ws);
    const u64 n = u64(capacity) * s.top_k;
    LayerScratch L{};
    L.routes.experts = c.take<u32>(n);
    L.routes.begins = c.take<u32>(n + 1);
    L.routes.rows = c.take<u32>(n);
    L.routes.slots = c.take<u32>(n);
    L.routes.order = c.take<u32>(n);
    L.routes.low_counts = c.take<u32>(capacity);
    L.routes.counts = c.take<u32>(4);
    L.routes_scratch = c.take<u32>(routes_scratch_words(capacity, s.top_k, s.experts));
    L.act.codes = c.take<i8>(n * s.inter);
    L.act.deltas = c.take<float>(n * (s.inter / 32));
    L.act.sums = c.take<i32>(n * (s.inter / 32));
    L.act.rows = static_cast<u32>(n); L.act.width = s.inter; L.act.stride = s.inter;
    L.raw = c.take<float>(n * s.hidden);
    L.summary = c.take<u32>(4);
    L.row_status = c.take<u32>(capacity);
    L.aux = c.take<u32>(n);
    L.bytes = (c.used + 255) & ~u64(255);
    return L;
}

struct FfnScratch {
    b200moe_a8_rows x;
    float* logits;
    u32* ids;
    float* weights;
    void* x_dev;
    float* y_dev;
    float* x_f32;  // bfloat16 activations widened for the router
    void* layer;
    u64 bytes;
};
FfnScratch carve_ffn(void* ws, const b200moe_shape& s, u32 capacity) {
    Carver c(ws);
    FfnScratch F{};
    F.x.codes = c.take<i8>(u64(capacity) * s.hidden);
    F.x.deltas = c.take<float>(u64(capacity) * (s.hidden / 32));
    F.x.sums = c.take<i32>(u64(capacity) * (s.hidden / 32));
    F.x.rows = capacity; F.x.width = s.hidden; F.x.stride = s.hidden;
    F.logits = c.take<float>(u64(capacity) * s.experts);
    F.ids = c.take<u32>(u64(capacity) * s.top_k);
    F.weights = c.take<float>(u64(capacity) * s.top_k);
    F.x_dev = c.take<float>(u64(capacity) * s.hidden);
    F.y_dev = c.take<float>(u64(capacity) * s.hidden);
    F.x_f32 = c.take<float>(u64(capacity) * s.hidden);
    const u64 at = (c.used + 255) & ~u64(255);
    F.layer = ws ? static_cast<unsigned char*>(ws) + at : nullptr;
    F.bytes = at + carve_layer(nullptr, s, capacity).bytes;
    return F;
}

// Zeroes the job summary (4 words) and, when it lives in the workspace, the per-row status behind it. The two sections
// are neighbours in the workspace (carve_layer), so one memset node covers both and the padding between them.
cudaError_t clear_status(const LayerScratch& L, bool with_row_status, u32 rows, cudaStream_t st) {
    const unsigned char* b = reinterpret_cast<const unsigned char*>(L.summary);
    const unsigned char* e = with_row_status ? reinterpret_cast<const unsigned char*>(L.row_status + rows) : b + 16;
    return cudaMemsetAsync(L.summary, 0, static_cast<size_t>(e - b), st);
}

// Plan by window size, chosen on the host from the row count (no environment reads inside numerical code): decode
// windows of Q4_K experts take the persistent bulk-copy form, everything else the plain per-block form.
// grouped_min_rows: 0 = the default threshold; windows of at least that many rows take the tensor-core form.
constexpr u32 kGroupedDefaultRows = 128;
bool use_grouped(const b200moe_shape& s, u32 rows, u32 grouped_min_rows, bool have_sums) {
    const u32 least = grouped_min_rows ? grouped_min_rows : kGroupedDefaultRows;
    return rows >= least && grouped_fits(s, have_sums);
}
// Decode forms of the Q4_K GEMVs: windows of one or two rows over rows of up to kRowStreamK weights take the row-streaming
// form (a ring of whole rows, its work split fixed per CTA), everything else the segment-streaming form (any row length;
// its items are dealt out dynamically), the per-block form being what is left. Measured on B200 at hidden 2048, 128
// experts, top-8: one row 36.0 against 37.1 us per step, eight rows 76.5 against 70.4 us. B200MOE_DEBUG_DECODE_FORM forces
// one of them where it applies.
constexpr u32 kRowStreamRows = 8, kRowStreamMaxRows = 2, kRowStreamK = 2048;
enum class DecodeForm { row_stream, wide, block };
DecodeForm pick_decode_form(bool row_stream_fits, bool wide_fits, u32 rows, u32 K) {
    const u32 forced = debug_value(B200MOE_DEBUG_DECODE_FORM);
    if (forced == 1 && row_stream_fits) return DecodeForm::row_stream;
    if (forced == 2 && wide_fits) return DecodeForm::wide;
    if (forced == 3) return DecodeForm::block;
    if (row_stream_fits && ((rows <= kRowStreamMaxRows && K <= kRowStreamK) || (rows <= kRowStreamRows && !wide_fits))) return DecodeForm::row_stream;
    if (wide_fits) return DecodeForm::wide;
    return row_stream_fits ? DecodeForm::row_stream : DecodeForm::block;
}
// The DS41 family (Q8_0 x A8): one weight row per warp below kRowStreamRows rows; from there on the tensor-core form of
// gemv_q8_mma.cu (rows of 1024 to 7168 weights), else the dp4a token-block form of gemv_q8_wide.cu. Measured on B200: a
// 7168 x 2048 dense block over 8 rows takes 49 + 18 us in the dp4a token-block form against 55 + 30 us with one row per
// warp; one row over four experts of 2048 x 1024 is 2 us faster with one row per warp.
enum class Q8Form { row_per_warp, wide, mma };
Q8Form pick_q8_form(bool wide_fits, bool mma_fits, u32 rows) {
    const u32 forced = debug_value(B200MOE_DEBUG_DECODE_FORM);
    if (forced == 3) return Q8Form::row_per_warp;
    if (forced == 4 && mma_fits) return Q8Form::mma;
    if (forced == 2 && wide_fits) return Q8Form::wide;
    if (forced == 0 && rows >= kRowStreamRows) {
        if (mma_fits) return Q8Form::mma;
        if (wide_fits) return Q8Form::wide;
    }
    return Q8Form::row_per_warp;
}
int enqueue_gate_up(const b200moe_gate_up_view& v, u32 rows, cudaStream_t st, u32 grouped_min_rows = 0) {
    if (v.shape.gate_type == B200MOE_TYPE_Q2_K) return launch_gate_up_ds41_any(v, st);  // the generic form of the family reads every block type
    if (!is_kquant(v.shape.gate_type)) {
        switch (pick_q8_form(q8_wide_gate_up_fits(v, rows), q8_mma_gate_up_fits(v, rows), rows)) {
            case Q8Form::mma: return launch_gate_up_q8_mma(v, rows, st);
            case Q8Form::wide: return launch_gate_up_q8_wide(v, rows, st);
            default: return launch_gate_up_q8(v, st);
        }
    }
    if (v.shape.gate_type == B200MOE_TYPE_Q5_K) return launch_gate_up_q4k(v, st);  // the per-block form reads both K-quant layouts
    if (use_grouped(v.shape, rows, grouped_min_rows, v.x.sums != nullptr)) return launch_gate_up_q4k_grouped(v, st);
    switch (pick_decode_form(stream_gate_up_fits(v, rows), wide_gate_up_fits(v, rows), rows, v.shape.hidden)) {
        case DecodeForm::row_stream: return launch_gate_up_q4k_stream(v, rows, st);
        case DecodeForm::wide: return launch_gate_up_q4k_wide(v, rows, st);
        default: return launch_gate_up_q4k(v, st);
    }
}
int enqueue_down(const b200moe_down_view& v, u32 rows, cudaStream_t st, u32 grouped_min_rows = 0) {
    if (v.shape.down_type == B200MOE_TYPE_Q4_K && use_grouped(v.shape, rows, grouped_min_rows, v.act.sums != nullptr)) return launch_down_q4k_grouped(v, st);
    if (v.shape.down_type == B200MOE_TYPE_Q4_K) {
        switch (pick_decode_form(stream_down_fits(v, rows), wide_down_fits(v, rows), rows, v.shape.inter)) {
            case DecodeForm::row_stream: return launch_down_q4k_stream(v, rows, st);
            case DecodeForm::wide: return launch_down_q4k_wide(v, rows, st);
            default: return launch_down_q4k(v, st);
        }
    }
    if (is_kquant(v.shape.gate_type)) return launch_down_q8_chain4(v, st);  // chain4: Q8_0 and Q5_1 blocks
    if (v.shape.down_type == B200MOE_TYPE_Q2_K) return launch_down_ds41_any(v, st);
    switch (pick_q8_form(q8_wide_down_fits(v, rows), q8_mma_down_fits(v, rows), rows)) {
        case Q8Form::mma: return launch_down_q8_mma(v, rows, st);
        case Q8Form::wide: return launch_down_q8_wide(v, rows, st);
        default: return launch_down_q8(v, st);
    }
}

}  // namespace
}  // namespace b200moe

using namespace b200moe;

extern "C" {

int b200moe_abi_version(void) { return B200MOE_ABI_VERSION; }
const char* b200moe_last_error(void) { return last_error_slot().c_str(); }
uint64_t b200moe_launch_count(void) { return launch_counter().load(std::memory_order_relaxed); }
int b200moe_debug_set(uint32_t key, uint32_t value) {
    B200_REQUIRE(key < 3, "debug_set: unknown key %u", key);
    g_debug[key].store(value, std::memory_order_relaxed);
    return B200MOE_OK;
}

uint64_t b200moe_gate_row_bytes(const b200moe_shape* s) { return s ? row_bytes_of(s->gate_type, s->hidden) : 0; }
uint64_t b200moe_down_row_bytes(const b200moe_shape* s) { return s ? row_bytes_of(s->down_type, s->inter) : 0; }
uint64_t b200moe_expert_bytes(const b200moe_shape* s) {
    return s ? 2 * row_bytes_of(s->gate_type, s->hidden) * s->inter + row_bytes_of(s->down_type, s->inter) * s->hidden : 0;
}

int b200moe_quantize_a8(const b200moe_quantize_a8_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->width % 32 == 0, "A8 activation width must be a multiple of 32 (got %u)", v->width);
    if (v->rows == 0 || v->width == 0) return B200MOE_OK;
    B200_REQUIRE(v->x, "quantize_a8: x is null");
    const u32 xs = v->x_stride ? v->x_stride : v->width;
    B200_REQUIRE(xs >= v->width, "quantize_a8: x_stride %u is below the width %u", xs, v->width);
    const u32 stride = v->out.stride ? v->out.stride : v->out.width;
    B200_REQUIRE(v->out.codes && v->out.deltas, "quantize_a8: output codes / deltas are null");
    B200_REQUIRE(v->out.width == v->width && stride >= v->width && stride % 32 == 0 && v->out.rows >= v->rows, "quantize_a8: output view does not fit rows %u x width %u", v->rows, v->width);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_quantize_a8(*v, as_stream(stream));
}

int b200moe_rmsnorm_a8(const b200moe_rmsnorm_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->n % 32 == 0, "rmsnorm: n must be a multiple of 32 (got %u)", v->n);
    if (v->rows == 0 || v->n == 0) return B200MOE_OK;
    B200_REQUIRE(v->x, "rmsnorm: x is null");
    B200_REQUIRE(v->out || v->a8.codes, "rmsnorm: neither out nor a8 is given");
    const u32 xs = v->x_stride ? v->x_stride : v->n, os = v->out_stride ? v->out_stride : v->n;
    B200_REQUIRE(xs >= v->n && os >= v->n, "rmsnorm: a stride is below n = %u", v->n);
    if (v->a8.codes) {
        const u32 stride = v->a8.stride ? v->a8.stride : v->a8.width;
        B200_REQUIRE(v->a8.deltas, "rmsnorm: a8.deltas is null");
        B200_REQUIRE(v->a8.width == v->n && stride >= v->n && stride % 32 == 0 && v->a8.rows >= v->rows, "rmsnorm: a8 view does not fit rows %u x n %u", v->rows, v->n);
    }
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_rmsnorm_a8(*v, as_stream(stream));
}

int b200moe_q8_0_a8(const b200moe_q8a8_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->width % 32 == 0, "Q8_0 product width must be a multiple of 32 (got %u)", v->width);
    if (v->count == 0 || v->x.rows == 0 || v->width == 0) return B200MOE_OK;
    B200_REQUIRE(v->weight && v->out, "q8_0_a8: weight / out are null");
    B200_REQUIRE(v->row_bytes >= v->width / 32 * kQ8Block, "q8_0_a8: row_bytes %u is below %u", v->row_bytes, v->width / 32 * kQ8Block);
    if (int rc = check_a8(v->x, v->x.rows, v->width, false, "q8_0_a8 x")) return rc;
    const u32 os = v->out_stride ? v->out_stride : v->count;
    B200_REQUIRE(os >= v->count, "q8_0_a8: out_stride %u is below count %u", os, v->count);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_q8_0_a8(*v, as_stream(stream));
}

int b200moe_router(const b200moe_router_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    if (int rc = check_policy(v->policy)) return rc;
    B200_REQUIRE(v->logits && v->ids && v->weights, "router: logits / ids / weights are null");
    B200_REQUIRE(!v->policy.selection_bias || v->bias, "router: the policy has a selection bias but bias is null");
    if (v->x) {
        B200_REQUIRE(v->weight && v->hidden, "router: weight is null or hidden is 0");
        const u32 xs = v->x_stride ? v->x_stride : v->hidden;
        B200_REQUIRE(xs >= v->hidden, "router: x_stride %u is below hidden %u", xs, v->hidden);
    }
    if (v->rows == 0) return B200MOE_OK;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    if (v->x) if (int rc = launch_router_logits(*v, as_stream(stream))) return rc;
    return launch_router_select(*v, as_stream(stream));
}

uint64_t b200moe_routes_scratch_words(uint32_t rows, uint32_t top_k, uint32_t experts) { return routes_scratch_words(rows, top_k, experts); }

}  // extern "C"
namespace b200moe {
int b200moe_check_routes_view(const b200moe_routes_view* v) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->rows && v->top_k && v->ids, "routes need rows * top_k expert ids");
    B200_REQUIRE(v->experts && v->experts <= kMaxExperts && v->top_k <= kMaxTopK && v->top_k <= v->experts, "routes: need top_k <= 32, top_k <= experts <= 1024");
    B200_REQUIRE(v->end <= v->experts && (v->end == 0 || v->first < v->end) && v->base <= v->first, "routes: expert range [%u, %u) base %u is inconsistent", v->first, v->end, v->base);
    if (int rc = check_routes(v->out)) return rc;
    B200_REQUIRE(v->out.order && v->out.low_counts, "routes: order / low_counts are null");
    B200_REQUIRE(u64(v->rows) * v->top_k <= 1024 || v->scratch, "routes: more than 1024 slots need scratch");
    return B200MOE_OK;
}
}  // namespace b200moe
extern "C" {

int b200moe_build_routes(const b200moe_routes_view* v, void* stream) {
    if (int rc = b200moe_check_routes_view(v)) return rc;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_routes(*v, as_stream(stream));
}

int b200moe_gate_up(const b200moe_gate_up_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    if (int rc = check_shape(v->shape)) return rc;
    if (int rc = check_routes(v->routes)) return rc;
    B200_REQUIRE(v->weights.gate && v->weights.up && aligned(v->weights.gate, 16) && aligned(v->weights.up, 16), "gate_up: gate / up tensors must be non-null and 16-byte aligned");
    B200_REQUIRE((v->gate_out == nullptr) == (v->up_out == nullptr), "gate_up: gate_out and up_out come together");
    const bool q4k = is_kquant(v->shape.gate_type);
    if (int rc = check_a8(v->x, 0, v->shape.hidden, q4k, "gate_up x")) return rc;
    if (int rc = check_a8(v->act, 0, v->shape.inter, down_reads_sums(v->shape.down_type), "gate_up act")) return rc;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return enqueue_gate_up(*v, v->x.rows, as_stream(stream));
}

int b200moe_down(const b200moe_down_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    if (int rc = check_shape(v->shape)) return rc;
    if (int rc = check_routes(v->routes)) return rc;
    B200_REQUIRE(v->weights.down && aligned(v->weights.down, 16) && v->raw, "down: the down tensor must be non-null and 16-byte aligned, raw non-null");
    if (int rc = check_a8(v->act, 0, v->shape.inter, down_reads_sums(v->shape.down_type), "down act")) return rc;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return enqueue_down(*v, v->act.rows / v->shape.top_k, as_stream(stream));
}

int b200moe_combine(const b200moe_combine_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->raw && v->weights && (v->y || v->y_blocks), "combine: raw / weights / y are null");
    B200_REQUIRE(!v->y_blocks || (v->y_block_rows && !v->y_bf16), "combine: y_blocks needs y_block_rows > 0 and no y_bf16");
    B200_REQUIRE(v->top_k && v->top_k <= kMaxTopK && v->hidden, "combine: need 0 < top_k <= 32 and hidden > 0");
    B200_REQUIRE(v->form <= B200MOE_COMBINE_FMA_SLOTS, "combine: unknown form %u", v->form);
    if (v->form == B200MOE_COMBINE_PARTS) {
        B200_REQUIRE((v->ids || v->low_counts) && v->order, "combine(parts): ids (or low_counts) / order are null");
        B200_REQUIRE(!v->low_counts || v->parts == 2, "combine(parts): low_counts describes a two-part split (parts must be 2)");
        B200_REQUIRE(v->parts && (v->part_experts || v->low_counts) && v->only_part < static_cast<int>(v->parts), "combine(parts): parts / part_experts / only_part are inconsistent");
        B200_REQUIRE(v->only_part_count <= 1 || (v->only_part >= 0 && v->only_part + v->only_part_count <= v->parts && v->part_stride && !v->y_bf16),
                     "combine(parts): only_part_count needs only_part >= 0, a part_stride and no y_bf16");
    }
    if (v->rows == 0) return B200MOE_OK;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_combine(*v, as_stream(stream));
}

int b200moe_canonical_sum(const float* a, const float* b, const float* c, uint64_t count, float* y, void* stream) {
    B200_REQUIRE(a && b && y, "canonical_sum: a / b / y are null");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_canonical_sum(a, b, c, count, y, as_stream(stream));
}

uint64_t b200moe_layer_workspace_bytes(const b200moe_shape* s, uint32_t capacity) {
    if (!s || check_shape(*s)) return 0;
    return carve_layer(nullptr, *s, capacity).bytes;
}

static int layer_impl(const b200moe_layer_view* v, void* stream, bool routes_ready);
int b200moe_layer(const b200moe_layer_view* v, void* stream) { return layer_impl(v, stream, false); }

// routes_ready: the caller (b200moe_ffn) has already built the routes of v->ids into this workspace and cleared the
// status words (the fused select + routes launch of decode windows).
static int layer_impl(const b200moe_layer_view* v, void* stream, bool routes_ready) {
    B200_REQUIRE(v, "null view");
    if (int rc = check_shape(v->shape)) return rc;
    const b200moe_shape& s = v->shape;
    B200_REQUIRE(v->rows <= v->capacity, "layer: rows %u exceed the workspace capacity %u", v->rows, v->capacity);
    if (v->rows == 0) return B200MOE_OK;
    B200_REQUIRE(v->ids && v->route_weights, "layer: ids / route_weights are null");
    B200_REQUIRE(v->weights.gate && v->weights.up && v->weights.down, "layer: expert tensors are null");
    B200_REQUIRE(aligned(v->weights.gate, 16) && aligned(v->weights.up, 16) && aligned(v->weights.down, 16), "layer: expert tensors must be 16-byte aligned");
    if (int rc = check_a8(v->x, v->rows, s.hidden, is_kquant(s.gate_type), "layer x")) return rc;
    B200_REQUIRE(v->end <= s.experts && (v->end == 0 || v->first < v->end) && v->base <= v->first, "layer: expert range [%u, %u) base %u is inconsistent", v->first, v->end, v->base);
    B200_REQUIRE(v->combine_form <= B200MOE_COMBINE_FMA_SLOTS, "layer: unknown combine form %u", v->combine_form);
    if (v->y && v->combine_form == B200MOE_COMBINE_PARTS)
        B200_REQUIRE(v->parts && v->part_experts && v->only_part < static_cast<int>(v->parts), "layer: parts / part_experts / only_part are inconsistent");
    B200_REQUIRE(v->only_part_count <= 1 || (v->combine_form == B200MOE_COMBINE_PARTS && v->only_part >= 0 && v->only_part + v->only_part_count <= v->parts &&
                                             v->part_stride && !v->y_bf16),
                 "layer: only_part_count needs the PARTS form, only_part >= 0, a part_stride and no y_bf16");
    const LayerScratch L = carve_layer(v->workspace, s, v->capacity);
    if (!v->workspace || v->workspace_bytes < L.bytes)
        return fail(B200MOE_ERR_WORKSPACE, "layer: workspace of %llu bytes needed, %llu given", (unsigned long long)L.bytes, (unsigned long long)v->workspace_bytes);
    B200_REQUIRE(aligned(v->workspace, 256), "layer: workspace must be 256-byte aligned");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);

    u32* row_status = v->row_status ? v->row_status : L.row_status;
    u32* summary = v->summary ? v->summary : L.summary;
    if (!routes_ready) {
        cudaError_t ce = clear_status(L, !v->row_status, v->rows, st);
        if (ce == cudaSuccess && v->summary) ce = cudaMemsetAsync(v->summary, 0, sizeof(u32), st);
        if (ce != cudaSuccess) return fail(B200MOE_ERR_CUDA, "layer: cudaMemsetAsync: %s", cudaGetErrorString(ce));
    }

    b200moe_routes_view rv{};
    rv.ids = v->ids; rv.rows = v->rows; rv.top_k = s.top_k; rv.experts = s.experts;
    rv.split = v->part_experts ? v->part_experts : s.experts / 2;
    rv.first = v->first; rv.end = v->end; rv.base = v->base;
    rv.scratch = L.routes_scratch; rv.row_status = row_status; rv.out = L.routes;
    auto tap = [&](int i) {
        if (v->stage_events && v->stage_events[i]) cudaEventRecord(static_cast<cudaEvent_t>(v->stage_events[i]), st);
    };
    tap(0);
    if (!routes_ready) if (int rc = launch_routes(rv, st)) return rc;
    tap(1);

    const u32 span = (v->end ? v->end : s.experts) - v->first;
    const u32 max_union = static_cast<u32>(std::min<u64>(u64(v->rows) * s.top_k, span));
    float* raw = v->raw ? v->raw : L.raw;

    b200moe_gate_up_view gu{};
    gu.shape = s; gu.weights = v->weights; gu.routes = L.routes; gu.max_union = max_union;
    gu.x = v->x; gu.act = L.act; gu.row_status = row_status; gu.summary = summary;
    tap(2);
    if (int rc = enqueue_gate_up(gu, v->rows, st, v->grouped_min_rows)) return rc;
    tap(3);

    b200moe_down_view dn{};
    dn.shape = s; dn.weights = v->weights; dn.routes = L.routes; dn.max_union = max_union;
    dn.act = L.act; dn.raw = raw; dn.summary = summary;
    tap(4);
    if (int rc = enqueue_down(dn, v->rows, st, v->grouped_min_rows)) return rc;
    tap(5);

    if (!v->y && !v->y_blocks) return B200MOE_OK;
    B200_REQUIRE(!v->y_blocks || (v->y_block_rows && !v->y_bf16), "layer: y_blocks needs y_block_rows > 0 and no y_bf16");
    b200moe_combine_view cv{};
    cv.raw = raw; cv.shared = v->shared; cv.weights = v->route_weights; cv.ids = v->ids; cv.order = L.routes.order;
    cv.rows = v->rows; cv.top_k = s.top_k; cv.hidden = s.hidden; cv.form = v->combine_form;
    cv.parts = v->parts; cv.part_experts = v->part_experts; cv.only_part = v->only_part;
    cv.only_part_count = v->only_part_count; cv.part_stride = v->part_stride;
    cv.y = v->y; cv.y_bf16 = v->y_bf16; cv.y_blocks = v->y_blocks; cv.y_block_rows = v->y_block_rows;
    cv.row_status = is_kquant(s.gate_type) ? row_status : nullptr;
    cv.summary = summary;
    tap(6);
    const int rc = launch_combine(cv, st);
    tap(7);
    return rc;
}

uint64_t b200moe_ffn_workspace_bytes(const b200moe_shape* s, uint32_t capacity) {
    if (!s || check_shape(*s)) return 0;
    return carve_ffn(nullptr, *s, capacity).bytes;
}

int b200moe_ffn(const b200moe_ffn_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    if (int rc = check_shape(v->shape)) return rc;
    if (int rc = check_policy(v->policy)) return rc;
    const b200moe_shape& s = v->shape;
    B200_REQUIRE(v->policy.experts == s.experts && v->policy.top_k == s.top_k, "ffn: the route policy and the shape disagree on experts / top_k");
    B200_REQUIRE(v->rows <= v->capacity, "ffn: rows %u exceed the workspace capacity %u", v->rows, v->capacity);
    if (v->rows == 0) return B200MOE_OK;
    B200_REQUIRE(v->x && v->y && v->router_weight, "ffn: x / y / router_weight are null");
    B200_REQUIRE(!v->policy.selection_bias || v->select_bias, "ffn: the policy has a selection bias but select_bias is null");
    const FfnScratch F = carve_ffn(v->workspace, s, v->capacity);
    if (!v->workspace || v->workspace_bytes < F.bytes)
        return fail(B200MOE_ERR_WORKSPACE, "ffn: workspace of %llu bytes needed, %llu given", (unsigned long long)F.bytes, (unsigned long long)v->workspace_bytes);
    B200_REQUIRE(aligned(v->workspace, 256), "ffn: workspace must be 256-byte aligned");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);

    // The router reads FP32 rows: bfloat16 activations are widened once (exactly) into the workspace, and both the A8
    // quantiser and the router read the widened rows (the Qwen prologue's input form, src/cuda/models/qwen/qwen_moe.cu:60-99).
    const float* x32 = static_cast<const float*>(v->x);
    if (v->x_is_bf16) {
        if (int rc = launch_widen_bf16(static_cast<const u16*>(v->x), F.x_f32, u64(v->rows) * s.hidden, st)) return rc;
        x32 = F.x_f32;
    }
    b200moe_quantize_a8_view q{};
    q.x = x32; q.rows = v->rows; q.width = s.hidden; q.x_stride = s.hidden; q.x_is_bf16 = 0; q.out = F.x;
    b200moe_router_view r{};
    r.x = x32; r.x_stride = s.hidden; r.rows = v->rows; r.hidden = s.hidden;
    r.weight = v->router_weight; r.logit_bias = v->logit_bias; r.bias = v->select_bias; r.policy = v->policy;
    r.logits = F.logits; r.scores = F.logits;
    r.ids = v->ids ? v->ids : F.ids; r.weights = v->route_weights ? v->route_weights : F.weights;
    // Decode windows: one launch for A8 + logits + selection + routes; 9..32 rows: selection and routes share a launch.
    const LayerScratch L = carve_layer(F.layer, s, v->capacity);
    const bool one_launch = prologue_fusable(r, s.top_k);
    const bool fused = one_launch || select_routes_fusable(r, s.top_k);
    b200moe_routes_view rv{};
    if (fused) {
        u32* row_status = v->row_status ? v->row_status : L.row_status;
        cudaError_t ce = clear_status(L, !v->row_status, v->rows, st);  // summary word, prologue ticket, row status
        if (ce == cudaSuccess && v->summary) ce = cudaMemsetAsync(v->summary, 0, sizeof(u32), st);
        if (ce != cudaSuccess) return fail(B200MOE_ERR_CUDA, "ffn: cudaMemsetAsync: %s", cudaGetErrorString(ce));
        rv.ids = r.ids; rv.rows = v->rows; rv.top_k = s.top_k; rv.experts = s.experts;
        rv.split = v->part_experts ? v->part_experts : s.experts / 2;
        rv.scratch = L.routes_scratch; rv.row_status = row_status; rv.out = L.routes;
    }
    if (one_launch) {
        if (int rc = launch_prologue(r, q, rv, L.summary + 1, st)) return rc;
    } else {
        if (int rc = launch_router_logits(r, st, &q)) return rc;
        if (fused) { if (int rc = launch_select_routes(r, rv, st)) return rc; }
        else if (int rc = launch_router_select(r, st)) return rc;
    }

    b200moe_layer_view lv{};
    lv.shape = s; lv.weights = v->weights; lv.rows = v->rows; lv.x = F.x; lv.ids = r.ids; lv.route_weights = r.weights;
    lv.shared = v->shared; lv.combine_form = v->combine_form; lv.parts = v->parts; lv.part_experts = v->part_experts; lv.only_part = -1;
    lv.y = v->y; lv.y_bf16 = v->y_bf16; lv.row_status = v->row_status;
    lv.workspace = F.layer; lv.workspace_bytes = v->workspace_bytes - (static_cast<unsigned char*>(F.layer) - static_cast<unsigned char*>(v->workspace));
    lv.capacity = v->capacity; lv.grouped_min_rows = v->grouped_min_rows; lv.stage_events = v->stage_events;
    lv.summary = v->summary;
    return layer_impl(&lv, stream, fused);
}

int b200moe_ffn_host(const b200moe_ffn_view* v, const void* x_host, float* y_host, void* stream) {
    B200_REQUIRE(v && x_host && y_host, "ffn_host: null view / host buffers");
    if (int rc = check_shape(v->shape)) return rc;
    B200_REQUIRE(v->rows <= v->capacity, "ffn_host: rows %u exceed the workspace capacity %u", v->rows, v->capacity);
    const FfnScratch F = carve_ffn(v->workspace, v->shape, v->capacity);
    if (!v->workspace || v->workspace_bytes < F.bytes)
        return fail(B200MOE_ERR_WORKSPACE, "ffn_host: workspace of %llu bytes needed, %llu given", (unsigned long long)F.bytes, (unsigned long long)v->workspace_bytes);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);
    const u64 n = u64(v->rows) * v->shape.hidden;
    cudaError_t e = cudaMemcpyAsync(F.x_dev, x_host, n * (v->x_is_bf16 ? 2 : 4), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "ffn_host: H2D copy: %s", cudaGetErrorString(e));
    b200moe_ffn_view d = *v;
    d.x = F.x_dev; d.y = F.y_dev;
    if (int rc = b200moe_ffn(&d, stream)) return rc;
    e = cudaMemcpyAsync(y_host, F.y_dev, n * 4, cudaMemcpyDeviceToHost, st);
    u32 job = 0;  // the job summary, read back with y: a bounded device wait that ran out must not look like success
    const u32* summary = v->summary ? v->summary : carve_layer(F.layer, v->shape, v->capacity).summary;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&job, summary, sizeof job, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "ffn_host: D2H copy / synchronize: %s", cudaGetErrorString(e));
    if (job & B200MOE_JOB_WAIT_ABORTED) return fail(B200MOE_ERR_ABORTED, "ffn_host: a bounded device wait ran out (job summary 0x%x); y_host is not valid", job);
    return B200MOE_OK;
}

int b200moe_dense_ffn(const b200moe_dense_view* v, void* stream) {
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->shape.experts == 1 && v->shape.top_k == 1, "dense_ffn: shape.experts and shape.top_k must be 1");
    if (int rc = check_shape(v->shape)) return rc;
    const b200moe_shape& s = v->shape;
    if (v->rows == 0) return B200MOE_OK;
    B200_REQUIRE(v->y, "dense_ffn: y is null");
    B200_REQUIRE(v->weights.gate && v->weights.up && v->weights.down, "dense_ffn: tensors are null");
    B200_REQUIRE(aligned(v->weights.gate, 16) && aligned(v->weights.up, 16) && aligned(v->weights.down, 16), "dense_ffn: tensors must be 16-byte aligned");
    if (int rc = check_a8(v->x, v->rows, s.hidden, is_kquant(s.gate_type), "dense_ffn x")) return rc;
    const LayerScratch L = carve_layer(v->workspace, s, v->rows);
    if (!v->workspace || v->workspace_bytes < L.bytes)
        return fail(B200MOE_ERR_WORKSPACE, "dense_ffn: workspace of %llu bytes needed, %llu given", (unsigned long long)L.bytes, (unsigned long long)v->workspace_bytes);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaStream_t st = as_stream(stream);
    // every row is one entry of the single expert (slot = row): the routes are written directly, the status words with them
    if (int rc = launch_dense_routes(L.routes, v->rows, L.row_status, L.summary, st)) return rc;
    b200moe_gate_up_view gu{};
    gu.shape = s; gu.weights = v->weights; gu.routes = L.routes; gu.max_union = 1; gu.x = v->x; gu.act = L.act;
    gu.row_status = L.row_status; gu.summary = L.summary;
    if (int rc = enqueue_gate_up(gu, v->rows, st)) return rc;
    b200moe_down_view dn{};
    dn.shape = s; dn.weights = v->weights; dn.routes = L.routes; dn.max_union = 1; dn.act = L.act; dn.raw = v->y; dn.summary = L.summary;
    if (int rc = enqueue_down(dn, v->rows, st)) return rc;
    if (v->y_bf16) {
        // bfloat16 RNE copy of y through the FMA_SLOTS combine with unit weights: fma(1, y, +0) = y exactly
        float* ones = reinterpret_cast<float*>(L.aux);  // the ids are no longer read once the routes exist
        if (int rc = launch_fill_u32(L.aux, 0x3f800000u, v->rows, st)) return rc;
        b200moe_combine_view cv{};
        cv.raw = v->y; cv.weights = ones; cv.rows = v->rows; cv.top_k = 1; cv.hidden = s.hidden; cv.form = B200MOE_COMBINE_FMA_SLOTS;
        cv.only_part = -1; cv.y = L.raw; cv.y_bf16 = v->y_bf16;
        return launch_combine(cv, st);
    }
    return B200MOE_OK;
}

}  // extern "C"

// ---- the launch-record seam (include/strix/weight/resolve.hpp:67-76, src/cuda/weight/registry.hpp:53-65) ----------------
namespace {
using SiteLaunch = int (*)(const void*, void*);
struct SiteRow { b200moe_registration reg; SiteLaunch launch; };
template <class View, int (*Fn)(const View*, void*)>
int site_thunk(const void* view, void* stream) { return Fn(static_cast<const View*>(view), stream); }
#define B200_SITE(id, View, fn) SiteRow{{id, B200MOE_ABI_VERSION, sizeof(View), alignof(View), #fn}, &site_thunk<View, fn>}
const SiteRow kSites[] = {
    B200_SITE(B200MOE_SITE_QUANTIZE_A8, b200moe_quantize_a8_view, b200moe_quantize_a8),
    B200_SITE(B200MOE_SITE_RMSNORM_A8, b200moe_rmsnorm_view, b200moe_rmsnorm_a8),
    B200_SITE(B200MOE_SITE_Q8_0_A8, b200moe_q8a8_view, b200moe_q8_0_a8),
    B200_SITE(B200MOE_SITE_ROUTER, b200moe_router_view, b200moe_router),
    B200_SITE(B200MOE_SITE_ROUTES, b200moe_routes_view, b200moe_build_routes),
    B200_SITE(B200MOE_SITE_ROUTES_STATIC, b200moe_routes_view, b200moe_build_routes_static),
    B200_SITE(B200MOE_SITE_GATE_UP, b200moe_gate_up_view, b200moe_gate_up),
    B200_SITE(B200MOE_SITE_DOWN, b200moe_down_view, b200moe_down),
    B200_SITE(B200MOE_SITE_COMBINE, b200moe_combine_view, b200moe_combine),
    B200_SITE(B200MOE_SITE_LAYER, b200moe_layer_view, b200moe_layer),
    B200_SITE(B200MOE_SITE_FFN, b200moe_ffn_view, b200moe_ffn),
    B200_SITE(B200MOE_SITE_DENSE_FFN, b200moe_dense_view, b200moe_dense_ffn),
};
#undef B200_SITE
constexpr uint32_t kSiteCount = sizeof(kSites) / sizeof(kSites[0]);
}  // namespace

extern "C" {

uint32_t b200moe_registry(const b200moe_registration** rows) {
    static b200moe_registration table[kSiteCount];
    static const bool filled = [] { for (uint32_t i = 0; i < kSiteCount; ++i) table[i] = kSites[i].reg; return true; }();
    (void)filled;
    if (rows) *rows = table;
    return kSiteCount;
}

int b200moe_enqueue(const b200moe_kernel_arguments* a, void* stream) {
    B200_REQUIRE(a, "enqueue: null launch record");
    for (const SiteRow& row : kSites) {
        if (row.reg.schema != a->schema) continue;
        B200_REQUIRE(a->abi_revision == row.reg.revision, "enqueue(%s): launch record of ABI revision %u, this build is revision %u", row.reg.name,
                     a->abi_revision, row.reg.revision);
        B200_REQUIRE(a->bytes == row.reg.bytes, "enqueue(%s): launch record of %llu bytes, the view has %llu", row.reg.name, (unsigned long long)a->bytes,
                     (unsigned long long)row.reg.bytes);
        B200_REQUIRE(a->data && reinterpret_cast<uintptr_t>(a->data) % row.reg.alignment == 0, "enqueue(%s): the view is null or not aligned to %llu bytes",
                     row.reg.name, (unsigned long long)row.reg.alignment);
        return row.launch(a->data, stream);
    }
    return fail(B200MOE_ERR_INVALID_ARGUMENT, "enqueue: unknown schema %u", a->schema);
}

}  // extern "C"

extern "C" {

int b200moe_merge_first_error(b200moe_first_error* record, const uint32_t* summary, uint32_t domain, void* stream) {
    B200_REQUIRE(record && summary, "merge_first_error: record / summary are null");
    B200_REQUIRE(domain == B200MOE_DOMAIN_LEGACY || domain == B200MOE_DOMAIN_Q4K_A8, "merge_first_error: domain %u is not one this library publishes", domain);
    if (!device_ready()) return B200MOE_ERR_CUDA;
    return launch_merge_first_error(record, summary, domain, as_stream(stream));
}

int b200moe_check_first_error(const b200moe_first_error* r) {
    B200_REQUIRE(r, "check_first_error: null record");
    if (r->domain == B200MOE_DOMAIN_NONE && r->bits == 0) return B200MOE_OK;
    if (r->domain == B200MOE_DOMAIN_LEGACY && r->bits != 0)
        return fail(B200MOE_ERR_INVALID_ARGUMENT, "routed experts rejected invalid routes or nonfinite weights (status bits %u)", r->bits);
    if (r->domain == B200MOE_DOMAIN_Q4K_A8 && r->bits != 0)
        return fail(B200MOE_ERR_INVALID_ARGUMENT, "Q4K A8 rejected status bits (route/weight=1,input=2,delta=4,pipeline=8%s): %u",
                    (r->bits & B200MOE_JOB_WAIT_ABORTED) ? ", bounded wait ran out=0x40000000" : "", r->bits);
    return fail(B200MOE_ERR_UNSUPPORTED, "deferred MoE completion record is malformed (domain %u, bits %u)", r->domain, r->bits);
}

}  // extern "C"
