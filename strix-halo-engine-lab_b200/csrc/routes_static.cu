// b200moe_build_routes_static: the window routes of b200moe_build_routes for callers that cannot hand over device
// scratch. The scratch of the chunked build (per-chunk histograms + expert begins) lives in a file-scope device array
// of fixed size; the entry point allocates nothing, on the host or on the device, and calls no routine that does.
//
// Nothing in the array has to start at zero: every word the scan and fill kernels read (hist[chunk][expert],
// ebegin[expert]) is written by the count and scan kernels of the same call before it is read, so the contents a
// previous call left behind are never observed. The array is one per device and shared by every caller in the
// process: two calls that overlap in time on the same device (different streams, or different threads) race on it.
#include <mutex>

#include "kernels.cuh"

namespace b200moe {
namespace {

// 64 chunks of 1024 slots at 1024 experts, plus the expert begins and the 4 spare words: (64 + 1) * 1024 + 4.
constexpr u64 kStaticRoutesWords = 65u * 1024u + 4u;  // 260 KiB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) u32 g_routes_scratch[kStaticRoutesWords];

// Device address of the array on the current device, looked up once per device with that device current.
int static_scratch(u32** out) {
    static std::mutex mu;
    static u32* ptrs[kMaxDevices] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B200MOE_ERR_CUDA, "build_routes_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(B200MOE_ERR_UNSUPPORTED, "build_routes_static: device ordinal %d is beyond %d", dev, kMaxDevices - 1);
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        u32* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_routes_scratch);
        if (e != cudaSuccess || !p) return fail(B200MOE_ERR_CUDA, "build_routes_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        ptrs[dev] = p;
    }
    *out = ptrs[dev];
    return B200MOE_OK;
}

}  // namespace
}  // namespace b200moe

namespace b200moe { int b200moe_check_routes_view(const b200moe_routes_view* v); }  // api.cu: the argument checks of b200moe_build_routes

extern "C" {

uint64_t b200moe_routes_static_max_words(void) { return b200moe::kStaticRoutesWords; }

int b200moe_build_routes_static(const b200moe_routes_view* v, void* stream) {
    using namespace b200moe;
    B200_REQUIRE(v, "null view");
    B200_REQUIRE(v->rows && v->top_k && v->experts, "build_routes_static: rows, top_k and experts must be non-zero");
    const u64 need = routes_scratch_words(v->rows, v->top_k, v->experts);
    if (need > kStaticRoutesWords)
        return fail(B200MOE_ERR_UNSUPPORTED,
                    "build_routes_static: %u rows x top-%u over %u experts need %llu scratch words, the built-in array holds %llu "
                    "(use b200moe_build_routes with caller scratch)",
                    v->rows, v->top_k, v->experts, (unsigned long long)need, (unsigned long long)kStaticRoutesWords);
    b200moe_routes_view w = *v;
    w.scratch = nullptr;
    if (u64(v->rows) * v->top_k > 1024) {  // the one-block form of small windows uses no scratch at all
        // argument errors come before the device is touched: the shared validation runs first, on a placeholder scratch
        static u32 placeholder;
        w.scratch = &placeholder;
        if (int rc = b200moe_check_routes_view(&w)) return rc;
        if (!device_ready()) return B200MOE_ERR_CUDA;
        if (int rc = static_scratch(&w.scratch)) return rc;
    }
    return b200moe_build_routes(&w, stream);  // same validation, same kernels
}

}  // extern "C"
