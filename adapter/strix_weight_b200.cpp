// Reference-side adapter: a launch function of the shape the reference's source registry stores
// (Launch in src/cuda/weight/registry.hpp:53-55), which hands the reference's checked launch-record envelope
// (strix::weight::KernelArguments, include/strix/weight/resolve.hpp:67-70) to b200moe_enqueue, and the registry rows
// {schema, revision, sizeof, alignof, launch} built from b200moe_registry.
//
// A maintainer appends `b200_registrations()` to the span source_registry() returns; strix::weight::enqueue then
// reaches this library through the same seam as the vendor's own kernels: the envelope's schema, ABI revision and size
// are checked twice, by enqueue_registered against the row and by b200moe_enqueue against the library's own table,
// before a view is read. Output and workspace travel inside the site's view (the C ABI's views carry their own pointers),
// so the seam's separate output / workspace arguments are only checked for consistency.
//
// tests/test_abi.py compiles this file against the reference checkout's headers (syntax and types only).
#include <cstddef>
#include <cstdint>
#include <vector>

#include "b200moe.h"
#include "strix/weight/cache.hpp"
#include "strix/weight/resolve.hpp"

namespace strix_b200 {

// The reference's Registration row, restated over its public types (the struct itself lives in a private header).
using Launch = ::strix::weight::Status (*)(const ::strix::weight::Plan&, const ::strix::weight::WeightView&, const ::strix::weight::KernelArguments&, void*,
                                           void*, std::size_t, ::strix::weight::ExecutionContext&);
struct Registration {
    ::strix::weight::KernelId schema;
    std::uint32_t revision;
    std::size_t bytes, alignment;
    Launch launch;
};

inline ::strix::weight::Status status_of(int rc) {
    using ::strix::weight::Error;
    switch (rc) {
        case B200MOE_OK: return {Error::ok, {}};
        case B200MOE_ERR_INVALID_ARGUMENT: return {Error::malformed, b200moe_last_error()};
        case B200MOE_ERR_UNSUPPORTED: return {Error::unsupported_shape, b200moe_last_error()};
        case B200MOE_ERR_WORKSPACE: return {Error::memory_budget, b200moe_last_error()};
        default: return {Error::device_failure, b200moe_last_error()};
    }
}

// Launch-shaped: the envelope goes through unchanged, the stream comes from the execution context.
inline ::strix::weight::Status launch_b200(const ::strix::weight::Plan&, const ::strix::weight::WeightView&, const ::strix::weight::KernelArguments& a, void*, void*,
                                           std::size_t, ::strix::weight::ExecutionContext& ctx) {
    if (ctx.backend != ::strix::weight::Backend::cuda) return {::strix::weight::Error::unsupported_backend, "b200moe runs on CUDA devices only"};
    const b200moe_kernel_arguments env{a.schema, a.abi_revision, a.data, static_cast<std::uint64_t>(a.bytes)};
    return status_of(b200moe_enqueue(&env, ctx.stream));
}

// One row per site of the library, ready to be appended to the backend's source registry.
inline std::vector<Registration> b200_registrations() {
    const b200moe_registration* rows = nullptr;
    const std::uint32_t n = b200moe_registry(&rows);
    std::vector<Registration> out;
    out.reserve(n);
    for (std::uint32_t i = 0; i < n; ++i)
        out.push_back({rows[i].schema, rows[i].revision, static_cast<std::size_t>(rows[i].bytes), static_cast<std::size_t>(rows[i].alignment), &launch_b200});
    return out;
}

// The typed way in for a caller that holds a view: strix::weight::arguments() needs ArgumentTraits, which a backend
// registration supplies (resolve.hpp:78-84); this is the same envelope built by hand.
template <class View>
inline ::strix::weight::KernelArguments envelope(std::uint32_t site, const View& view) {
    return {site, B200MOE_ABI_VERSION, &view, sizeof(View)};
}

}  // namespace strix_b200

// instantiate what the file defines, so that the syntax check covers it
static ::strix::weight::KernelArguments b200_example(const b200moe_quantize_a8_view& v) { return strix_b200::envelope(B200MOE_SITE_QUANTIZE_A8, v); }
static std::vector<strix_b200::Registration> (*const b200_rows)() = &strix_b200::b200_registrations;
static const void* const b200_use[] = {reinterpret_cast<const void*>(&b200_example), reinterpret_cast<const void*>(b200_rows)};
