// Home-rank side of expert parallelism: what a rank does with the pieces its peers return.
//
//  * fold_parts: y = (((shared + P_0) + P_1) + ...) + P_{n-1}, one FP32 add per step in rank order. P_r is the partial
//    sum of the experts owned by rank r (b200moe_layer with only_part = r, i.e. reference_half_sum,
//    src/ds41_moe.cpp:99-115); the fold is the reference's (shared + low) + high (include/strix/ds41_moe.hpp:7-11)
//    with n ranges instead of two, so one GPU folding n virtual ranks and n GPUs give the same bits.
//  * select_owner_slots: the Qwen-form combine is one fused multiply-add chain in slot order and cannot be split by
//    rank, so the owners return raw slot vectors (same file, :5-8: "a rank that computes a subset of the experts
//    produces the same raw vectors"). Every peer returns a full [slots][hidden] block of which only the slots of its
//    own experts are meaningful; this picks slot s from the block of the rank that owns expert ids[s].
// Pure data movement and FP32 adds: HBM-bound, tiny at decode sizes.
#include <cstring>

#include "kernels.cuh"

namespace b200moe {
namespace {

__global__ void __launch_bounds__(256) fold_parts_kernel(const float* __restrict__ parts, u32 n_parts, u64 part_stride,
                                                         const float* __restrict__ shared, u64 count, float* __restrict__ y,
                                                         u16* __restrict__ y_bf16) {
    const u64 i = u64(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float acc = shared ? shared[i] : 0.0f;
    for (u32 p = 0; p < n_parts; ++p) acc = __fadd_rn(acc, parts[u64(p) * part_stride + i]);
    y[i] = acc;
    if (y_bf16) y_bf16[i] = static_cast<u16>(bf16_rne_bits(acc));
}

__global__ void __launch_bounds__(256) select_owner_slots_kernel(const float* __restrict__ blocks, u64 block_stride, u32 n_blocks,
                                                                 u32 experts_per_block, const u32* __restrict__ ids, u32 slots, u32 hidden,
                                                                 float* __restrict__ raw) {
    for (u32 slot = blockIdx.y; slot < slots; slot += gridDim.y) {  // grid.y is capped at 65,535
        const u32 owner = min(ids[slot] / experts_per_block, n_blocks - 1u);
        const float* src = blocks + u64(owner) * block_stride + u64(slot) * hidden;
        for (u32 o = blockIdx.x * blockDim.x + threadIdx.x; o < hidden; o += gridDim.x * blockDim.x) raw[u64(slot) * hidden + o] = src[o];
    }
}

}  // namespace
}  // namespace b200moe

extern "C" {

int b200moe_peer_buffer_create(uint64_t bytes, void** dev_ptr, void* ipc_handle_64) {
    using namespace b200moe;
    B200_REQUIRE(bytes && dev_ptr && ipc_handle_64, "peer_buffer_create: bytes / dev_ptr / ipc_handle are null");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the IPC handle is sent as 64 bytes");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    cudaIpcMemHandle_t h{};
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        return fail(B200MOE_ERR_CUDA, "peer_buffer_create: %s", cudaGetErrorString(e));
    }
    std::memcpy(ipc_handle_64, &h, 64);
    *dev_ptr = p;
    return B200MOE_OK;
}
int b200moe_peer_buffer_open(const void* ipc_handle_64, void** dev_ptr) {
    using namespace b200moe;
    B200_REQUIRE(ipc_handle_64 && dev_ptr, "peer_buffer_open: ipc_handle / dev_ptr are null");
    if (!device_ready()) return B200MOE_ERR_CUDA;
    cudaIpcMemHandle_t h{};
    std::memcpy(&h, ipc_handle_64, 64);
    void* p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(B200MOE_ERR_COMM, "peer_buffer_open: %s", cudaGetErrorString(e));
    *dev_ptr = p;
    return B200MOE_OK;
}
int b200moe_peer_buffer_close(void* dev_ptr) {
    using namespace b200moe;
    B200_REQUIRE(dev_ptr, "peer_buffer_close: null pointer");
    const cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    return e == cudaSuccess ? B200MOE_OK : fail(B200MOE_ERR_COMM, "peer_buffer_close: %s", cudaGetErrorString(e));
}
int b200moe_peer_buffer_destroy(void* dev_ptr) {
    using namespace b200moe;
    B200_REQUIRE(dev_ptr, "peer_buffer_destroy: null pointer");
    const cudaError_t e = cudaFree(dev_ptr);
    return e == cudaSuccess ? B200MOE_OK : fail(B200MOE_ERR_CUDA, "peer_buffer_destroy: %s", cudaGetErrorString(e));
}

int b200moe_fold_parts(const float* parts, uint32_t n_parts, uint64_t part_stride, const float* shared, uint64_t count, float* y,
                       uint16_t* y_bf16, void* stream) {
    using namespace b200moe;
    B200_REQUIRE(parts && y && n_parts >= 1, "fold_parts: parts / y are null or n_parts is 0");
    B200_REQUIRE(part_stride >= count, "fold_parts: part_stride %llu is below count %llu", (unsigned long long)part_stride, (unsigned long long)count);
    if (count == 0) return B200MOE_OK;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    fold_parts_kernel<<<static_cast<u32>((count + 255) / 256), 256, 0, as_stream(stream)>>>(parts, n_parts, part_stride, shared, count, y, y_bf16);
    return after_launch("fold_parts");
}

int b200moe_select_owner_slots(const float* blocks, uint64_t block_stride, uint32_t n_blocks, uint32_t experts_per_block,
                               const uint32_t* ids, uint32_t slots, uint32_t hidden, float* raw, void* stream) {
    using namespace b200moe;
    B200_REQUIRE(blocks && ids && raw, "select_owner_slots: blocks / ids / raw are null");
    B200_REQUIRE(n_blocks >= 1 && experts_per_block >= 1 && hidden >= 1, "select_owner_slots: n_blocks, experts_per_block and hidden must be non-zero");
    B200_REQUIRE(block_stride >= u64(slots) * hidden, "select_owner_slots: block_stride is below slots * hidden");
    if (slots == 0) return B200MOE_OK;
    if (!device_ready()) return B200MOE_ERR_CUDA;
    select_owner_slots_kernel<<<dim3((hidden + 1023) / 1024, slots < 65535u ? slots : 65535u), 256, 0, as_stream(stream)>>>(blocks, block_stride, n_blocks, experts_per_block, ids, slots, hidden, raw);
    return after_launch("select_owner_slots");
}

}  // extern "C"
