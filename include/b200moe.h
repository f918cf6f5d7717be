/*
 * b200moe.h - C ABI of the B200 (sm_100a) block-quantized MoE FFN path.
 *
 * The path: router top-k -> dequant-fused expert gate/up projection with SwiGLU and A8 re-quantisation -> down
 * projection -> weighted combine, on GGUF Q8_0 / Q4_K expert tensors kept in their stored byte layout.
 *
 * Conventions (the reference CUDA operator layer's, include/strix/cuda/ds41_common.hpp:6-19):
 *   - every entry point only ENQUEUES on the caller's stream (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream): no synchronisation, no allocation, no hidden threads;
 *   - views are plain structs of device pointers, sizes and strides; storage and lifetime belong to the caller;
 *     scratch comes from the caller and is sized by the matching *_workspace_bytes function;
 *   - rows are independent tokens: a row's bits never depend on how many rows the call carries;
 *   - argument errors return a non-zero status BEFORE anything is written or launched (the reference throws
 *     std::invalid_argument there, ds41_common.hpp:33-35; exceptions do not cross a C ABI) and the text is kept in a
 *     thread-local string read with b200moe_last_error();
 *   - data errors (non-finite activations, invalid routes) never fail a call: they set per-row status bits and a
 *     job summary word, later stages return early, exactly like include/strix/cuda/qwen_moe.hpp:30-31.
 * All pointers are device pointers unless a name ends in _host.
 *
 * There is no CPU fallback behind this interface: without a CUDA device (or without the sm_100a image) every
 * compute entry point fails with B200MOE_ERR_CUDA.
 */
#ifndef B200MOE_H
#define B200MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 4

/* Status codes (values follow strix::weight::Error's role, include/strix/weight/types.hpp:35-40). */
enum {
    B200MOE_OK = 0,
    B200MOE_ERR_INVALID_ARGUMENT = 1, /* a view is inconsistent (sizes, alignment, null pointers) */
    B200MOE_ERR_UNSUPPORTED = 2,      /* a format / policy this build does not bind */
    B200MOE_ERR_WORKSPACE = 3,        /* caller-owned scratch is missing or too small */
    B200MOE_ERR_CUDA = 4,             /* a CUDA runtime call failed (text in b200moe_last_error) */
    B200MOE_ERR_COMM = 5,             /* an NCCL call failed */
    B200MOE_ERR_ABORTED = 6           /* a bounded device wait ran out (B200MOE_JOB_WAIT_ABORTED): the outputs are not valid */
};

/* ggml tensor type ids of the stored expert tensors (include/strix/cuda/qwen_moe.hpp:33). */
#define B200MOE_TYPE_Q5_1 7u  /* 24-byte blocks {fp16 d, fp16 m, 32 high bits, 16 B nibbles}: down tensors of the Qwen A8 family
                               * (strix::cpu::expert::DownFormat::q5_1, src/cpu/core/routed_expert.hpp:28) */
#define B200MOE_TYPE_Q8_0 8u  /* 34-byte blocks {fp16 d, int8 q[32]} */
#define B200MOE_TYPE_Q2_K 10u /* 84-byte super-blocks {16 B of (4-bit scale | 4-bit min << 4) per 16 weights, 64 B of 2-bit quants, fp16 d,
                              * fp16 dmin}: gate / up / down tensors of the DS41 family (include/strix/ds41_formats.hpp:16-19) */
#define B200MOE_TYPE_Q4_K 12u /* 144-byte super-blocks {fp16 d, fp16 dmin, 12 B 6-bit scales/mins, 128 B nibbles} */
#define B200MOE_TYPE_Q5_K 13u /* 176-byte super-blocks {fp16 d, fp16 dmin, 12 B scales/mins, 32 B high bits, 128 B nibbles}: gate / up
                               * tensors (GateFormat::q5_k, routed_expert.hpp:27); the Q4_K row rule with 5-bit quants */

/* Row status / job summary bits (include/strix/cuda/qwen_moe.hpp:31). */
#define B200MOE_ROW_INVALID_ROUTE 1u
#define B200MOE_ROW_NONFINITE_ACTIVATION 2u
#define B200MOE_ROW_INVALID_DELTA 4u
#define B200MOE_ROW_PROJECTION_NONFINITE 8u
/* Job summary only: a bounded wait inside a kernel of the job ran out (a copy that never landed, a peer that never
 * signalled). Every wait on the device has a poll limit instead of hanging (the reference's bounded wait with a watchdog,
 * src/cuda/tiered_experts.cu:107-127); the kernel that gives up sets this bit and returns, later stages of the job see it and
 * write nothing (down, combine), so y keeps what the caller put there. The *_host call returns B200MOE_ERR_ABORTED. */
#define B200MOE_JOB_WAIT_ABORTED 0x40000000u

int b200moe_abi_version(void);
/* Text of the last failure on the calling thread ("" when none). Valid until the thread's next failing call. */
const char* b200moe_last_error(void);
/* Number of kernels this library has launched in the calling process (all threads); a plain counter for reports. */
uint64_t b200moe_launch_count(void);

/* Test and measurement hooks: process-wide values read when a kernel is launched. They exist so that the tests can make a
 * bounded wait run out WITHOUT a device fault and so that the forms of the decode GEMVs can be compared on one input; a
 * production caller never sets them. The reference has the same kind of seam (TierDev::timeout_ns,
 * src/cuda/tiered_experts.cu:107-127). Returns B200MOE_ERR_INVALID_ARGUMENT for an unknown key. */
#define B200MOE_DEBUG_WAIT_LIMIT 0u  /* polls of every bounded wait in the streaming kernels; 0 = the default (2^22) */
#define B200MOE_DEBUG_STALL_STAGE 1u /* n > 0: in every CTA of the segment-streaming kernels the first producer stops feeding
                                      * before its n-th stage (no copy of that stage is issued, none is left in flight); 0 = never */
#define B200MOE_DEBUG_DECODE_FORM 2u /* decode windows: 0 = chosen by the plan, 1 = row streaming (Q4_K), 2 = segment streaming (Q4_K;
                                      * Q8_0: the dp4a token-block form), 3 = per-block (Q8_0: one row per warp), 4 = the Q8_0
                                      * tensor-core form (each only where it applies) */
int b200moe_debug_set(uint32_t key, uint32_t value);

/* ------------------------------------------------------------------------------------------------ A8 activations
 * A8 rows: codes [row][stride] int8, deltas / sums [row][stride / 32]; width <= stride, both multiples of 32.
 * Mirrors strix::cuda::core::A8Rows (include/strix/cuda/core/types.hpp:16-21). */
typedef struct b200moe_a8_rows {
    int8_t* codes;
    float* deltas;
    int32_t* sums; /* optional (NULL) where a consumer does not read sums */
    uint32_t rows, width, stride; /* stride 0 = width */
} b200moe_a8_rows;

/* out row r = quantize_a8(x[r * x_stride .. + width)): per 32 values delta = amax / 127 (1 when amax == 0 or
 * amax < 2^-119, codes then 0), code = clamp(rint(x / delta), +-127), sum = sum of codes. Bitwise the host rule
 * (src/cpu/core/reference.cpp:35-55, src/ds41_formats.cpp:146-165).
 * Replaces strix::ds41::cuda::enqueue_quantize_a8(QuantizeA8View) (include/strix/cuda/ds41_core.hpp:17-22) and
 * strix::cpu::Kernels::quantize_a8 (src/cpu/core/backend.hpp:68-69). x_is_bf16 != 0: x holds bfloat16 bit patterns
 * (uint16) widened exactly, the input form of the Qwen prologue (src/cuda/models/qwen/qwen_moe.cu:60-99). */
typedef struct b200moe_quantize_a8_view {
    const void* x;
    uint32_t rows, width, x_stride; /* x_stride in elements, 0 = width */
    uint32_t x_is_bf16;
    b200moe_a8_rows out;
    uint32_t* status; /* optional [rows]: |= NONFINITE_ACTIVATION for a row holding a NaN / Inf */
} b200moe_quantize_a8_view;
int b200moe_quantize_a8(const b200moe_quantize_a8_view* view, void* stream);

/* ------------------------------------------------------------------------------------------- RMSNorm (+ A8) before the FFN
 * The step in front of the FFN in a layer, fused with the A8 quantiser the router / experts read:
 *   y[r][i] = (x[r][i] * s_r) * weight[i]   (weight NULL: x * s_r),   s_r = 1 / sqrt(sumsq_r / n + eps),
 * sumsq_r in the host rule's order: L = 256 lanes (128 when n < 512), lane l = fma(x[i], x[i], .) over i = l, l + L, ...
 * from +0, then the halving tree lane[l] += lane[l + h], h = L/2 .. 1. Bitwise strix::cpu::Kernels::rmsnorm_f32
 * (src/cpu/core/backend.hpp:71-72; src/cpu/core/reference.cpp:86-103), which it replaces together with the norm + A8
 * outputs of strix::ds41::cuda::enqueue_norm(NormView) (include/strix/cuda/ds41_core.hpp:86-100).
 * out (optional, may alias x) gets y; a8 (optional: a8.codes NULL = none) gets quantize_a8(y). n a multiple of 32. */
typedef struct b200moe_rmsnorm_view {
    const float* x;
    uint32_t rows, n, x_stride; /* x_stride in elements, 0 = n */
    const float* weight;        /* [n] or NULL */
    float eps;
    float* out;                 /* optional [rows][out_stride] */
    uint32_t out_stride;        /* 0 = n */
    b200moe_a8_rows a8;         /* optional */
    uint32_t* status;           /* optional [rows]: |= NONFINITE_ACTIVATION for a row whose y holds a NaN / Inf */
} b200moe_rmsnorm_view;
int b200moe_rmsnorm_a8(const b200moe_rmsnorm_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ Q8_0 x A8 GEMV
 * out[r * out_stride + o] = product_q8_0(weight row (first + o), A8 row r) for o in [0, count): per 32-weight group
 * float(int32 dot) * (scale * delta); group g into lane class g % 32, classes accumulated ascending from +0, combined
 * by the butterfly v[l] += v[l ^ d], d = 16..1, result lane 0; accumulate != 0: out = out + product.
 * Replaces strix::ds41::cuda::enqueue_q8_0_a8(Q8A8View) (include/strix/cuda/ds41_core.hpp:46-74) and
 * strix::cpu::Kernels::gemv_q8_0_a8(Q8a8View) (src/cpu/core/backend.hpp:47-55, :70). */
typedef struct b200moe_q8a8_view {
    const uint8_t* weight; /* row o at weight + o * row_bytes */
    uint32_t row_bytes;    /* >= width / 32 * 34, a multiple of 2 */
    uint32_t width;        /* K, a multiple of 32 */
    uint32_t first, count;
    b200moe_a8_rows x;
    float* out;
    uint32_t out_stride; /* 0 = count */
    uint32_t accumulate;
} b200moe_q8a8_view;
int b200moe_q8_0_a8(const b200moe_q8a8_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ router
 * Mirrors strix::moe::RoutePolicy (include/strix/moe/route_policy.hpp:40-53), enum values included. */
enum { B200MOE_SCORE_SOFTMAX = 0, B200MOE_SCORE_SIGMOID = 1, B200MOE_SCORE_SQRT_SOFTPLUS = 2 };
enum { B200MOE_KEY_FLOAT_SERIAL = 0, B200MOE_KEY_ORDERED_BITS = 1 };
enum { B200MOE_ORDER_SELECTION = 0, B200MOE_ORDER_ASCENDING_ID = 1 };
typedef struct b200moe_route_policy {
    uint32_t score;
    uint32_t selection_bias; /* choice = score + bias[e] (selection only; weights use the unbiased score) */
    uint32_t key;
    uint32_t order;
    uint32_t experts, top_k;
    /* n_group > 1: group-limited selection. The reference rejects it (route_policy.hpp:56-60); here it is an
     * extension in the same declared style: experts split into n_group contiguous groups, group score = c1 + c2 of
     * the group's two best choices (picked with the policy's key), topk_group groups kept by k passes (ties -> lower
     * group id), then the usual k-pass expert selection over the kept groups only. */
    uint32_t n_group, topk_group;
    uint32_t renormalize;
    uint32_t renorm_single;
    float renorm_eps;
    float scale;
} b200moe_route_policy;

/* logits[r][e] = lane-strided FP32 dot of weight row e with x[r] (lane l takes elements l, l + 32, ... ascending,
 * acc = acc + w * x with no fused multiply-add, then the butterfly d = 16..1), + logit_bias[e] when given; scores by
 * the policy transform (declared_exp / declared_log1p, include/strix/ds41_moe.hpp:38-100); k-pass selection
 * (choice desc, id asc; a NaN stays only as a first candidate); weights = score / (sum + eps) * scale, the sum in
 * output order. Expert ids and weight bits equal strix::ds41::reference_router (src/ds41_moe.cpp:63-97) +
 * strix::moe::route_select_ref (route_policy.hpp:99-129).
 * Replaces strix::ds41::cuda::enqueue_router(RouterView) (include/strix/cuda/ds41_core.hpp:153-167) and
 * hc::route_logits / route_select (src/cuda/models/qwen/qwen_hc.cu:1131-1361). */
typedef struct b200moe_router_view {
    const float* x;          /* [rows][x_stride] FP32; NULL when logits are given */
    uint32_t x_stride;       /* 0 = hidden */
    uint32_t rows, hidden;   /* hidden a multiple of 32 */
    const float* weight;     /* [experts][hidden] FP32 */
    const float* logit_bias; /* optional [experts], added to the logit before the score transform */
    const float* bias;       /* [experts] when policy.selection_bias */
    b200moe_route_policy policy;
    float* logits;           /* [rows][experts]: written when x is given, read otherwise */
    float* scores;           /* [rows][experts] output (may alias logits) */
    uint32_t* ids;           /* [rows][top_k] */
    float* weights;          /* [rows][top_k] */
} b200moe_router_view;
int b200moe_router(const b200moe_router_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ routes (permute)
 * Expert-major CSR over the union of the window's experts; activations are never moved, kernels gather through it.
 * Mirrors strix::ds41::cuda::MoeRoutes / MoeRoutesView (include/strix/cuda/ds41_moe.hpp:41-72) =
 * build_window_routes + restrict_routes (src/ds41_moe.cpp:11-61): experts ascending, entries of an expert in
 * ascending row; slots[i] = row * top_k + k; order[row][k] = the row's slots in ascending expert id;
 * low_counts[row] = how many of them have id < split; counts[0] = union experts, counts[1] = most entries of one
 * expert, counts[2] = entries, counts[3] = 0: a scratch word of the expert kernels (they deal their work items out through
 * it and leave it zero; routes built by other means must provide it zeroed, and two launches that run at the same time
 * must not share one routes object). Only experts in [first, end) get entries (end 0 = all); experts[] holds id - base.
 * Sizes: rows * top_k for experts / rows / slots / order, + 1 for begins, rows for low_counts, 4 for counts. */
typedef struct b200moe_routes {
    uint32_t* experts;
    uint32_t* begins;
    uint32_t* rows;
    uint32_t* slots;
    uint32_t* order;
    uint32_t* low_counts;
    uint32_t* counts;
} b200moe_routes;
typedef struct b200moe_routes_view {
    const uint32_t* ids;
    uint32_t rows, top_k, experts, split;
    uint32_t first, end, base;
    uint32_t* scratch;    /* b200moe_routes_scratch_words(rows, top_k, experts) words; may be NULL up to 1024 slots */
    uint32_t* row_status; /* optional [rows]: |= INVALID_ROUTE for an id >= experts or repeated within a row */
    b200moe_routes out;
} b200moe_routes_view;
uint64_t b200moe_routes_scratch_words(uint32_t rows, uint32_t top_k, uint32_t experts);
int b200moe_build_routes(const b200moe_routes_view* view, void* stream);

/* The same build with the library's own scratch: view->scratch is ignored, and the call allocates no device memory
 * (no cudaMalloc / cudaFree, no allocating library routine). This entry point has no counterpart in the reference; it
 * exists for callers that own no device allocator and whose buffers were all fixed when the engine loaded. The scratch
 * is one fixed array per device inside the library, b200moe_routes_static_max_words() words long: a window whose
 * b200moe_routes_scratch_words(rows, top_k, experts) exceeds that is refused with B200MOE_ERR_UNSUPPORTED and a message
 * that names both numbers (65,536 slots at 1024 experts fit). The array keeps whatever the previous call left; no word
 * of it is read before the same call has written it, so nothing needs clearing. It is shared by every caller of the
 * process: two calls that overlap in time on one device (two streams, two threads) race on it - serialise them. The
 * first call on each device looks up the array's address with that device current; make that call during set-up,
 * before any stream capture begins. Results are identical to b200moe_build_routes. */
uint64_t b200moe_routes_static_max_words(void);
int b200moe_build_routes_static(const b200moe_routes_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ experts
 * Geometry and formats of the routed experts of one layer. The gate/up type fixes the arithmetic family:
 *   Q8_0 (DS41 family, src/ds41_formats.cpp:188-197, src/ds41_moe.cpp:124-165): product_q8_0 lane classes and
 *     butterfly for gate, up and down; h = swiglu_clamped(g, u, limit) with declared_exp; quantize_a8 per 32 outputs.
 *   Q4_K (Qwen A8 family, src/cpu/core/routed_expert.hpp:9-15): x_j = E_g * ((d*sc_j) * float(dot_j) - (dmin*m_j) *
 *     float(S_g)), pair sums into four chains over ascending super-blocks, (a0 + a1) + (a2 + a3);
 *     h = (g / (1 + exp(-g))) * u with the gfx1151 v_exp twin at zero correction tables
 *     (src/cpu/core/routed_expert.cpp:208-261); down Q4_K with the same row rule over K = inter
 *     (src/moe_a8_down_contract.cpp:141-146) or Q8_0 with the four-chain rule (routed_expert.cpp:110-144).
 * Tensors keep their GGUF bytes: gate, up [experts][inter][hidden / B blocks]; down [experts][hidden][inter / B]. */
typedef struct b200moe_shape {
    uint32_t hidden, inter, experts, top_k;
    uint32_t gate_type, down_type;
    float limit; /* SwiGLU clamp of the DS41 family (+inf = none); ignored by the Qwen family */
} b200moe_shape;
typedef struct b200moe_expert_weights {
    const uint8_t* gate;
    const uint8_t* up;
    const uint8_t* down;
} b200moe_expert_weights;
uint64_t b200moe_gate_row_bytes(const b200moe_shape* shape);
uint64_t b200moe_down_row_bytes(const b200moe_shape* shape);
uint64_t b200moe_expert_bytes(const b200moe_shape* shape);

/* act[slot] = quantize_a8(swiglu(gate . x[row], up . x[row])) for every routed entry.
 * Replaces enqueue_routed_gate_up(RoutedGateUpView) (include/strix/cuda/ds41_moe.hpp:78-107), qwen_moe::enqueue_project
 * (include/strix/cuda/qwen_moe.hpp:100) and phase 1 of strix::cpu::expert::Executor::run
 * (src/cpu/core/routed_expert.cpp:403-427). */
typedef struct b200moe_gate_up_view {
    b200moe_shape shape;
    b200moe_expert_weights weights;
    b200moe_routes routes;
    uint32_t max_union;     /* a bound of counts[0]: min(rows * top_k, experts) */
    b200moe_a8_rows x;      /* [rows][hidden] */
    b200moe_a8_rows act;    /* [slots][inter] */
    float* gate_out;        /* optional [slots][inter] FP32 taps (both or neither) */
    float* up_out;
    uint32_t* row_status;   /* optional [rows] */
    uint32_t* summary;      /* optional [1]: OR of every status bit set by the job */
} b200moe_gate_up_view;
int b200moe_gate_up(const b200moe_gate_up_view* view, void* stream);

/* raw[slot][o] = down row o of the slot's expert . act[slot] (unweighted raw slot vector).
 * Replaces enqueue_routed_down(RoutedDownView) (include/strix/cuda/ds41_moe.hpp:91-107), qwen_moe::enqueue_down
 * (qwen_moe.hpp:101) and phase 2 of Executor::run (routed_expert.cpp:429-447). */
typedef struct b200moe_down_view {
    b200moe_shape shape;
    b200moe_expert_weights weights;
    b200moe_routes routes;
    uint32_t max_union;
    b200moe_a8_rows act;
    float* raw;          /* [slots][hidden] */
    const uint32_t* summary; /* optional: a non-zero word skips the whole stage (routed_expert.hpp:17-19) */
} b200moe_down_view;
int b200moe_down(const b200moe_down_view* view, void* stream);

/* Combine forms.
 *   PARTS (DS41, src/ds41_moe.cpp:152-163 generalised to `parts` expert ranges): y = (((shared + S_0) + S_1) ... ),
 *     S_p = sum over the row's slots whose expert id lies in part p (p = min(id / part_experts, parts - 1)), in
 *     ascending expert id from +0, each step one product then one add. parts = 2, part_experts = split is
 *     (shared + low) + high. `only_part` >= 0 writes S_only_part alone (reference_half_sum, ds41_moe.cpp:99-115:
 *     what a rank owning that part sends).
 *   FMA_SLOTS (Qwen merge, src/cuda/models/qwen/qwen_moe.cu:286-310 = combine_ref fma_f32,
 *     include/strix/moe/combine.hpp:36-59): acc = +0; acc = fma(w[k], raw[k], acc) in slot order; y = acc (+ shared).
 * y_bf16 (optional) receives the bfloat16 RNE commit of y (qwen_moe.cu:330-335). */
enum { B200MOE_COMBINE_PARTS = 0, B200MOE_COMBINE_FMA_SLOTS = 1 };
typedef struct b200moe_combine_view {
    const float* raw;          /* [rows * top_k][hidden] */
    const float* shared;       /* optional [rows][hidden] */
    const float* weights;      /* [rows * top_k] */
    const uint32_t* ids;       /* [rows * top_k] expert id of each slot (PARTS) */
    const uint32_t* order;     /* [rows * top_k] slots in ascending expert id (PARTS) */
    uint32_t rows, top_k, hidden;
    uint32_t form;
    uint32_t parts, part_experts;
    int32_t only_part;         /* -1: the whole combine */
    float* y;                  /* [rows][hidden] */
    uint16_t* y_bf16;          /* optional */
    const uint32_t* row_status; /* optional: a row with status != 0 is not written (fail closed) */
    /* Optional scatter of y by row blocks (expert parallelism: each block of y_block_rows rows belongs to another home
     * rank and is written straight into that rank's memory by this kernel - plain peer stores over NVLink, no
     * collective in between): a DEVICE array of ceil(rows / y_block_rows) pointers; row r goes to
     * y_blocks[r / y_block_rows] + (r % y_block_rows) * hidden. When set, y may be NULL and y_bf16 must be NULL. */
    float* const* y_blocks;
    uint32_t y_block_rows;
    const uint32_t* summary;   /* optional job summary: with B200MOE_JOB_WAIT_ABORTED set nothing is written */
    /* only_part >= 0 with only_part_count = n > 1: the n partial sums S_only_part .. S_only_part+n-1 are written, sum i at
     * the destination of sum 0 plus i * part_stride floats (a rank that owns n consecutive expert ranges of the fold). */
    uint32_t only_part_count;  /* 0 or 1: one sum */
    uint64_t part_stride;
    /* PARTS with parts = 2, as strix::ds41::cuda::MoeCombineView gives it (include/strix/cuda/ds41_moe.hpp:113-131): the
     * first low_counts[row] slots of the row's order are the low part, the others the high part. When set, ids is not read. */
    const uint32_t* low_counts;
} b200moe_combine_view;
int b200moe_combine(const b200moe_combine_view* view, void* stream);

/* y = (a + b) + c elementwise (enqueue_moe_canonical_sum, include/strix/cuda/ds41_moe.hpp:135-137); c may be NULL. */
int b200moe_canonical_sum(const float* a, const float* b, const float* c, uint64_t count, float* y, void* stream);

/* ------------------------------------------------------------------------------------------ expert parallelism
 * What the home rank of a token block does with the pieces its peers return. The reference moves them with
 * Communicator::exchange (include/strix/dist/communicator.hpp, two ranks); here they arrive by NCCL and these two
 * calls are the arithmetic either side of it.
 *
 * fold_parts: y = (((shared + P_0) + P_1) + ...) + P_{n-1}, one FP32 add per step in rank order; P_r = the partial sum
 *   of rank r's experts (b200moe_layer with only_part = r: reference_half_sum, src/ds41_moe.cpp:99-115). This is the
 *   reference's y = (shared + low) + high (include/strix/ds41_moe.hpp:7-11) with n expert ranges instead of two.
 *   parts: n_parts blocks of `count` floats, `part_stride` floats apart. shared may be NULL (+0). y_bf16 optional.
 * select_owner_slots: raw[s] = blocks[owner(s)][s] with owner(s) = min(ids[s] / experts_per_block, n_blocks - 1): every
 *   peer returned a [slots][hidden] block of raw slot vectors of which only its own experts' slots are meaningful
 *   (include/strix/ds41_moe.hpp:5-8); the result feeds b200moe_combine (the Qwen form's chain cannot be split by rank). */
/* Buffers other ranks of the node write into (CUDA IPC; set-up time, these calls allocate / map memory and
 * synchronise). create: cudaMalloc + the 64-byte IPC handle to send to the peers; open: map a peer's buffer from its
 * handle (peer access is enabled on first use); close / destroy undo them. The reference's counterpart is the
 * DirectTransport's registered windows (docs/engine/transport/communicator.md: "registered windows, submit, repost"). */
int b200moe_peer_buffer_create(uint64_t bytes, void** dev_ptr, void* ipc_handle_64);
int b200moe_peer_buffer_open(const void* ipc_handle_64, void** dev_ptr);
int b200moe_peer_buffer_close(void* dev_ptr);
int b200moe_peer_buffer_destroy(void* dev_ptr);
int b200moe_fold_parts(const float* parts, uint32_t n_parts, uint64_t part_stride, const float* shared, uint64_t count, float* y,
                       uint16_t* y_bf16, void* stream);
int b200moe_select_owner_slots(const float* blocks, uint64_t block_stride, uint32_t n_blocks, uint32_t experts_per_block,
                               const uint32_t* ids, uint32_t slots, uint32_t hidden, float* raw, void* stream);

/* ------------------------------------------------------------------------------------------ expert parallelism, one call
 * The whole expert-parallel step of a rank behind one enqueue-only call: route the rank's home rows, dispatch them to the
 * ranks whose experts they selected, run the local experts, return the partial sums, fold. Both exchanges are kernels of
 * this library storing into the peers' memory over NVLink (windows created with b200moe_peer_buffer_create and mapped with
 * b200moe_peer_buffer_open on every rank; plain peer stores, no multicast, no collective library, no host wait), each
 * followed by per-source arrival flags that the receiver polls with a BOUNDED wait: a peer that never signals costs
 * wait_polls polls (about a second by default), then the job summary gets B200MOE_JOB_WAIT_ABORTED and y is not written.
 * Stands where the reference has its two-rank split over Communicator::exchange (include/strix/dist/communicator.hpp:180;
 * include/strix/ds41_moe.hpp:5-11; restrict_routes / reference_half_sum, src/ds41_moe.cpp:45-61, :99-115): rank r owns
 * experts [r * E / W, (r + 1) * E / W) and passes only those tensors; a row's A8 record goes only to the ranks that own
 * one of its experts (the all-to-all-v of the dispatch; positions are fixed by the global row index, so no counts are
 * negotiated); y = (((shared + S_0) + S_1) + ...) + S_{F-1} over F = fold_parts expert ranges (a rank returns the sums of
 * its F / W ranges): the bits of b200moe_ffn with combine PARTS and parts = F.
 * Every rank calls b200moe_ep_ffn once per step with the same rows_per_rank; steps alternate between two halves of
 * the window, so a captured CUDA graph must hold an even number of steps. Set-up calls (create / destroy) allocate and
 * synchronise; b200moe_ep_ffn does neither. */
typedef struct b200moe_ep_desc {
    b200moe_shape shape;           /* experts = all routed experts of the layer */
    b200moe_route_policy policy;
    uint32_t world, rank;          /* 1 <= world <= 8 (one node), experts % world == 0 */
    uint32_t rows_per_rank;        /* home rows of every rank per step */
    uint32_t wait_polls;           /* bound of the flag waits, 0 = the default (about a second) */
    uint32_t fold_parts;           /* expert ranges of the fold, a multiple of world dividing experts; 0 = world. With the same
                                    * value at every world size (8, say) 1, 2, 4 and 8 GPUs give the same bits */
    void* const* windows;          /* HOST array [world]: device address, in this process, of every rank's window (own included),
                                    * each b200moe_ep_window_bytes() long and zero-filled before the first step */
} b200moe_ep_desc;
typedef struct b200moe_ep_step_view {
    b200moe_expert_weights weights; /* the rank's experts only: [experts / world][...] */
    const float* router_weight;     /* [experts][hidden], replicated */
    const float* logit_bias;        /* optional */
    const float* select_bias;       /* when policy.selection_bias */
    const void* x;                  /* [rows][hidden] FP32 or bfloat16: the rank's home rows */
    uint32_t x_is_bf16;
    uint32_t rows;                  /* == rows_per_rank */
    const float* shared;            /* optional [rows][hidden]: the shared expert's output for the home rows */
    float* y;                       /* [rows][hidden] */
    uint16_t* y_bf16;               /* optional */
    uint32_t* summary;              /* optional [1]: job summary (see b200moe_layer_view) */
    void* workspace;
    uint64_t workspace_bytes;       /* b200moe_ep_workspace_bytes(ep) */
    uint32_t grouped_min_rows;      /* as b200moe_layer_view, applied to the world * rows_per_rank window */
    void* const* stage_events;      /* optional timing taps of the local experts (see b200moe_layer_view) */
} b200moe_ep_step_view;
uint64_t b200moe_ep_window_bytes(const b200moe_shape* shape, uint32_t world, uint32_t rows_per_rank, uint32_t fold_parts);
int b200moe_ep_create(const b200moe_ep_desc* desc, void** ep);
void b200moe_ep_destroy(void* ep);
uint64_t b200moe_ep_workspace_bytes(const void* ep);
int b200moe_ep_ffn(void* ep, const b200moe_ep_step_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ whole layer
 * Routes from the router's ids, gate/up, down and the combine. Decode GEMVs below grouped_min_rows rows, the grouped
 * tensor-core GEMM from there (0 = never). Replaces enqueue_moe_layer(MoeLayerView)
 * (include/strix/cuda/ds41_moe.hpp:139-156) and qwen_moe::enqueue_routed + enqueue_combine (qwen_moe.hpp:105-107). */
typedef struct b200moe_layer_view {
    b200moe_shape shape;
    b200moe_expert_weights weights;
    uint32_t rows;
    b200moe_a8_rows x;
    const uint32_t* ids;        /* [rows][top_k] */
    const float* route_weights; /* [rows][top_k] */
    const float* shared;        /* optional [rows][hidden] */
    uint32_t first, end, base;  /* expert range owned by this call (end 0 = all) */
    uint32_t combine_form, parts, part_experts;
    int32_t only_part;
    float* raw;                 /* optional [rows * top_k][hidden] (else in the workspace) */
    float* y;                   /* [rows][hidden]; NULL skips the combine */
    uint16_t* y_bf16;
    uint32_t* row_status;       /* optional [rows] */
    void* workspace;
    uint64_t workspace_bytes;
    uint32_t capacity;          /* rows <= capacity */
    uint32_t grouped_min_rows;
    /* Timing taps (optional, like MoeRange::wait_begin / wait_end, include/strix/cuda/ds41_moe.hpp:172-179): eight
     * cudaEvent_t handles recorded on the stream before / after the stages routes, gate/up, down, combine
     * ([2 * stage], [2 * stage + 1]). NULL: nothing is recorded. */
    void* const* stage_events;
    float* const* y_blocks;     /* optional, with y_block_rows: see b200moe_combine_view */
    uint32_t y_block_rows;
    uint32_t* summary;          /* optional [1]: receives the job summary (OR of the row status bits and B200MOE_JOB_WAIT_ABORTED);
                                 * cleared by the call. NULL: the word stays in the workspace */
    uint32_t only_part_count;   /* see b200moe_combine_view */
    uint64_t part_stride;
} b200moe_layer_view;
uint64_t b200moe_layer_workspace_bytes(const b200moe_shape* shape, uint32_t capacity);
int b200moe_layer(const b200moe_layer_view* view, void* stream);

/* Router + A8 + layer from FP32 (or bfloat16) activations: one token block through the whole FFN. */
typedef struct b200moe_ffn_view {
    b200moe_shape shape;
    b200moe_expert_weights weights;
    b200moe_route_policy policy;
    const float* router_weight;  /* [experts][hidden] */
    const float* logit_bias;     /* optional */
    const float* select_bias;    /* when policy.selection_bias */
    const void* x;               /* [rows][hidden] FP32 or bfloat16 */
    uint32_t x_is_bf16;
    uint32_t rows;
    const float* shared;         /* optional [rows][hidden] */
    uint32_t combine_form, parts, part_experts;
    float* y;                    /* [rows][hidden] */
    uint16_t* y_bf16;
    uint32_t* ids;               /* optional outputs [rows][top_k] */
    float* route_weights;
    uint32_t* row_status;
    void* workspace;
    uint64_t workspace_bytes;    /* b200moe_ffn_workspace_bytes(shape, capacity) */
    uint32_t capacity;
    uint32_t grouped_min_rows;
    void* const* stage_events;   /* passed to the layer (see b200moe_layer_view) */
    uint32_t* summary;           /* optional [1]: the job summary (see b200moe_layer_view) */
} b200moe_ffn_view;
uint64_t b200moe_ffn_workspace_bytes(const b200moe_shape* shape, uint32_t capacity);
int b200moe_ffn(const b200moe_ffn_view* view, void* stream);
/* The same call from HOST activations: x_host / y_host are host buffers (pinned for overlap); the call copies
 * x to the workspace, runs b200moe_ffn, copies y back and waits for the stream: what a caller holding tokens in host
 * memory pays end to end. view->x and view->y are ignored. Having waited, it reads the job summary: B200MOE_ERR_ABORTED
 * when a bounded device wait ran out (y_host is then not valid). */
int b200moe_ffn_host(const b200moe_ffn_view* view, const void* x_host, float* y_host, void* stream);

/* Dense SwiGLU FFN block (one "expert" applied to every row): y_partial[r] = down . A8(swiglu(gate . x_r, up . x_r))
 * over this call's slice of inter (tensor parallel: gate/up column shares and the matching down K share are stored
 * compacted, so a rank passes its own tensors and inter = its share; the partials are summed by the caller's
 * allreduce). Row rule as the routed experts of the same types. */
typedef struct b200moe_dense_view {
    b200moe_shape shape;          /* experts = 1, top_k = 1 */
    b200moe_expert_weights weights;
    uint32_t rows;
    b200moe_a8_rows x;
    float* y;                     /* [rows][hidden] FP32 */
    uint16_t* y_bf16;             /* optional bfloat16 RNE copy (the allreduce payload) */
    void* workspace;
    uint64_t workspace_bytes;     /* b200moe_layer_workspace_bytes(shape, rows) */
} b200moe_dense_view;
int b200moe_dense_ffn(const b200moe_dense_view* view, void* stream);

/* ------------------------------------------------------------------------------------------ tensor parallelism, one call
 * The dense block under tensor parallelism behind one enqueue-only call: the rank's share of b200moe_dense_ffn (gate / up
 * column shares and the matching down K share stored compacted: shape.inter = the share) and the exchange of the partial
 * sums. Every rank stores its [rows][hidden] partial - FP32, or rounded to bfloat16 when payload_bf16 is set, the payload of
 * the usual row-parallel all-reduce - into block `rank` of every rank's window (b200moe_peer_buffer_create / _open; plain
 * peer stores over NVLink, no collective library, no host wait) followed by an arrival flag; then every rank folds the W
 * blocks in rank order, y = (((+0 + P_0) + P_1) + ...) + P_{W-1} in FP32: an all-reduce with a fixed association order, the
 * reference's rule for its two-rank shared expert (include/strix/ds41_shexp_tp.hpp:7-9; src/core/tp_join.hpp:16-78). The
 * flag wait is bounded as in b200moe_ep_ffn (B200MOE_JOB_WAIT_ABORTED, y not written). x is replicated: every rank passes
 * the same rows. Steps alternate between two halves of the window: a captured CUDA graph holds an even number of steps. */
typedef struct b200moe_tp_desc {
    b200moe_shape shape;          /* experts = top_k = 1; inter = THIS rank's share (whole 256-wide super-blocks) */
    uint32_t world, rank;         /* 1 <= world <= 8 */
    uint32_t rows;                /* most rows of a step */
    uint32_t payload_bf16;        /* != 0: the partials cross NVLink as bfloat16 (RNE) and are widened before the FP32 fold */
    uint32_t wait_polls;          /* 0 = the default (about a second) */
    void* const* windows;         /* HOST array [world] of device addresses, each b200moe_tp_window_bytes() long, zero-filled */
} b200moe_tp_desc;
typedef struct b200moe_tp_step_view {
    b200moe_expert_weights weights; /* the rank's share */
    uint32_t rows;
    b200moe_a8_rows x;              /* [rows][hidden], the same on every rank */
    float* y;                       /* [rows][hidden]: the folded sum, on every rank */
    uint16_t* y_bf16;               /* optional */
    uint32_t* summary;              /* optional [1] */
    void* workspace;
    uint64_t workspace_bytes;       /* b200moe_tp_workspace_bytes(tp) */
} b200moe_tp_step_view;
uint64_t b200moe_tp_window_bytes(uint32_t hidden, uint32_t world, uint32_t rows, uint32_t payload_bf16);
int b200moe_tp_create(const b200moe_tp_desc* desc, void** tp);
void b200moe_tp_destroy(void* tp);
uint64_t b200moe_tp_workspace_bytes(const void* tp);
int b200moe_tp_dense(void* tp, const b200moe_tp_step_view* view, void* stream);

/* ------------------------------------------------------------------------------------------------ GGUF container
 * Reader for the files the expert tensors come in, with the reference reader's admission rules (strix::gguf::read_file,
 * include/strix/gguf_reader.hpp:104-111; src/gguf_reader.cpp:23-99, :330-373): GGUF v3 little-endian, bounded counts,
 * no duplicate keys or names, zero padding, aligned / in-file / non-overlapping tensor ranges, sizes from the block
 * geometry. Host-only calls (no CUDA); the handle owns the strings the infos point to. */
typedef struct b200moe_gguf_tensor_info {
    const char* name;
    uint32_t n_dims;
    uint64_t dims[4];     /* GGUF order: dims[0] is the innermost (row length in elements) */
    uint32_t ggml_type;
    uint64_t offset;      /* absolute file offset of the data */
    uint64_t bytes;
} b200moe_gguf_tensor_info;
/* The expert tensors and the router of layer L under their conventional names blk.<L>.ffn_{gate,up,down}_exps.weight and
 * blk.<L>.ffn_gate_inp.weight (roles expert_gate / expert_up / expert_down / router of include/strix/weight/types.hpp:30-34),
 * cross-checked ([hidden, inter, experts] / [inter, hidden, experts] / F32 [hidden, experts]); shape.top_k is left 0
 * (routing metadata is not tensor geometry). The byte ranges are the kernels' layout as they lie in the file. */
typedef struct b200moe_gguf_moe_layer {
    b200moe_gguf_tensor_info gate, up, down, router;
    b200moe_shape shape;
} b200moe_gguf_moe_layer;
int b200moe_gguf_open(const char* path, void** file);
void b200moe_gguf_close(void* file);
uint64_t b200moe_gguf_tensor_count(const void* file);
uint64_t b200moe_gguf_data_offset(const void* file);
uint64_t b200moe_gguf_alignment(const void* file);
int b200moe_gguf_tensor_at(const void* file, uint64_t index, b200moe_gguf_tensor_info* out);
int b200moe_gguf_find(const void* file, const char* name, b200moe_gguf_tensor_info* out);
int b200moe_gguf_find_moe_layer(const void* file, uint32_t layer, b200moe_gguf_moe_layer* out);

/* ------------------------------------------------------------------------------------------------ Expert residency
 * A layer whose experts do not all live in HBM: `slots` of the `experts` are resident (caller-owned slot tensors, the
 * per-expert layout of the full tensors), the rest stays in host memory. Stands where the reference has its tiered
 * expert residency (include/strix/cuda/tiered_experts.hpp:1-17: publish maps expert ids to slots through a device table,
 * a miss goes to the host; planner include/strix/residency/expert_residency.hpp:121-147: decayed use scores, free slots
 * first, an expert seen in the current step is never evicted, ties ascending) - with one deliberate difference: the
 * reference COMPUTES a missing expert on the CPU and a device kernel spins on a host flag for the answer; here a miss
 * is a COPY (host -> slot over the same stream) and every expert is computed on the GPU, so no kernel ever waits on
 * the host and this library keeps having no CPU arithmetic path.
 *
 * b200moe_residency_map, per window and in stream order: marks the experts the ids use, waits for that mark list on
 * the host (one stream synchronisation: the only host wait), copies the missing experts into victim slots, updates the
 * device table and writes slot_ids[i] = slot of ids[i] (0xffffffff for an id >= experts, which the routes builder then
 * flags as invalid). The caller runs b200moe_layer / b200moe_ffn stages with shape.experts = slots, the slot tensors
 * and slot_ids. Results equal the all-resident run bit for bit in the FMA_SLOTS combine form (slot order does not depend
 * on the expert numbers); the PARTS form orders by expert id and is therefore not offered through slot ids.
 * A window that uses more distinct experts than there are slots is refused (B200MOE_ERR_WORKSPACE), state unchanged. */
typedef struct b200moe_residency_desc {
    b200moe_shape shape;          /* experts = all experts of the layer */
    const uint8_t* gate_host;     /* full tensors in host memory (pinned memory makes the copies asynchronous) */
    const uint8_t* up_host;
    const uint8_t* down_host;
    uint32_t slots;               /* 1 .. experts */
    uint8_t* gate_slots;          /* device, slots x per-expert bytes (b200moe_gate_row_bytes * inter) */
    uint8_t* up_slots;
    uint8_t* down_slots;          /* device, slots x b200moe_down_row_bytes * hidden */
    float decay;                  /* score decay per window, 0 = 0.97 (the reference planner's default) */
} b200moe_residency_desc;
typedef struct b200moe_residency_stats {
    uint64_t windows, hits, misses, evictions, bytes_loaded; /* hits / misses count distinct experts per window */
} b200moe_residency_stats;
int b200moe_residency_create(const b200moe_residency_desc* desc, void** residency);
void b200moe_residency_destroy(void* residency);
int b200moe_residency_map(void* residency, const uint32_t* ids, uint32_t count, uint32_t* slot_ids, void* stream);
int b200moe_residency_get_stats(const void* residency, b200moe_residency_stats* out);
/* expert -> slot or -1, host copy of the table ([experts]). */
int b200moe_residency_table(const void* residency, int32_t* table_host);
/* The eviction rule on its own (pure host function, no CUDA): slot_expert [slots] (expert in the slot or -1), score
 * [experts], used [experts] (1 = the window uses it), missing [n_missing] -> victims [n_missing] (slot for each missing
 * expert, in order): free slots ascending first, then the slots whose expert the window does not use by (score ascending,
 * expert ascending). B200MOE_ERR_WORKSPACE when there are fewer such slots than missing experts (nothing written). */
int b200moe_residency_choose_victims(const int32_t* slot_expert, uint32_t slots, const double* score, const uint8_t* used,
                                     uint32_t experts, const uint32_t* missing, uint32_t n_missing, uint32_t* victims);

/* ------------------------------------------------------------------------------------------------ deferred first error
 * strix::DeferredMoeFirstError (include/strix/deferred_moe_status.hpp:9-28): two words {domain, bits} in device memory
 * that keep the COMPLETE first non-zero job summary of a stream of layers. The caller enqueues the merge after a layer
 * with that layer's summary word; a later layer - failed or not - never overwrites the record. The publishers are
 * serialised by the stream. b200moe_check_first_error reads a HOST copy of the record: B200MOE_OK for {0, 0},
 * B200MOE_ERR_INVALID_ARGUMENT with the bits named in b200moe_last_error for a recorded failure,
 * B200MOE_ERR_UNSUPPORTED for a malformed record (check_deferred_moe_status, :30-42). */
enum { B200MOE_DOMAIN_NONE = 0, B200MOE_DOMAIN_LEGACY = 1, B200MOE_DOMAIN_Q4K_A8 = 2 };
typedef struct b200moe_first_error {
    uint32_t domain, bits;
} b200moe_first_error;
int b200moe_merge_first_error(b200moe_first_error* record, const uint32_t* summary, uint32_t domain, void* stream);
int b200moe_check_first_error(const b200moe_first_error* record_host);

/* ------------------------------------------------------------------------------------------------ residency planner
 * Which experts to bring into HBM slots AHEAD of need, under an upload budget per step: the host-side planner of
 * strix::residency::Planner (include/strix/residency/expert_residency.hpp:102-147). Pure host code (no CUDA call).
 * seed (optional prior) -> fill_from_seed (initial residency) -> per step: observe(layer, ids) ..., end_step, plan -> for
 * every move the caller copies the expert into the slot (b200moe_residency_promote) and commits it. plan() is a pure
 * function of the state: twice without a commit gives the same moves. */
#define B200MOE_MOVE_NO_EVICTION 0xffffffffu
typedef struct b200moe_planner_desc {
    uint32_t layers, experts, top_k, slots;  /* slots per layer */
    const uint64_t* expert_bytes;            /* [layers]: bytes of one expert (gate + up + down) of the layer */
    double decay;                            /* 0 = 0.97 */
    double margin_reuses;                    /* 0 = 1.5: a candidate replaces a victim only if its score leads by more */
    uint64_t upload_bytes_per_step;          /* 0 = 64 MiB; one expert larger than the budget may still move alone */
} b200moe_planner_desc;
typedef struct b200moe_move {
    uint32_t layer, slot;
    uint32_t evict;   /* the expert leaving the slot, or B200MOE_MOVE_NO_EVICTION */
    uint32_t expert;  /* the expert moving in */
} b200moe_move;
typedef struct b200moe_planner_receipt {
    uint64_t active_bytes, hit_bytes, promoted_bytes, promotions, evictions, steps;
} b200moe_planner_receipt;
int b200moe_planner_create(const b200moe_planner_desc* desc, void** planner);
void b200moe_planner_destroy(void* planner);
int b200moe_planner_seed(void* planner, uint32_t layer, const uint32_t* counts);               /* counts [experts] */
int b200moe_planner_observe(void* planner, uint32_t layer, const uint32_t* ids, uint32_t n);  /* one step's ids, duplicates allowed */
int b200moe_planner_end_step(void* planner);
/* moves [capacity] <- the step's moves, *count <- how many there are (more than capacity: enlarge the array and call again). */
int b200moe_planner_plan(const void* planner, b200moe_move* moves, uint32_t capacity, uint32_t* count);
int b200moe_planner_commit(void* planner, const b200moe_move* move);
int b200moe_planner_fill_from_seed(void* planner);
int b200moe_planner_table(const void* planner, uint32_t layer, int32_t* table);   /* [experts]: slot or -1 */
int b200moe_planner_scores(const void* planner, uint32_t layer, double* scores);  /* [experts] */
int b200moe_planner_get_receipt(const void* planner, b200moe_planner_receipt* out);
/* Applies planner moves of ONE layer to its residency object: copies each move's expert from host memory into the slot on
 * `stream` (a stream of the caller's choice - a side stream keeps the copies off the compute stream; the caller orders it
 * before the next b200moe_residency_map, e.g. with an event) and updates the residency's table. Moves whose slot holds an
 * expert other than `evict`, or whose expert is already resident, are refused before anything is copied. */
int b200moe_residency_promote(void* residency, const b200moe_move* moves, uint32_t count, void* stream);

/* ------------------------------------------------------------------------------------------------ the launch-record seam
 * The reference dispatches its weight kernels through a registry of {schema, revision, sizeof, alignof, launch} rows and a
 * checked, typed launch-record envelope instead of an untyped pointer (strix::weight::KernelArguments and
 * strix::weight::enqueue, include/strix/weight/resolve.hpp:67-76; Registration / enqueue_registered,
 * src/cuda/weight/registry.hpp:53-65). The same seam over this library's sites: b200moe_registry lists one row per
 * enqueue entry point, b200moe_enqueue takes an envelope, checks it against the row (known schema, this ABI revision,
 * bytes == sizeof of the site's view, data aligned for it) before anything is touched, and forwards to the site. */
enum {
    B200MOE_SITE_QUANTIZE_A8 = 1, B200MOE_SITE_RMSNORM_A8 = 2, B200MOE_SITE_Q8_0_A8 = 3, B200MOE_SITE_ROUTER = 4,
    B200MOE_SITE_ROUTES = 5, B200MOE_SITE_ROUTES_STATIC = 6, B200MOE_SITE_GATE_UP = 7, B200MOE_SITE_DOWN = 8,
    B200MOE_SITE_COMBINE = 9, B200MOE_SITE_LAYER = 10, B200MOE_SITE_FFN = 11, B200MOE_SITE_DENSE_FFN = 12
};
typedef struct b200moe_kernel_arguments {
    uint32_t schema;        /* B200MOE_SITE_* */
    uint32_t abi_revision;  /* B200MOE_ABI_VERSION the caller was compiled against */
    const void* data;       /* the site's view */
    uint64_t bytes;         /* sizeof of that view in the caller's build */
} b200moe_kernel_arguments;
typedef struct b200moe_registration {
    uint32_t schema, revision;
    uint64_t bytes, alignment;  /* sizeof / alignof of the site's view in this build */
    const char* name;           /* the entry point's name */
} b200moe_registration;
/* Rows of the registry (static storage); returns how many. */
uint32_t b200moe_registry(const b200moe_registration** rows);
int b200moe_enqueue(const b200moe_kernel_arguments* arguments, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H */
