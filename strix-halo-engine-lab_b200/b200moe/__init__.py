"""Host-side Python binding of the B200 MoE FFN library: ctypes over the C ABI of include/b200moe.h.

The structures below mirror the header field for field; device memory and streams come from torch (plumbing only).
There is no CPU path here: loading fails loudly when libb200moe.so has not been built, and every compute call fails
with B200MoeError when no sm_100 device is usable.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB_PATH = os.path.join(PKG, "libb200moe.so")

OK, ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_COMM, ERR_ABORTED = range(7)
TYPE_Q8_0, TYPE_Q4_K = 8, 12
ROW_INVALID_ROUTE, ROW_NONFINITE_ACTIVATION, ROW_INVALID_DELTA, ROW_PROJECTION_NONFINITE = 1, 2, 4, 8
JOB_WAIT_ABORTED = 0x40000000
DEBUG_WAIT_LIMIT, DEBUG_STALL_STAGE, DEBUG_DECODE_FORM = 0, 1, 2
FORM_AUTO, FORM_ROW_STREAM, FORM_SEGMENT_STREAM, FORM_PER_BLOCK, FORM_TENSOR = 0, 1, 2, 3, 4
SCORE_SOFTMAX, SCORE_SIGMOID, SCORE_SQRT_SOFTPLUS = 0, 1, 2
KEY_FLOAT_SERIAL, KEY_ORDERED_BITS = 0, 1
ORDER_SELECTION, ORDER_ASCENDING_ID = 0, 1
COMBINE_PARTS, COMBINE_FMA_SLOTS = 0, 1

u32, i32, u64, f32, vp = C.c_uint32, C.c_int32, C.c_uint64, C.c_float, C.c_void_p


class B200MoeError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"b200moe status {code}: {text}")
        self.code = code


class InvalidArgument(B200MoeError, ValueError):
    """The reference's std::invalid_argument: raised before anything was written or launched."""


class A8Rows(C.Structure):
    _fields_ = [("codes", vp), ("deltas", vp), ("sums", vp), ("rows", u32), ("width", u32), ("stride", u32)]


class QuantizeA8View(C.Structure):
    _fields_ = [("x", vp), ("rows", u32), ("width", u32), ("x_stride", u32), ("x_is_bf16", u32), ("out", A8Rows), ("status", vp)]


class RmsnormView(C.Structure):
    _fields_ = [("x", vp), ("rows", u32), ("n", u32), ("x_stride", u32), ("weight", vp), ("eps", C.c_float), ("out", vp),
                ("out_stride", u32), ("a8", A8Rows), ("status", vp)]


class Q8A8View(C.Structure):
    _fields_ = [("weight", vp), ("row_bytes", u32), ("width", u32), ("first", u32), ("count", u32), ("x", A8Rows), ("out", vp),
                ("out_stride", u32), ("accumulate", u32)]


class RoutePolicy(C.Structure):
    _fields_ = [("score", u32), ("selection_bias", u32), ("key", u32), ("order", u32), ("experts", u32), ("top_k", u32),
                ("n_group", u32), ("topk_group", u32), ("renormalize", u32), ("renorm_single", u32), ("renorm_eps", f32),
                ("scale", f32)]


class RouterView(C.Structure):
    _fields_ = [("x", vp), ("x_stride", u32), ("rows", u32), ("hidden", u32), ("weight", vp), ("logit_bias", vp), ("bias", vp),
                ("policy", RoutePolicy), ("logits", vp), ("scores", vp), ("ids", vp), ("weights", vp)]


class Routes(C.Structure):
    _fields_ = [("experts", vp), ("begins", vp), ("rows", vp), ("slots", vp), ("order", vp), ("low_counts", vp), ("counts", vp)]


class RoutesView(C.Structure):
    _fields_ = [("ids", vp), ("rows", u32), ("top_k", u32), ("experts", u32), ("split", u32), ("first", u32), ("end", u32),
                ("base", u32), ("scratch", vp), ("row_status", vp), ("out", Routes)]


class Shape(C.Structure):
    _fields_ = [("hidden", u32), ("inter", u32), ("experts", u32), ("top_k", u32), ("gate_type", u32), ("down_type", u32),
                ("limit", f32)]


class ExpertWeights(C.Structure):
    _fields_ = [("gate", vp), ("up", vp), ("down", vp)]


class GateUpView(C.Structure):
    _fields_ = [("shape", Shape), ("weights", ExpertWeights), ("routes", Routes), ("max_union", u32), ("x", A8Rows), ("act", A8Rows),
                ("gate_out", vp), ("up_out", vp), ("row_status", vp), ("summary", vp)]


class DownView(C.Structure):
    _fields_ = [("shape", Shape), ("weights", ExpertWeights), ("routes", Routes), ("max_union", u32), ("act", A8Rows), ("raw", vp),
                ("summary", vp)]


class CombineView(C.Structure):
    _fields_ = [("raw", vp), ("shared", vp), ("weights", vp), ("ids", vp), ("order", vp), ("rows", u32), ("top_k", u32),
                ("hidden", u32), ("form", u32), ("parts", u32), ("part_experts", u32), ("only_part", i32), ("y", vp),
                ("y_bf16", vp), ("row_status", vp), ("y_blocks", vp), ("y_block_rows", u32), ("summary", vp), ("only_part_count", u32),
                ("part_stride", u64), ("low_counts", vp)]


class LayerView(C.Structure):
    _fields_ = [("shape", Shape), ("weights", ExpertWeights), ("rows", u32), ("x", A8Rows), ("ids", vp), ("route_weights", vp),
                ("shared", vp), ("first", u32), ("end", u32), ("base", u32), ("combine_form", u32), ("parts", u32),
                ("part_experts", u32), ("only_part", i32), ("raw", vp), ("y", vp), ("y_bf16", vp), ("row_status", vp),
                ("workspace", vp), ("workspace_bytes", u64), ("capacity", u32), ("grouped_min_rows", u32), ("stage_events", vp),
                ("y_blocks", vp), ("y_block_rows", u32), ("summary", vp), ("only_part_count", u32), ("part_stride", u64)]


class FfnView(C.Structure):
    _fields_ = [("shape", Shape), ("weights", ExpertWeights), ("policy", RoutePolicy), ("router_weight", vp), ("logit_bias", vp),
                ("select_bias", vp), ("x", vp), ("x_is_bf16", u32), ("rows", u32), ("shared", vp), ("combine_form", u32),
                ("parts", u32), ("part_experts", u32), ("y", vp), ("y_bf16", vp), ("ids", vp), ("route_weights", vp),
                ("row_status", vp), ("workspace", vp), ("workspace_bytes", u64), ("capacity", u32), ("grouped_min_rows", u32),
                ("stage_events", vp), ("summary", vp)]


class EpDesc(C.Structure):
    _fields_ = [("shape", Shape), ("policy", RoutePolicy), ("world", u32), ("rank", u32), ("rows_per_rank", u32), ("wait_polls", u32),
                ("fold_parts", u32), ("windows", vp)]


class EpStepView(C.Structure):
    _fields_ = [("weights", ExpertWeights), ("router_weight", vp), ("logit_bias", vp), ("select_bias", vp), ("x", vp), ("x_is_bf16", u32),
                ("rows", u32), ("shared", vp), ("y", vp), ("y_bf16", vp), ("summary", vp), ("workspace", vp), ("workspace_bytes", u64),
                ("grouped_min_rows", u32), ("stage_events", vp)]


class TpDesc(C.Structure):
    _fields_ = [("shape", Shape), ("world", u32), ("rank", u32), ("rows", u32), ("payload_bf16", u32), ("wait_polls", u32), ("windows", vp)]


class TpStepView(C.Structure):
    _fields_ = [("weights", ExpertWeights), ("rows", u32), ("x", A8Rows), ("y", vp), ("y_bf16", vp), ("summary", vp), ("workspace", vp),
                ("workspace_bytes", u64)]


class DenseView(C.Structure):
    _fields_ = [("shape", Shape), ("weights", ExpertWeights), ("rows", u32), ("x", A8Rows), ("y", vp), ("y_bf16", vp),
                ("workspace", vp), ("workspace_bytes", u64)]


class GgufTensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", u32), ("dims", u64 * 4), ("ggml_type", u32), ("offset", u64), ("bytes", u64)]


class GgufMoeLayer(C.Structure):
    _fields_ = [("gate", GgufTensorInfo), ("up", GgufTensorInfo), ("down", GgufTensorInfo), ("router", GgufTensorInfo), ("shape", Shape)]


class ResidencyDesc(C.Structure):
    _fields_ = [("shape", Shape), ("gate_host", vp), ("up_host", vp), ("down_host", vp), ("slots", u32), ("gate_slots", vp),
                ("up_slots", vp), ("down_slots", vp), ("decay", f32)]


class ResidencyStats(C.Structure):
    _fields_ = [("windows", u64), ("hits", u64), ("misses", u64), ("evictions", u64), ("bytes_loaded", u64)]


ABI_VERSION = 4  # B200MOE_ABI_VERSION of include/b200moe.h: the layout of the views mirrored above

# every symbol include/b200moe.h declares (tests check that the library exports each of them)
class PlannerDesc(C.Structure):
    _fields_ = [("layers", u32), ("experts", u32), ("top_k", u32), ("slots", u32), ("expert_bytes", vp), ("decay", C.c_double),
                ("margin_reuses", C.c_double), ("upload_bytes_per_step", u64)]


class Move(C.Structure):
    _fields_ = [("layer", u32), ("slot", u32), ("evict", u32), ("expert", u32)]


class PlannerReceipt(C.Structure):
    _fields_ = [("active_bytes", u64), ("hit_bytes", u64), ("promoted_bytes", u64), ("promotions", u64), ("evictions", u64), ("steps", u64)]


MOVE_NO_EVICTION = 0xFFFFFFFF


class FirstError(C.Structure):
    """strix::DeferredMoeFirstError: {domain, bits}."""
    _fields_ = [("domain", u32), ("bits", u32)]


DOMAIN_NONE, DOMAIN_LEGACY, DOMAIN_Q4K_A8 = 0, 1, 2


class KernelArguments(C.Structure):
    """The checked launch-record envelope (b200moe_kernel_arguments)."""
    _fields_ = [("schema", u32), ("abi_revision", u32), ("data", vp), ("bytes", u64)]


class Registration(C.Structure):
    _fields_ = [("schema", u32), ("revision", u32), ("bytes", u64), ("alignment", u64), ("name", C.c_char_p)]


(SITE_QUANTIZE_A8, SITE_RMSNORM_A8, SITE_Q8_0_A8, SITE_ROUTER, SITE_ROUTES, SITE_ROUTES_STATIC, SITE_GATE_UP, SITE_DOWN, SITE_COMBINE,
 SITE_LAYER, SITE_FFN, SITE_DENSE_FFN) = range(1, 13)


def registry():
    """The library's registry rows as {schema: Registration}."""
    rows = C.POINTER(Registration)()
    n = lib().b200moe_registry(C.byref(rows))
    return {rows[i].schema: rows[i] for i in range(n)}


def enqueue(schema, view, stream=None, abi_revision=None, nbytes=None):
    """A site through the launch-record seam: the view travels as a typed, size-checked envelope."""
    a = KernelArguments(schema, ABI_VERSION if abi_revision is None else abi_revision, C.cast(C.pointer(view), C.c_void_p),
                        C.sizeof(view) if nbytes is None else nbytes)
    return lib().b200moe_enqueue(C.byref(a), stream)


EXPORTS = ["b200moe_abi_version", "b200moe_last_error", "b200moe_launch_count", "b200moe_debug_set", "b200moe_quantize_a8", "b200moe_rmsnorm_a8", "b200moe_q8_0_a8",
           "b200moe_router", "b200moe_routes_scratch_words", "b200moe_build_routes", "b200moe_routes_static_max_words",
           "b200moe_build_routes_static", "b200moe_gate_row_bytes",
           "b200moe_down_row_bytes", "b200moe_expert_bytes", "b200moe_gate_up", "b200moe_down", "b200moe_combine",
           "b200moe_canonical_sum", "b200moe_fold_parts", "b200moe_select_owner_slots", "b200moe_peer_buffer_create",
           "b200moe_peer_buffer_open", "b200moe_peer_buffer_close", "b200moe_peer_buffer_destroy",
           "b200moe_tp_window_bytes", "b200moe_tp_create", "b200moe_tp_destroy", "b200moe_tp_workspace_bytes", "b200moe_tp_dense",
           "b200moe_ep_window_bytes", "b200moe_ep_create", "b200moe_ep_destroy", "b200moe_ep_workspace_bytes", "b200moe_ep_ffn", "b200moe_layer_workspace_bytes", "b200moe_layer", "b200moe_ffn_workspace_bytes",
           "b200moe_ffn", "b200moe_ffn_host", "b200moe_dense_ffn", "b200moe_gguf_open", "b200moe_gguf_close",
           "b200moe_residency_create", "b200moe_residency_destroy", "b200moe_residency_map",
           "b200moe_residency_get_stats", "b200moe_residency_table", "b200moe_residency_choose_victims",
           "b200moe_gguf_tensor_count", "b200moe_gguf_data_offset", "b200moe_gguf_alignment", "b200moe_gguf_tensor_at", "b200moe_gguf_find",
           "b200moe_gguf_find_moe_layer", "b200moe_registry", "b200moe_enqueue",
           "b200moe_planner_create", "b200moe_planner_destroy", "b200moe_planner_seed", "b200moe_planner_observe", "b200moe_planner_end_step",
           "b200moe_planner_plan", "b200moe_planner_commit", "b200moe_planner_fill_from_seed", "b200moe_planner_table", "b200moe_planner_scores",
           "b200moe_planner_get_receipt", "b200moe_residency_promote", "b200moe_merge_first_error", "b200moe_check_first_error"]

_lib = None


def lib():
    """The loaded C library. Raises when it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it first (python -c 'import __graft_entry__ as g; g.build()')")
        L = C.CDLL(LIB_PATH)
        L.b200moe_last_error.restype = C.c_char_p
        L.b200moe_launch_count.restype = u64
        L.b200moe_debug_set.restype = C.c_int
        L.b200moe_debug_set.argtypes = [u32, u32]
        for n in ("b200moe_gate_row_bytes", "b200moe_down_row_bytes", "b200moe_expert_bytes"):
            getattr(L, n).restype = u64
            getattr(L, n).argtypes = [C.POINTER(Shape)]
        L.b200moe_routes_static_max_words.restype = u64
        L.b200moe_routes_static_max_words.argtypes = []
        L.b200moe_routes_scratch_words.restype = u64
        L.b200moe_routes_scratch_words.argtypes = [u32, u32, u32]
        for n in ("b200moe_layer_workspace_bytes", "b200moe_ffn_workspace_bytes"):
            getattr(L, n).restype = u64
            getattr(L, n).argtypes = [C.POINTER(Shape), u32]
        for n, t in (("b200moe_quantize_a8", QuantizeA8View), ("b200moe_rmsnorm_a8", RmsnormView), ("b200moe_q8_0_a8", Q8A8View), ("b200moe_router", RouterView),
                     ("b200moe_build_routes", RoutesView), ("b200moe_build_routes_static", RoutesView),
                     ("b200moe_gate_up", GateUpView), ("b200moe_down", DownView),
                     ("b200moe_combine", CombineView), ("b200moe_layer", LayerView), ("b200moe_ffn", FfnView),
                     ("b200moe_dense_ffn", DenseView)):
            getattr(L, n).restype = C.c_int
            getattr(L, n).argtypes = [C.POINTER(t), vp]
        L.b200moe_ffn_host.restype = C.c_int
        L.b200moe_ffn_host.argtypes = [C.POINTER(FfnView), vp, vp, vp]
        L.b200moe_gguf_open.restype = C.c_int
        L.b200moe_gguf_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        L.b200moe_gguf_close.restype = None
        L.b200moe_gguf_close.argtypes = [vp]
        for n in ("b200moe_gguf_tensor_count", "b200moe_gguf_data_offset", "b200moe_gguf_alignment"):
            getattr(L, n).restype = u64
            getattr(L, n).argtypes = [vp]
        L.b200moe_gguf_tensor_at.restype = C.c_int
        L.b200moe_gguf_tensor_at.argtypes = [vp, u64, C.POINTER(GgufTensorInfo)]
        L.b200moe_gguf_find.restype = C.c_int
        L.b200moe_gguf_find.argtypes = [vp, C.c_char_p, C.POINTER(GgufTensorInfo)]
        L.b200moe_gguf_find_moe_layer.restype = C.c_int
        L.b200moe_gguf_find_moe_layer.argtypes = [vp, u32, C.POINTER(GgufMoeLayer)]
        L.b200moe_residency_create.restype = C.c_int
        L.b200moe_residency_create.argtypes = [C.POINTER(ResidencyDesc), C.POINTER(vp)]
        L.b200moe_residency_destroy.restype = None
        L.b200moe_residency_destroy.argtypes = [vp]
        L.b200moe_residency_map.restype = C.c_int
        L.b200moe_residency_map.argtypes = [vp, vp, u32, vp, vp]
        L.b200moe_residency_get_stats.restype = C.c_int
        L.b200moe_residency_get_stats.argtypes = [vp, C.POINTER(ResidencyStats)]
        L.b200moe_residency_table.restype = C.c_int
        L.b200moe_residency_table.argtypes = [vp, vp]
        L.b200moe_residency_choose_victims.restype = C.c_int
        L.b200moe_residency_choose_victims.argtypes = [vp, u32, vp, vp, u32, vp, u32, vp]
        L.b200moe_peer_buffer_create.restype = C.c_int
        L.b200moe_peer_buffer_create.argtypes = [u64, C.POINTER(vp), vp]
        L.b200moe_peer_buffer_open.restype = C.c_int
        L.b200moe_peer_buffer_open.argtypes = [vp, C.POINTER(vp)]
        for n in ("b200moe_peer_buffer_close", "b200moe_peer_buffer_destroy"):
            getattr(L, n).restype = C.c_int
            getattr(L, n).argtypes = [vp]
        L.b200moe_ep_window_bytes.restype = u64
        L.b200moe_ep_window_bytes.argtypes = [C.POINTER(Shape), u32, u32, u32]
        L.b200moe_ep_create.restype = C.c_int
        L.b200moe_ep_create.argtypes = [C.POINTER(EpDesc), C.POINTER(vp)]
        L.b200moe_ep_destroy.restype = None
        L.b200moe_ep_destroy.argtypes = [vp]
        L.b200moe_ep_workspace_bytes.restype = u64
        L.b200moe_ep_workspace_bytes.argtypes = [vp]
        L.b200moe_ep_ffn.restype = C.c_int
        L.b200moe_ep_ffn.argtypes = [vp, C.POINTER(EpStepView), vp]
        L.b200moe_tp_window_bytes.restype = u64
        L.b200moe_tp_window_bytes.argtypes = [u32, u32, u32, u32]
        L.b200moe_tp_create.restype = C.c_int
        L.b200moe_tp_create.argtypes = [C.POINTER(TpDesc), C.POINTER(vp)]
        L.b200moe_tp_destroy.restype = None
        L.b200moe_tp_destroy.argtypes = [vp]
        L.b200moe_tp_workspace_bytes.restype = u64
        L.b200moe_tp_workspace_bytes.argtypes = [vp]
        L.b200moe_tp_dense.restype = C.c_int
        L.b200moe_tp_dense.argtypes = [vp, C.POINTER(TpStepView), vp]
        L.b200moe_fold_parts.restype = C.c_int
        L.b200moe_fold_parts.argtypes = [vp, u32, u64, vp, u64, vp, vp, vp]
        L.b200moe_select_owner_slots.restype = C.c_int
        L.b200moe_select_owner_slots.argtypes = [vp, u64, u32, u32, vp, u32, u32, vp, vp]
        L.b200moe_canonical_sum.restype = C.c_int
        L.b200moe_canonical_sum.argtypes = [vp, vp, vp, u64, vp, vp]
        # every pointer / handle argument is declared: an undeclared Python int would travel as a 32-bit C int
        L.b200moe_registry.restype = u32
        L.b200moe_registry.argtypes = [C.POINTER(C.POINTER(Registration))]
        L.b200moe_enqueue.restype = C.c_int
        L.b200moe_enqueue.argtypes = [C.POINTER(KernelArguments), vp]
        L.b200moe_merge_first_error.restype = C.c_int
        L.b200moe_merge_first_error.argtypes = [vp, vp, u32, vp]
        L.b200moe_check_first_error.restype = C.c_int
        L.b200moe_check_first_error.argtypes = [C.POINTER(FirstError)]
        L.b200moe_planner_create.restype = C.c_int
        L.b200moe_planner_create.argtypes = [C.POINTER(PlannerDesc), C.POINTER(vp)]
        L.b200moe_planner_destroy.restype = None
        L.b200moe_planner_destroy.argtypes = [vp]
        L.b200moe_planner_seed.restype = C.c_int
        L.b200moe_planner_seed.argtypes = [vp, u32, vp]
        L.b200moe_planner_observe.restype = C.c_int
        L.b200moe_planner_observe.argtypes = [vp, u32, vp, u32]
        for n in ("b200moe_planner_end_step", "b200moe_planner_fill_from_seed"):
            getattr(L, n).restype = C.c_int
            getattr(L, n).argtypes = [vp]
        L.b200moe_planner_plan.restype = C.c_int
        L.b200moe_planner_plan.argtypes = [vp, C.POINTER(Move), u32, C.POINTER(u32)]
        L.b200moe_planner_commit.restype = C.c_int
        L.b200moe_planner_commit.argtypes = [vp, C.POINTER(Move)]
        for n in ("b200moe_planner_table", "b200moe_planner_scores"):
            getattr(L, n).restype = C.c_int
            getattr(L, n).argtypes = [vp, u32, vp]
        L.b200moe_planner_get_receipt.restype = C.c_int
        L.b200moe_planner_get_receipt.argtypes = [vp, C.POINTER(PlannerReceipt)]
        L.b200moe_residency_promote.restype = C.c_int
        L.b200moe_residency_promote.argtypes = [vp, C.POINTER(Move), u32, vp]
        L.b200moe_abi_version.restype = C.c_int
        L.b200moe_abi_version.argtypes = []
        L.b200moe_last_error.argtypes = []
        L.b200moe_launch_count.argtypes = []
        _lib = L
    return _lib


def check(rc):
    if rc == OK:
        return
    text = lib().b200moe_last_error().decode()
    if rc == ERR_INVALID_ARGUMENT:
        raise InvalidArgument(rc, text)
    raise B200MoeError(rc, text)


def debug_set(key, value):
    """b200moe_debug_set: a process-wide test / measurement hook (DEBUG_* keys). Tests restore 0 when done."""
    check(lib().b200moe_debug_set(key, value))


def launch_count():
    return int(lib().b200moe_launch_count())


def ptr(t):
    """Device (or pinned host) address of a torch tensor; None stays NULL."""
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def a8_rows(codes, deltas, sums, rows=None, width=None, stride=0):
    return A8Rows(ptr(codes), ptr(deltas), ptr(sums), codes.shape[0] if rows is None else rows,
                  codes.shape[1] if width is None else width, stride)
