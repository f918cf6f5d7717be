"""Operator-level host wrappers: one function per entry point of the C ABI, taking torch CUDA tensors.

Names follow the reference's operator layer (enqueue_quantize_a8, enqueue_q8_0_a8, enqueue_router, enqueue_moe_routes,
enqueue_routed_gate_up / _down, enqueue_moe_combine, enqueue_moe_layer: include/strix/cuda/ds41_core.hpp,
include/strix/cuda/ds41_moe.hpp). Every call only enqueues on the current torch stream.
"""
import ctypes as C
import math

import torch

from . import (A8Rows, CombineView, DenseView, DownView, ExpertWeights, FfnView, GateUpView, LayerView, Q8A8View,
               QuantizeA8View, RoutePolicy, RouterView, Routes, RoutesView, Shape, a8_rows, check, lib, ptr, stream_ptr,
               COMBINE_FMA_SLOTS, COMBINE_PARTS, TYPE_Q4_K, TYPE_Q8_0)


def _dev(t):
    return t.device if t is not None else torch.device("cuda")


def enqueue_quantize_a8(x, status=None, stride=0):
    """x [rows][width] float32 or bfloat16 -> (codes int8, deltas float32, sums int32)."""
    rows, width = x.shape
    st = stride or width
    codes = torch.empty((rows, st), dtype=torch.int8, device=x.device)
    deltas = torch.empty((rows, st // 32 if st % 32 == 0 else 1), dtype=torch.float32, device=x.device)
    sums = torch.empty_like(deltas, dtype=torch.int32)
    v = QuantizeA8View(ptr(x), rows, width, x.stride(0), int(x.dtype == torch.bfloat16),
                       A8Rows(ptr(codes), ptr(deltas), ptr(sums), rows, width, st), ptr(status))
    check(lib().b200moe_quantize_a8(C.byref(v), stream_ptr()))
    return codes, deltas, sums


def enqueue_rmsnorm_a8(x, weight=None, eps=1e-6, want_out=True, want_a8=True, status=None):
    """x [rows][n] float32 -> (y float32 or None, (codes, deltas, sums) or None): RMSNorm and the A8 of its output in one launch."""
    from . import RmsnormView
    rows, n = x.shape
    y = torch.empty((rows, n), dtype=torch.float32, device=x.device) if want_out else None
    a8, rows_view = None, A8Rows()
    if want_a8:
        codes = torch.empty((rows, n), dtype=torch.int8, device=x.device)
        deltas = torch.empty((rows, max(n // 32, 1)), dtype=torch.float32, device=x.device)
        sums = torch.empty_like(deltas, dtype=torch.int32)
        a8, rows_view = (codes, deltas, sums), A8Rows(ptr(codes), ptr(deltas), ptr(sums), rows, n, n)
    v = RmsnormView(ptr(x), rows, n, x.stride(0), ptr(weight), eps, ptr(y), 0, rows_view, ptr(status))
    check(lib().b200moe_rmsnorm_a8(C.byref(v), stream_ptr()))
    return y, a8


def enqueue_q8_0_a8(weight, width, codes, deltas, out=None, accumulate=False, first=0, count=None):
    """weight uint8 [n][row_bytes] Q8_0 rows; A8 rows (codes, deltas) -> out [rows][count]."""
    n, row_bytes = weight.shape
    count = n - first if count is None else count
    rows = codes.shape[0]
    if out is None:
        out = torch.zeros((rows, count), dtype=torch.float32, device=weight.device)
    v = Q8A8View(ptr(weight), row_bytes, width, first, count, A8Rows(ptr(codes), ptr(deltas), None, rows, width, codes.shape[1]),
                 ptr(out), out.stride(0), int(accumulate))
    check(lib().b200moe_q8_0_a8(C.byref(v), stream_ptr()))
    return out


def enqueue_router(policy, x=None, weight=None, logits=None, logit_bias=None, bias=None):
    """Returns (logits, scores, ids, weights). Either x and weight, or logits."""
    if x is not None:
        rows, hidden = x.shape
        logits = torch.empty((rows, policy.experts), dtype=torch.float32, device=x.device)
    else:
        rows, hidden = logits.shape[0], 0
    dev = logits.device
    scores = torch.empty_like(logits)
    ids = torch.empty((rows, policy.top_k), dtype=torch.int32, device=dev)
    wts = torch.empty((rows, policy.top_k), dtype=torch.float32, device=dev)
    v = RouterView(ptr(x), x.stride(0) if x is not None else 0, rows, hidden, ptr(weight), ptr(logit_bias), ptr(bias), policy,
                   ptr(logits), ptr(scores), ptr(ids), ptr(wts))
    check(lib().b200moe_router(C.byref(v), stream_ptr()))
    return logits, scores, ids, wts


class MoeRoutes:
    """Device arrays of one window's routes (include/b200moe.h b200moe_routes)."""

    def __init__(self, rows, top_k, experts, device):
        n = rows * top_k
        z = lambda k: torch.zeros(k, dtype=torch.int32, device=device)
        self.experts, self.begins, self.rows, self.slots, self.order = z(n), z(n + 1), z(n), z(n), z(n)
        self.low_counts, self.counts = z(rows), z(4)
        self.scratch = z(int(lib().b200moe_routes_scratch_words(rows, top_k, experts)))

    def struct(self):
        return Routes(ptr(self.experts), ptr(self.begins), ptr(self.rows), ptr(self.slots), ptr(self.order),
                      ptr(self.low_counts), ptr(self.counts))


def enqueue_moe_routes(ids, experts, split, first=0, end=0, base=0, row_status=None):
    rows, top_k = ids.shape
    r = MoeRoutes(rows, top_k, experts, ids.device)
    v = RoutesView(ptr(ids), rows, top_k, experts, split, first, end, base, ptr(r.scratch), ptr(row_status), r.struct())
    check(lib().b200moe_build_routes(C.byref(v), stream_ptr()))
    return r


def enqueue_moe_routes_static(ids, experts, split, first=0, end=0, base=0, row_status=None, out=None):
    """b200moe_build_routes_static: the same routes with the library's built-in scratch (no scratch argument)."""
    rows, top_k = ids.shape
    r = out if out is not None else MoeRoutes(rows, top_k, experts, ids.device)
    v = RoutesView(ptr(ids), rows, top_k, experts, split, first, end, base, None, ptr(row_status), r.struct())
    check(lib().b200moe_build_routes_static(C.byref(v), stream_ptr()))
    return r


def enqueue_routed_gate_up(shape, gate, up, routes, max_union, x, slots, taps=False, row_status=None, summary=None):
    """x = (codes, deltas, sums) of the MoE input; returns act = (codes, deltas, sums) [slots][inter] (+ gate, up taps)."""
    dev = gate.device
    act = (torch.zeros((slots, shape.inter), dtype=torch.int8, device=dev),
           torch.zeros((slots, shape.inter // 32), dtype=torch.float32, device=dev),
           torch.zeros((slots, shape.inter // 32), dtype=torch.int32, device=dev))
    g = torch.zeros((slots, shape.inter), dtype=torch.float32, device=dev) if taps else None
    u = torch.zeros_like(g) if taps else None
    v = GateUpView(shape, ExpertWeights(ptr(gate), ptr(up), None), routes.struct(), max_union, a8_rows(*x), a8_rows(*act),
                   ptr(g), ptr(u), ptr(row_status), ptr(summary))
    check(lib().b200moe_gate_up(C.byref(v), stream_ptr()))
    return (act, g, u) if taps else act


def enqueue_routed_down(shape, down, routes, max_union, act, raw=None, summary=None):
    slots = act[0].shape[0]
    if raw is None:
        raw = torch.zeros((slots, shape.hidden), dtype=torch.float32, device=down.device)
    v = DownView(shape, ExpertWeights(None, None, ptr(down)), routes.struct(), max_union, a8_rows(*act), ptr(raw), ptr(summary))
    check(lib().b200moe_down(C.byref(v), stream_ptr()))
    return raw


def enqueue_moe_combine(form, raw, weights, ids, order=None, shared=None, parts=2, part_experts=1, only_part=-1, bf16=False,
                        row_status=None, summary=None, fill=0.0):
    rows, top_k = ids.shape
    hidden = raw.shape[1]
    y = torch.full((rows, hidden), fill, dtype=torch.float32, device=raw.device)
    yb = torch.zeros((rows, hidden), dtype=torch.bfloat16, device=raw.device) if bf16 else None
    v = CombineView(ptr(raw), ptr(shared), ptr(weights), ptr(ids), ptr(order), rows, top_k, hidden, form, parts, part_experts,
                    only_part, ptr(y), ptr(yb), ptr(row_status), None, 0, ptr(summary))
    check(lib().b200moe_combine(C.byref(v), stream_ptr()))
    return (y, yb) if bf16 else y


class MoeLayer:
    """The routed experts of one layer: weights resident on the device, caller-style workspace held here.

    Mirrors enqueue_moe_layer(MoeLayerView) (include/strix/cuda/ds41_moe.hpp:139-156)."""

    def __init__(self, shape, gate, up, down, capacity, combine_form, parts=2, part_experts=None, grouped_min_rows=0):
        self.shape, self.gate, self.up, self.down, self.capacity = shape, gate, up, down, capacity
        self.combine_form, self.parts = combine_form, parts
        self.part_experts = part_experts if part_experts is not None else max(1, shape.experts // parts)
        self.grouped_min_rows = grouped_min_rows
        self.ws_bytes = int(lib().b200moe_layer_workspace_bytes(C.byref(shape), capacity))
        if self.ws_bytes == 0:
            check(lib().b200moe_layer(C.byref(LayerView(shape=shape)), None))  # surfaces the shape error
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=gate.device)

    def __call__(self, x_a8, ids, route_weights, shared=None, first=0, end=0, base=0, only_part=-1, want_raw=False, bf16=False,
                 row_status=None, combine=True, y_blocks=None, y_block_rows=0):
        """y_blocks: int64 device tensor of destination pointers (one per block of y_block_rows rows): the combine writes
        there (peer buffers under expert parallelism) and no y is returned."""
        rows = ids.shape[0]
        dev = self.gate.device
        y = torch.zeros((rows, self.shape.hidden), dtype=torch.float32, device=dev) if combine and y_blocks is None else None
        yb = torch.zeros((rows, self.shape.hidden), dtype=torch.bfloat16, device=dev) if bf16 else None
        raw = torch.zeros((rows * self.shape.top_k, self.shape.hidden), dtype=torch.float32, device=dev) if want_raw else None
        v = LayerView(self.shape, ExpertWeights(ptr(self.gate), ptr(self.up), ptr(self.down)), rows, a8_rows(*x_a8), ptr(ids),
                      ptr(route_weights), ptr(shared), first, end, base, self.combine_form, self.parts, self.part_experts, only_part,
                      ptr(raw), ptr(y), ptr(yb), ptr(row_status), ptr(self.ws), self.ws_bytes, self.capacity, self.grouped_min_rows, None,
                      ptr(y_blocks), y_block_rows)
        check(lib().b200moe_layer(C.byref(v), stream_ptr()))
        out = [y]
        if want_raw:
            out.append(raw)
        if bf16:
            out.append(yb)
        return out[0] if len(out) == 1 else tuple(out)


class MoeFfn:
    """Router + A8 + routed experts + combine of one layer from FP32 activations (b200moe_ffn / b200moe_ffn_host)."""

    def __init__(self, shape, policy, gate, up, down, router_weight, capacity, combine_form, parts=2, part_experts=None,
                 logit_bias=None, select_bias=None, grouped_min_rows=0):
        self.shape, self.policy, self.capacity = shape, policy, capacity
        self.gate, self.up, self.down, self.router_weight = gate, up, down, router_weight
        self.logit_bias, self.select_bias = logit_bias, select_bias
        self.combine_form, self.parts = combine_form, parts
        self.part_experts = part_experts if part_experts is not None else max(1, shape.experts // parts)
        self.grouped_min_rows = grouped_min_rows
        self.ws_bytes = int(lib().b200moe_ffn_workspace_bytes(C.byref(shape), capacity))
        if self.ws_bytes == 0:
            check(lib().b200moe_ffn(C.byref(FfnView(shape=shape, policy=policy)), None))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=gate.device)

    @staticmethod
    def stage_events(handles):
        """Eight cudaEvent_t values (ints or None) as the array the views point to; the caller keeps it alive."""
        return (C.c_void_p * 8)(*handles)

    def _view(self, rows, x, y, ids=None, wts=None, shared=None, row_status=None, events=None, summary=None, x_is_bf16=None):
        ev = C.cast(events, C.c_void_p) if events is not None else None
        if x_is_bf16 is None:
            x_is_bf16 = x is not None and x.dtype == torch.bfloat16
        return FfnView(self.shape, ExpertWeights(ptr(self.gate), ptr(self.up), ptr(self.down)), self.policy, ptr(self.router_weight),
                       ptr(self.logit_bias), ptr(self.select_bias), ptr(x), int(x_is_bf16), rows, ptr(shared), self.combine_form, self.parts,
                       self.part_experts, ptr(y), None, ptr(ids), ptr(wts), ptr(row_status), ptr(self.ws), self.ws_bytes,
                       self.capacity, self.grouped_min_rows, ev, ptr(summary))

    def __call__(self, x, y=None, shared=None, want_routes=False, row_status=None, summary=None):
        """x: [rows][hidden] float32 or bfloat16 (widened exactly before the router and the A8 quantiser)."""
        rows = x.shape[0]
        if y is None:
            y = torch.empty((rows, self.shape.hidden), dtype=torch.float32, device=x.device)
        ids = torch.empty((rows, self.shape.top_k), dtype=torch.int32, device=x.device) if want_routes else None
        wts = torch.empty((rows, self.shape.top_k), dtype=torch.float32, device=x.device) if want_routes else None
        v = self._view(rows, x, y, ids, wts, shared, row_status, summary=summary)
        check(lib().b200moe_ffn(C.byref(v), stream_ptr()))
        return (y, ids, wts) if want_routes else y

    def host(self, x_host, y_host):
        """x_host / y_host: pinned host tensors; copies in, runs, copies out and waits (the end-to-end call)."""
        v = self._view(x_host.shape[0], None, None, x_is_bf16=x_host.dtype == torch.bfloat16)
        check(lib().b200moe_ffn_host(C.byref(v), x_host.data_ptr(), y_host.data_ptr(), stream_ptr()))
        return y_host


def enqueue_dense_ffn(shape, gate, up, down, x_a8, bf16=False):
    rows = x_a8[0].shape[0]
    dev = gate.device
    ws_bytes = int(lib().b200moe_layer_workspace_bytes(C.byref(shape), rows))
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev)
    y = torch.zeros((rows, shape.hidden), dtype=torch.float32, device=dev)
    yb = torch.zeros((rows, shape.hidden), dtype=torch.bfloat16, device=dev) if bf16 else None
    v = DenseView(shape, ExpertWeights(ptr(gate), ptr(up), ptr(down)), rows, a8_rows(*x_a8), ptr(y), ptr(yb), ptr(ws), ws_bytes)
    check(lib().b200moe_dense_ffn(C.byref(v), stream_ptr()))
    return (y, yb) if bf16 else y


def make_shape(hidden, inter, experts, top_k, gate_type, down_type, limit=math.inf):
    return Shape(hidden, inter, experts, top_k, gate_type, down_type, limit)


def softmax_policy(experts, top_k):
    return RoutePolicy(0, 0, 0, 0, experts, top_k, 1, 1, 1, 1, 1e-20, 1.0)


def sigmoid_group_policy(experts, top_k, n_group, topk_group, scale=1.0):
    return RoutePolicy(1, 1, 0, 0, experts, top_k, n_group, topk_group, 1, 1, 1e-20, scale)
