"""TEST INFRASTRUCTURE: ctypes loaders for the CPU oracle (liboracle.so, the restatement in moe_oracle.cpp) and for the
reference's own CPU code (oracle/_ref/libstrixref.so, built by oracle/Makefile from the reference checkout).

Only tests, the smoke check and the benchmark's CPU-baseline / reference arm import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libstrixref.so")

u8p = C.POINTER(C.c_uint8)
i8p = C.POINTER(C.c_int8)
u16p = C.POINTER(C.c_uint16)
u32p = C.POINTER(C.c_uint32)
i32p = C.POINTER(C.c_int32)
f32p = C.POINTER(C.c_float)


class RoutePolicy(C.Structure):
    """Layout of b200moe_route_policy (include/b200moe.h)."""
    _fields_ = [("score", C.c_uint32), ("selection_bias", C.c_uint32), ("key", C.c_uint32), ("order", C.c_uint32),
                ("experts", C.c_uint32), ("top_k", C.c_uint32), ("n_group", C.c_uint32), ("topk_group", C.c_uint32),
                ("renormalize", C.c_uint32), ("renorm_single", C.c_uint32), ("renorm_eps", C.c_float),
                ("scale", C.c_float)]

    def words(self):
        return np.array([self.score, self.selection_bias, self.key, self.order, self.experts, self.top_k, self.n_group,
                         self.topk_group, self.renormalize, self.renorm_single], dtype=np.uint32)


class Shape(C.Structure):
    """Layout of b200moe_shape (include/b200moe.h)."""
    _fields_ = [("hidden", C.c_uint32), ("inter", C.c_uint32), ("experts", C.c_uint32), ("top_k", C.c_uint32),
                ("gate_type", C.c_uint32), ("down_type", C.c_uint32), ("limit", C.c_float)]


SOFTMAX, SIGMOID, SQRT_SOFTPLUS = 0, 1, 2
FLOAT_SERIAL, ORDERED_BITS = 0, 1
SELECTION, ASCENDING_ID = 0, 1
Q8_0, Q4_K = 8, 12
COMBINE_PARTS, COMBINE_FMA_SLOTS = 0, 1


def softmax_policy(experts, top_k):
    """Configs 1-3: softmax over FP32 logits, top-k, renormalised weights (route_policy.hpp fields)."""
    return RoutePolicy(SOFTMAX, 0, FLOAT_SERIAL, SELECTION, experts, top_k, 1, 1, 1, 1, 1e-20, 1.0)


def ds41_policy(experts, top_k, scale):
    """strix::moe::preset::ds41 (include/strix/moe/route_policy.hpp:64-66)."""
    return RoutePolicy(SQRT_SOFTPLUS, 1, FLOAT_SERIAL, SELECTION, experts, top_k, 1, 1, 1, 0, 1e-20, scale)


def sigmoid_group_policy(experts, top_k, n_group, topk_group, scale=1.0):
    """Config 4: sigmoid + selection bias, group-limited top-k."""
    return RoutePolicy(SIGMOID, 1, FLOAT_SERIAL, SELECTION, experts, top_k, n_group, topk_group, 1, 1, 1e-20, scale)


def _p(a, t):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"], "array must be contiguous"
    return a.ctypes.data_as(t)


def build(ref=True):
    """Compile liboracle.so (and the reference build when its checkout is present). Idempotent (make)."""
    subprocess.run(["make", "-C", HERE, "-j8"] + ([] if ref else ["oracle"]), check=True, stdout=subprocess.DEVNULL)


class Oracle:
    """The restated contracts (oracle/moe_oracle.cpp)."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        self.lib = L = C.CDLL(ORACLE_SO)
        for n in ("orc_half_to_float",):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_uint16]
        for n in ("orc_declared_exp", "orc_declared_log1p", "orc_sqrt_softplus", "orc_gfx1151_expf"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        L.orc_swiglu_ds41.restype = C.c_float
        L.orc_swiglu_ds41.argtypes = [C.c_float] * 3
        L.orc_swiglu_qwen.restype = C.c_float
        L.orc_swiglu_qwen.argtypes = [C.c_float] * 2
        L.orc_row_q4k.restype = C.c_float
        L.orc_row_q8_chain4.restype = C.c_float

    # -- A8 -------------------------------------------------------------------------------------------------------
    def quantize_a8(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, width = x.shape
        codes = np.zeros((rows, width), np.int8)
        deltas = np.zeros((rows, width // 32), np.float32)
        sums = np.zeros((rows, width // 32), np.int32)
        rc = self.lib.orc_quantize_a8(_p(x, f32p), rows, width, 0, _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p), 0)
        if rc:
            raise ValueError("A8 width must be a multiple of 32")
        return codes, deltas, sums

    def rmsnorm(self, x, w=None, eps=1e-6):
        x = np.ascontiguousarray(x, dtype=np.float32)
        rows, n = x.shape
        y = np.zeros_like(x)
        wp = _p(np.ascontiguousarray(w, dtype=np.float32), f32p) if w is not None else None
        self.lib.orc_rmsnorm_f32(_p(x, f32p), wp, n, C.c_float(eps), _p(y, f32p), rows)
        return y

    def gemv_q8_0_a8(self, weight, width, codes, deltas, out=None, accumulate=False):
        weight = np.ascontiguousarray(weight, dtype=np.uint8)
        count, row_bytes = weight.shape
        rows = codes.shape[0]
        if out is None:
            out = np.zeros((rows, count), np.float32)
        rc = self.lib.orc_gemv_q8_0_a8(_p(weight, u8p), row_bytes, width, count, rows, _p(codes, i8p), _p(deltas, f32p),
                                       codes.shape[1], _p(out, f32p), out.shape[1], int(accumulate))
        if rc:
            raise ValueError("Q8_0 width must be a multiple of 32")
        return out

    def row_q4k(self, row, codes, deltas, sums):
        row = np.ascontiguousarray(row, dtype=np.uint8)
        return self.lib.orc_row_q4k(_p(row, u8p), C.c_uint32(row.size // 144), _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p))

    def row_q8_chain4(self, row, codes, deltas):
        row = np.ascontiguousarray(row, dtype=np.uint8)
        return self.lib.orc_row_q8_chain4(_p(row, u8p), C.c_uint32(row.size // 34), _p(codes, i8p), _p(deltas, f32p))

    # -- router ---------------------------------------------------------------------------------------------------
    def router_logits(self, x, w, logit_bias=None):
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        rows, hidden = x.shape
        experts = w.shape[0]
        out = np.zeros((rows, experts), np.float32)
        self.lib.orc_router_logits(_p(x, f32p), rows, hidden, hidden, _p(w, f32p), experts, _p(logit_bias, f32p), _p(out, f32p))
        return out

    def route_scores(self, score, logits):
        logits = np.ascontiguousarray(logits, np.float32)
        out = np.zeros_like(logits)
        for r in range(logits.shape[0]):
            self.lib.orc_route_scores(score, _p(logits[r], f32p), logits.shape[1], _p(out[r], f32p))
        return out

    def route_select(self, policy, scores, bias=None):
        scores = np.ascontiguousarray(scores, np.float32)
        rows = scores.shape[0]
        ids = np.zeros((rows, policy.top_k), np.uint32)
        w = np.zeros((rows, policy.top_k), np.float32)
        for r in range(rows):
            rc = self.lib.orc_route_select(C.byref(policy), _p(scores[r], f32p), _p(bias, f32p), _p(ids[r], u32p), _p(w[r], f32p))
            if rc:
                raise ValueError("route policy rejected")
        return ids, w

    def router(self, policy, x=None, w=None, logits=None, logit_bias=None, bias=None):
        """Returns logits, scores, ids, weights."""
        if x is not None:
            logits = self.router_logits(x, w, logit_bias)
        logits = np.ascontiguousarray(logits, np.float32)
        scores = self.route_scores(policy.score, logits)
        ids, wt = self.route_select(policy, scores, bias)
        return logits, scores, ids, wt

    # -- routes ---------------------------------------------------------------------------------------------------
    def routes(self, ids, experts, split, first=0, end=0, base=0):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, top_k = ids.shape
        n = rows * top_k
        r = {k: np.zeros(n, np.uint32) for k in ("experts", "rows", "slots", "order")}
        r["begins"] = np.zeros(n + 1, np.uint32)
        r["low_counts"] = np.zeros(rows, np.uint32)
        r["counts"] = np.zeros(4, np.uint32)
        rc = self.lib.orc_routes(_p(ids, u32p), rows, top_k, experts, split, first, end, base, _p(r["experts"], u32p),
                                 _p(r["begins"], u32p), _p(r["rows"], u32p), _p(r["slots"], u32p), _p(r["order"], u32p),
                                 _p(r["low_counts"], u32p), _p(r["counts"], u32p))
        if rc < 0:
            raise ValueError("routes: an expert repeats within a row or is out of range")
        return r

    # -- experts / combine ----------------------------------------------------------------------------------------
    def experts(self, shape, gate, up, down, ids, x_codes, x_deltas, x_sums, first=0, end=0, taps=False):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, K = ids.shape
        H, I = shape.hidden, shape.inter
        out = {"raw": np.zeros((rows * K, H), np.float32), "status": np.zeros(rows, np.uint32)}
        if taps:
            out.update(gate=np.zeros((rows * K, I), np.float32), up=np.zeros((rows * K, I), np.float32),
                       act_codes=np.zeros((rows * K, I), np.int8), act_deltas=np.zeros((rows * K, I // 32), np.float32),
                       act_sums=np.zeros((rows * K, I // 32), np.int32))
        rc = self.lib.orc_experts(C.byref(shape), _p(gate, u8p), _p(up, u8p), _p(down, u8p), _p(ids, u32p), rows,
                                  _p(x_codes, i8p), _p(x_deltas, f32p), _p(x_sums, i32p), first, end, _p(out["raw"], f32p),
                                  _p(out.get("gate"), f32p), _p(out.get("up"), f32p), _p(out.get("act_codes"), i8p),
                                  _p(out.get("act_deltas"), f32p), _p(out.get("act_sums"), i32p), _p(out["status"], u32p))
        if rc:
            raise ValueError("experts: unsupported shape / formats")
        return out

    def combine(self, form, raw, weights, ids, shared=None, parts=2, part_experts=1, only_part=-1, bf16=False):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, K = ids.shape
        H = raw.shape[1]
        y = np.zeros((rows, H), np.float32)
        yb = np.zeros((rows, H), np.uint16) if bf16 else None
        weights = np.ascontiguousarray(weights, np.float32)
        rc = self.lib.orc_combine(form, _p(raw, f32p), _p(shared, f32p), _p(weights, f32p), _p(ids, u32p), rows, K, H, parts,
                                  part_experts, only_part, _p(y, f32p), _p(yb, u16p))
        if rc:
            raise ValueError("combine: bad parts")
        return (y, yb) if bf16 else y

    def float_truth(self, shape, gate, up, down, ids, weights, x):
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.uint32)
        weights = np.ascontiguousarray(weights, np.float32)
        y = np.zeros((x.shape[0], shape.hidden), np.float32)
        self.lib.orc_float_truth(C.byref(shape), _p(gate, u8p), _p(up, u8p), _p(down, u8p), _p(ids, u32p), _p(weights, f32p),
                                 x.shape[0], _p(x, f32p), _p(y, f32p))
        return y

    def ffn(self, shape, policy, gate, up, down, router_w, x, combine_form, parts=2, part_experts=None, shared=None,
            logit_bias=None, select_bias=None):
        """Whole path on FP32 rows: router -> A8 -> experts -> combine. Returns a dict of every stage's output."""
        x = np.ascontiguousarray(x, np.float32)
        logits, scores, ids, wts = self.router(policy, x=x, w=router_w, logit_bias=logit_bias, bias=select_bias)
        codes, deltas, sums = self.quantize_a8(x)
        ex = self.experts(shape, gate, up, down, ids, codes, deltas, sums)
        if part_experts is None:
            part_experts = max(1, shape.experts // parts)
        y = self.combine(combine_form, ex["raw"], wts, ids, shared=shared, parts=parts, part_experts=part_experts)
        return dict(logits=logits, scores=scores, ids=ids, weights=wts, raw=ex["raw"], status=ex["status"], y=y,
                    x_codes=codes, x_deltas=deltas, x_sums=sums)


class Ref:
    """The reference's own CPU functions (oracle/ref_shim.cpp over the reference's object files)."""

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        self.lib = L = C.CDLL(REF_SO)
        L.ref_half_to_float.restype = C.c_float
        L.ref_half_to_float.argtypes = [C.c_uint16]
        for n in ("ref_declared_exp", "ref_router_score", "ref_gfx1151_expf"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        L.ref_swiglu_clamped.restype = C.c_float
        L.ref_swiglu_clamped.argtypes = [C.c_float] * 3
        L.ref_product_q8_0.restype = C.c_float
        L.ref_gate_row_q4k.restype = C.c_float
        L.ref_down_row_q8_0.restype = C.c_float
        L.ref_evaluate_row_q4k.restype = C.c_float
        L.ref_evaluate_down_row.restype = C.c_float
        L.ref_cpu_isa.restype = C.c_char_p
        L.ref_expert_isa.restype = C.c_char_p
        L.ref_time_layer_q4k.restype = C.c_double

    def rmsnorm(self, x, w=None, eps=1e-6):
        x = np.ascontiguousarray(x, np.float32)
        rows, n = x.shape
        y = np.zeros_like(x)
        wp = _p(np.ascontiguousarray(w, np.float32), f32p) if w is not None else None
        self.lib.ref_rmsnorm_f32(_p(x, f32p), wp, n, C.c_float(eps), _p(y, f32p), rows)
        return y

    def quantize_a8(self, x, ds41=False):
        x = np.ascontiguousarray(x, np.float32)
        rows, width = x.shape
        codes = np.zeros((rows, width), np.int8)
        deltas = np.zeros((rows, width // 32), np.float32)
        sums = np.zeros((rows, width // 32), np.int32)
        for r in range(rows):
            if ds41:
                self.lib.ref_ds41_quantize_a8(_p(x[r], f32p), C.c_size_t(width), _p(codes[r], i8p), _p(deltas[r], f32p), _p(sums[r], i32p))
            elif self.lib.ref_quantize_a8(_p(x[r], f32p), C.c_size_t(width), _p(codes[r], i8p), _p(deltas[r], f32p), _p(sums[r], i32p)):
                raise ValueError("rejected")
        return codes, deltas, sums

    def gemv_q8_0_a8(self, weight, width, codes, deltas, out=None, accumulate=False):
        weight = np.ascontiguousarray(weight, np.uint8)
        count, row_bytes = weight.shape
        rows = codes.shape[0]
        if out is None:
            out = np.zeros((rows, count), np.float32)
        if self.lib.ref_gemv_q8_0_a8(_p(weight, u8p), row_bytes, width, count, rows, _p(codes, i8p), _p(deltas, f32p),
                                     codes.shape[1], _p(out, f32p), out.shape[1], int(accumulate)):
            raise ValueError("rejected")
        return out

    def product_q8_0(self, row, codes, deltas):
        row = np.ascontiguousarray(row, np.uint8)
        return self.lib.ref_product_q8_0(_p(row, u8p), _p(codes, i8p), _p(deltas, f32p), C.c_size_t(codes.size))

    def reference_router(self, x, w, bias, top_k, scale, bias_image=None, image_rows=None):
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        rows, hidden = x.shape
        experts = w.shape[0]
        scores = np.zeros((rows, experts), np.float32)
        ids = np.zeros((rows, top_k), np.uint32)
        wt = np.zeros((rows, top_k), np.float32)
        if self.lib.ref_reference_router(_p(x, f32p), rows, hidden, _p(w, f32p), experts, _p(bias, f32p), _p(bias_image, f32p),
                                         _p(image_rows, u8p), top_k, C.c_float(scale), _p(scores, f32p), _p(ids, u32p), _p(wt, f32p)):
            raise ValueError("rejected")
        return scores, ids, wt

    def route_scores(self, score, logits):
        logits = np.ascontiguousarray(logits, np.float32)
        out = np.zeros_like(logits)
        for r in range(logits.shape[0]):
            if self.lib.ref_route_scores(score, _p(logits[r], f32p), logits.shape[1], _p(out[r], f32p)):
                raise ValueError("rejected")
        return out

    def route_select(self, policy, scores, bias=None):
        scores = np.ascontiguousarray(scores, np.float32)
        rows = scores.shape[0]
        ids = np.zeros((rows, policy.top_k), np.uint32)
        w = np.zeros((rows, policy.top_k), np.float32)
        words = policy.words()
        for r in range(rows):
            if self.lib.ref_route_select(_p(words, u32p), C.c_float(policy.renorm_eps), C.c_float(policy.scale),
                                         _p(scores[r], f32p), _p(bias, f32p), _p(ids[r], u32p), _p(w[r], f32p)):
                raise ValueError("route policy rejected")
        return ids, w

    def select_softmax(self, logits, top_k, normalize=True):
        logits = np.ascontiguousarray(logits, np.float32)
        ids = np.zeros((logits.shape[0], top_k), np.uint32)
        w = np.zeros((logits.shape[0], top_k), np.float32)
        for r in range(logits.shape[0]):
            if self.lib.ref_select_softmax(_p(logits[r], f32p), logits.shape[1], top_k, int(normalize), _p(ids[r], u32p), _p(w[r], f32p)):
                raise ValueError("rejected")
        return ids, w

    def window_routes(self, ids, split, first=0, end=0):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, top_k = ids.shape
        n = rows * top_k
        r = {k: np.zeros(n, np.uint32) for k in ("experts", "rows", "slots", "order")}
        r["begins"] = np.zeros(n + 1, np.uint32)
        r["low_counts"] = np.zeros(rows, np.uint32)
        mx = C.c_uint32(0)
        rc = self.lib.ref_window_routes(_p(ids, u32p), rows, top_k, split, first, end, _p(r["experts"], u32p), _p(r["begins"], u32p),
                                        _p(r["rows"], u32p), _p(r["slots"], u32p), _p(r["order"], u32p), _p(r["low_counts"], u32p),
                                        C.byref(mx))
        if rc < 0:
            raise ValueError("rejected")
        r["union"], r["max_rows"] = rc, mx.value
        return r

    def window_ds41(self, gate_type, down_type, gate, up, down, experts, hidden, inter, limit, x, ids, weights, shared, split, first=0, end=0):
        """reference_window over Q8_0 (8) / Q2_K (10) tensors."""
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.uint32)
        weights = np.ascontiguousarray(weights, np.float32)
        rows, K = ids.shape
        slots = rows * K
        out = dict(gate=np.zeros((slots, inter), np.float32), up=np.zeros((slots, inter), np.float32),
                   act_codes=np.zeros((slots, inter), np.int8), act_deltas=np.zeros((slots, inter // 32), np.float32),
                   act_sums=np.zeros((slots, inter // 32), np.int32), raw=np.zeros((slots, hidden), np.float32),
                   y=np.zeros((rows, hidden), np.float32))
        if shared is None:
            shared = np.zeros((rows, hidden), np.float32)
        rc = self.lib.ref_window_ds41(gate_type, down_type, _p(gate, u8p), _p(up, u8p), _p(down, u8p), experts, hidden, inter, C.c_float(limit),
                                      _p(x, f32p), rows, _p(ids, u32p), _p(weights, f32p), _p(shared, f32p), K, split, first, end,
                                      _p(out["gate"], f32p), _p(out["up"], f32p), _p(out["act_codes"], i8p),
                                      _p(out["act_deltas"], f32p), _p(out["act_sums"], i32p), _p(out["raw"], f32p), _p(out["y"], f32p))
        if rc:
            raise ValueError("rejected")
        return out


    def window_q8_0(self, gate, up, down, experts, hidden, inter, limit, x, ids, weights, shared, split, first=0, end=0):
        return self.window_ds41(8, 8, gate, up, down, experts, hidden, inter, limit, x, ids, weights, shared, split, first, end)
    def half_sum(self, ids, split, weights, raw, half):
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, K = ids.shape
        H = raw.shape[1]
        out = np.zeros((rows, H), np.float32)
        weights = np.ascontiguousarray(weights, np.float32)
        if self.lib.ref_half_sum(_p(ids, u32p), rows, K, split, _p(weights, f32p), _p(raw, f32p), H, half, _p(out, f32p)):
            raise ValueError("rejected")
        return out

    def expert_run(self, gate, up, down, gate_format, down_format, hidden, ffn, codes, deltas, sums, ids, threads=0, simd=True):
        """reference_run (threads 0) or Executor over every (row, k) assignment of ids. Returns rawdots, status."""
        ids = np.ascontiguousarray(ids, np.uint32)
        rows, K = ids.shape
        asg = np.zeros((rows * K, 3), np.uint32)
        asg[:, 0] = np.repeat(np.arange(rows), K)
        asg[:, 1] = np.tile(np.arange(K), rows)
        asg[:, 2] = ids.reshape(-1)
        raw = np.zeros((rows, K, hidden), np.float32)
        status = np.zeros(rows, np.uint32)
        self.lib.ref_expert_run(_p(gate, u8p), _p(up, u8p), _p(down, u8p), gate_format, down_format, hidden, ffn, _p(codes, i8p),
                                _p(deltas, f32p), _p(sums, i32p), rows, _p(asg, u32p), rows * K, K, _p(raw, f32p), _p(status, u32p),
                                threads, int(simd))
        return raw.reshape(rows * K, hidden), status

    def gate_row_q4k(self, row, codes, deltas, sums, simd=False):
        row = np.ascontiguousarray(row, np.uint8)
        return self.lib.ref_gate_row_q4k(_p(row, u8p), C.c_uint32(row.size // 144), _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p), int(simd))

    def down_row_q8_0(self, row, codes, deltas, sums):
        row = np.ascontiguousarray(row, np.uint8)
        return self.lib.ref_down_row_q8_0(_p(row, u8p), C.c_uint32(row.size // 34), _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p))

    def evaluate_row_q4k(self, row, codes, deltas, sums):
        row = np.ascontiguousarray(row, np.uint8)
        return self.lib.ref_evaluate_row_q4k(_p(row, u8p), _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p), C.c_uint32(codes.size))

    def evaluate_down_row(self, row, codes, deltas, sums, ggml_type):
        row = np.ascontiguousarray(row, np.uint8)
        return self.lib.ref_evaluate_down_row(_p(row, u8p), _p(codes, i8p), _p(deltas, f32p), _p(sums, i32p), C.c_uint32(codes.size), ggml_type)

    def combine(self, form, w, eo, base, rows, top_k, width):
        y = np.zeros((rows, width), np.float32)
        if self.lib.ref_combine(form, rows, top_k, width, _p(w, f32p), _p(eo, f32p), _p(base, f32p), _p(y, f32p)):
            raise ValueError("rejected")
        return y

    def time_layer_q4k(self, gate, up, down, experts, hidden, inter, top_k, router_w, x, threads, reps):
        x = np.ascontiguousarray(x, np.float32)
        rows = x.shape[0]
        y = np.zeros((rows, hidden), np.float32)
        ids = np.zeros((rows, top_k), np.uint32)
        sec = self.lib.ref_time_layer_q4k(_p(gate, u8p), _p(up, u8p), _p(down, u8p), experts, hidden, inter, top_k,
                                          _p(router_w, f32p), _p(x, f32p), rows, threads, reps, _p(y, f32p), _p(ids, u32p))
        return sec, y, ids

    def time_experts_q4k(self, gate, up, down, hidden, inter, top_k, x, ids, threads, reps):
        """Seconds for `reps` calls of the routed Q4_K experts (reference row kernels) on the given routes; raw of the last call."""
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.uint32)
        rows = x.shape[0]
        raw = np.zeros((rows * top_k, hidden), np.float32)
        self.lib.ref_time_experts_q4k.restype = C.c_double
        sec = self.lib.ref_time_experts_q4k(_p(gate, u8p), _p(up, u8p), _p(down, u8p), hidden, inter, top_k, _p(x, f32p), rows,
                                            _p(ids, u32p), threads, reps, _p(raw, f32p))
        return sec, raw

    def time_gemv_q8_0_a8(self, weight, width, codes, deltas, threads, reps):
        """Seconds for `reps` dense Q8_0 x A8 products (the CPU backend's kernel, output rows split over the threads)."""
        weight = np.ascontiguousarray(weight, np.uint8).reshape(-1)
        row_bytes = width // 32 * 34
        count, rows = weight.size // row_bytes, codes.shape[0]
        out = np.zeros((rows, count), np.float32)
        self.lib.ref_time_gemv_q8_0_a8.restype = C.c_double
        sec = self.lib.ref_time_gemv_q8_0_a8(_p(weight, u8p), row_bytes, width, count, rows, _p(codes, i8p), _p(deltas, f32p), threads, reps,
                                             _p(out, f32p))
        return sec, out

    def planner_trace(self, layers, experts, top_k, slots, expert_bytes, decay, margin, budget, ids, seed_counts=None, fill=False, max_moves=256):
        """The reference's residency planner over a scripted trace (ids [steps][layers][n]); every planned move is committed.
        Returns (moves per step as lists of (layer, slot, evict, expert), final tables [layers][experts], receipt dict)."""
        ids = np.ascontiguousarray(ids, np.uint32)
        steps, _, n = ids.shape
        eb = np.ascontiguousarray(expert_bytes, np.uint64)
        moves = np.zeros((steps, max_moves, 4), np.uint32)
        counts = np.zeros(steps, np.uint32)
        tables = np.zeros((layers, experts), np.int32)
        receipt = np.zeros(6, np.uint64)
        sc = np.ascontiguousarray(seed_counts, np.uint32) if seed_counts is not None else None
        self.lib.ref_planner_trace.argtypes = [C.c_uint32] * 4 + [C.c_void_p, C.c_double, C.c_double, C.c_uint64, C.c_void_p, C.c_int, C.c_uint32, C.c_void_p,
                                               C.c_uint32, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
        rc = self.lib.ref_planner_trace(layers, experts, top_k, slots, eb.ctypes.data, decay, margin, budget, sc.ctypes.data if sc is not None else None,
                                        int(fill), steps, ids.ctypes.data, n, moves.ctypes.data, max_moves, counts.ctypes.data, tables.ctypes.data, None,
                                        receipt.ctypes.data)
        assert rc == 0, f"ref_planner_trace failed ({rc})"
        assert int(counts.max(initial=0)) <= max_moves
        per_step = [[tuple(int(v) for v in moves[s, i]) for i in range(int(counts[s]))] for s in range(steps)]
        keys = ("active_bytes", "hit_bytes", "promoted_bytes", "promotions", "evictions", "steps")
        return per_step, tables, dict(zip(keys, (int(v) for v in receipt)))

    def host_read_gbs(self, data, threads, reps=3):
        """Read bandwidth of the host over `data` (a uint8 array far larger than the caches) with `threads` threads, GB/s."""
        data = np.ascontiguousarray(data, np.uint8).reshape(-1)
        self.lib.ref_time_read.restype = C.c_double
        self.lib.ref_time_read.argtypes = [C.c_void_p, C.c_size_t, C.c_uint, C.c_uint32, C.c_void_p]
        self.lib.ref_time_read(data.ctypes.data, data.size, threads, 1, None)          # warm the pool and the pages
        sec = self.lib.ref_time_read(data.ctypes.data, data.size, threads, reps, None)
        return data.size * reps / sec / 1e9

    def isa(self):
        """Row-kernel table of the routed-expert executor on this host."""
        return self.lib.ref_expert_isa().decode()
