"""Pins of the CPU oracle (oracle/moe_oracle.cpp).

(a) Known-answer literals held by the reference's own tests, restated here as data:
      tests/route_policy_tests.cpp (digest :211-242/:302, ties / -0 / NaN / top-1 :143-190),
      tests/cpu_backend_host_tests.cpp (width rejection :65-92, cancellation order :94-117, subnormal halves :119-149).
(b) Agreement with the reference's own CPU code (oracle/_ref) on seeded inputs, bit for bit.
(c) Agreement with the committed vectors under tests/golden/ (generated from oracle/_ref by make_golden.py).
"""
import os

import numpy as np
import pytest

from oracle import loader as L
from b200moe import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "moe_golden.npz")


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def same(a, b):
    return np.array_equal(bits(a), bits(b))


# ---- the reference test's deterministic generators (tests/route_policy_tests.cpp:60-85), restated ----------------
class Lcg:
    def __init__(self, s):
        self.s = s

    def next(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return (self.s >> 33) & 0xFFFFFFFF


def lcg_logits(g, n):
    z = np.zeros(n, np.float32)
    for i in range(n):
        r = g.next()
        z[i] = np.float32(20.0 + (r % 7) * 0.5) if r % 97 == 0 else np.float32((int(r % 1025) - 512) / 64.0)
    return z


def lcg_biases(g, n):
    b = np.zeros(n, np.float32)
    for i in range(n):
        r = g.next()
        b[i] = 0.0 if r % 3 == 0 else np.float32((int(r % 257) - 128) / 256.0)
    return b


def fnv(values, h=1469598103934665603):
    for v in values:
        v = int(v)
        for i in range(4):
            h ^= (v >> (8 * i)) & 0xFF
            h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_router_digest_pinned(oracle):
    """kDs41Digest of tests/route_policy_tests.cpp:302: ids and weight bits of 4 shapes x 16 rows."""
    g = Lcg(41)
    h = 1469598103934665603
    for experts, top_k, scale in ((256, 8, 2.5), (384, 6, 1.5), (64, 1, 2.0), (512, 16, 3.998)):
        rows = 16
        w = lcg_logits(g, experts)
        b, bi = lcg_biases(g, experts), lcg_biases(g, experts)
        x = np.ones((rows, 1), np.float32)
        pol = L.ds41_policy(experts, top_k, scale)
        logits = oracle.router_logits(x, w.reshape(experts, 1))
        assert same(logits, np.tile(w, (rows, 1)))  # hidden 1: 0 + w * 1 exactly
        scores = oracle.route_scores(pol.score, logits)
        for r in range(rows):
            ids, wt = oracle.route_select(pol, scores[r:r + 1], bi if r % 2 else b)
            vals = []
            for k in range(top_k):
                vals += [ids[0, k], bits(wt)[0, k]]
            h = fnv(vals, h)
    assert h == 0x168F06B494AE3B13


def test_router_literals(oracle):
    sig512 = L.RoutePolicy(L.SIGMOID, 1, L.ORDERED_BITS, L.ASCENDING_ID, 512, 16, 1, 1, 1, 1, 1e-20, 3.998)
    s = np.full((1, 512), 0.25, np.float32)
    b = np.zeros(512, np.float32)
    ids, w = oracle.route_select(sig512, s, b)
    assert list(ids[0]) == list(range(16))  # ties -> lower id first
    b[300] = 0.5
    ids, w = oracle.route_select(sig512, s, b)
    assert ids[0, 0] == 0 and ids[0, 14] == 14 and ids[0, 15] == 300
    assert bits(w)[0, 0] == bits(w)[0, 15]  # the bias does not enter the weights
    q = L.RoutePolicy(L.SIGMOID, 0, L.ORDERED_BITS, L.SELECTION, 4, 2, 1, 1, 1, 1, 1e-20, 1.0)
    zeros = np.array([[-0.0, 0.0, -1.0, -2.0]], np.float32)
    assert list(oracle.route_select(q, zeros)[0][0]) == [0, 1]
    q.key = L.FLOAT_SERIAL
    assert list(oracle.route_select(q, zeros)[0][0]) == [0, 1]
    nan_first = np.array([[np.nan, 3.0, 2.0, 1.0]], np.float32)
    assert list(oracle.route_select(q, nan_first)[0][0]) == [0, 1]  # a first-candidate NaN is kept
    q.order = L.ASCENDING_ID
    desc = np.array([[1.0, 3.0, 2.0, 0.5]], np.float32)
    assert list(oracle.route_select(q, desc)[0][0]) == [1, 2]
    one = L.ds41_policy(4, 1, 2.0)
    ids, w = oracle.route_select(one, desc, np.zeros(4, np.float32))
    assert ids[0, 0] == 1 and bits(w)[0, 0] == bits(np.float32(6.0))  # top-1 keeps raw score x scale
    sm = oracle.route_scores(L.SOFTMAX, desc)[0]
    assert sm[1] > sm[2] > sm[0] and abs(float(sm.sum()) - 1.0) < 1e-6


def half_bytes(h):
    return [h & 0xFF, h >> 8]


def test_q8_0_cancellation_order(oracle):
    """Lane 0 rounds (2^24 + 1) before cancelling lane 16; lane 1 leaves 1 (cpu_backend_host_tests.cpp:94-117)."""
    w = np.zeros((1, 33 * 34), np.uint8)
    for g in range(33):
        w[0, g * 34 + 1] = 0x3C
        w[0, g * 34 + 2] = 1
    codes = np.ones((1, 33 * 32), np.int8)
    deltas = np.zeros((1, 33), np.float32)
    deltas[0, 0], deltas[0, 16], deltas[0, 1], deltas[0, 32] = 2.0 ** 24, -2.0 ** 24, 1.0, 1.0
    y = oracle.gemv_q8_0_a8(w, 33 * 32, codes, deltas, out=np.full((1, 1), -1.0, np.float32))
    assert bits(y)[0, 0] == bits(np.float32(1.0))
    y = oracle.gemv_q8_0_a8(w, 33 * 32, codes, deltas, out=np.full((1, 1), -1.0, np.float32), accumulate=True)
    assert bits(y)[0, 0] == bits(np.float32(0.0))


def test_q8_0_tiny_and_subnormal(oracle):
    """cpu_backend_host_tests.cpp:119-149."""
    w = np.zeros((2, 35), np.uint8)
    w[0, 0] = 1  # +2^-24
    w[1, 0], w[1, 1] = 0xFF, 0x83  # -1023 * 2^-24
    w[:, 2:34] = 1
    x = np.zeros((2, 32), np.float32)
    x[0, :] = 2.0 ** -120
    x[1, :] = 127.0
    codes, deltas, sums = oracle.quantize_a8(x)
    assert bits(deltas)[0, 0] == bits(np.float32(1.0)) and bits(deltas)[1, 0] == bits(np.float32(1.0))
    assert sums[0, 0] == 0 and sums[1, 0] == 4064
    assert (codes[0] == 0).all() and (codes[1] == 127).all()
    y = oracle.gemv_q8_0_a8(w, 32, codes, deltas)
    assert bits(y)[0, 0] == 0 and bits(y)[0, 1] == 0
    assert bits(y)[1, 0] == bits(np.float32(4064.0 * 2.0 ** -24))
    assert bits(y)[1, 1] == bits(np.float32(-4157472.0 * 2.0 ** -24))


def test_width_rejection(oracle):
    with pytest.raises(ValueError):
        oracle.quantize_a8(np.ones((1, 31), np.float32))
    with pytest.raises(ValueError):
        oracle.gemv_q8_0_a8(np.zeros((1, 68), np.uint8), 33, np.zeros((1, 64), np.int8), np.zeros((1, 2), np.float32))


# ---- (b) against the reference's own CPU code -------------------------------------------------------------------
def special_rows(rng, rows, width):
    x = rng.standard_normal((rows, width), dtype=np.float32)
    if rows > 1 and width >= 96:
        x[1, :32] = 0.0          # an all-zero group
        x[1, 32:64] = 1e-37      # below 2^-119: the tiny rule
        x[1, 64] = 3.0e38
    return x


def test_quantize_a8_vs_reference(oracle, ref):
    rng = np.random.default_rng(1)
    for width in (32, 256, 2048):
        x = special_rows(rng, 3, width) * np.float32(rng.uniform(0.01, 50.0))
        got = oracle.quantize_a8(x)
        for ds41 in (False, True):
            want = ref.quantize_a8(x, ds41=ds41)
            assert np.array_equal(got[0], want[0]) and same(got[1], want[1]) and np.array_equal(got[2], want[2])


def test_gemv_q8_0_vs_reference(oracle, ref):
    rng = np.random.default_rng(2)
    for width, count, rows in ((32, 5, 1), (1024, 17, 3), (2048, 9, 2), (7168, 3, 1)):
        w = synth.q8_0_blocks(rng, count * width // 32).reshape(count, -1)
        w[::3, 1] |= 0x80  # some negative scales
        x = special_rows(rng, rows, width)
        x[np.abs(x) > 1e30] = 1.0
        codes, deltas, _ = oracle.quantize_a8(x)
        got = oracle.gemv_q8_0_a8(w, width, codes, deltas)
        want = ref.gemv_q8_0_a8(w, width, codes, deltas)
        assert same(got, want)
        for r in range(rows):
            for o in range(0, count, 4):
                assert bits(np.float32(ref.product_q8_0(w[o], codes[r], deltas[r]))) == bits(got)[r, o]
        init = rng.standard_normal(got.shape, dtype=np.float32)
        assert same(oracle.gemv_q8_0_a8(w, width, codes, deltas, out=init.copy(), accumulate=True),
                    ref.gemv_q8_0_a8(w, width, codes, deltas, out=init.copy(), accumulate=True))


def test_q4k_row_vs_reference(oracle, ref):
    rng = np.random.default_rng(3)
    for width in (256, 768, 2048, 2560, 7168):
        blocks = width // 256
        w = synth.q4_k_blocks(rng, 6 * blocks, scale=0.01).reshape(6, -1)
        x = rng.standard_normal((2, width), dtype=np.float32) * np.float32(3.0)
        x[1, :32] = 127.0  # extreme codes
        codes, deltas, sums = oracle.quantize_a8(x)
        for o in range(6):
            for r in range(2):
                got = np.float32(oracle.row_q4k(w[o], codes[r], deltas[r], sums[r]))
                assert bits(got) == bits(np.float32(ref.gate_row_q4k(w[o], codes[r], deltas[r], sums[r], simd=False)))
                assert bits(got) == bits(np.float32(ref.gate_row_q4k(w[o], codes[r], deltas[r], sums[r], simd=True)))
                if width <= 2560:  # the contract-level oracle's admitted widths (moe_q4k_a8_contract.cpp:26-27)
                    assert bits(got) == bits(np.float32(ref.evaluate_row_q4k(w[o], codes[r], deltas[r], sums[r])))
                if width <= 1536:  # Q4_K down = the same row rule (moe_a8_down_contract.cpp:146)
                    assert bits(got) == bits(np.float32(ref.evaluate_down_row(w[o], codes[r], deltas[r], sums[r], 12)))


def test_q8_chain4_down_vs_reference(oracle, ref):
    rng = np.random.default_rng(4)
    for width in (128, 640, 768, 1024):
        w = synth.q8_0_blocks(rng, 4 * width // 32).reshape(4, -1)
        x = rng.standard_normal((1, width), dtype=np.float32)
        codes, deltas, sums = oracle.quantize_a8(x)
        for o in range(4):
            got = np.float32(oracle.row_q8_chain4(w[o], codes[0], deltas[0]))
            assert bits(got) == bits(np.float32(ref.down_row_q8_0(w[o], codes[0], deltas[0], sums[0])))
            if width <= 640:  # the contract-level oracle admits at most 640 inputs for the 32-group formats
                assert bits(got) == bits(np.float32(ref.evaluate_down_row(w[o], codes[0], deltas[0], sums[0], 8)))


def test_scalar_math_vs_reference(oracle, ref):
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(4000) * 8, rng.uniform(-110, 95, 2000),
                         [0.0, -0.0, 88.0, 88.5, -103.0, -103.5, np.inf, -np.inf, np.nan, 20.0, 20.5]]).astype(np.float32)
    for v in xs:
        assert bits(np.float32(oracle.lib.orc_declared_exp(v))) == bits(np.float32(ref.lib.ref_declared_exp(v)))
        assert bits(np.float32(oracle.lib.orc_gfx1151_expf(v))) == bits(np.float32(ref.lib.ref_gfx1151_expf(v)))
        if np.isfinite(v):
            assert bits(np.float32(oracle.lib.orc_sqrt_softplus(v))) == bits(np.float32(ref.lib.ref_router_score(v)))
    for _ in range(3000):
        g, u = (rng.standard_normal(2) * 6).astype(np.float32)
        for lim in (10.0, np.inf):
            assert bits(np.float32(oracle.lib.orc_swiglu_ds41(g, u, np.float32(lim)))) == \
                bits(np.float32(ref.lib.ref_swiglu_clamped(g, u, np.float32(lim))))
    for h in list(range(0, 0x8000, 97)) + [0x0001, 0x83FF, 0x7BFF, 0xFBFF, 0x7C00, 0x8000]:
        assert bits(np.float32(oracle.lib.orc_half_to_float(h))) == bits(np.float32(ref.lib.ref_half_to_float(h)))


def test_router_vs_reference(oracle, ref):
    rng = np.random.default_rng(6)
    # reference_router: declared dot order + sqrt-softplus + ds41 preset
    for experts, top_k, hidden, rows in ((64, 4, 2048, 3), (256, 8, 7168, 2), (128, 1, 96, 2)):
        x = rng.standard_normal((rows, hidden), dtype=np.float32)
        w = synth.router_weight(rng, experts, hidden, std=0.05)
        bias = (rng.standard_normal(experts) * 0.1).astype(np.float32)
        scores, ids, wt = ref.reference_router(x, w, bias, top_k, 1.5)
        pol = L.ds41_policy(experts, top_k, 1.5)
        lg, sc, gi, gw = oracle.router(pol, x=x, w=w, bias=bias)
        assert same(sc, scores) and np.array_equal(gi, ids) and same(gw, wt)
    # every score transform and selection option through route_scores_ref / route_select_ref
    for score in (L.SOFTMAX, L.SIGMOID, L.SQRT_SOFTPLUS):
        for key in (L.FLOAT_SERIAL, L.ORDERED_BITS):
            for order in (L.SELECTION, L.ASCENDING_ID):
                for experts, top_k in ((64, 4), (128, 8), (512, 16)):
                    logits = (rng.integers(-512, 513, size=(4, experts)) / 64.0).astype(np.float32)  # exact ties
                    bias = (rng.integers(-128, 129, size=experts) / 256.0).astype(np.float32)
                    pol = L.RoutePolicy(score, 1, key, order, experts, top_k, 1, 1, 1, 1, 1e-20, 2.5)
                    s_ref = ref.route_scores(score, logits)
                    s_orc = oracle.route_scores(score, logits)
                    assert same(s_ref, s_orc)
                    i_ref, w_ref = ref.route_select(pol, s_ref, bias)
                    i_orc, w_orc = oracle.route_select(pol, s_orc, bias)
                    assert np.array_equal(i_ref, i_orc) and same(w_ref, w_orc)


def test_softmax_select_cross_check(oracle, ref):
    """select_moe_experts_deterministic (std::exp softmax, src/moe_plan.cpp:101-162) picks the same experts as the
    declared-exp policy on well separated logits; weights agree to float rounding."""
    rng = np.random.default_rng(7)
    logits = rng.uniform(-1, 1, size=(16, 128)).astype(np.float32)
    pol = L.softmax_policy(128, 8)
    _, _, ids, w = oracle.router(pol, logits=logits)
    ids2, w2 = ref.select_softmax(logits, 8)
    assert np.array_equal(ids, ids2)
    np.testing.assert_allclose(w, w2, rtol=2e-6)


def test_routes_vs_reference(oracle, ref):
    rng = np.random.default_rng(8)
    for rows, top_k, experts in ((1, 4, 64), (8, 8, 128), (40, 6, 32)):
        ids = np.stack([rng.permutation(experts)[:top_k] for _ in range(rows)]).astype(np.uint32)
        split = experts // 2
        for first, end in ((0, 0), (experts // 4, experts // 2), (experts // 2, experts)):
            a = oracle.routes(ids, experts, split, first, end, base=0)
            b = ref.window_routes(ids, split, first, end)
            n, m = b["union"], int(a["counts"][2])
            assert a["counts"][0] == n and a["counts"][1] == b["max_rows"]
            assert np.array_equal(a["experts"][:n], b["experts"][:n]) and np.array_equal(a["begins"][:n + 1], b["begins"][:n + 1])
            assert np.array_equal(a["rows"][:m], b["rows"][:m]) and np.array_equal(a["slots"][:m], b["slots"][:m])
            assert np.array_equal(a["order"], b["order"]) and np.array_equal(a["low_counts"], b["low_counts"])
    dup = np.array([[3, 3, 1, 2]], np.uint32)
    with pytest.raises(ValueError):
        oracle.routes(dup, 8, 4)
    with pytest.raises(ValueError):
        ref.window_routes(dup, 4)


def test_window_q8_0_vs_reference(oracle, ref):
    """Whole DS41-family window (reference_window, src/ds41_moe.cpp:124-165): every intermediate bit for bit."""
    rng = np.random.default_rng(9)
    E, H, I, K, rows = 8, 256, 128, 3, 5
    gate, up, down = synth.expert_tensors(rng, E, H, I, 8, 8)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
    shared = rng.standard_normal((rows, H), dtype=np.float32)
    for limit in (10.0, np.inf):
        sh = L.Shape(H, I, E, K, 8, 8, limit)
        want = ref.window_q8_0(gate, up, down, E, H, I, limit, x, ids, wts, shared, split=E // 2)
        codes, deltas, sums = oracle.quantize_a8(x)
        got = oracle.experts(sh, gate, up, down, ids, codes, deltas, sums, taps=True)
        for k in ("gate", "up", "raw", "act_deltas"):
            assert same(got[k], want[k]), k
        assert np.array_equal(got["act_codes"], want["act_codes"]) and np.array_equal(got["act_sums"], want["act_sums"])
        y = oracle.combine(L.COMBINE_PARTS, got["raw"], wts, ids, shared=shared, parts=2, part_experts=E // 2)
        assert same(y, want["y"])
        for half in (0, 1):
            hs = oracle.combine(L.COMBINE_PARTS, got["raw"], wts, ids, parts=2, part_experts=E // 2, only_part=half)
            assert same(hs, ref.half_sum(ids, E // 2, wts, want["raw"], half))
    # expert-parallel restriction: a rank owning [first, end) produces the same raw vectors for its slots
    sh = L.Shape(H, I, E, K, 8, 8, 10.0)
    part = ref.window_q8_0(gate, up, down, E, H, I, 10.0, x, ids, wts, shared, split=E // 2, first=2, end=6)
    got = oracle.experts(sh, gate, up, down, ids, codes, deltas, sums, first=2, end=6)
    own = ((ids >= 2) & (ids < 6)).reshape(-1)
    assert same(got["raw"][own], part["raw"][own])


def test_window_q2_k_vs_reference(oracle, ref):
    """The family's Q2_K tensors (product_q2_k, src/ds41_formats.cpp:198-218) alone and mixed with Q8_0: the oracle's
    window equals reference_window bit for bit in every intermediate."""
    rng = np.random.default_rng(19)
    E, H, I, K, rows = 6, 512, 256, 2, 4
    x = rng.standard_normal((rows, H), dtype=np.float32)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
    shared = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    for gt, dt in ((10, 10), (10, 8), (8, 10)):
        gate, up, down = synth.expert_tensors(rng, E, H, I, gt, dt)
        want = ref.window_ds41(gt, dt, gate, up, down, E, H, I, 7.0, x, ids, wts, shared, split=E // 2)
        got = oracle.experts(L.Shape(H, I, E, K, gt, dt, 7.0), gate, up, down, ids, codes, deltas, sums, taps=True)
        for k in ("gate", "up", "raw", "act_deltas"):
            assert same(got[k], want[k]), (gt, dt, k)
        assert np.array_equal(got["act_codes"], want["act_codes"]) and np.array_equal(got["act_sums"], want["act_sums"])
        y = oracle.combine(L.COMBINE_PARTS, got["raw"], wts, ids, shared=shared, parts=2, part_experts=E // 2)
        assert same(y, want["y"])


def test_qwen_experts_vs_reference(oracle, ref):
    """Qwen-family job (reference_run and the threaded Executor, src/cpu/core/routed_expert.cpp:264-489): Q4_K
    gate/up, gfx1151 exp SwiGLU, A8 of h, Q8_0 four-chain down."""
    rng = np.random.default_rng(10)
    E, H, I, K, rows = 6, 512, 256, 2, 7
    gate, up, _ = synth.expert_tensors(rng, E, H, I, 12, 12)
    down = synth.q8_0_blocks(rng, E * H * (I // 32)).reshape(-1)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    sh = L.Shape(H, I, E, K, 12, 8, np.inf)
    got = oracle.experts(sh, gate, up, down, ids, codes, deltas, sums)
    for threads, simd in ((0, False), (3, False), (4, True)):
        raw, status = ref.expert_run(gate, up, down, 0, 1, H, I, codes, deltas, sums, ids, threads=threads, simd=simd)
        assert same(got["raw"], raw) and not status.any()
    # merge: combine_ref fma_f32 with base 0
    wts = rng.uniform(0.1, 0.5, size=(rows, K)).astype(np.float32)
    y = oracle.combine(L.COMBINE_FMA_SLOTS, got["raw"], wts, ids)
    want = ref.combine(0, wts, got["raw"], np.zeros((rows, H), np.float32), rows, K, H)
    assert same(y, want)
    # fail closed on a non-finite projection: poison one input delta (routed_expert_host_tests.cpp:393-399)
    bad = deltas.copy()
    bad[2, 0] = 3e38
    got = oracle.experts(sh, gate, up, down, ids, codes, bad, sums)
    raw, status = ref.expert_run(gate, up, down, 0, 1, H, I, codes, bad, sums, ids, threads=0)
    assert np.array_equal(got["status"] != 0, status != 0) and status[2] != 0


# ---- (c) committed golden vectors --------------------------------------------------------------------------------
def test_golden_vectors(oracle):
    g = np.load(GOLDEN)
    codes, deltas, sums = oracle.quantize_a8(g["a8_x"])
    assert np.array_equal(codes, g["a8_codes"]) and same(deltas, g["a8_deltas"]) and np.array_equal(sums, g["a8_sums"])
    assert same(oracle.gemv_q8_0_a8(g["q8_w"], int(g["q8_width"]), g["q8_codes"], g["q8_deltas"]), g["q8_y"])
    for o in range(g["q4k_w"].shape[0]):
        assert bits(np.float32(oracle.row_q4k(g["q4k_w"][o], g["q4k_codes"][0], g["q4k_deltas"][0], g["q4k_sums"][0]))) == bits(g["q4k_y"])[o]
    pol = L.ds41_policy(int(g["rt_w"].shape[0]), int(g["rt_ids"].shape[1]), 1.5)
    _, sc, ids, wt = oracle.router(pol, x=g["rt_x"], w=g["rt_w"], bias=g["rt_bias"])
    assert same(sc, g["rt_scores"]) and np.array_equal(ids, g["rt_ids"]) and same(wt, g["rt_weights"])
    pol = L.softmax_policy(int(g["sm_logits"].shape[1]), int(g["sm_ids"].shape[1]))
    _, sc, ids, wt = oracle.router(pol, logits=g["sm_logits"])
    assert same(sc, g["sm_scores"]) and np.array_equal(ids, g["sm_ids"]) and same(wt, g["sm_weights"])
    # DS41 window (Q8_0)
    E, H, I, K = (int(v) for v in g["win_shape"])
    sh = L.Shape(H, I, E, K, 8, 8, float(g["win_limit"]))
    codes, deltas, sums = oracle.quantize_a8(g["win_x"])
    ex = oracle.experts(sh, g["win_gate"], g["win_up"], g["win_down"], g["win_ids"], codes, deltas, sums)
    assert same(ex["raw"], g["win_raw"])
    y = oracle.combine(L.COMBINE_PARTS, ex["raw"], g["win_weights"], g["win_ids"], shared=g["win_shared"], parts=2, part_experts=E // 2)
    assert same(y, g["win_y"])
    # Qwen job (Q4_K gate/up, Q8_0 down)
    E, H, I, K = (int(v) for v in g["qw_shape"])
    sh = L.Shape(H, I, E, K, 12, 8, np.inf)
    codes, deltas, sums = oracle.quantize_a8(g["qw_x"])
    ex = oracle.experts(sh, g["qw_gate"], g["qw_up"], g["qw_down"], g["qw_ids"], codes, deltas, sums)
    assert same(ex["raw"], g["qw_raw"])


# ---- RMSNorm in front of the FFN (src/cpu/core/reference.cpp:86-103) ---------------------------------------------
def test_rmsnorm_golden_vectors(oracle):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "norm_golden.npz"))
    for n in (96, 512, 2048):
        assert same(oracle.rmsnorm(g[f"x_{n}"], g[f"w_{n}"], 1e-6), g[f"y_{n}"])
        assert same(oracle.rmsnorm(g[f"x_{n}"], None, 1e-6), g[f"y_unscaled_{n}"])


def test_rmsnorm_against_reference(oracle, ref):
    """Both lane counts (128 below n = 512, 256 from there), with and without the weight, as the reference's own
    test_norm does (tests/cpu_backend_host_tests.cpp:220-239)."""
    rng = np.random.default_rng(77)
    for n in (32, 480, 512, 1024, 7168):
        x = (rng.standard_normal((4, n)) * 3.0).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        for ww in (w, None):
            assert same(oracle.rmsnorm(x, ww, 1e-6), ref.rmsnorm(x, ww, 1e-6))


# ---- the executor's other stored formats: Q5_K gate/up, Q5_1 down (src/cpu/core/routed_expert.hpp:27-28) -----------
FORMAT_CASES = ((13, 7, 1, 0), (12, 7, 0, 0), (13, 8, 1, 1), (13, 12, 1, None))


def test_other_formats_against_reference_executor(oracle, ref):
    """reference_run (scalar) and Executor (AVX2 + VNNI table, 4 threads) on Q5_K / Q5_1 tensors = the oracle, bit for bit.
    Q4_K down has no executor form (its reference is evaluate_down_row, pinned above): gate/up taps only there."""
    rng = np.random.default_rng(91)
    E, H, I, K, rows = 4, 512, 256, 2, 3
    for gt, dt, gf, df in FORMAT_CASES:
        g, u, d = synth.expert_tensors(rng, E, H, I, gt, dt)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        c, dl, s = ref.quantize_a8(x)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        ex = oracle.experts(L.Shape(H, I, E, K, gt, dt, np.inf), g, u, d, ids, c, dl, s)
        if df is None:
            continue
        for threads in (0, 4):
            raw, st = ref.expert_run(g, u, d, gf, df, H, I, c, dl, s, ids, threads=threads)
            assert not st.any() and same(ex["raw"], raw)


def test_other_formats_golden_vectors(oracle):
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "formats_golden.npz"))
    E, H, I, K = (int(v) for v in g["shape"])
    for gt, dt, _, df in FORMAT_CASES:
        if df is None:
            continue
        t = f"{gt}_{dt}"
        c, dl, s = oracle.quantize_a8(g[f"x_{t}"])
        ex = oracle.experts(L.Shape(H, I, E, K, gt, dt, np.inf), g[f"gate_{t}"], g[f"up_{t}"], g[f"down_{t}"], g[f"ids_{t}"], c, dl, s)
        assert same(ex["raw"], g[f"raw_{t}"])
    # Q2_K tensors of the DS41 family (reference_window outputs)
    E, H, I, K = (int(v) for v in g["shape_q2k"])
    for gt, dt in ((10, 10), (10, 8), (8, 10)):
        t = f"{gt}_{dt}"
        c, dl, s = oracle.quantize_a8(g[f"x_{t}"])
        ex = oracle.experts(L.Shape(H, I, E, K, gt, dt, 7.0), g[f"gate_{t}"], g[f"up_{t}"], g[f"down_{t}"], g[f"ids_{t}"], c, dl, s, taps=True)
        assert same(ex["raw"], g[f"raw_{t}"]) and np.array_equal(ex["act_codes"], g[f"act_codes_{t}"])
