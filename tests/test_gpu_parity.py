"""GPU parity: every stage of the CUDA path, called through the C ABI, against the CPU oracle on the same seeded
inputs - bit for bit (integer work, ids, and every FP32 value whose contract is declared as single IEEE operations).

The one place where exactness is not structural: the Qwen-family SwiGLU evaluates exp2 in double precision on both sides
(C library on the host, CUDA math library on the device); the two may differ by one double ulp, which flips the rounded
float in about one evaluation per 2^29. The tests of that family COUNT the A8 groups of h that differ and allow
`evaluations >> 26` of them - zero at every size used here - so they assert bit equality of every stage; the north-star
tolerance (max relative error 1e-3) is asserted beside it on whole-layer outputs.
"""
import math

import numpy as np
import pytest

from oracle import loader as O

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

REL_TOL = 1e-3  # north-star tolerance for MoE outputs (max relative error, fp32 accumulate)


@pytest.fixture(scope="module")
def gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import b200moe
    b200moe.lib()  # fails loudly when the extension is missing
    return torch.device("cuda:0")


def dv(a, dev):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def host(t):
    return t.detach().cpu().numpy()


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def same(a, b):
    return np.array_equal(bits(a), bits(b))


def u32(t):
    return host(t).view(np.uint32)


def max_rel(y, ref):
    return float(np.max(np.abs(y - ref).max(axis=-1) / np.maximum(np.abs(ref).max(axis=-1), 1e-30)))


def shape_pair(H, I, E, K, gt, dt, limit=math.inf):
    from b200moe import ops
    return ops.make_shape(H, I, E, K, gt, dt, limit), O.Shape(H, I, E, K, gt, dt, limit)


def policy_pair(p):
    import b200moe
    return b200moe.RoutePolicy(*[getattr(p, f[0]) for f in p._fields_])


# ---------------------------------------------------------------------------------------------------------- A8
def test_quantize_a8(gpu, oracle):
    from b200moe import ops, synth
    rng = np.random.default_rng(11)
    for rows, width in ((1, 32), (3, 256), (8, 2048), (5, 7168)):
        x = rng.standard_normal((rows, width), dtype=np.float32) * np.float32(rng.uniform(0.01, 40))
        if width >= 128:
            x[0, :32] = 0.0
            x[0, 32:64] = 1e-37          # tiny rule: below 2^-119
            x[0, 64:96] = 127.0
            x[-1, 96] = 3.0e38
        c, d, s = ops.enqueue_quantize_a8(dv(x, gpu))
        wc, wd, ws = oracle.quantize_a8(x)
        assert np.array_equal(host(c), wc) and same(host(d), wd) and np.array_equal(host(s), ws)
        xb = synth.bf16_round(x)
        c, d, s = ops.enqueue_quantize_a8(dv(xb, gpu).to(torch.bfloat16))
        wc, wd, ws = oracle.quantize_a8(xb)
        assert np.array_equal(host(c), wc) and same(host(d), wd) and np.array_equal(host(s), ws)


def test_site_through_the_launch_record_seam(gpu, oracle):
    """b200moe_enqueue forwards a checked envelope to the site: the A8 quantiser through it equals the oracle."""
    import ctypes as C
    import b200moe
    rng = np.random.default_rng(12)
    x = rng.standard_normal((6, 512), dtype=np.float32)
    xd = dv(x, gpu)
    codes = torch.empty((6, 512), dtype=torch.int8, device=gpu)
    deltas = torch.empty((6, 16), dtype=torch.float32, device=gpu)
    sums = torch.empty((6, 16), dtype=torch.int32, device=gpu)
    v = b200moe.QuantizeA8View(b200moe.ptr(xd), 6, 512, 512, 0, b200moe.A8Rows(b200moe.ptr(codes), b200moe.ptr(deltas), b200moe.ptr(sums), 6, 512, 512), None)
    b200moe.check(b200moe.enqueue(b200moe.SITE_QUANTIZE_A8, v, b200moe.stream_ptr()))
    wc, wd, ws = oracle.quantize_a8(x)
    assert np.array_equal(host(codes), wc) and same(host(deltas), wd) and np.array_equal(host(sums), ws)
    with pytest.raises(b200moe.B200MoeError):
        b200moe.check(b200moe.enqueue(b200moe.SITE_QUANTIZE_A8, v, b200moe.stream_ptr(), nbytes=C.sizeof(v) - 8))


def test_deferred_first_error_record(gpu):
    """The record keeps the COMPLETE first non-zero summary of a stream of layers; a clean layer or a later failure never
    overwrites it (include/strix/deferred_moe_status.hpp:16-28). The summaries are real ones: a window with an id out of
    range sets INVALID_ROUTE in the routes' row status, folded into the word the merge reads."""
    import ctypes as C
    import b200moe
    from b200moe import ops
    L = b200moe.lib()
    record = torch.zeros(2, dtype=torch.int32, device=gpu)
    clean = torch.zeros(1, dtype=torch.int32, device=gpu)
    ids = torch.tensor([[0, 1], [2, 900]], dtype=torch.int32, device=gpu)        # 900 >= 8 experts
    status = torch.zeros(2, dtype=torch.int32, device=gpu)
    ops.enqueue_moe_routes(ids, 8, 4, row_status=status)
    first = status.max().reshape(1).contiguous()                                   # the job summary of that window
    later = torch.tensor([b200moe.ROW_PROJECTION_NONFINITE], dtype=torch.int32, device=gpu)
    st = b200moe.stream_ptr()
    for summary, domain in ((clean, b200moe.DOMAIN_Q4K_A8), (first, b200moe.DOMAIN_Q4K_A8), (clean, b200moe.DOMAIN_LEGACY),
                            (later, b200moe.DOMAIN_LEGACY)):
        b200moe.check(L.b200moe_merge_first_error(b200moe.ptr(record), b200moe.ptr(summary), domain, st))
    got = record.cpu().numpy().view(np.uint32)
    assert int(first.item()) == b200moe.ROW_INVALID_ROUTE and got.tolist() == [b200moe.DOMAIN_Q4K_A8, b200moe.ROW_INVALID_ROUTE]
    assert L.b200moe_check_first_error(C.byref(b200moe.FirstError(int(got[0]), int(got[1])))) == b200moe.ERR_INVALID_ARGUMENT
    with pytest.raises(b200moe.B200MoeError):
        b200moe.check(L.b200moe_merge_first_error(b200moe.ptr(record), b200moe.ptr(clean), 9, st))


def test_quantize_a8_padding_and_rejection(gpu, oracle):
    """Padded output stride keeps the padding (cpu_backend_host_tests.cpp:119-149); a partial group is rejected with
    every output untouched (:65-92)."""
    import b200moe
    from b200moe import ops
    x = np.full((2, 32), 127.0, np.float32)
    x[0, :] = 2.0 ** -120
    c, d, s = ops.enqueue_quantize_a8(dv(x, gpu))
    assert (host(c)[0] == 0).all() and (host(c)[1] == 127).all() and host(s)[1, 0] == 4064 and host(d)[0, 0] == 1.0
    codes = torch.full((2, 64), 17, dtype=torch.int8, device=gpu)
    deltas = torch.full((2, 2), 19.0, device=gpu)
    sums = torch.full((2, 2), 23, dtype=torch.int32, device=gpu)
    xs = dv(x, gpu)
    v = b200moe.QuantizeA8View(xs.data_ptr(), 2, 32, 32, 0, b200moe.A8Rows(codes.data_ptr(), deltas.data_ptr(), sums.data_ptr(), 2, 32, 64), None)
    b200moe.check(b200moe.lib().b200moe_quantize_a8(v, b200moe.stream_ptr()))
    assert (host(codes)[:, 32:] == 17).all() and (host(deltas)[:, 1] == 19.0).all() and (host(sums)[:, 1] == 23).all()
    for width in (31, 33):
        v = b200moe.QuantizeA8View(xs.data_ptr(), 1, width, 64, 0, b200moe.A8Rows(codes.data_ptr(), deltas.data_ptr(), sums.data_ptr(), 2, width, 64), None)
        before = host(codes).copy()
        with pytest.raises(b200moe.InvalidArgument):
            b200moe.check(b200moe.lib().b200moe_quantize_a8(v, b200moe.stream_ptr()))
        assert np.array_equal(host(codes), before)


def test_rmsnorm_a8(gpu, oracle):
    """RMSNorm + the A8 of its output in one launch, bit for bit the host rule (both lane counts, with / without the
    weight, in place, A8 only); a partial group is rejected; a non-finite row is flagged."""
    import b200moe
    from b200moe import ops
    rng = np.random.default_rng(12)
    for rows, n in ((1, 32), (3, 480), (8, 2048), (5, 7168)):
        x = (rng.standard_normal((rows, n)) * 3.0).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        for ww in (w, None):
            want = oracle.rmsnorm(x, ww, 1e-6)
            wc, wd, ws = oracle.quantize_a8(want)
            y, (c, d, sm) = ops.enqueue_rmsnorm_a8(dv(x, gpu), dv(ww, gpu) if ww is not None else None, 1e-6)
            assert same(host(y), want)
            assert np.array_equal(host(c), wc) and same(host(d), wd) and np.array_equal(host(sm), ws)
            y2, a8 = ops.enqueue_rmsnorm_a8(dv(x, gpu), dv(ww, gpu) if ww is not None else None, 1e-6, want_out=False)
            assert y2 is None and np.array_equal(host(a8[0]), wc)
    # in place
    xs = dv(x, gpu)
    v = b200moe.RmsnormView(xs.data_ptr(), rows, n, n, None, 1e-6, xs.data_ptr(), 0, b200moe.A8Rows(), None)
    b200moe.check(b200moe.lib().b200moe_rmsnorm_a8(v, b200moe.stream_ptr()))
    assert same(host(xs), oracle.rmsnorm(x, None, 1e-6))
    # rejection and status
    v = b200moe.RmsnormView(xs.data_ptr(), 1, 33, 64, None, 1e-6, xs.data_ptr(), 0, b200moe.A8Rows(), None)
    with pytest.raises(b200moe.InvalidArgument):
        b200moe.check(b200moe.lib().b200moe_rmsnorm_a8(v, b200moe.stream_ptr()))
    bad = x.copy()
    bad[1, 7] = np.inf
    status = torch.zeros(rows, dtype=torch.int32, device=gpu)
    ops.enqueue_rmsnorm_a8(dv(bad, gpu), None, 1e-6, status=status)
    st = host(status)
    assert st[1] == 2 and st[0] == 0


# ---------------------------------------------------------------------------------------------------------- Q8_0 GEMV
def test_q8_0_a8_dense(gpu, oracle):
    from b200moe import ops, synth
    rng = np.random.default_rng(12)
    for width, count, rows in ((32, 5, 1), (1024, 40, 3), (2048, 33, 8), (7168, 9, 11), (96, 7, 2), (2080, 6, 1)):
        w = synth.q8_0_blocks(rng, count * width // 32).reshape(count, -1)
        w[::3, 1] |= 0x80
        x = rng.standard_normal((rows, width), dtype=np.float32)
        if rows > 1:
            x[1, :32] = 0.0
        codes, deltas, _ = oracle.quantize_a8(x)
        want = oracle.gemv_q8_0_a8(w, width, codes, deltas)
        got = ops.enqueue_q8_0_a8(dv(w, gpu), width, dv(codes, gpu), dv(deltas, gpu))
        assert same(host(got), want), (width, count, rows)
        init = rng.standard_normal(want.shape, dtype=np.float32)
        want2 = oracle.gemv_q8_0_a8(w, width, codes, deltas, out=init.copy(), accumulate=True)
        got2 = ops.enqueue_q8_0_a8(dv(w, gpu), width, dv(codes, gpu), dv(deltas, gpu), out=dv(init, gpu), accumulate=True)
        assert same(host(got2), want2)


def test_q8_0_known_answers(gpu):
    """The reference's literal fixtures on the device: cancellation order (cpu_backend_host_tests.cpp:94-117) and
    subnormal half scales with an odd row stride (:119-149)."""
    from b200moe import ops
    w = np.zeros((1, 33 * 34), np.uint8)
    for g in range(33):
        w[0, g * 34 + 1] = 0x3C
        w[0, g * 34 + 2] = 1
    codes = np.ones((1, 33 * 32), np.int8)
    deltas = np.zeros((1, 33), np.float32)
    deltas[0, 0], deltas[0, 16], deltas[0, 1], deltas[0, 32] = 2.0 ** 24, -2.0 ** 24, 1.0, 1.0
    y = ops.enqueue_q8_0_a8(dv(w, gpu), 33 * 32, dv(codes, gpu), dv(deltas, gpu), out=torch.full((1, 1), -1.0, device=gpu))
    assert bits(host(y))[0, 0] == bits(np.float32(1.0))
    y = ops.enqueue_q8_0_a8(dv(w, gpu), 33 * 32, dv(codes, gpu), dv(deltas, gpu), out=torch.full((1, 1), -1.0, device=gpu), accumulate=True)
    assert bits(host(y))[0, 0] == bits(np.float32(0.0))
    w = np.zeros((2, 35), np.uint8)  # odd stride: rows are only byte aligned
    w[0, 0] = 1
    w[1, 0], w[1, 1] = 0xFF, 0x83
    w[:, 2:34] = 1
    codes = np.zeros((2, 64), np.int8)
    codes[1, :32] = 127
    deltas = np.ones((2, 2), np.float32)
    out = torch.full((2, 3), 29.0, device=gpu)
    ops.enqueue_q8_0_a8(dv(w, gpu), 32, dv(codes, gpu), dv(deltas, gpu), out=out, count=2)
    y = host(out)
    assert bits(y)[0, 0] == 0 and bits(y)[0, 1] == 0
    assert bits(y)[1, 0] == bits(np.float32(4064.0 * 2.0 ** -24)) and bits(y)[1, 1] == bits(np.float32(-4157472.0 * 2.0 ** -24))
    assert y[0, 2] == 29.0 and y[1, 2] == 29.0  # output padding untouched


def test_q8_0_rejects_partial_group(gpu):
    import b200moe
    from b200moe import ops
    w = torch.zeros((1, 68), dtype=torch.uint8, device=gpu)
    codes = torch.zeros((1, 64), dtype=torch.int8, device=gpu)
    deltas = torch.ones((1, 2), device=gpu)
    out = torch.full((1, 1), 29.0, device=gpu)
    for width in (31, 33):
        with pytest.raises(b200moe.InvalidArgument):
            ops.enqueue_q8_0_a8(w, width, codes, deltas, out=out)
    assert host(out)[0, 0] == 29.0


# ---------------------------------------------------------------------------------------------------------- router
class Lcg:
    def __init__(self, s):
        self.s = s

    def next(self):
        self.s = (self.s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        return (self.s >> 33) & 0xFFFFFFFF


def test_router_digest_on_device(gpu):
    """kDs41Digest (tests/route_policy_tests.cpp:211-242, :302) reproduced by the CUDA router."""
    from b200moe import ops
    g = Lcg(41)

    def logits(n):
        z = np.zeros(n, np.float32)
        for i in range(n):
            r = g.next()
            z[i] = np.float32(20.0 + (r % 7) * 0.5) if r % 97 == 0 else np.float32((int(r % 1025) - 512) / 64.0)
        return z

    def biases(n):
        b = np.zeros(n, np.float32)
        for i in range(n):
            r = g.next()
            b[i] = 0.0 if r % 3 == 0 else np.float32((int(r % 257) - 128) / 256.0)
        return b

    h = 1469598103934665603
    for experts, top_k, scale in ((256, 8, 2.5), (384, 6, 1.5), (64, 1, 2.0), (512, 16, 3.998)):
        w = logits(experts)
        b, bi = biases(experts), biases(experts)
        pol = policy_pair(O.ds41_policy(experts, top_k, scale))
        x = torch.ones((8, 1), device=gpu)
        out = {}
        for which, bb in (("b", b), ("bi", bi)):  # image rows alternate; each bias handles its 8 rows
            _, _, ids, wt = ops.enqueue_router(pol, x=x, weight=dv(w.reshape(experts, 1), gpu), bias=dv(bb, gpu))
            out[which] = (u32(ids), u32(wt))
        for r in range(16):
            ids, wt = out["bi" if r % 2 else "b"]
            for k in range(top_k):
                for v in (int(ids[r // 2, k]), int(wt[r // 2, k])):
                    for i in range(4):
                        h ^= (v >> (8 * i)) & 0xFF
                        h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    assert h == 0x168F06B494AE3B13


def test_router_policies(gpu, oracle):
    from b200moe import ops, synth
    rng = np.random.default_rng(13)
    # logits in the declared dot order, every config's router shape
    for experts, top_k, hidden, rows in ((64, 4, 2048, 1), (128, 8, 2048, 8), (256, 8, 7168, 5), (128, 8, 2048, 37), (32, 2, 96, 3),
                                        (256, 8, 7168, 64), (40, 3, 1100, 21), (24, 2, 100, 17), (16, 2, 98, 18)):
        x = rng.standard_normal((rows, hidden), dtype=np.float32)
        w = synth.router_weight(rng, experts, hidden)
        lb = synth.zipf_logit_bias(rng, experts)
        pol = O.softmax_policy(experts, top_k)
        for logit_bias in (None, lb):
            wl, ws, wi, ww = oracle.router(pol, x=x, w=w, logit_bias=logit_bias)
            gl, gs, gi, gw = ops.enqueue_router(policy_pair(pol), x=dv(x, gpu), weight=dv(w, gpu), logit_bias=dv(logit_bias, gpu))
            assert same(host(gl), wl) and same(host(gs), ws) and np.array_equal(u32(gi), wi) and same(host(gw), ww)
    # every transform / key / order with exact ties in the choices
    for score in (O.SOFTMAX, O.SIGMOID, O.SQRT_SOFTPLUS):
        for key in (O.FLOAT_SERIAL, O.ORDERED_BITS):
            for order in (O.SELECTION, O.ASCENDING_ID):
                for experts, top_k in ((64, 4), (128, 8), (512, 16), (1024, 32), (48, 1)):
                    logits = (rng.integers(-512, 513, size=(6, experts)) / 64.0).astype(np.float32)
                    logits[0, :] = 0.25
                    bias = (rng.integers(-128, 129, size=experts) / 256.0).astype(np.float32)
                    pol = O.RoutePolicy(score, 1, key, order, experts, top_k, 1, 1, 1, 1, 1e-20, 2.5)
                    _, ws, wi, ww = oracle.router(pol, logits=logits, bias=bias)
                    _, gs, gi, gw = ops.enqueue_router(policy_pair(pol), logits=dv(logits, gpu), bias=dv(bias, gpu))
                    assert same(host(gs), ws) and np.array_equal(u32(gi), wi) and same(host(gw), ww), (score, key, order, experts)


def test_router_nan_and_zero_literals(gpu, oracle):
    """tests/route_policy_tests.cpp:143-190 on the device (scores given through the sigmoid-free path: choice = bias)."""
    from b200moe import ops
    # selection works on choice = score + bias; a logit of 0 with sigmoid gives score 0.5 for all, so the bias decides
    z = np.zeros((1, 4), np.float32)
    for key in (O.FLOAT_SERIAL, O.ORDERED_BITS):
        for bias, want in (([-0.5, -0.5, -1.0, -2.0], [0, 1]), ([1.0, 3.0, 2.0, 0.5], [1, 2]), ([0.0, 0.0, 0.0, 0.0], [0, 1])):
            pol = O.RoutePolicy(O.SIGMOID, 1, key, O.SELECTION, 4, 2, 1, 1, 1, 1, 1e-20, 1.0)
            b = np.array(bias, np.float32)
            wi = oracle.router(pol, logits=z, bias=b)[2]
            gi = ops.enqueue_router(policy_pair(pol), logits=dv(z, gpu), bias=dv(b, gpu))[2]
            assert list(wi[0]) == want and list(u32(gi)[0]) == want
    # NaN choices: kept only as the first candidate under float_serial
    pol = O.RoutePolicy(O.SIGMOID, 1, O.FLOAT_SERIAL, O.SELECTION, 6, 3, 1, 1, 1, 1, 1e-20, 1.0)
    for b in ([np.nan, 3.0, 2.0, 1.0, 0.0, 0.5], [1.0, np.nan, 2.0, 3.0, np.nan, 0.0], [np.nan, np.nan, 1.0, 2.0, 0.0, 0.5]):
        b = np.array(b, np.float32)
        z6 = np.zeros((1, 6), np.float32)
        wi = oracle.router(pol, logits=z6, bias=b)[2]
        gi = ops.enqueue_router(policy_pair(pol), logits=dv(z6, gpu), bias=dv(b, gpu))[2]
        assert np.array_equal(u32(gi), wi), (b, wi, u32(gi))


def test_router_group_limited(gpu, oracle):
    """Config 4's router: sigmoid + bias, 8 groups, best 4 groups, top-8. The group step is this build's extension:
    checked against the oracle's restatement only (unpinned against the reference, which rejects n_group != 1)."""
    from b200moe import ops, synth
    rng = np.random.default_rng(14)
    for experts, top_k, ng, tg, hidden, rows in ((256, 8, 8, 4, 7168, 6), (64, 6, 4, 2, 256, 9), (32, 4, 8, 2, 64, 4)):
        x = rng.standard_normal((rows, hidden), dtype=np.float32)
        w = synth.router_weight(rng, experts, hidden)
        bias = (rng.standard_normal(experts) * 0.1).astype(np.float32)
        pol = O.sigmoid_group_policy(experts, top_k, ng, tg, 2.5)
        wl, ws, wi, ww = oracle.router(pol, x=x, w=w, bias=bias)
        gl, gs, gi, gw = ops.enqueue_router(policy_pair(pol), x=dv(x, gpu), weight=dv(w, gpu), bias=dv(bias, gpu))
        assert same(host(gs), ws) and np.array_equal(u32(gi), wi) and same(host(gw), ww)
        groups = np.unique(wi // (experts // ng), axis=None)
        assert all(len(np.unique(r // (experts // ng))) <= tg for r in wi)
    # ties between groups -> lower group id
    pol = O.sigmoid_group_policy(32, 4, 8, 2)
    z = np.zeros((1, 32), np.float32)
    b = np.zeros(32, np.float32)
    wi = oracle.router(pol, logits=z, bias=b)[2]
    gi = ops.enqueue_router(policy_pair(pol), logits=dv(z, gpu), bias=dv(b, gpu))[2]
    assert list(wi[0]) == [0, 1, 2, 3] and np.array_equal(u32(gi), wi)


# ---------------------------------------------------------------------------------------------------------- routes
def check_routes(r, want):
    n, m = int(want["counts"][0]), int(want["counts"][2])
    got_counts = u32(r.counts)
    assert np.array_equal(got_counts[:3], want["counts"][:3])
    assert np.array_equal(u32(r.experts)[:n], want["experts"][:n]) and np.array_equal(u32(r.begins)[:n + 1], want["begins"][:n + 1])
    assert np.array_equal(u32(r.rows)[:m], want["rows"][:m]) and np.array_equal(u32(r.slots)[:m], want["slots"][:m])
    assert np.array_equal(u32(r.order), want["order"]) and np.array_equal(u32(r.low_counts), want["low_counts"])


def test_routes(gpu, oracle):
    from b200moe import ops
    rng = np.random.default_rng(15)
    for rows, top_k, experts in ((1, 4, 64), (8, 8, 128), (40, 6, 32), (128, 8, 128), (129, 8, 256), (700, 8, 128), (4096, 8, 128), (33, 32, 1024)):
        ids = np.stack([rng.permutation(experts)[:top_k] for _ in range(rows)]).astype(np.uint32)
        split = experts // 2
        for first, end, base in ((0, 0, 0), (experts // 4, experts // 2, experts // 4), (experts // 2, experts, 0)):
            want = oracle.routes(ids, experts, split, first, end, base)
            r = ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), experts, split, first, end, base)
            check_routes(r, want)


def test_routes_invalid_ids_set_status(gpu):
    import b200moe
    from b200moe import ops
    ids = np.array([[3, 3, 1, 2], [0, 1, 2, 99], [4, 5, 6, 7]], np.int32)
    status = torch.zeros(3, dtype=torch.int32, device=gpu)
    r = ops.enqueue_moe_routes(dv(ids, gpu), 8, 4, row_status=status)
    st = host(status)
    assert st[0] == b200moe.ROW_INVALID_ROUTE and st[1] == b200moe.ROW_INVALID_ROUTE and st[2] == 0
    assert u32(r.counts)[2] == 10  # neither the out-of-range id nor the second occurrence of a repeated id gets an entry
    with pytest.raises(b200moe.InvalidArgument):
        ops.enqueue_moe_routes(dv(ids, gpu), 2000, 4)


# ---------------------------------------------------------------------------------------------------------- experts
def run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, form, parts=2, shared=None, first=0, end=0, exact=True, want=None):
    """Runs routes -> gate/up -> down -> combine stage by stage with taps; compares every stage with the oracle, bit for
    bit. exact=False (Qwen family): the A8 groups of h that differ are counted and `evaluations >> 26` of them allowed
    (the exp2 note in the file header; zero at the sizes used here), the stages behind them within the tolerance then."""
    from b200moe import ops
    rows, K = ids.shape
    H, I, E = sh.hidden, sh.inter, sh.experts
    codes, deltas, sums = oracle.quantize_a8(x)
    if want is None:
        want = oracle.experts(osh, gate, up, down, ids, codes, deltas, sums, first=first, end=end, taps=True)
    routes = ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), E, E // 2, first, end, 0)
    xa = (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu))
    g_gate, g_up, g_down = dv(gate, gpu), dv(up, gpu), dv(down, gpu)
    span = (end or E) - first
    mu = min(rows * K, span)
    act, g, u = ops.enqueue_routed_gate_up(sh, g_gate, g_up, routes, mu, xa, rows * K, taps=True)
    own = ((ids >= first) & (ids < (end or E))).reshape(-1)
    assert same(host(g)[own], want["gate"][own]) and same(host(u)[own], want["up"][own])
    raw = ops.enqueue_routed_down(sh, g_down, routes, mu, act)
    if exact:
        assert np.array_equal(host(act[0])[own], want["act_codes"][own])
        assert same(host(act[1])[own], want["act_deltas"][own]) and np.array_equal(host(act[2])[own], want["act_sums"][own])
        assert same(host(raw)[own], want["raw"][own])
    else:
        diff = (host(act[0])[own].reshape(-1, 32) != want["act_codes"][own].reshape(-1, 32)).any(axis=1)
        diff |= bits(host(act[1])[own]).reshape(-1) != bits(want["act_deltas"][own]).reshape(-1)
        allowed = (int(own.sum()) * I) >> 26
        assert int(diff.sum()) <= allowed, f"{int(diff.sum())} A8 groups of h differ, {allowed} allowed"
        if diff.any():
            assert max_rel(host(raw)[own], want["raw"][own]) <= REL_TOL
        else:
            assert np.array_equal(host(act[2])[own], want["act_sums"][own]) and same(host(raw)[own], want["raw"][own])
    exact = exact or not diff.any()
    if first == 0 and end == 0:
        pe = max(1, E // parts)
        wy = oracle.combine(form, want["raw"], wts, ids, shared=shared, parts=parts, part_experts=pe)
        gy = ops.enqueue_moe_combine(form, raw, dv(wts, gpu), dv(ids.view(np.int32), gpu), order=routes.order, shared=dv(shared, gpu),
                                     parts=parts, part_experts=pe)
        if exact:
            assert same(host(gy), wy)
        else:
            assert max_rel(host(gy), wy) <= REL_TOL
    return host(raw), want


def test_experts_q8_0_ds41_family(gpu, oracle):
    """Config-1 family (Q8_0 gate/up/down, declared_exp SwiGLU, (shared + low) + high): bit for bit."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(16)
    for E, H, I, K, rows, limit in ((8, 256, 128, 3, 5, 10.0), (16, 512, 256, 4, 1, math.inf), (6, 2048, 1024, 2, 19, math.inf),
                                    (4, 1280, 768, 2, 70, 7.0), (3, 256, 1536, 1, 33, math.inf), (2, 2304, 1024, 2, 9, math.inf)):
        gate, up, down = synth.expert_tensors(rng, E, H, I, 8, 8)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        shared = rng.standard_normal((rows, H), dtype=np.float32)
        sh, osh = shape_pair(H, I, E, K, 8, 8, limit)
        # one row per warp, the dp4a token-block form and the tensor-core form (each where the shape admits it; runs of 32
        # blocks, the last one partial)
        for form in (b200moe.FORM_AUTO, b200moe.FORM_SEGMENT_STREAM, b200moe.FORM_PER_BLOCK, b200moe.FORM_TENSOR):
            b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, form)
            try:
                run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_PARTS, shared=shared)
                run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_PARTS, first=E // 4, end=E // 2 + 1)
            finally:
                b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, b200moe.FORM_AUTO)


def test_experts_q2_k_ds41_family(gpu, oracle):
    """Q2_K tensors of the DS41 family (84-byte super-blocks, product_q2_k), alone and mixed with Q8_0, through the
    family's generic form: every stage bit for bit, with restricted expert ranges and experts of more than eight entries."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(17)
    for E, H, I, K, rows, limit in ((6, 512, 256, 2, 5, 7.0), (4, 2048, 1024, 2, 19, math.inf)):
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        shared = rng.standard_normal((rows, H), dtype=np.float32)
        for gt, dt in ((10, 10), (10, 8), (8, 10)):
            gate, up, down = synth.expert_tensors(rng, E, H, I, gt, dt)
            sh, osh = shape_pair(H, I, E, K, gt, dt, limit)
            run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_PARTS, shared=shared)
            run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_PARTS, first=E // 4, end=E // 2 + 1)


def test_experts_q4k_qwen_family(gpu, oracle):
    """Config-2 family (Q4_K gate/up, Q4_K or Q8_0 down, gfx1151-exp SwiGLU, fma merge)."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(17)
    for E, H, I, K, rows, dt in ((6, 512, 256, 2, 7, 12), (16, 2048, 768, 8, 4, 12), (8, 256, 512, 3, 21, 12), (6, 512, 256, 2, 7, 8),
                                 (4, 7168, 2048, 2, 3, 12), (4, 1280, 1024, 2, 2, 12), (5, 2560, 640, 3, 3, 8),
                                 (4, 256, 256, 2, 70, 12), (3, 512, 768, 2, 64, 12), (3, 256, 256, 2, 40, 12)):
        gate, up, _ = synth.expert_tensors(rng, E, H, I, 12, 12)
        down = (synth.q4_k_blocks(rng, E * H * (I // 256)) if dt == 12 else synth.q8_0_blocks(rng, E * H * (I // 32))).reshape(-1)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        sh, osh = shape_pair(H, I, E, K, 12, dt)
        want = want_part = None
        # every decode form of the Q4_K GEMVs on the same inputs: by plan, row streaming, segment streaming, per block
        for form in (b200moe.FORM_AUTO, b200moe.FORM_ROW_STREAM, b200moe.FORM_SEGMENT_STREAM, b200moe.FORM_PER_BLOCK):
            b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, form)
            try:
                _, want = run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, exact=False, want=want)
                _, want_part = run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, first=1, end=E - 1,
                                          exact=False, want=want_part)
            finally:
                b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, b200moe.FORM_AUTO)


def test_experts_other_formats_q5_k_q5_1(gpu, oracle):
    """The other stored formats of the same executor (routed_expert.hpp:27-28): Q5_K gate/up (the Q4_K rule with 5-bit
    quants) and Q5_1 down (four chains, d * dot + m * S): bit for bit, every combination with Q4_K / Q8_0, through
    the stages and through the layer call; a decode window and one beyond it."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(27)
    for E, H, I, K, rows, gt, dt in ((6, 512, 256, 2, 7, 13, 7), (8, 2048, 768, 4, 4, 13, 12), (5, 1280, 640, 3, 3, 12, 7),
                                     (4, 768, 512, 2, 9, 13, 8), (4, 256, 256, 2, 70, 13, 7), (3, 7168, 2048, 2, 2, 13, 7)):
        gate, up, down = synth.expert_tensors(rng, E, H, I, gt, dt)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        sh, osh = shape_pair(H, I, E, K, gt, dt)
        run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS)
        run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, first=1, end=E - 1)


def test_experts_q4k_grouped_tensor_core_form(gpu, oracle):
    """Windows of 128 rows and more take the grouped form (tcgen05 integer MMAs + the same FP32 chains): stage by stage
    against the oracle like the decode forms. Cases: several token tiles per expert with a ragged last one, experts with
    few tokens, an expert range (first / end), K = 256 (two stages per tile) and a wide K."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(31)
    for E, H, I, K, rows in ((4, 512, 256, 2, 300), (8, 256, 256, 3, 130), (16, 1024, 512, 4, 128), (3, 2048, 768, 2, 200)):
        gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        sh, osh = shape_pair(H, I, E, K, 12, 12)
        run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, exact=False)
        run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, first=1, end=E - 1, exact=False)


def test_experts_q4k_collisions_and_empty_experts(gpu, oracle):
    """Every row routed to the same two experts (64 entries per expert: many passes of the decode form; 200 entries:
    several token tiles of the grouped form), all other experts empty; and the opposite, one entry per expert."""
    import b200moe
    from b200moe import synth
    rng = np.random.default_rng(33)
    E, H, I, K = 12, 512, 256, 2
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    for rows in (64, 200):
        x = rng.standard_normal((rows, H), dtype=np.float32)
        ids = np.tile(np.array([[7, 2]], np.uint32), (rows, 1))
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        want = None
        for form in (b200moe.FORM_AUTO, b200moe.FORM_ROW_STREAM, b200moe.FORM_SEGMENT_STREAM):  # 64 entries: 8 virtual experts of 8
            b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, form)
            try:
                _, want = run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, wts, b200moe.COMBINE_FMA_SLOTS, exact=False, want=want)
            finally:
                b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, b200moe.FORM_AUTO)
    x = rng.standard_normal((6, H), dtype=np.float32)
    ids = np.arange(12, dtype=np.uint32).reshape(6, 2)
    run_stages(gpu, oracle, sh, osh, gate, up, down, x, ids, rng.uniform(0.05, 0.6, size=(6, K)).astype(np.float32),
               b200moe.COMBINE_FMA_SLOTS, exact=False)


def test_repeated_id_leaves_valid_rows_exact(gpu, oracle):
    """A row that names one expert twice is flagged INVALID_ROUTE and keeps only the first occurrence's entry; a valid row
    sharing that expert must stay bit-exact in every decode form (an expert never has more entries than the window has
    rows). The host builder throws on such a row (src/ds41_moe.cpp:22-23); a device path flags it and fails closed."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(35)
    E, H, I, K, rows = 6, 512, 256, 2, 2
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    ids = np.array([[3, 3], [3, 1]], np.uint32)   # row 0 repeats expert 3, row 1 uses it once
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    good = oracle.experts(osh, gate, up, down, np.array([[3, 1]], np.uint32), codes[1:], deltas[1:], sums[1:])["raw"]
    for form in (b200moe.FORM_AUTO, b200moe.FORM_ROW_STREAM, b200moe.FORM_SEGMENT_STREAM, b200moe.FORM_PER_BLOCK):
        b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, form)
        try:
            status = torch.zeros(rows, dtype=torch.int32, device=gpu)
            routes = ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), E, E // 2, row_status=status)
            assert list(host(status)) == [b200moe.ROW_INVALID_ROUTE, 0]
            assert u32(routes.counts)[2] == 3 and u32(routes.counts)[1] == 2   # three entries, at most two for one expert
            act = ops.enqueue_routed_gate_up(sh, dv(gate, gpu), dv(up, gpu), routes, 3, (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu)), rows * K)
            raw = host(ops.enqueue_routed_down(sh, dv(down, gpu), routes, 3, act))
            assert same(raw[2:4], good), form
        finally:
            b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, b200moe.FORM_AUTO)


def test_bounded_wait_runs_out_and_fails_closed(gpu, oracle):
    """No device wait is unbounded. With a poll limit of a few thousand and a producer that stops feeding before its first
    stage (both test hooks; nothing faults, no copy is left in flight), the segment-streaming gate/up kernel returns with
    B200MOE_JOB_WAIT_ABORTED in the job summary; the down stage and the combine then write nothing, and the host-buffer
    call reports B200MOE_ERR_ABORTED. The same call without the hooks is bit-exact afterwards."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(36)
    E, H, I, K, rows = 8, 512, 256, 2, 4
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    xa = (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu))
    ffn = ops.MoeFfn(sh, ops.softmax_policy(E, K), dv(gate, gpu), dv(up, gpu), dv(down, gpu), dv(rw, gpu), capacity=rows,
                     combine_form=b200moe.COMBINE_FMA_SLOTS)
    xh, yh = torch.from_numpy(x).pin_memory(), torch.full((rows, H), 5.0).pin_memory()
    b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, b200moe.FORM_SEGMENT_STREAM)
    b200moe.debug_set(b200moe.DEBUG_WAIT_LIMIT, 4096)
    b200moe.debug_set(b200moe.DEBUG_STALL_STAGE, 1)
    try:
        routes = ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), E, E // 2)
        summary = torch.zeros(4, dtype=torch.int32, device=gpu)
        act = ops.enqueue_routed_gate_up(sh, dv(gate, gpu), dv(up, gpu), routes, rows * K, xa, rows * K, summary=summary)
        torch.cuda.synchronize()                                   # the launch returned: nothing hangs
        assert u32(summary)[0] & b200moe.JOB_WAIT_ABORTED
        sentinel = torch.full((rows * K, H), 7.0, device=gpu)
        ops.enqueue_routed_down(sh, dv(down, gpu), routes, rows * K, act, raw=sentinel, summary=summary)
        y = ops.enqueue_moe_combine(b200moe.COMBINE_FMA_SLOTS, sentinel, dv(wts, gpu), dv(ids.view(np.int32), gpu), summary=summary, fill=9.0)
        assert (host(sentinel) == 7.0).all() and (host(y) == 9.0).all()
        with pytest.raises(b200moe.B200MoeError) as err:
            ffn.host(xh, yh)
        assert err.value.code == b200moe.ERR_ABORTED
    finally:
        for key in (b200moe.DEBUG_DECODE_FORM, b200moe.DEBUG_WAIT_LIMIT, b200moe.DEBUG_STALL_STAGE):
            b200moe.debug_set(key, 0)
    want = oracle.ffn(osh, O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_FMA_SLOTS)
    ffn.host(xh, yh)
    assert same(yh.numpy(), want["y"])


def test_routes_maximum_sizes(gpu, oracle):
    """1024 experts and top-32 (the ABI's limits), one-block and chunked windows, with an owned expert range."""
    from b200moe import ops
    rng = np.random.default_rng(34)
    for rows, first, end in ((8, 0, 0), (70, 0, 0), (70, 256, 768)):
        ids = np.stack([rng.permutation(1024)[:32] for _ in range(rows)]).astype(np.uint32)
        want = oracle.routes(ids, 1024, 512, first, end, first)
        check_routes(ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), 1024, 512, first, end, first), want)


def test_experts_fail_closed(gpu, oracle):
    """A non-finite projection sets status bit 8 on its row, the summary word, and the down stage writes nothing
    (src/cpu/core/routed_expert.hpp:17-19; host-side injection as tests/cpu/routed_expert_host_tests.cpp:393-399)."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(18)
    E, H, I, K, rows = 6, 512, 256, 2, 4
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    deltas[2, 0] = 3e38
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    want = oracle.experts(osh, gate, up, down, ids, codes, deltas, sums)
    routes = ops.enqueue_moe_routes(dv(ids.view(np.int32), gpu), E, E // 2)
    status = torch.zeros(rows, dtype=torch.int32, device=gpu)
    summary = torch.zeros(4, dtype=torch.int32, device=gpu)
    act = ops.enqueue_routed_gate_up(sh, dv(gate, gpu), dv(up, gpu), routes, rows * K, (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu)),
                                     rows * K, row_status=status, summary=summary)
    sentinel = torch.full((rows * K, H), 7.0, device=gpu)
    ops.enqueue_routed_down(sh, dv(down, gpu), routes, rows * K, act, raw=sentinel, summary=summary)
    st = host(status)
    assert np.array_equal(st != 0, want["status"] != 0) and st[2] == b200moe.ROW_PROJECTION_NONFINITE
    assert host(summary)[0] == b200moe.ROW_PROJECTION_NONFINITE and (host(sentinel) == 7.0).all()


# ---------------------------------------------------------------------------------------------------------- whole layer
def test_ffn_config1_q8_0(gpu, oracle):
    """Config 1: hidden 2048, 64 experts, top-4, inter 1024, Q8_0, batch 1, 16 decode steps, seed 0 - bit for bit."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(0)
    E, H, I, K = 64, 2048, 1024, 4
    gate, up, down = synth.expert_tensors(rng, E, H, I, 8, 8)
    rw = synth.router_weight(rng, E, H)
    sh, osh = shape_pair(H, I, E, K, 8, 8)
    ffn = ops.MoeFfn(sh, ops.softmax_policy(E, K), dv(gate, gpu), dv(up, gpu), dv(down, gpu), dv(rw, gpu), capacity=1,
                     combine_form=b200moe.COMBINE_PARTS, parts=2)
    for step in range(16):
        x = synth.activations(rng, 1, H)
        want = oracle.ffn(osh, O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_PARTS, parts=2)
        y, ids, wts = ffn(dv(x, gpu), want_routes=True)
        assert np.array_equal(u32(ids), want["ids"]) and same(host(wts), want["weights"]), step
        assert same(host(y), want["y"]), step


def test_ffn_config2_q4k(gpu, oracle):
    """Config 2: hidden 2048, 128 experts, top-8, inter 768, Q4_K; batch 1, 4 and 8. Expert ids bit-exact, outputs
    within 1e-3 (reported exact when they are), against the A8-contract oracle; the distance of both to float truth
    is reported beside it."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(2)
    E, H, I, K = 128, 2048, 768, 8
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    ffn = ops.MoeFfn(sh, ops.softmax_policy(E, K), dv(gate, gpu), dv(up, gpu), dv(down, gpu), dv(rw, gpu), capacity=8,
                     combine_form=b200moe.COMBINE_FMA_SLOTS)
    for batch in (1, 4, 8):
        x = synth.activations(rng, batch, H)
        want = oracle.ffn(osh, O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_FMA_SLOTS)
        y, ids, wts = ffn(dv(x, gpu), want_routes=True)
        assert np.array_equal(u32(ids), want["ids"]) and same(host(wts), want["weights"])
        err = max_rel(host(y), want["y"])
        assert err <= REL_TOL
        truth = oracle.float_truth(osh, gate, up, down, want["ids"], want["weights"], x)
        print(f"config2 batch {batch}: bit-exact={same(host(y), want['y'])} max_rel vs A8 oracle {err:.2e}; "
              f"A8 contract vs float truth {max_rel(want['y'], truth):.2e}")
    # the host-buffer call gives the same bits as the device call
    x = synth.activations(rng, 8, H)
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty((8, H), dtype=torch.float32).pin_memory()
    ffn.host(xh, yh)
    y = ffn(dv(x, gpu))
    torch.cuda.synchronize()
    assert same(yh.numpy(), host(y))


def test_ffn_config3_prefill_zipf(gpu, oracle):
    """Config 3 at reduced size: a token block with bf16-rounded activations and a Zipf(1.1) logit bias (skewed expert
    load, some experts empty) through the whole call: tiled router logits, chunked routes, grouped tensor-core experts,
    slot-order merge. Ids bit-exact, outputs within tolerance (reported exact when they are)."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(3)
    E, H, I, K, rows = 32, 512, 256, 4, 700
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    bias = synth.zipf_logit_bias(rng, E)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    ffn = ops.MoeFfn(sh, ops.softmax_policy(E, K), dv(gate, gpu), dv(up, gpu), dv(down, gpu), dv(rw, gpu), capacity=rows,
                     combine_form=b200moe.COMBINE_FMA_SLOTS, logit_bias=dv(bias, gpu))
    x = synth.bf16_round(synth.activations(rng, rows, H))
    want = oracle.ffn(osh, O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_FMA_SLOTS, logit_bias=bias)
    y, ids, wts = ffn(dv(x, gpu), want_routes=True)
    assert np.array_equal(u32(ids), want["ids"]) and same(host(wts), want["weights"])
    counts = np.bincount(want["ids"].reshape(-1), minlength=E)
    assert max_rel(host(y), want["y"]) <= REL_TOL
    print(f"config3-like: rows/expert max {counts.max()} min {counts.min()}; bit-exact={same(host(y), want['y'])}")


def test_ffn_config4_group_limited_shared_expert(gpu, oracle):
    """Config 4 at reduced size: sigmoid scores + selection bias, group-limited top-k (8 groups, best 4), Q4_K routed
    experts folded in 8 expert ranges onto a dense Q8_0 shared expert: y = ((shared + S_0) + ...) + S_7. A decode window
    and a token block. The group step is this build's extension: the oracle restates it (parity unpinned for it)."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(4)
    E, H, I, K = 64, 512, 256, 8
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    sg, su, sd = synth.expert_tensors(rng, 1, H, I, 8, 8)
    rw = synth.router_weight(rng, E, H)
    sbias = (rng.standard_normal(E) * 0.1).astype(np.float32)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    ssh, sosh = shape_pair(H, I, 1, 1, 8, 8)
    pol, opol = ops.sigmoid_group_policy(E, K, 8, 4), O.sigmoid_group_policy(E, K, 8, 4)
    for rows in (64, 200):
        ffn = ops.MoeFfn(sh, pol, dv(gate, gpu), dv(up, gpu), dv(down, gpu), dv(rw, gpu), capacity=rows, combine_form=b200moe.COMBINE_PARTS,
                         parts=8, select_bias=dv(sbias, gpu))
        x = synth.bf16_round(synth.activations(rng, rows, H))
        codes, deltas, sums = oracle.quantize_a8(x)
        shared_want = oracle.experts(sosh, sg, su, sd, np.zeros((rows, 1), np.uint32), codes, deltas, sums)["raw"]
        shared = ops.enqueue_dense_ffn(ssh, dv(sg, gpu), dv(su, gpu), dv(sd, gpu), ops.enqueue_quantize_a8(dv(x, gpu)))
        assert same(host(shared), shared_want)   # the Q8_0 family is bit-exact
        want = oracle.ffn(osh, opol, gate, up, down, rw, x, O.COMBINE_PARTS, parts=8, part_experts=E // 8, shared=shared_want, select_bias=sbias)
        y, ids, wts = ffn(dv(x, gpu), shared=shared, want_routes=True)
        assert np.array_equal(u32(ids), want["ids"]) and same(host(wts), want["weights"])
        assert max_rel(host(y), want["y"]) <= REL_TOL
        print(f"config4-like rows {rows}: bit-exact={same(host(y), want['y'])}")


def test_layer_expert_parallel_fold(gpu, oracle):
    """Expert-parallel split on one device: each of `parts` virtual ranks owns a contiguous expert range, produces its
    partial sum (only_part), and the fixed-order fold equals the unsplit layer bit for bit (the reference's 2-rank
    form, src/ds41_moe.cpp:45-61, :99-115, generalised to 8 ranks)."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(19)
    E, H, I, K, rows, parts = 32, 512, 256, 6, 9, 8
    gate, up, down = synth.expert_tensors(rng, E, H, I, 8, 8)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
    shared = rng.standard_normal((rows, H), dtype=np.float32)
    sh, osh = shape_pair(H, I, E, K, 8, 8)
    codes, deltas, sums = oracle.quantize_a8(x)
    xa = (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu))
    layer = ops.MoeLayer(sh, dv(gate, gpu), dv(up, gpu), dv(down, gpu), rows, b200moe.COMBINE_PARTS, parts=parts)
    gi, gw = dv(ids.view(np.int32), gpu), dv(wts, gpu)
    full = host(layer(xa, gi, gw, shared=dv(shared, gpu)))
    ex = oracle.experts(osh, gate, up, down, ids, codes, deltas, sums)
    want = oracle.combine(O.COMBINE_PARTS, ex["raw"], wts, ids, shared=shared, parts=parts, part_experts=E // parts)
    assert same(full, want)
    per = E // parts
    acc = torch.from_numpy(shared).to(gpu)
    for p in range(parts):
        part = layer(xa, gi, gw, first=p * per, end=(p + 1) * per, base=0, only_part=p)
        wp = oracle.combine(O.COMBINE_PARTS, ex["raw"], wts, ids, parts=parts, part_experts=per, only_part=p)
        assert same(host(part), wp)
        acc = acc + part  # one FP32 add per rank, in rank order
    assert same(host(acc), want)
    # a rank holding only its slice of the tensors: base = first
    p = 3
    sl = slice(p * per, (p + 1) * per)
    gsl = gate.reshape(E, -1)[sl].reshape(-1)
    usl = up.reshape(E, -1)[sl].reshape(-1)
    dsl = down.reshape(E, -1)[sl].reshape(-1)
    layer_p = ops.MoeLayer(sh, dv(gsl, gpu), dv(usl, gpu), dv(dsl, gpu), rows, b200moe.COMBINE_PARTS, parts=parts)
    part = layer_p(xa, gi, gw, first=p * per, end=(p + 1) * per, base=p * per, only_part=p)
    assert same(host(part), oracle.combine(O.COMBINE_PARTS, ex["raw"], wts, ids, parts=parts, part_experts=per, only_part=p))


def test_ep_entry_point_single_rank(gpu, oracle):
    """b200moe_ep_ffn with one rank: the same kernels as on N GPUs (route, dispatch into the rank's own window, flag
    waits, restricted routes, combine through the block table, fold), compared with the oracle's PARTS combine with one
    part; FP32 and bfloat16 inputs, five steps (both halves of the window, the device step counter)."""
    import b200moe
    from b200moe import ep, ops, synth
    rng = np.random.default_rng(41)
    E, H, I, K, rows = 16, 512, 256, 4, 5
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    sh, osh = shape_pair(H, I, E, K, 12, 12)
    for fold in (0, 4):   # 0: one expert range per rank; 4: the rank returns the sums of four ranges, folded in order
        layer = ep.PeerEpFfn(sh, ops.softmax_policy(E, K), dv(rw, gpu), dv(gate, gpu), dv(up, gpu), dv(down, gpu), rows, fold_parts=fold)
        summary = torch.zeros(1, dtype=torch.int32, device=gpu)
        try:
            for step in range(5):
                x = synth.bf16_round(synth.activations(rng, rows, H))
                shared = rng.standard_normal((rows, H), dtype=np.float32)
                want = oracle.ffn(osh, O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_PARTS, parts=max(fold, 1), part_experts=E // max(fold, 1),
                                  shared=shared)
                gx = dv(x, gpu).to(torch.bfloat16) if step % 2 else dv(x, gpu)
                y = layer(gx, dv(shared, gpu), summary=summary)
                assert same(host(y), want["y"]), (fold, step)
                assert host(summary)[0] == 0
        finally:
            layer.close()


def test_ep_wait_for_a_silent_peer_is_bounded(gpu, oracle):
    """Failure detection without a fault: a two-rank set-up whose second window belongs to nobody, so no peer ever signals.
    The dispatch wait gives up after wait_polls polls (well under a second here), the step returns, the job summary holds
    B200MOE_JOB_WAIT_ABORTED and y keeps the caller's bytes; the device stays usable (a normal call follows)."""
    import b200moe
    from b200moe import ep, ops, synth
    rng = np.random.default_rng(42)
    E, H, I, K, rows = 16, 512, 256, 4, 3
    gate, up, down = synth.expert_tensors(rng, E // 2, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    sh, _ = shape_pair(H, I, E, K, 12, 12)
    layer = ep.PeerEpFfn(sh, ops.softmax_policy(E, K), dv(rw, gpu), dv(gate, gpu), dv(up, gpu), dv(down, gpu), rows, wait_polls=2000,
                         extra_windows=1)
    try:
        summary = torch.zeros(1, dtype=torch.int32, device=gpu)
        y = torch.full((rows, H), 3.0, device=gpu)
        layer(dv(synth.activations(rng, rows, H), gpu), y=y, summary=summary)
        torch.cuda.synchronize()
        assert u32(summary)[0] & b200moe.JOB_WAIT_ABORTED
        assert (host(y) == 3.0).all()
    finally:
        layer.close()
    test_quantize_a8(gpu, oracle)   # the context is intact


def test_tp_entry_point_single_rank(gpu, oracle):
    """b200moe_tp_dense with one rank (the kernels of the N-GPU path: share, scatter into the rank's own window, flag
    wait, fold): FP32 payload = the dense block's bits, bfloat16 payload = its bfloat16 rounding widened; four steps."""
    from b200moe import ops, synth, tp
    rng = np.random.default_rng(43)
    H, I, rows = 512, 768, 3
    gate, up, down = synth.expert_tensors(rng, 1, H, I, 12, 12)
    sh, osh = shape_pair(H, I, 1, 1, 12, 12)
    for bf16 in (False, True):
        layer = tp.PeerTpDense(sh, dv(gate, gpu), dv(up, gpu), dv(down, gpu), rows, payload_bf16=bf16)
        summary = torch.zeros(1, dtype=torch.int32, device=gpu)
        try:
            for step in range(4):
                x = rng.standard_normal((rows, H), dtype=np.float32)
                codes, deltas, sums = oracle.quantize_a8(x)
                want = oracle.experts(osh, gate, up, down, np.zeros((rows, 1), np.uint32), codes, deltas, sums)["raw"]
                if bf16:
                    want = (synth.bf16_bits(want).astype(np.uint32) << 16).view(np.float32)
                y = layer(dv(x, gpu), summary=summary)
                assert same(host(y), want), (bf16, step)
                assert host(summary)[0] == 0
        finally:
            layer.close()
    # a silent second rank: the fold's bounded wait runs out, y is not written, the status says so
    layer = tp.PeerTpDense(sh, dv(gate, gpu), dv(up, gpu), dv(down, gpu), rows, wait_polls=2000, extra_windows=1)
    try:
        summary = torch.zeros(1, dtype=torch.int32, device=gpu)
        y = torch.full((rows, H), 3.0, device=gpu)
        layer(dv(rng.standard_normal((rows, H), dtype=np.float32), gpu), summary=summary, y=y)
        torch.cuda.synchronize()
        import b200moe
        assert u32(summary)[0] & b200moe.JOB_WAIT_ABORTED and (host(y) == 3.0).all()
    finally:
        layer.close()


def test_dense_ffn_tensor_parallel_split(gpu, oracle):
    """Config-5 family at reduced size: dense Q4_K SwiGLU block, column-parallel gate/up and row-parallel down over
    whole super-blocks; each share's partial equals the oracle's partial bit for bit (modulo the SwiGLU note above),
    and their rank-ordered sum stays within the tolerance of the unsplit block."""
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(20)
    H, I, rows = 512, 1792, 5  # 7 super-blocks of inter: uneven shares 2, 2, 2, 1
    gate, up, down = synth.expert_tensors(rng, 1, H, I, 12, 12)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    codes, deltas, sums = oracle.quantize_a8(x)
    xa = (dv(codes, gpu), dv(deltas, gpu), dv(sums, gpu))
    ids = np.zeros((rows, 1), np.uint32)
    sh, osh = shape_pair(H, I, 1, 1, 12, 12)
    want = oracle.experts(osh, gate, up, down, ids, codes, deltas, sums)["raw"]
    y, yb = ops.enqueue_dense_ffn(sh, dv(gate, gpu), dv(up, gpu), dv(down, gpu), xa, bf16=True)
    assert max_rel(host(y), want) <= REL_TOL
    assert np.array_equal(host(yb.view(torch.int16)).view(np.uint16), synth.bf16_bits(host(y)))
    shares = [(0, 2), (2, 4), (4, 6), (6, 7)]
    g2 = gate.reshape(I, -1)
    u2 = up.reshape(I, -1)
    d3 = down.reshape(H, I // 256, 144)
    total = np.zeros_like(want)
    for b0, b1 in shares:
        Il = (b1 - b0) * 256
        gs, us = g2[b0 * 256:b1 * 256].reshape(-1), u2[b0 * 256:b1 * 256].reshape(-1)
        ds = np.ascontiguousarray(d3[:, b0:b1]).reshape(-1)
        shl, oshl = shape_pair(H, Il, 1, 1, 12, 12)
        wp = oracle.experts(oshl, gs, us, ds, ids, codes, deltas, sums)["raw"]
        gp = host(ops.enqueue_dense_ffn(shl, dv(gs, gpu), dv(us, gpu), dv(ds, gpu), xa))
        assert max_rel(gp, wp) <= REL_TOL
        total = total + gp
    assert max_rel(total, want) <= REL_TOL


def test_empty_and_argument_errors(gpu):
    import b200moe
    from b200moe import ops, synth
    rng = np.random.default_rng(21)
    sh, _ = shape_pair(512, 256, 8, 2, 12, 12)
    gate, up, down = (dv(a, gpu) for a in synth.expert_tensors(rng, 8, 512, 256, 12, 12))
    rw = dv(synth.router_weight(rng, 8, 512), gpu)
    ffn = ops.MoeFfn(sh, ops.softmax_policy(8, 2), gate, up, down, rw, capacity=4, combine_form=b200moe.COMBINE_FMA_SLOTS)
    y = torch.full((4, 512), 5.0, device=gpu)
    ffn(torch.zeros((0, 512), device=gpu), y=y)  # zero rows: nothing is written
    assert (host(y) == 5.0).all()
    with pytest.raises(b200moe.InvalidArgument):
        ffn(torch.zeros((5, 512), device=gpu))  # beyond the workspace capacity
    with pytest.raises(b200moe.InvalidArgument):
        ops.MoeFfn(shape_pair(500, 256, 8, 2, 12, 12)[0], ops.softmax_policy(8, 2), gate, up, down, rw, 4, b200moe.COMBINE_FMA_SLOTS)
    with pytest.raises(b200moe.InvalidArgument):
        ops.MoeFfn(shape_pair(512, 256, 8, 2, 8, 12)[0], ops.softmax_policy(8, 2), gate, up, down, rw, 4, b200moe.COMBINE_FMA_SLOTS)
    # all-zero activations: delta 1, codes 0, outputs exactly +0
    y = ffn(torch.zeros((2, 512), device=gpu))
    assert (bits(host(y)) == 0).all()


def test_golden_vectors_on_device(gpu):
    """The committed vectors generated from the reference's own CPU code (tests/golden/make_golden.py)."""
    import os
    import b200moe
    from b200moe import ops
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "moe_golden.npz"))
    c, d, s = ops.enqueue_quantize_a8(dv(g["a8_x"], gpu))
    assert np.array_equal(host(c), g["a8_codes"]) and same(host(d), g["a8_deltas"]) and np.array_equal(host(s), g["a8_sums"])
    y = ops.enqueue_q8_0_a8(dv(g["q8_w"], gpu), int(g["q8_width"]), dv(g["q8_codes"], gpu), dv(g["q8_deltas"], gpu))
    assert same(host(y), g["q8_y"])
    pol = policy_pair(O.ds41_policy(int(g["rt_w"].shape[0]), int(g["rt_ids"].shape[1]), 1.5))
    _, sc, ids, wt = ops.enqueue_router(pol, x=dv(g["rt_x"], gpu), weight=dv(g["rt_w"], gpu), bias=dv(g["rt_bias"], gpu))
    assert same(host(sc), g["rt_scores"]) and np.array_equal(u32(ids), g["rt_ids"]) and same(host(wt), g["rt_weights"])
    pol = policy_pair(O.softmax_policy(int(g["sm_logits"].shape[1]), int(g["sm_ids"].shape[1])))
    _, sc, ids, wt = ops.enqueue_router(pol, logits=dv(g["sm_logits"], gpu))
    assert same(host(sc), g["sm_scores"]) and np.array_equal(u32(ids), g["sm_ids"]) and same(host(wt), g["sm_weights"])
    # DS41 window
    E, H, I, K = (int(v) for v in g["win_shape"])
    sh, _ = shape_pair(H, I, E, K, 8, 8, float(g["win_limit"]))
    xa = ops.enqueue_quantize_a8(dv(g["win_x"], gpu))
    layer = ops.MoeLayer(sh, dv(g["win_gate"], gpu), dv(g["win_up"], gpu), dv(g["win_down"], gpu), g["win_x"].shape[0], b200moe.COMBINE_PARTS, parts=2)
    y, raw = layer(xa, dv(g["win_ids"].view(np.int32), gpu), dv(g["win_weights"], gpu), shared=dv(g["win_shared"], gpu), want_raw=True)
    assert same(host(raw), g["win_raw"]) and same(host(y), g["win_y"])
    # Qwen job: Q4_K gate/up, Q8_0 four-chain down (reference_run)
    E, H, I, K = (int(v) for v in g["qw_shape"])
    sh, _ = shape_pair(H, I, E, K, 12, 8)
    xa = ops.enqueue_quantize_a8(dv(g["qw_x"], gpu))
    layer = ops.MoeLayer(sh, dv(g["qw_gate"], gpu), dv(g["qw_up"], gpu), dv(g["qw_down"], gpu), g["qw_x"].shape[0], b200moe.COMBINE_FMA_SLOTS)
    rows = g["qw_x"].shape[0]
    _, raw = layer(xa, dv(g["qw_ids"].view(np.int32), gpu), torch.ones((rows, K), device=gpu), want_raw=True)
    assert max_rel(host(raw), g["qw_raw"]) <= REL_TOL
    print("golden qwen job bit-exact:", same(host(raw), g["qw_raw"]))
