"""b200moe_build_routes_static: the routes build with the library's built-in device scratch.

Collected last (file name) so that it also runs after every other GPU test has used the device; it passes alone too.
Every call goes through the C ABI. The check is equality with b200moe_build_routes (caller scratch) on the same ids, on
two calls in a row with different windows, so that what the first call leaves in the shared array cannot leak into the
second."""
import ctypes as C

import numpy as np
import pytest
import torch

import b200moe
from b200moe import ops

FIELDS = ("experts", "begins", "rows", "slots", "order", "low_counts", "counts")


def _ids(rows, top_k, experts, seed):
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(experts)[:top_k] for _ in range(rows)]).astype(np.int32)
    return torch.from_numpy(ids).cuda()


def _same(a, b, rows, top_k):
    n = rows * top_k
    union = int(a.counts[0].item())
    assert torch.equal(a.counts, b.counts)
    assert torch.equal(a.experts[:union], b.experts[:union])
    assert torch.equal(a.begins[:union + 1], b.begins[:union + 1])
    total = int(a.counts[2].item())
    assert torch.equal(a.rows[:total], b.rows[:total]) and torch.equal(a.slots[:total], b.slots[:total])
    assert torch.equal(a.order[:n], b.order[:n]) and torch.equal(a.low_counts, b.low_counts)


@pytest.mark.gpu
def test_static_routes_match_on_two_calls_in_a_row():
    # chunked form (more than 1024 slots), then a different window with fewer experts and another expert range,
    # then a one-block window (no scratch at all)
    cases = [(3000, 8, 128, 0, 0, 0, 11), (1500, 6, 256, 64, 192, 64, 12), (5, 8, 128, 0, 0, 0, 13)]
    for rows, top_k, experts, first, end, base, seed in cases:
        ids = _ids(rows, top_k, experts, seed)
        want = ops.enqueue_moe_routes(ids, experts, experts // 2, first, end, base)
        got = ops.enqueue_moe_routes_static(ids, experts, experts // 2, first, end, base)
        torch.cuda.synchronize()
        _same(want, got, rows, top_k)
    # and the very same window twice into the same outputs: the second call sees the first call's leftovers
    ids = _ids(3000, 8, 128, 21)
    want = ops.enqueue_moe_routes(ids, 128, 64)
    got = ops.enqueue_moe_routes_static(ids, 128, 64)
    got = ops.enqueue_moe_routes_static(ids, 128, 64, out=got)
    torch.cuda.synchronize()
    _same(want, got, 3000, 8)
    # the point of the entry: calls made after the per-device set-up take no device memory - neither from the driver
    # (cudaMemGetInfo) nor from torch's allocator - with every output preallocated by the caller
    L = b200moe.lib()
    v = b200moe.RoutesView(b200moe.ptr(ids), 3000, 8, 128, 64, 0, 0, 0, None, None, got.struct())
    torch.cuda.synchronize()
    free0, stats0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(20):
        assert L.b200moe_build_routes_static(C.byref(v), b200moe.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == stats0 and torch.cuda.memory_reserved() == reserved0
    _same(want, got, 3000, 8)


def test_static_routes_refuse_windows_beyond_the_array():
    L = b200moe.lib()
    limit = int(L.b200moe_routes_static_max_words())
    assert limit == 65 * 1024 + 4
    rows, top_k, experts = 70000, 1, 1024  # 69 chunks at 1024 experts
    assert int(L.b200moe_routes_scratch_words(rows, top_k, experts)) > limit
    v = b200moe.RoutesView(rows=rows, top_k=top_k, experts=experts)
    rc = L.b200moe_build_routes_static(C.byref(v), None)
    assert rc == b200moe.ERR_UNSUPPORTED
    msg = L.b200moe_last_error().decode()
    assert "scratch words" in msg and str(limit) in msg
