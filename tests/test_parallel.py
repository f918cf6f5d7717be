"""Multi-rank paths: expert parallelism (b200moe.ep) and the tensor-parallel dense block (b200moe.tp).

CPU (not gpu): world_size 2 over gloo. The exchange logic is the shipped one; the per-rank arithmetic is the oracle
stand-in of tests/parallel_worker.py. The result must equal the oracle's single-process run over the whole window with
`world` virtual ranks, bit for bit.
GPU (needs 2 devices, skipped otherwise): the same over NCCL with the C library on every rank.
"""
import os
import socket
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from oracle import loader as O

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import parallel_worker as W  # noqa: E402

REL_TOL = 1e-3


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(case, backend, world):
    out = tempfile.mkdtemp(prefix="b200moe_ranks_")
    port = free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "parallel_worker.py"), "--case", case, "--backend", backend,
                                       "--out", out], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace"))
    assert all(p.returncode == 0 for p in procs), "\n".join(logs)
    return [np.load(os.path.join(out, f"rank{r}.npy")) for r in range(world)]


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def max_rel(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


def ep_expected(oracle, form, world, x_scale=1.0):
    gate, up, down, rw, x, shared = W.ep_inputs(world)
    sh = O.Shape(W.H, W.I, W.E, W.K, 12, 12, float("inf"))
    return oracle.ffn(sh, O.softmax_policy(W.E, W.K), gate, up, down, rw, x * np.float32(x_scale), form, parts=world, part_experts=W.E // world,
                      shared=shared)["y"]


def tp_expected(oracle, world, x_scale=1.0, bf16=False):
    from b200moe import synth
    gate, up, down, x = W.tp_inputs()
    codes, deltas, sums = oracle.quantize_a8(x * np.float32(x_scale))
    ids = np.zeros((W.DROWS, 1), np.uint32)
    acc = np.zeros((W.DROWS, W.DH), np.float32)
    for start, size in __import__("b200moe").tp.tp_shares(W.DI, world):
        gs, us, ds = W.tp_slices(gate, up, down, start, size)
        part = oracle.experts(O.Shape(W.DH, size, 1, 1, 12, 12, float("inf")), gs, us, ds, ids, codes, deltas, sums)["raw"]
        if bf16:   # the payload crosses the link as bfloat16 (RNE) and is widened before the FP32 fold
            part = (synth.bf16_bits(part).astype(np.uint32) << 16).view(np.float32)
        acc = (acc + part).astype(np.float32)
    return acc


def test_tp_shares():
    from b200moe import tp
    assert [s for _, s in tp.tp_shares(17408, 8)] == [9 * 256] * 4 + [8 * 256] * 4
    assert [s for _, s in tp.tp_shares(17408, 2)] == [34 * 256] * 2
    assert tp.tp_shares(1792, 2) == [(0, 1024), (1024, 768)]


@pytest.mark.parametrize("case,form,world", [("ep_parts", 0, 2), ("ep_fma", 1, 2), ("ep_parts", 0, 4)])
def test_expert_parallel_ranks_gloo(oracle, case, form, world):
    ys = run_ranks(case, "gloo", world)
    want = ep_expected(oracle, form, world)
    got = np.concatenate(ys)
    assert np.array_equal(bits(got), bits(want))


def test_tensor_parallel_two_ranks_gloo(oracle):
    world = 2
    ys = run_ranks("tp", "gloo", world)
    want = tp_expected(oracle, world)
    for y in ys:                                  # every rank holds the whole y
        assert np.array_equal(bits(y), bits(want))
    ya = run_ranks("tp_allreduce", "gloo", world)  # sum order is the library's: tolerance, and the ranks agree
    assert max_rel(ya[0], want) <= REL_TOL and np.array_equal(bits(ya[0]), bits(ya[1]))


def _two_gpus():
    torch = pytest.importorskip("torch")
    return torch.cuda.is_available() and torch.cuda.device_count() >= 2


@pytest.mark.gpu
@pytest.mark.parametrize("case,form", [("ep_parts", 0), ("ep_parts_peer", 0), ("ep_fma", 1)])
def test_expert_parallel_two_gpus_nccl(oracle, case, form):
    if not _two_gpus():
        pytest.skip("needs 2 CUDA devices")
    world = 2
    got = np.concatenate(run_ranks(case, "nccl", world))
    want = ep_expected(oracle, form, world)
    # the Qwen-family SwiGLU may differ by one code in rare elements (see test_gpu_parity.py): tolerance, bits reported
    assert max_rel(got, want) <= REL_TOL
    print("bit-exact:", np.array_equal(bits(got), bits(want)))


@pytest.mark.gpu
def test_expert_parallel_two_gpus_c_abi(oracle):
    """b200moe_ep_ffn on two GPUs: dispatch and return are the library's peer stores with flag waits (no collective);
    five steps, the last one compared with the oracle's single-process run over the whole window, bit for bit."""
    if not _two_gpus():
        pytest.skip("needs 2 CUDA devices")
    world = 2
    got = np.concatenate(run_ranks("ep_c_abi", "nccl", world))
    want = ep_expected(oracle, 0, world, x_scale=2.0)   # step 4 of the worker: x * (1 + 0.25 * 4)
    assert max_rel(got, want) <= REL_TOL
    assert np.array_equal(bits(got), bits(want))


@pytest.mark.gpu
@pytest.mark.parametrize("case,bf16", [("tp_c_abi", False), ("tp_c_abi_bf16", True)])
def test_tensor_parallel_two_gpus_c_abi(oracle, case, bf16):
    """b200moe_tp_dense on two GPUs: the partials cross NVLink by the library's peer stores (FP32 or bfloat16), both ranks
    fold them in rank order; the fourth step against the oracle's rank-ordered sum of the shares' partials, bit for bit."""
    if not _two_gpus():
        pytest.skip("needs 2 CUDA devices")
    ys = run_ranks(case, "nccl", 2)
    want = tp_expected(oracle, 2, x_scale=2.5, bf16=bf16)
    assert np.array_equal(bits(ys[0]), bits(ys[1]))
    assert max_rel(ys[0], want) <= REL_TOL
    assert np.array_equal(bits(ys[0]), bits(want))


@pytest.mark.gpu
def test_tensor_parallel_two_gpus_nccl(oracle):
    if not _two_gpus():
        pytest.skip("needs 2 CUDA devices")
    world = 2
    ys = run_ranks("tp", "nccl", world)
    want = tp_expected(oracle, world)
    assert max_rel(ys[0], want) <= REL_TOL and np.array_equal(bits(ys[0]), bits(ys[1]))
