"""One rank of the multi-rank tests (launched by tests/test_parallel.py with RANK / WORLD_SIZE / MASTER_* set).

--backend gloo: CPU ranks. The exchange logic of b200moe.ep / b200moe.tp (what is gathered, which block goes home to
  whom, the order of the folds) runs for real over gloo; the per-rank arithmetic is a stand-in written here on top of
  the CPU oracle, which is test infrastructure: the library itself has no CPU path.
--backend nccl: one GPU per rank, the shipped DeviceKernels through the C ABI.
Every rank builds the same seeded inputs, keeps its share, and writes its y to <out>/rank<r>.npy.
"""
import argparse
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path[:0] = [ROOT, os.path.join(ROOT, "strix-halo-engine-lab_b200")]

import b200moe  # noqa: E402
from b200moe import ep, ops, synth, tp  # noqa: E402

H, I, E, K, ROWS = 512, 256, 16, 4, 3           # EP case: per-rank rows
DH, DI, DROWS = 512, 1792, 3                    # TP case: 7 super-blocks of inter


def ep_inputs(world):
    rng = np.random.default_rng(100)
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    rw = synth.router_weight(rng, E, H)
    x = rng.standard_normal((world * ROWS, H), dtype=np.float32)
    shared = rng.standard_normal((world * ROWS, H), dtype=np.float32)
    return gate, up, down, rw, x, shared


def tp_inputs():
    rng = np.random.default_rng(101)
    gate, up, down = synth.expert_tensors(rng, 1, DH, DI, 12, 12)
    x = rng.standard_normal((DROWS, DH), dtype=np.float32)
    return gate, up, down, x


def tp_slices(gate, up, down, start, size):
    g2, u2 = gate.reshape(DI, -1), up.reshape(DI, -1)
    d3 = down.reshape(DH, DI // 256, 144)
    return (np.ascontiguousarray(g2[start:start + size]).reshape(-1), np.ascontiguousarray(u2[start:start + size]).reshape(-1),
            np.ascontiguousarray(d3[:, start // 256:(start + size) // 256]).reshape(-1))


class OracleEpKernels:
    """CPU stand-in of b200moe.ep.DeviceKernels for the gloo tests (same five steps, oracle arithmetic)."""

    def __init__(self, orc, oshape, policy, rw, gate, up, down, form, world, rank):
        self.o, self.shape, self.policy, self.rw, self.form, self.world, self.rank = orc, oshape, policy, rw, form, world, rank
        self.gate, self.up, self.down = gate, up, down
        self.per = oshape.experts // world

    @staticmethod
    def _t(a):
        a = np.ascontiguousarray(a)
        return torch.from_numpy(a.view(np.int32) if a.dtype == np.uint32 else a)

    def route(self, x):
        x = x.numpy()
        codes, deltas, sums = self.o.quantize_a8(x)
        _, _, ids, wts = self.o.router(self.policy, x=x, w=self.rw)
        return tuple(self._t(a) for a in (codes, deltas, sums, ids, wts))

    def experts(self, a8, ids, wts):
        idn = ids.numpy().view(np.uint32)
        first = self.rank * self.per
        ex = self.o.experts(self.shape, self.gate, self.up, self.down, idn, a8[0].numpy(), a8[1].numpy(), a8[2].numpy(),
                            first=first, end=first + self.per)
        if self.form == b200moe.COMBINE_PARTS:
            return self._t(self.o.combine(self.form, ex["raw"], wts.numpy(), idn, parts=self.world, part_experts=self.per,
                                          only_part=self.rank))
        return self._t(ex["raw"])

    def fold(self, parts, shared):
        acc = shared.numpy().copy() if shared is not None else np.zeros(parts.shape[1:], np.float32)
        for p in range(parts.shape[0]):
            acc = (acc + parts[p].numpy()).astype(np.float32)
        return self._t(acc)

    def combine_slots(self, blocks, ids, wts, shared):
        idn = ids.numpy().view(np.uint32)
        b = blocks.numpy()
        flat = idn.reshape(-1)
        raw = np.stack([b[min(int(flat[s]) // self.per, self.world - 1), s] for s in range(flat.size)])
        return self._t(self.o.combine(self.form, raw, wts.numpy(), idn, shared=None if shared is None else shared.numpy()))


class OracleDenseKernels:
    def __init__(self, orc, oshape, gate, up, down):
        self.o, self.shape, self.gate, self.up, self.down = orc, oshape, gate, up, down

    def partial(self, x):
        x = x.numpy()
        codes, deltas, sums = self.o.quantize_a8(x)
        ids = np.zeros((x.shape[0], 1), np.uint32)
        return torch.from_numpy(self.o.experts(self.shape, self.gate, self.up, self.down, ids, codes, deltas, sums)["raw"])

    def fold(self, parts):
        acc = np.zeros(parts.shape[1:], np.float32)
        for p in range(parts.shape[0]):
            acc = (acc + parts[p].numpy()).astype(np.float32)
        return torch.from_numpy(acc)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["ep_parts", "ep_parts_peer", "ep_fma", "ep_c_abi", "tp", "tp_allreduce", "tp_c_abi", "tp_c_abi_bf16"])
    ap.add_argument("--backend", default="gloo")
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    gpu = a.backend == "nccl"
    if gpu:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        from oracle import loader as O
        orc = O.Oracle()
    put = lambda arr: torch.from_numpy(np.ascontiguousarray(arr)).to(dev)

    if a.case == "ep_c_abi":   # the whole step behind b200moe_ep_ffn: peer-store dispatch and return, no collective on the path
        gate, up, down, rw, x, shared = ep_inputs(world)
        per = E // world
        gb, db = (I * (H // 256) * 144), (H * (I // 256) * 144)
        sl = lambda t, b: put(t.reshape(-1)[rank * per * b:(rank + 1) * per * b])
        layer = ep.PeerEpFfn(ops.make_shape(H, I, E, K, 12, 12), ops.softmax_policy(E, K), put(rw), sl(gate, gb), sl(up, gb), sl(down, db), ROWS)
        summary = torch.zeros(1, dtype=torch.int32, device=dev)
        for step in range(5):          # odd and even steps: both halves of the window, the step counters, a changing x
            scale = np.float32(1.0 + 0.25 * step)
            y = layer(put(x[rank * ROWS:(rank + 1) * ROWS] * scale), put(shared[rank * ROWS:(rank + 1) * ROWS]), summary=summary)
        torch.cuda.synchronize()
        assert int(summary.item()) == 0, f"job summary {int(summary.item()):#x}"
        layer.close()
    elif a.case.startswith("ep"):
        form = b200moe.COMBINE_PARTS if a.case.startswith("ep_parts") else b200moe.COMBINE_FMA_SLOTS
        gate, up, down, rw, x, shared = ep_inputs(world)
        per = E // world
        x_l, sh_l = x[rank * ROWS:(rank + 1) * ROWS], shared[rank * ROWS:(rank + 1) * ROWS]
        if gpu:
            gb, db = (I * (H // 256) * 144), (H * (I // 256) * 144)   # bytes of one expert's gate (= up) / down tensor
            sl = lambda t, b: put(t.reshape(-1)[rank * per * b:(rank + 1) * per * b])
            shape = ops.make_shape(H, I, E, K, 12, 12)
            k = ep.DeviceKernels(shape, ops.softmax_policy(E, K), put(rw), sl(gate, gb), sl(up, gb), sl(down, db), world * ROWS, form,
                                 world, rank)
        else:
            k = OracleEpKernels(orc, O.Shape(H, I, E, K, 12, 12, float("inf")), O.softmax_policy(E, K), rw, gate, up, down, form, world, rank)
        layer = ep.EpMoeFfn(k, ROWS, K, H, form, peer_return=a.case == "ep_parts_peer", device=dev)
        y = layer(put(x_l), put(sh_l))
        if layer.peers is not None:       # a second and third step: the alternating buffers
            y = layer(put(x_l), put(sh_l))
            y = layer(put(x_l), put(sh_l))
            torch.cuda.synchronize()
            layer.peers.close()
    else:
        gate, up, down, x = tp_inputs()
        start, size = tp.tp_shares(DI, world)[rank]
        gs, us, ds = tp_slices(gate, up, down, start, size)
        if a.case.startswith("tp_c_abi"):   # share + exchange + rank-ordered fold behind b200moe_tp_dense (no collective on the path)
            layer = tp.PeerTpDense(ops.make_shape(DH, size, 1, 1, 12, 12), put(gs), put(us), put(ds), DROWS, payload_bf16=a.case.endswith("bf16"))
            summary = torch.zeros(1, dtype=torch.int32, device=dev)
            for step in range(4):
                y = layer(put(x * np.float32(1.0 + 0.5 * step)), summary=summary).clone()
            torch.cuda.synchronize()
            assert int(summary.item()) == 0, f"job summary {int(summary.item()):#x}"
            layer.close()
            np.save(os.path.join(a.out, f"rank{rank}.npy"), y.cpu().numpy())
            dist.barrier()
            dist.destroy_process_group()
            return
        if gpu:
            k = tp.DeviceDenseKernels(ops.make_shape(DH, size, 1, 1, 12, 12), put(gs), put(us), put(ds))
        else:
            k = OracleDenseKernels(orc, O.Shape(DH, size, 1, 1, 12, 12, float("inf")), gs, us, ds)
        y = tp.TpDenseFfn(k, allreduce=a.case == "tp_allreduce")(put(x))
    if gpu:
        torch.cuda.synchronize()
    np.save(os.path.join(a.out, f"rank{rank}.npy"), y.cpu().numpy())
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
