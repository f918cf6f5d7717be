"""Expert parallelism over torch.distributed: one process per GPU, rank r owns experts [r * E / W, (r + 1) * E / W).

The reference runs this split on two ranks through Communicator::exchange (include/strix/dist/communicator.hpp;
docs/engine/transport/communicator.md): a rank that owns a subset of the experts restricts the window routes to its range
(restrict_routes, src/ds41_moe.cpp:45-61), and the combine over ranks is a fixed-order fold
(include/strix/ds41_moe.hpp:5-11). Sizes are never sent: every rank derives them from shared data (rows per rank).

One step, every rank alike:
  1. route:    A8 of the local token rows + router (local rows are independent).
  2. dispatch: all-gather of the A8 rows (codes, deltas, sums), the ids and the route weights -> the global window.
               (Every rank sees every row; at decode sizes the volume is a few hundred KB and the step is latency bound.)
  3. experts:  b200moe_layer over the global window restricted to the rank's expert range, on its local tensors.
               PARTS form: the rank's partial sum S_r per row (only_part = r).  FMA_SLOTS form: raw slot vectors.
  4. return:   all-to-all, the block of home rank h goes to h - or, with peer_return (PARTS form, one node), no
               collective at all: the combine kernel stores each home rank's rows straight into that rank's buffer
               (CUDA IPC peer memory over NVLink), then a one-word all-reduce as the barrier.
  5. combine:  PARTS: y = ((shared + S_0) + S_1) ... in rank order (b200moe_fold_parts).
               FMA_SLOTS: slot s is taken from the block of the rank that owns ids[s] (b200moe_select_owner_slots), then
               the ordinary slot-order chain (b200moe_combine).
With W virtual ranks on one GPU (b200moe_ffn, parts = W) the bits are the same.

The collectives are torch.distributed's (NCCL on GPUs, gloo in the CPU tests); the arithmetic is the C library's.
`kernels` is the seam between the two: DeviceKernels calls the C ABI and is the only implementation shipped; the CPU
tests of the exchange logic pass a stand-in of their own.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import COMBINE_FMA_SLOTS, COMBINE_PARTS, EpDesc, EpStepView, ExpertWeights, check, lib, ptr, stream_ptr
from . import ops


class PeerEpFfn:
    """b200moe_ep_ffn: the whole expert-parallel step of a rank behind ONE C call - route, dispatch, local experts, return,
    fold - with both exchanges done by the library's own kernels storing into the peers' windows over NVLink (no
    collective, no host wait; bounded flag waits on the device). torch.distributed is used once, at set-up, to hand the
    windows' CUDA IPC handles round; world 1 (no process group) runs the same kernels against the rank's own window.
    gate / up / down hold the rank's experts only; every rank passes the same number of rows per step. fold_parts: the
    number of expert ranges of the fold (0 = world); the same value at every world size gives the same bits."""

    def __init__(self, shape, policy, router_weight, gate, up, down, rows, group=None, logit_bias=None, select_bias=None,
                 wait_polls=0, grouped_min_rows=0, extra_windows=0, fold_parts=0):
        L = lib()
        multi = dist.is_available() and dist.is_initialized()
        self.group = group
        self.world = dist.get_world_size(group) if multi else 1 + extra_windows
        self.rank = dist.get_rank(group) if multi else 0
        self.shape, self.policy, self.rows = shape, policy, rows
        self.router_weight, self.gate, self.up, self.down = router_weight, gate, up, down
        self.logit_bias, self.select_bias, self.grouped_min_rows = logit_bias, select_bias, grouped_min_rows
        nbytes = int(L.b200moe_ep_window_bytes(C.byref(shape), self.world, rows, fold_parts))
        if nbytes == 0:
            raise ValueError("expert parallelism: 1 <= world <= 8, rows >= 1, fold_parts a multiple of world")
        self.mine, self.opened, self.silent = C.c_void_p(), [], []
        handle = C.create_string_buffer(64)
        check(L.b200moe_peer_buffer_create(nbytes, C.byref(self.mine), handle))
        windows = (C.c_void_p * self.world)()
        if multi:
            everyone = [None] * self.world
            dist.all_gather_object(everyone, handle.raw, group=group)
            for r in range(self.world):
                if r == self.rank:
                    windows[r] = self.mine.value
                else:
                    q = C.c_void_p()
                    check(L.b200moe_peer_buffer_open(everyone[r], C.byref(q)))
                    self.opened.append(q.value)
                    windows[r] = q.value
        else:
            windows[0] = self.mine.value
            for r in range(1, self.world):   # windows nobody serves (tests of the bounded wait): plain local buffers
                q, h = C.c_void_p(), C.create_string_buffer(64)
                check(L.b200moe_peer_buffer_create(nbytes, C.byref(q), h))
                self.silent.append(q.value)
                windows[r] = q.value
        desc = EpDesc(shape, policy, self.world, self.rank, rows, wait_polls, fold_parts, C.cast(windows, C.c_void_p))
        self.handle = C.c_void_p()
        check(L.b200moe_ep_create(C.byref(desc), C.byref(self.handle)))
        self.ws_bytes = int(L.b200moe_ep_workspace_bytes(self.handle))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=gate.device)
        if multi:
            dist.barrier(group=group)

    def view(self, x, y, shared=None, summary=None, events=None):
        ev = C.cast(events, C.c_void_p) if events is not None else None
        return EpStepView(ExpertWeights(ptr(self.gate), ptr(self.up), ptr(self.down)), ptr(self.router_weight), ptr(self.logit_bias),
                          ptr(self.select_bias), ptr(x), int(x.dtype == torch.bfloat16), x.shape[0], ptr(shared), ptr(y), None,
                          ptr(summary), ptr(self.ws), self.ws_bytes, self.grouped_min_rows, ev)

    def __call__(self, x, shared=None, y=None, summary=None):
        if y is None:
            y = torch.empty((x.shape[0], self.shape.hidden), dtype=torch.float32, device=x.device)
        check(lib().b200moe_ep_ffn(self.handle, C.byref(self.view(x, y, shared, summary)), stream_ptr()))
        return y

    def close(self):
        L = lib()
        torch.cuda.synchronize()
        if self.group is not None or (dist.is_available() and dist.is_initialized()):
            dist.barrier(group=self.group)
        if self.handle:
            L.b200moe_ep_destroy(self.handle)
            self.handle = None
        for q in self.opened:
            L.b200moe_peer_buffer_close(q)
        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=self.group)
        for q in self.silent + ([self.mine.value] if self.mine else []):
            L.b200moe_peer_buffer_destroy(q)
        self.opened, self.silent, self.mine = [], [], None


class DeviceKernels:
    """The five compute steps of one rank, through the C ABI (CUDA only: there is no other implementation)."""

    def __init__(self, shape, policy, router_weight, gate, up, down, window_rows, combine_form, world, rank,
                 logit_bias=None, select_bias=None):
        if shape.experts % world:
            raise ValueError(f"{shape.experts} experts do not split over {world} ranks")
        self.shape, self.policy, self.world, self.rank = shape, policy, world, rank
        self.per = shape.experts // world
        self.router_weight, self.logit_bias, self.select_bias = router_weight, logit_bias, select_bias
        self.combine_form = combine_form
        # local tensors hold experts [rank * per, (rank + 1) * per): base = first
        self.layer = ops.MoeLayer(shape, gate, up, down, window_rows, combine_form, parts=world, part_experts=self.per)

    def route(self, x):
        codes, deltas, sums = ops.enqueue_quantize_a8(x)
        _, _, ids, wts = ops.enqueue_router(self.policy, x=x, weight=self.router_weight, logit_bias=self.logit_bias, bias=self.select_bias)
        return codes, deltas, sums, ids, wts

    def experts(self, a8, ids, wts, y_blocks=None, y_block_rows=0):
        first = self.rank * self.per
        if self.combine_form == COMBINE_PARTS:
            return self.layer(a8, ids, wts, first=first, end=first + self.per, base=first, only_part=self.rank,
                              y_blocks=y_blocks, y_block_rows=y_block_rows)
        return self.layer(a8, ids, wts, first=first, end=first + self.per, base=first, want_raw=True, combine=False)[1]

    def fold(self, parts, shared):
        world, rows, hidden = parts.shape
        y = torch.empty((rows, hidden), dtype=torch.float32, device=parts.device)
        check(lib().b200moe_fold_parts(ptr(parts), world, rows * hidden, ptr(shared), rows * hidden, ptr(y), None, stream_ptr()))
        return y

    def fold_at(self, parts_ptr, world, rows, hidden, shared, device):
        """fold over a raw device pointer (a peer buffer of this rank)."""
        y = torch.empty((rows, hidden), dtype=torch.float32, device=device)
        check(lib().b200moe_fold_parts(parts_ptr, world, rows * hidden, ptr(shared), rows * hidden, ptr(y), None, stream_ptr()))
        return y

    def combine_slots(self, blocks, ids, wts, shared):
        world, slots, hidden = blocks.shape
        raw = torch.empty((slots, hidden), dtype=torch.float32, device=blocks.device)
        check(lib().b200moe_select_owner_slots(ptr(blocks), slots * hidden, world, self.per, ptr(ids), slots, hidden, ptr(raw),
                                               stream_ptr()))
        return ops.enqueue_moe_combine(COMBINE_FMA_SLOTS, raw, wts, ids, shared=shared)


class PeerBuffers:
    """Receive buffers of the PARTS return step that the peers write DIRECTLY (CUDA IPC, one node): two buffers per rank
    ([world][rows][hidden] FP32, alternating by step), every rank maps every other rank's. The combine kernel of rank r
    stores the partial sums of home rank h's rows straight into block r of h's buffer - peer stores over NVLink from
    the kernel that computes them, no all-to-all. A stream-ordered NCCL all-reduce of one word is the barrier between
    "everyone has written" and the home rank's fold; alternating buffers keep step s + 1's stores away from a fold of
    step s that may still be running."""

    def __init__(self, rows, hidden, group, device):
        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.rows, self.hidden, self.device = rows, hidden, device
        L = lib()
        nbytes = self.world * rows * hidden * 4
        self.mine, handles = [], []
        for _ in range(2):
            p, h = C.c_void_p(), C.create_string_buffer(64)
            check(L.b200moe_peer_buffer_create(nbytes, C.byref(p), h))
            self.mine.append(p.value)
            handles.append(h.raw)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handles, group=group)
        self.opened = []
        self.tables = []                       # per parity: device array of world pointers (block `rank` of each home's buffer)
        block = rows * hidden * 4
        for parity in range(2):
            ptrs = []
            for h in range(self.world):
                if h == self.rank:
                    base = self.mine[parity]
                else:
                    p = C.c_void_p()
                    check(L.b200moe_peer_buffer_open(everyone[h][parity], C.byref(p)))
                    self.opened.append(p.value)
                    base = p.value
                ptrs.append(base + self.rank * block)
            self.tables.append(torch.tensor(ptrs, dtype=torch.int64, device=device))
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.step = 0
        dist.barrier(group=group)

    def barrier(self):
        dist.all_reduce(self.flag, group=self.group)   # stream-ordered: runs after this rank's stores, before its fold

    def close(self):
        L = lib()
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self.opened:
            L.b200moe_peer_buffer_close(p)
        dist.barrier(group=self.group)
        for p in self.mine:
            L.b200moe_peer_buffer_destroy(p)
        self.opened, self.mine = [], []


class EpMoeFfn:
    """One MoE FFN layer under expert parallelism. Every rank calls it with the same number of local rows.
    peer_return=True (PARTS form, CUDA ranks of one node): the return step is the combine kernel's own peer stores
    (PeerBuffers) instead of an all-to-all."""

    def __init__(self, kernels, rows, top_k, hidden, combine_form, group=None, peer_return=False, device=None):
        self.k, self.rows, self.top_k, self.hidden, self.form = kernels, rows, top_k, hidden, combine_form
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.peers = PeerBuffers(rows, hidden, group, device) if peer_return and combine_form == COMBINE_PARTS else None

    def _all_gather(self, t):
        out = torch.empty((self.world * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        dist.all_gather(list(out.chunk(self.world)), t.contiguous(), group=self.group)
        return out

    def _return_home(self, blocks):
        """blocks [world][n][hidden]: block h is for home rank h. Returns [world][n][hidden], block r came from rank r."""
        out = torch.empty_like(blocks)
        dist.all_to_all_single(out, blocks.contiguous(), group=self.group)
        return out

    def __call__(self, x, shared=None):
        if x.shape[0] != self.rows:
            raise ValueError(f"every rank passes {self.rows} rows, got {x.shape[0]}")
        codes, deltas, sums, ids, wts = self.k.route(x)
        g = [self._all_gather(t) for t in (codes, deltas, sums, ids, wts)]
        if self.peers is not None:
            pb = self.peers
            parity = pb.step & 1
            pb.step += 1
            self.k.experts((g[0], g[1], g[2]), g[3], g[4], y_blocks=pb.tables[parity], y_block_rows=self.rows)
            pb.barrier()
            return self.k.fold_at(pb.mine[parity], self.world, self.rows, self.hidden, shared, x.device)
        out = self.k.experts((g[0], g[1], g[2]), g[3], g[4])
        if self.form == COMBINE_PARTS:      # out [world * rows][hidden]: the rank's partial sums of every row
            parts = self._return_home(out.view(self.world, self.rows, self.hidden))
            return self.k.fold(parts, shared)
        blocks = self._return_home(out.view(self.world, self.rows * self.top_k, self.hidden))
        return self.k.combine_slots(blocks, ids, wts, shared)
