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
  4. return:   all-to-all, the block of home rank h goes to h.
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

from . import COMBINE_FMA_SLOTS, COMBINE_PARTS, check, lib, ptr, stream_ptr
from . import ops


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

    def experts(self, a8, ids, wts):
        first = self.rank * self.per
        if self.combine_form == COMBINE_PARTS:
            return self.layer(a8, ids, wts, first=first, end=first + self.per, base=first, only_part=self.rank)
        return self.layer(a8, ids, wts, first=first, end=first + self.per, base=first, want_raw=True, combine=False)[1]

    def fold(self, parts, shared):
        world, rows, hidden = parts.shape
        y = torch.empty((rows, hidden), dtype=torch.float32, device=parts.device)
        check(lib().b200moe_fold_parts(ptr(parts), world, rows * hidden, ptr(shared), rows * hidden, ptr(y), None, stream_ptr()))
        return y

    def combine_slots(self, blocks, ids, wts, shared):
        world, slots, hidden = blocks.shape
        raw = torch.empty((slots, hidden), dtype=torch.float32, device=blocks.device)
        check(lib().b200moe_select_owner_slots(ptr(blocks), slots * hidden, world, self.per, ptr(ids), slots, hidden, ptr(raw),
                                               stream_ptr()))
        return ops.enqueue_moe_combine(COMBINE_FMA_SLOTS, raw, wts, ids, shared=shared)


class EpMoeFfn:
    """One MoE FFN layer under expert parallelism. Every rank calls it with the same number of local rows."""

    def __init__(self, kernels, rows, top_k, hidden, combine_form, group=None):
        self.k, self.rows, self.top_k, self.hidden, self.form = kernels, rows, top_k, hidden, combine_form
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

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
        out = self.k.experts((g[0], g[1], g[2]), g[3], g[4])
        if self.form == COMBINE_PARTS:      # out [world * rows][hidden]: the rank's partial sums of every row
            parts = self._return_home(out.view(self.world, self.rows, self.hidden))
            return self.k.fold(parts, shared)
        blocks = self._return_home(out.view(self.world, self.rows * self.top_k, self.hidden))
        return self.k.combine_slots(blocks, ids, wts, shared)
