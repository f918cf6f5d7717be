"""Tensor parallelism of the dense (shared-expert style) FFN over torch.distributed.

gate / up are split by output (column parallel over `inter`, in whole 256-wide super-blocks so that every share is a
valid Q4_K row set), SwiGLU and the A8 of h stay local to the share, down is split along K over the same shares and
yields one [rows][hidden] partial per rank. The partials are summed in RANK ORDER - y = ((+0 + P_0) + P_1) ... - so that
W GPUs and W virtual ranks on one GPU give the same bits (the reference's rule for its two-rank shared expert:
include/strix/ds41_shexp_tp.hpp:7-9). That fixed order is why the partials are all-gathered and folded by
b200moe_fold_parts instead of handed to an all-reduce, whose association order is the library's choice; `allreduce=True`
takes the all-reduce anyway (one collective less on the wire, sum order not pinned).

x is replicated on every rank. The collectives are torch.distributed's; the arithmetic is the C library's.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import check, lib, ptr, stream_ptr
from . import ops


def tp_shares(inter, world):
    """Whole super-blocks per rank, the larger shares first: 68 blocks over 8 ranks -> 9,9,9,9,8,8,8,8."""
    blocks = inter // 256
    base, extra = divmod(blocks, world)
    sizes = [(base + (1 if r < extra else 0)) * 256 for r in range(world)]
    starts = [sum(sizes[:r]) for r in range(world)]
    return list(zip(starts, sizes))


class DeviceDenseKernels:
    """A rank's share of the dense FFN through the C ABI (CUDA only)."""

    def __init__(self, shape_local, gate, up, down):
        self.shape, self.gate, self.up, self.down = shape_local, gate, up, down

    def partial(self, x):
        """The rank's partial sum [rows][hidden]. Workspace, A8 rows and output are kept per row count (the caller-owned
        buffers of the C contract): a step is then two library calls and no allocation. The output is overwritten by the
        next call with the same row count."""
        from . import A8Rows, DenseView, ExpertWeights, QuantizeA8View
        rows, width = x.shape
        buf = self._buffers.get(rows) if hasattr(self, "_buffers") else None
        if buf is None:
            if not hasattr(self, "_buffers"):
                self._buffers = {}
            dev = self.gate.device
            ws_bytes = int(lib().b200moe_layer_workspace_bytes(C.byref(self.shape), rows))
            buf = dict(ws=torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device=dev), ws_bytes=ws_bytes,
                       codes=torch.empty((rows, width), dtype=torch.int8, device=dev),
                       deltas=torch.empty((rows, width // 32), dtype=torch.float32, device=dev),
                       sums=torch.empty((rows, width // 32), dtype=torch.int32, device=dev),
                       y=torch.empty((rows, self.shape.hidden), dtype=torch.float32, device=dev))
            self._buffers[rows] = buf
        a8 = A8Rows(ptr(buf["codes"]), ptr(buf["deltas"]), ptr(buf["sums"]), rows, width, width)
        q = QuantizeA8View(ptr(x), rows, width, x.stride(0), int(x.dtype == torch.bfloat16), a8, None)
        check(lib().b200moe_quantize_a8(C.byref(q), stream_ptr()))
        v = DenseView(self.shape, ExpertWeights(ptr(self.gate), ptr(self.up), ptr(self.down)), rows, a8, ptr(buf["y"]), None,
                      ptr(buf["ws"]), buf["ws_bytes"])
        check(lib().b200moe_dense_ffn(C.byref(v), stream_ptr()))
        return buf["y"]

    def fold(self, parts):
        world, rows, hidden = parts.shape
        y = torch.empty((rows, hidden), dtype=torch.float32, device=parts.device)
        check(lib().b200moe_fold_parts(ptr(parts), world, rows * hidden, None, rows * hidden, ptr(y), None, stream_ptr()))
        return y


class PeerTpDense:
    """b200moe_tp_dense: the rank's share of the dense block and the exchange of the partial sums behind ONE C call. The
    partials go to every rank's window by the library's peer stores (FP32, or bfloat16 with payload_bf16), every rank folds
    them in rank order: an all-reduce with a fixed association order and no collective library on the path.
    torch.distributed is used once, at set-up, to hand the windows' CUDA IPC handles round; world 1 needs no process group."""

    def __init__(self, shape_local, gate, up, down, rows, group=None, payload_bf16=False, wait_polls=0, extra_windows=0):
        from . import TpDesc
        L = lib()
        multi = dist.is_available() and dist.is_initialized()
        self.group, self.shape, self.rows = group, shape_local, rows
        self.world = dist.get_world_size(group) if multi else 1 + extra_windows
        self.rank = dist.get_rank(group) if multi else 0
        self.gate, self.up, self.down = gate, up, down
        nbytes = int(L.b200moe_tp_window_bytes(shape_local.hidden, self.world, rows, int(payload_bf16)))
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
            for r in range(1, self.world):
                q, h = C.c_void_p(), C.create_string_buffer(64)
                check(L.b200moe_peer_buffer_create(nbytes, C.byref(q), h))
                self.silent.append(q.value)
                windows[r] = q.value
        desc = TpDesc(shape_local, self.world, self.rank, rows, int(payload_bf16), wait_polls, C.cast(windows, C.c_void_p))
        self.handle = C.c_void_p()
        check(L.b200moe_tp_create(C.byref(desc), C.byref(self.handle)))
        self.ws_bytes = int(L.b200moe_tp_workspace_bytes(self.handle))
        dev = gate.device
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        H = shape_local.hidden
        self.codes = torch.empty((rows, H), dtype=torch.int8, device=dev)
        self.deltas = torch.empty((rows, H // 32), dtype=torch.float32, device=dev)
        self.sums = torch.empty((rows, H // 32), dtype=torch.int32, device=dev)
        self.y = torch.empty((rows, H), dtype=torch.float32, device=dev)
        if multi:
            dist.barrier(group=group)

    def __call__(self, x, summary=None, y=None):
        """x [rows][hidden] float32 (the same on every rank) -> y, the folded sum (kept in a buffer of this object)."""
        from . import A8Rows, ExpertWeights, QuantizeA8View, TpStepView
        rows, width = x.shape
        a8 = A8Rows(ptr(self.codes), ptr(self.deltas), ptr(self.sums), rows, width, width)
        q = QuantizeA8View(ptr(x), rows, width, x.stride(0), int(x.dtype == torch.bfloat16), a8, None)
        check(lib().b200moe_quantize_a8(C.byref(q), stream_ptr()))
        y = self.y[:rows] if y is None else y
        v = TpStepView(ExpertWeights(ptr(self.gate), ptr(self.up), ptr(self.down)), rows, a8, ptr(y), None, ptr(summary), ptr(self.ws), self.ws_bytes)
        check(lib().b200moe_tp_dense(self.handle, C.byref(v), stream_ptr()))
        return y

    def close(self):
        L = lib()
        torch.cuda.synchronize()
        multi = dist.is_available() and dist.is_initialized()
        if multi:
            dist.barrier(group=self.group)
        if self.handle:
            L.b200moe_tp_destroy(self.handle)
            self.handle = None
        for q in self.opened:
            L.b200moe_peer_buffer_close(q)
        if multi:
            dist.barrier(group=self.group)
        for q in self.silent + ([self.mine.value] if self.mine else []):
            L.b200moe_peer_buffer_destroy(q)
        self.opened, self.silent, self.mine = [], [], None


class TpDenseFfn:
    def __init__(self, kernels, group=None, allreduce=False):
        self.k, self.group, self.allreduce = kernels, group, allreduce
        self.world = dist.get_world_size(group)

    def __call__(self, x):
        part = self.k.partial(x)
        if self.allreduce:
            dist.all_reduce(part, group=self.group)
            return part
        parts = torch.empty((self.world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
        dist.all_gather(list(parts.unbind(0)), part.contiguous(), group=self.group)
        return self.k.fold(parts)
