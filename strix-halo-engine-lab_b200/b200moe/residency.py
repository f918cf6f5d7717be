"""Expert residency: a layer whose experts do not all fit the HBM budget given to it.

Mirror of the reference's tiered expert residency (include/strix/cuda/tiered_experts.hpp; planner
include/strix/residency/expert_residency.hpp:121-147) with the one difference the C header states: a miss is a host -> slot
COPY on the caller's stream and the expert is then computed on the GPU; nothing is computed on the CPU and no kernel waits
on the host.

    res = ExpertResidency(shape, gate_host, up_host, down_host, slots)     # host tensors: pinned uint8 torch tensors
    slot_ids = res.map(ids)                                                 # ids int32 [rows][top_k] on the device
    layer = ops.MoeLayer(res.slot_shape, res.gate, res.up, res.down, rows, COMBINE_FMA_SLOTS)
    y = layer(x_a8, slot_ids, weights)
"""
import ctypes as C

import numpy as np
import torch

from . import ResidencyDesc, ResidencyStats, Shape, check, lib, ptr, stream_ptr


class ExpertResidency:
    def __init__(self, shape, gate_host, up_host, down_host, slots, device=None, decay=0.0):
        L = lib()
        self.shape, self.slots = shape, slots
        self.host = (gate_host, up_host, down_host)           # kept alive: the copies read them
        dev = device or torch.device("cuda", torch.cuda.current_device())
        gate_bytes = int(L.b200moe_gate_row_bytes(C.byref(shape))) * shape.inter
        down_bytes = int(L.b200moe_down_row_bytes(C.byref(shape))) * shape.hidden
        self.gate = torch.zeros(slots * gate_bytes, dtype=torch.uint8, device=dev)
        self.up = torch.zeros(slots * gate_bytes, dtype=torch.uint8, device=dev)
        self.down = torch.zeros(slots * down_bytes, dtype=torch.uint8, device=dev)
        self.slot_shape = Shape(shape.hidden, shape.inter, slots, shape.top_k, shape.gate_type, shape.down_type, shape.limit)
        desc = ResidencyDesc(shape, gate_host.data_ptr(), up_host.data_ptr(), down_host.data_ptr(), slots, ptr(self.gate), ptr(self.up),
                             ptr(self.down), decay)
        self.handle = C.c_void_p()
        check(L.b200moe_residency_create(C.byref(desc), C.byref(self.handle)))

    def map(self, ids):
        """ids: int32 device tensor of expert ids (any shape) -> slot ids of the same shape; loads what is missing."""
        out = torch.empty_like(ids)
        check(lib().b200moe_residency_map(self.handle, ptr(ids), ids.numel(), ptr(out), stream_ptr()))
        return out

    def promote(self, moves, stream=None):
        """Planner moves of this layer ((layer, slot, evict, expert) tuples): the experts are copied into their slots on
        `stream` (an int handle; default: the current stream) and the table follows; the caller orders that stream before
        the next map()."""
        from . import Move
        arr = (Move * len(moves))(*[Move(*m) for m in moves])
        check(lib().b200moe_residency_promote(self.handle, arr, len(moves), stream if stream is not None else stream_ptr()))

    def stats(self):
        s = ResidencyStats()
        check(lib().b200moe_residency_get_stats(self.handle, C.byref(s)))
        return {k: int(getattr(s, k)) for k, _ in ResidencyStats._fields_}

    def table(self):
        t = np.zeros(self.shape.experts, np.int32)
        check(lib().b200moe_residency_table(self.handle, t.ctypes.data_as(C.c_void_p)))
        return t

    def close(self):
        if self.handle:
            torch.cuda.synchronize()
            lib().b200moe_residency_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def choose_victims(slot_expert, score, used, missing):
    """The eviction rule on its own (pure host function of the library, no CUDA)."""
    slot_expert = np.ascontiguousarray(slot_expert, np.int32)
    score = np.ascontiguousarray(score, np.float64)
    used = np.ascontiguousarray(used, np.uint8)
    missing = np.ascontiguousarray(missing, np.uint32)
    victims = np.zeros(len(missing), np.uint32)
    p = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    check(lib().b200moe_residency_choose_victims(p(slot_expert), len(slot_expert), p(score), p(used), len(score), p(missing), len(missing), p(victims)))
    return victims


class Planner:
    """b200moe_planner_*: which experts to bring into slots ahead of need under an upload budget per step (host code only;
    the counterpart of strix::residency::Planner, include/strix/residency/expert_residency.hpp:102-147)."""

    def __init__(self, layers, experts, top_k, slots, expert_bytes, decay=0.0, margin_reuses=0.0, upload_bytes_per_step=0):
        from . import PlannerDesc
        self.layers, self.experts, self.slots = layers, experts, slots
        self._bytes = (C.c_uint64 * layers)(*[int(b) for b in expert_bytes])
        desc = PlannerDesc(layers, experts, top_k, slots, C.cast(self._bytes, C.c_void_p), decay, margin_reuses, upload_bytes_per_step)
        self.handle = C.c_void_p()
        check(lib().b200moe_planner_create(C.byref(desc), C.byref(self.handle)))

    def seed(self, layer, counts):
        a = np.ascontiguousarray(counts, np.uint32)
        check(lib().b200moe_planner_seed(self.handle, layer, a.ctypes.data_as(C.c_void_p)))

    def observe(self, layer, ids):
        a = np.ascontiguousarray(ids, np.uint32).reshape(-1)
        check(lib().b200moe_planner_observe(self.handle, layer, a.ctypes.data_as(C.c_void_p), a.size))

    def end_step(self):
        check(lib().b200moe_planner_end_step(self.handle))

    def plan(self):
        """The step's moves as (layer, slot, evict, expert) tuples; evict is MOVE_NO_EVICTION for a free slot."""
        from . import Move
        n = C.c_uint32()
        cap = 64
        while True:
            moves = (Move * cap)()
            check(lib().b200moe_planner_plan(self.handle, moves, cap, C.byref(n)))
            if n.value <= cap:
                return [(m.layer, m.slot, m.evict, m.expert) for m in moves[:n.value]]
            cap = n.value

    def commit(self, move):
        from . import Move
        check(lib().b200moe_planner_commit(self.handle, C.byref(Move(*move))))

    def fill_from_seed(self):
        check(lib().b200moe_planner_fill_from_seed(self.handle))

    def table(self, layer):
        t = np.zeros(self.experts, np.int32)
        check(lib().b200moe_planner_table(self.handle, layer, t.ctypes.data_as(C.c_void_p)))
        return t

    def scores(self, layer):
        s = np.zeros(self.experts, np.float64)
        check(lib().b200moe_planner_scores(self.handle, layer, s.ctypes.data_as(C.c_void_p)))
        return s

    def receipt(self):
        from . import PlannerReceipt
        r = PlannerReceipt()
        check(lib().b200moe_planner_get_receipt(self.handle, C.byref(r)))
        return {k: int(getattr(r, k)) for k, _ in PlannerReceipt._fields_}

    def close(self):
        if self.handle:
            lib().b200moe_planner_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass
