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
