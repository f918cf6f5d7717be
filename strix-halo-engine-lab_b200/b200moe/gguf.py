"""Expert tensors from a GGUF file: parse with the C library's reader, copy the byte ranges to the device as they lie.

The reference loads the same tensors through strix::gguf::read_file and its weight seam (src/gguf_reader.cpp,
src/weight/readers/gguf.cpp; roles expert_gate / expert_up / expert_down / router of include/strix/weight/types.hpp:30-34).
Nothing is repacked: dims [hidden, inter, experts] on disk are [experts][inter][hidden / B] in memory order, which is
the layout the kernels read.
"""
import ctypes as C

import numpy as np

from . import GgufMoeLayer, GgufTensorInfo, Shape, check, lib


class GgufFile:
    def __init__(self, path):
        self.path = str(path)
        self._h = C.c_void_p()
        check(lib().b200moe_gguf_open(self.path.encode(), C.byref(self._h)))

    def close(self):
        if self._h:
            lib().b200moe_gguf_close(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def data_offset(self):
        return int(lib().b200moe_gguf_data_offset(self._h))

    @property
    def alignment(self):
        return int(lib().b200moe_gguf_alignment(self._h))

    @staticmethod
    def _info(t):
        return dict(name=t.name.decode(), dims=[int(t.dims[i]) for i in range(t.n_dims)], ggml_type=int(t.ggml_type),
                    offset=int(t.offset), bytes=int(t.bytes))

    def tensors(self):
        out, t = [], GgufTensorInfo()
        for i in range(int(lib().b200moe_gguf_tensor_count(self._h))):
            check(lib().b200moe_gguf_tensor_at(self._h, i, C.byref(t)))
            out.append(self._info(t))
        return out

    def find(self, name):
        t = GgufTensorInfo()
        check(lib().b200moe_gguf_find(self._h, name.encode(), C.byref(t)))
        return self._info(t)

    def moe_layer(self, layer):
        """(shape with top_k = 0, {gate, up, down, router} infos) of layer `layer`."""
        m = GgufMoeLayer()
        check(lib().b200moe_gguf_find_moe_layer(self._h, layer, C.byref(m)))
        shape = Shape(m.shape.hidden, m.shape.inter, m.shape.experts, m.shape.top_k, m.shape.gate_type, m.shape.down_type, m.shape.limit)
        return shape, {k: self._info(getattr(m, k)) for k in ("gate", "up", "down", "router")}

    def read(self, info):
        """The tensor's bytes as a read-only numpy view of the memory-mapped file."""
        return np.memmap(self.path, dtype=np.uint8, mode="r", offset=info["offset"], shape=(info["bytes"],))

    def load_moe_layer(self, layer, top_k, device):
        """Uploads one layer: returns (shape, gate, up, down, router_weight) with torch tensors on `device`."""
        import torch
        shape, infos = self.moe_layer(layer)
        shape.top_k = top_k
        up = lambda k: torch.from_numpy(np.ascontiguousarray(self.read(infos[k]))).to(device)
        router = torch.from_numpy(np.ascontiguousarray(self.read(infos["router"])).view(np.float32).reshape(shape.experts, shape.hidden)).to(device)
        return shape, up("gate"), up("up"), up("down"), router
