"""Minimal GGUF v3 writer for the tests (public container format: magic, version, counts, key/value metadata, tensor
infos, zero padding to `general.alignment`, tensor data at aligned offsets)."""
import struct

import numpy as np

TYPES = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7, "str": 8, "arr": 9, "u64": 10, "i64": 11, "f64": 12}
FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


def _str(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(t, v):
    if t == 8:
        return _str(v)
    if t == 9:
        et, items = v
        return struct.pack("<IQ", et, len(items)) + b"".join(_value(et, i) for i in items)
    return struct.pack(FMT[t], v)


def write(path, metadata, tensors, alignment=32, version=3, magic=b"GGUF", pad_byte=0, offsets=None, truncate=None):
    """metadata: list of (key, type name, value); tensors: list of (name, dims (GGUF order), ggml type, bytes-like).
    offsets: optional explicit relative offsets (to build malformed files)."""
    out = bytearray(magic + struct.pack("<IQQ", version, len(tensors), len(metadata)))
    for key, tname, v in metadata:
        t = TYPES[tname]
        out += _str(key) + struct.pack("<I", t) + _value(t, v)
    rel, rels = 0, []
    for i, (name, dims, gt, data) in enumerate(tensors):
        r = offsets[i] if offsets is not None else rel
        rels.append(r)
        out += _str(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", gt, r)
        rel = (r + len(data) + alignment - 1) // alignment * alignment
    pad = (-len(out)) % alignment
    out += bytes([pad_byte]) * pad
    base = len(out)
    end = max([r + len(t[3]) for r, t in zip(rels, tensors)], default=0)
    out += bytes(end)
    for r, (_, _, _, data) in zip(rels, tensors):
        out[base + r:base + r + len(data)] = bytes(data)
    if truncate is not None:
        out = out[:truncate]
    with open(path, "wb") as f:
        f.write(out)
    return base, rels
