"""GGUF reader (include/b200moe.h, b200moe_gguf_*): synthetic files, valid and malformed, written by tests/gguf_writer.py.
Admission rules follow the reference reader (src/gguf_reader.cpp:23-99, :330-373). The reference's own reader is not
linked here (it pulls in its weight registry): these checks pin the container format, not the reference's code."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import gguf_writer as W  # noqa: E402

import b200moe  # noqa: E402
from b200moe import gguf, synth  # noqa: E402

torch = pytest.importorskip("torch")


def moe_tensors(rng, layer, E, H, I, gt, dt):
    gate, up, down = synth.expert_tensors(rng, E, H, I, gt, dt)
    rw = synth.router_weight(rng, E, H)
    return [(f"blk.{layer}.ffn_gate_exps.weight", [H, I, E], gt, gate), (f"blk.{layer}.ffn_up_exps.weight", [H, I, E], gt, up),
            (f"blk.{layer}.ffn_down_exps.weight", [I, H, E], dt, down), (f"blk.{layer}.ffn_gate_inp.weight", [H, E], 0, rw.tobytes())], (gate, up, down, rw)


META = [("general.architecture", "str", "synthetic-moe"), ("general.alignment", "u32", 64), ("synthetic.expert_count", "u32", 4),
        ("tokenizer.tokens", "arr", (8, ["a", "bc", ""])), ("synthetic.scales", "arr", (6, [0.5, 1.5])), ("synthetic.flag", "bool", 1),
        ("synthetic.big", "u64", 1 << 40), ("synthetic.neg", "i32", -7)]


def test_reads_layers_and_offsets(tmp_path):
    rng = np.random.default_rng(60)
    t0, raw0 = moe_tensors(rng, 0, 4, 512, 256, 12, 12)
    t1, raw1 = moe_tensors(rng, 1, 4, 512, 256, 8, 8)
    extra = [("output_norm.weight", [512], 0, np.ones(512, np.float32).tobytes())]
    path = tmp_path / "m.gguf"
    base, rels = W.write(path, META, t0 + extra + t1, alignment=64)
    with gguf.GgufFile(path) as f:
        assert f.alignment == 64 and f.data_offset == base and base % 64 == 0
        ts = f.tensors()
        assert [t["name"] for t in ts] == [t[0] for t in t0 + extra + t1]
        for t, r, src in zip(ts, rels, t0 + extra + t1):
            assert t["offset"] == base + r and t["bytes"] == len(bytes(src[3])) and t["dims"] == src[1] and t["ggml_type"] == src[2]
        for layer, raw, gt in ((0, raw0, 12), (1, raw1, 8)):
            shape, infos = f.moe_layer(layer)
            assert (shape.hidden, shape.inter, shape.experts, shape.top_k, shape.gate_type, shape.down_type) == (512, 256, 4, 0, gt, gt)
            assert np.array_equal(f.read(infos["gate"]), raw[0]) and np.array_equal(f.read(infos["down"]), raw[2])
            assert np.array_equal(np.asarray(f.read(infos["router"])).view(np.float32).reshape(4, 512), raw[3])
        with pytest.raises(b200moe.B200MoeError):
            f.find("blk.9.ffn_gate_exps.weight")
        with pytest.raises(b200moe.B200MoeError):
            f.moe_layer(2)


@pytest.mark.parametrize("kind", ["magic", "version", "truncated_header", "truncated_data", "unaligned", "overlap", "duplicate_name",
                                  "duplicate_key", "padding", "block", "alignment", "alignment_signed", "bad_key", "rank"])
def test_rejects_malformed_files(tmp_path, kind):
    rng = np.random.default_rng(61)
    ts, _ = moe_tensors(rng, 0, 2, 256, 256, 12, 12)
    path = tmp_path / "bad.gguf"
    kw, meta = {}, list(META)
    if kind == "magic":
        kw["magic"] = b"GGUX"
    elif kind == "version":
        kw["version"] = 2
    elif kind == "truncated_header":
        kw["truncate"] = 40
    elif kind == "truncated_data":
        base, _ = W.write(path, meta, ts, alignment=64)
        kw["truncate"] = base + 1000
    elif kind == "unaligned":
        kw["offsets"] = [0, len(ts[0][3]) + 8, 4 * len(ts[0][3]), 8 * len(ts[0][3])]
    elif kind == "overlap":
        kw["offsets"] = [0, 64, 4 * len(ts[0][3]), 8 * len(ts[0][3])]
    elif kind == "duplicate_name":
        ts[1] = (ts[0][0],) + ts[1][1:]
    elif kind == "duplicate_key":
        meta.append(META[0])
    elif kind == "padding":
        kw["pad_byte"] = 1
    elif kind == "block":
        ts[0] = (ts[0][0], [250, 256, 2], 12, ts[0][3])
    elif kind == "alignment":       # a non-zero multiple of 8 is required (the reference reader's rule): 12 is not
        meta[1] = ("general.alignment", "u32", 12)
    elif kind == "alignment_signed":  # ... and an unsigned integer type
        meta[1] = ("general.alignment", "i32", 64)
    elif kind == "bad_key":
        meta.append(("Synthetic.Upper", "u32", 1))
    elif kind == "rank":
        ts[3] = (ts[3][0], [256, 2, 1, 1, 1], 0, ts[3][3])
    W.write(path, meta, ts, alignment=64, **kw)
    with pytest.raises(b200moe.B200MoeError):
        gguf.GgufFile(path)


def test_alignment_rule_is_the_reference_readers(tmp_path):
    """general.alignment: any non-zero multiple of 8 is admitted - 24 is, although it is no power of two."""
    rng = np.random.default_rng(63)
    ts, _ = moe_tensors(rng, 0, 2, 256, 256, 12, 12)
    meta = list(META)
    meta[1] = ("general.alignment", "u32", 24)
    path = tmp_path / "a24.gguf"
    base, _ = W.write(path, meta, ts, alignment=24)
    with gguf.GgufFile(path) as f:
        assert f.alignment == 24 and f.data_offset == base


def test_missing_file():
    with pytest.raises(b200moe.B200MoeError):
        gguf.GgufFile("/nonexistent/file.gguf")


@pytest.mark.gpu
def test_ffn_from_gguf_file_matches_oracle(tmp_path, oracle):
    """A layer loaded from the file runs through b200moe_ffn and equals the oracle on the same bytes."""
    from oracle import loader as O
    from b200moe import ops
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    rng = np.random.default_rng(62)
    E, H, I, K, rows = 8, 512, 256, 2, 5
    ts, (gate, up, down, rw) = moe_tensors(rng, 3, E, H, I, 12, 12)
    path = tmp_path / "layer.gguf"
    W.write(path, META, ts, alignment=32)
    dev = torch.device("cuda:0")
    with gguf.GgufFile(path) as f:
        shape, g, u, d, r = f.load_moe_layer(3, K, dev)
    ffn = ops.MoeFfn(shape, ops.softmax_policy(E, K), g, u, d, r, capacity=rows, combine_form=b200moe.COMBINE_FMA_SLOTS)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    y = ffn(torch.from_numpy(x).to(dev)).cpu().numpy()
    want = oracle.ffn(O.Shape(H, I, E, K, 12, 12, float("inf")), O.softmax_policy(E, K), gate, up, down, rw, x, O.COMBINE_FMA_SLOTS)["y"]
    assert float(np.max(np.abs(y - want)) / np.max(np.abs(want))) <= 1e-3
    print("bit-exact:", np.array_equal(y.view(np.uint32), want.view(np.uint32)))
