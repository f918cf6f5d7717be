"""CPU-side checks of the drop-in boundary: the C-ABI library loads, exports every symbol include/b200moe.h
declares, its structures have the layout the Python binding assumes, argument errors are reported before any device
work, and - with no GPU - compute entry points fail loudly instead of falling back to a CPU path."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200moe.h")


@pytest.fixture(scope="module")
def lib():
    import b200moe
    if not os.path.exists(b200moe.LIB_PATH):
        sys.path.insert(0, ROOT)
        import __graft_entry__
        __graft_entry__.build()
    return b200moe.lib()


def test_exports_match_header(lib):
    import b200moe
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text))
    assert declared == set(b200moe.EXPORTS), declared ^ set(b200moe.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
        # ctypes sends an undeclared Python int as a 32-bit C int: every export declares its arguments
        assert getattr(lib, name).argtypes is not None, f"{name}: argtypes not declared in b200moe/__init__.py"
    assert lib.b200moe_abi_version() == b200moe.ABI_VERSION == header_abi_version()


def test_struct_layouts(tmp_path):
    """sizeof of every view as the C compiler sees it equals the ctypes mirror."""
    import b200moe
    names = {"b200moe_a8_rows": b200moe.A8Rows, "b200moe_quantize_a8_view": b200moe.QuantizeA8View,
             "b200moe_q8a8_view": b200moe.Q8A8View, "b200moe_route_policy": b200moe.RoutePolicy,
             "b200moe_router_view": b200moe.RouterView, "b200moe_routes": b200moe.Routes,
             "b200moe_routes_view": b200moe.RoutesView, "b200moe_shape": b200moe.Shape,
             "b200moe_expert_weights": b200moe.ExpertWeights, "b200moe_gate_up_view": b200moe.GateUpView,
             "b200moe_down_view": b200moe.DownView, "b200moe_combine_view": b200moe.CombineView,
             "b200moe_layer_view": b200moe.LayerView, "b200moe_ffn_view": b200moe.FfnView,
             "b200moe_dense_view": b200moe.DenseView, "b200moe_rmsnorm_view": b200moe.RmsnormView,
             "b200moe_residency_desc": b200moe.ResidencyDesc, "b200moe_residency_stats": b200moe.ResidencyStats,
             "b200moe_gguf_tensor_info": b200moe.GgufTensorInfo, "b200moe_gguf_moe_layer": b200moe.GgufMoeLayer,
             "b200moe_kernel_arguments": b200moe.KernelArguments, "b200moe_registration": b200moe.Registration,
             "b200moe_first_error": b200moe.FirstError, "b200moe_move": b200moe.Move, "b200moe_planner_desc": b200moe.PlannerDesc,
             "b200moe_planner_receipt": b200moe.PlannerReceipt}
    src = tmp_path / "sizes.c"
    body = "\n".join(f'    printf("{n} %zu\\n", sizeof({n}));' for n in names)
    src.write_text(f'#include <stdio.h>\n#include "{HEADER}"\nint main(void) {{\n{body}\n    return 0;\n}}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)  # the header is plain C
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    for line in out.strip().splitlines():
        n, size = line.split()
        assert C.sizeof(names[n]) == int(size), n
    # field offsets of the deepest view
    src.write_text(f'#include <stdio.h>\n#include <stddef.h>\n#include "{HEADER}"\nint main(void) {{\n'
                   '    printf("%zu %zu %zu %zu\\n", offsetof(b200moe_layer_view, x), offsetof(b200moe_layer_view, only_part),'
                   ' offsetof(b200moe_layer_view, workspace_bytes), offsetof(b200moe_ffn_view, policy));\n    return 0;\n}\n')
    subprocess.run(["gcc", "-std=c99", str(src), "-o", str(exe)], check=True)
    a, b, c, d = (int(v) for v in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split())
    assert (a, b, c) == (b200moe.LayerView.x.offset, b200moe.LayerView.only_part.offset, b200moe.LayerView.workspace_bytes.offset)
    assert d == b200moe.FfnView.policy.offset


def test_argument_errors_come_first(lib):
    """Host-side validation needs no device: bad views are rejected with a message and nothing else happens."""
    import b200moe
    v = b200moe.QuantizeA8View(1, 1, 31, 31, 0, b200moe.A8Rows(1, 1, 1, 1, 31, 32), None)
    assert lib.b200moe_quantize_a8(v, None) == b200moe.ERR_INVALID_ARGUMENT
    assert b"multiple of 32" in lib.b200moe_last_error()
    q = b200moe.Q8A8View(1, 68, 33, 0, 1, b200moe.A8Rows(1, 1, None, 1, 64, 64), 1, 1, 0)
    assert lib.b200moe_q8_0_a8(q, None) == b200moe.ERR_INVALID_ARGUMENT
    bad = b200moe.Shape(500, 256, 8, 2, 12, 12, float("inf"))
    assert lib.b200moe_layer_workspace_bytes(bad, 4) == 0
    assert lib.b200moe_layer(b200moe.LayerView(shape=bad), None) == b200moe.ERR_INVALID_ARGUMENT
    grouped = b200moe.RoutePolicy(1, 1, 0, 0, 256, 8, 8, 9, 1, 1, 1e-20, 1.0)  # topk_group > n_group
    r = b200moe.RouterView(policy=grouped, logits=1, ids=1, weights=1, bias=1)
    assert lib.b200moe_router(r, None) == b200moe.ERR_INVALID_ARGUMENT
    for gt, dt in ((12, 10), (10, 12), (10, 7)):            # Q2_K belongs to the Q8_0 / Q2_K family on both sides
        assert lib.b200moe_layer_workspace_bytes(b200moe.Shape(2048, 1024, 8, 2, gt, dt, float("inf")), 4) == 0
    q2 = b200moe.Shape(2048, 1024, 8, 2, 10, 10, float("inf"))
    assert lib.b200moe_layer_workspace_bytes(q2, 4) > 0 and lib.b200moe_gate_row_bytes(q2) == 8 * 84 and lib.b200moe_down_row_bytes(q2) == 4 * 84
    assert lib.b200moe_layer_workspace_bytes(b200moe.Shape(2048 + 32, 1024, 8, 2, 10, 8, float("inf")), 4) == 0   # hidden not in super-blocks
    ok = b200moe.Shape(2048, 768, 128, 8, 12, 12, float("inf"))
    assert lib.b200moe_gate_row_bytes(ok) == 8 * 144 and lib.b200moe_down_row_bytes(ok) == 3 * 144
    assert lib.b200moe_expert_bytes(ok) == 2654208  # config 2's bytes per expert
    assert lib.b200moe_layer_workspace_bytes(ok, 8) > 0
    lv = b200moe.LayerView(shape=ok, rows=9, capacity=8)
    assert lib.b200moe_layer(lv, None) == b200moe.ERR_INVALID_ARGUMENT and b"capacity" in lib.b200moe_last_error()


def test_registry_rows_and_envelope_checks(lib):
    """The launch-record seam: one registry row per enqueue site whose size equals the ctypes mirror of its view, and an
    envelope with the wrong schema, revision or size is refused before the site sees it."""
    import b200moe
    views = {b200moe.SITE_QUANTIZE_A8: b200moe.QuantizeA8View, b200moe.SITE_RMSNORM_A8: b200moe.RmsnormView, b200moe.SITE_Q8_0_A8: b200moe.Q8A8View,
             b200moe.SITE_ROUTER: b200moe.RouterView, b200moe.SITE_ROUTES: b200moe.RoutesView, b200moe.SITE_ROUTES_STATIC: b200moe.RoutesView,
             b200moe.SITE_GATE_UP: b200moe.GateUpView, b200moe.SITE_DOWN: b200moe.DownView, b200moe.SITE_COMBINE: b200moe.CombineView,
             b200moe.SITE_LAYER: b200moe.LayerView, b200moe.SITE_FFN: b200moe.FfnView, b200moe.SITE_DENSE_FFN: b200moe.DenseView}
    rows = b200moe.registry()
    assert set(rows) == set(views)
    for schema, view in views.items():
        assert rows[schema].revision == b200moe.ABI_VERSION and rows[schema].bytes == C.sizeof(view), rows[schema].name
        assert rows[schema].alignment == C.alignment(view) and rows[schema].name.startswith(b"b200moe_")
    v = b200moe.QuantizeA8View(1, 1, 31, 31, 0, b200moe.A8Rows(1, 1, 1, 1, 31, 32), None)
    assert b200moe.enqueue(b200moe.SITE_QUANTIZE_A8, v) == b200moe.ERR_INVALID_ARGUMENT and b"multiple of 32" in lib.b200moe_last_error()  # reached the site
    assert b200moe.enqueue(99, v) == b200moe.ERR_INVALID_ARGUMENT and b"unknown schema" in lib.b200moe_last_error()
    assert b200moe.enqueue(b200moe.SITE_QUANTIZE_A8, v, abi_revision=b200moe.ABI_VERSION - 1) == b200moe.ERR_INVALID_ARGUMENT
    assert b"revision" in lib.b200moe_last_error()
    assert b200moe.enqueue(b200moe.SITE_ROUTER, v) == b200moe.ERR_INVALID_ARGUMENT and b"bytes" in lib.b200moe_last_error()
    assert lib.b200moe_enqueue(None, None) == b200moe.ERR_INVALID_ARGUMENT


def test_first_error_record_check(lib):
    """b200moe_check_first_error on host copies of the record: the cases of check_deferred_moe_status
    (include/strix/deferred_moe_status.hpp:30-42)."""
    import b200moe
    assert lib.b200moe_check_first_error(C.byref(b200moe.FirstError(0, 0))) == b200moe.OK
    assert lib.b200moe_check_first_error(C.byref(b200moe.FirstError(b200moe.DOMAIN_Q4K_A8, 9))) == b200moe.ERR_INVALID_ARGUMENT
    assert b"route/weight=1" in lib.b200moe_last_error() and b": 9" in lib.b200moe_last_error()
    assert lib.b200moe_check_first_error(C.byref(b200moe.FirstError(b200moe.DOMAIN_LEGACY, 1))) == b200moe.ERR_INVALID_ARGUMENT
    assert b"invalid routes" in lib.b200moe_last_error()
    for malformed in ((0, 5), (b200moe.DOMAIN_Q4K_A8, 0), (7, 1)):
        assert lib.b200moe_check_first_error(C.byref(b200moe.FirstError(*malformed))) == b200moe.ERR_UNSUPPORTED
        assert b"malformed" in lib.b200moe_last_error()
    assert lib.b200moe_merge_first_error(None, None, 2, None) == b200moe.ERR_INVALID_ARGUMENT


def test_no_cpu_fallback(lib):
    """Without a usable sm_100 device a well-formed compute call fails with ERR_CUDA."""
    import torch
    import b200moe
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    v = b200moe.QuantizeA8View(256, 1, 32, 32, 0, b200moe.A8Rows(256, 256, 256, 1, 32, 32), None)
    assert lib.b200moe_quantize_a8(v, None) == b200moe.ERR_CUDA
    assert b"no CPU fallback" in lib.b200moe_last_error()
    with pytest.raises(b200moe.B200MoeError):
        b200moe.check(lib.b200moe_quantize_a8(v, None))


def header_abi_version():
    import re
    text = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "b200moe.h")).read()
    return int(re.search(r"#define\s+B200MOE_ABI_VERSION\s+(\d+)", text).group(1))


def test_graft_entry_build_runs():
    """build() compiles (incrementally) the library and the oracle and checks exports and ABI version: what the build check runs."""
    import __graft_entry__ as entry
    entry.build()


REFERENCE_INCLUDE = os.environ.get("STRIX_REFERENCE_INCLUDE", "/root/reference/include")


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_INCLUDE, "strix", "cuda", "ds41_moe.hpp")),
                    reason="the reference checkout is absent: the adapters are compiled against its headers")
@pytest.mark.parametrize("source,compiler", [("strix_ds41_b200.cpp", "g++"), ("strix_qwen_b200.cpp", "nvcc"), ("strix_weight_b200.cpp", "g++")])
def test_adapters_compile_against_the_reference_headers(tmp_path, source, compiler):
    """adapter/*.cpp re-expose the C ABI under the reference's operator names; compiling them against the reference's
    own headers is what shows that every view maps field for field (types included). The DS41 operator header is plain
    C++ (g++ -fsyntax-only); the Qwen header pulls in a .cuh with device intrinsics and needs nvcc."""
    import shutil
    path = os.path.join(ROOT, "adapter", source)
    inc = ["-I" + REFERENCE_INCLUDE, "-I" + os.path.join(ROOT, "include")]
    if compiler == "g++":
        cmd = ["g++", "-std=c++20", "-fsyntax-only", "-Wall", "-I/usr/local/cuda/include"] + inc + [path]
    else:
        nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
        if not os.path.exists(nvcc):
            pytest.skip("nvcc not found")
        cmd = [nvcc, "-x", "cu", "-std=c++20", "-arch=sm_100a"] + inc + ["-c", path, "-o", str(tmp_path / "adapter.o")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
