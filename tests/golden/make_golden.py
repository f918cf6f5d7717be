"""Generates tests/golden/moe_golden.npz from the reference's OWN CPU code (oracle/_ref/libstrixref.so, built from
the reference checkout by oracle/Makefile). Run where the reference checkout exists:

    make -C oracle && python tests/golden/make_golden.py

norm_golden.npz (the RMSNorm in front of the FFN) is written by the same run; `--norm-only` writes just that file; formats_golden.npz (Q5_K / Q5_1 tensors) likewise with `--formats-only`, planner_golden.npz (the residency planner's traces) with `--planner-only`.
The vectors are small seeded cases of every contract on the path; tests/test_oracle_pins.py::test_golden_vectors
replays them against the restated oracle wherever the reference itself is absent (e.g. on the GPU box).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "strix-halo-engine-lab_b200")]
from oracle.loader import Ref  # noqa: E402
from b200moe import synth  # noqa: E402


def main():
    ref = Ref()
    rng = np.random.default_rng(20250)
    out = {}
    # A8
    x = rng.standard_normal((3, 256), dtype=np.float32) * np.float32(2.5)
    x[1, :32] = 0.0
    x[1, 32:64] = 1e-37
    out["a8_x"] = x
    out["a8_codes"], out["a8_deltas"], out["a8_sums"] = ref.quantize_a8(x)
    # Q8_0 x A8 GEMV
    width, count = 1024, 12
    w = synth.q8_0_blocks(rng, count * width // 32).reshape(count, -1)
    xx = rng.standard_normal((2, width), dtype=np.float32)
    c, d, _ = ref.quantize_a8(xx)
    out.update(q8_w=w, q8_width=np.int64(width), q8_codes=c, q8_deltas=d, q8_y=ref.gemv_q8_0_a8(w, width, c, d))
    # Q4_K x A8 rows (executor scalar table)
    width = 2048
    w4 = synth.q4_k_blocks(rng, 10 * width // 256, scale=0.002).reshape(10, -1)
    x4 = rng.standard_normal((1, width), dtype=np.float32)
    c, d, s = ref.quantize_a8(x4)
    y4 = np.array([ref.gate_row_q4k(w4[o], c[0], d[0], s[0]) for o in range(10)], np.float32)
    out.update(q4k_w=w4, q4k_codes=c, q4k_deltas=d, q4k_sums=s, q4k_y=y4)
    # reference_router (sqrt-softplus, ds41 preset)
    E, H, K = 64, 512, 6
    rx = rng.standard_normal((4, H), dtype=np.float32)
    rw = synth.router_weight(rng, E, H, std=0.05)
    rb = (rng.standard_normal(E) * 0.1).astype(np.float32)
    sc, ids, wt = ref.reference_router(rx, rw, rb, K, 1.5)
    out.update(rt_x=rx, rt_w=rw, rt_bias=rb, rt_scores=sc, rt_ids=ids, rt_weights=wt)
    # softmax policy through route_scores_ref + route_select_ref
    from oracle.loader import softmax_policy
    lg = rng.uniform(-1, 1, size=(6, 128)).astype(np.float32)
    pol = softmax_policy(128, 8)
    sc = ref.route_scores(pol.score, lg)
    ids, wt = ref.route_select(pol, sc)
    out.update(sm_logits=lg, sm_scores=sc, sm_ids=ids, sm_weights=wt)
    # DS41 window, Q8_0
    E, H, I, K, rows = 6, 256, 128, 3, 4
    g, u, dn = synth.expert_tensors(rng, E, H, I, 8, 8)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
    shared = rng.standard_normal((rows, H), dtype=np.float32)
    win = ref.window_q8_0(g, u, dn, E, H, I, 10.0, x, ids, wts, shared, split=E // 2)
    out.update(win_shape=np.array([E, H, I, K]), win_limit=np.float32(10.0), win_gate=g, win_up=u, win_down=dn, win_x=x,
               win_ids=ids, win_weights=wts, win_shared=shared, win_raw=win["raw"], win_y=win["y"])
    # Qwen job: Q4_K gate/up, Q8_0 four-chain down (reference_run)
    E, H, I, K, rows = 4, 256, 128, 2, 3
    g, u, _ = synth.expert_tensors(rng, E, H, I, 12, 12)
    dn = synth.q8_0_blocks(rng, E * H * (I // 32)).reshape(-1)
    x = rng.standard_normal((rows, H), dtype=np.float32)
    c, d, s = ref.quantize_a8(x)
    ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
    raw, status = ref.expert_run(g, u, dn, 0, 1, H, I, c, d, s, ids, threads=0)
    assert not status.any()
    out.update(qw_shape=np.array([E, H, I, K]), qw_gate=g, qw_up=u, qw_down=dn, qw_x=x, qw_ids=ids, qw_raw=raw)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "moe_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def norm_vectors():
    """tests/golden/norm_golden.npz: RMSNorm of the CPU backend (rmsnorm_f32) on small seeded rows, both lane counts."""
    ref = Ref()
    rng = np.random.default_rng(20251)
    out = {}
    for n in (96, 512, 2048):
        x = (rng.standard_normal((3, n)) * 3.0).astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        out[f"x_{n}"], out[f"w_{n}"] = x, w
        out[f"y_{n}"] = ref.rmsnorm(x, w, 1e-6)
        out[f"y_unscaled_{n}"] = ref.rmsnorm(x, None, 1e-6)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "norm_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


def format_vectors():
    """tests/golden/formats_golden.npz: reference_run on Q5_K gate/up and Q5_1 / Q8_0 down tensors."""
    ref = Ref()
    rng = np.random.default_rng(20252)
    E, H, I, K, rows = 2, 256, 128, 2, 2
    out = {"shape": np.array([E, H, I, K])}
    for gt, dt, gf, df in ((13, 7, 1, 0), (12, 7, 0, 0), (13, 8, 1, 1)):
        g, u, d = synth.expert_tensors(rng, E, H, I, gt, dt)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        c, dl, s = ref.quantize_a8(x)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        raw, status = ref.expert_run(g, u, d, gf, df, H, I, c, dl, s, ids, threads=0)
        assert not status.any()
        t = f"{gt}_{dt}"
        out.update({f"gate_{t}": g, f"up_{t}": u, f"down_{t}": d, f"x_{t}": x, f"ids_{t}": ids, f"raw_{t}": raw})
    # Q2_K tensors of the DS41 family, alone and mixed with Q8_0 (reference_window, limit 7)
    H2, I2 = 512, 256
    out["shape_q2k"] = np.array([E, H2, I2, K])
    for gt, dt in ((10, 10), (10, 8), (8, 10)):
        g, u, d = synth.expert_tensors(rng, E, H2, I2, gt, dt)
        x = rng.standard_normal((rows, H2), dtype=np.float32)
        ids = np.stack([rng.permutation(E)[:K] for _ in range(rows)]).astype(np.uint32)
        wts = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        win = ref.window_ds41(gt, dt, g, u, d, E, H2, I2, 7.0, x, ids, wts, None, split=E // 2)
        t = f"{gt}_{dt}"
        out.update({f"gate_{t}": g, f"up_{t}": u, f"down_{t}": d, f"x_{t}": x, f"ids_{t}": ids, f"raw_{t}": win["raw"], f"act_codes_{t}": win["act_codes"]})
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "formats_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")



def planner_vectors():
    """planner_golden.npz: the reference Planner's moves, tables and receipt on the traces of tests/test_planner.py."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import test_planner as tp
    ref = Ref()
    out = {}
    for k, case in enumerate(tp.CASES):
        layers, experts, top_k, slots, eb, decay, margin, budget, steps, n, seeded, _ = case
        ids, seed_counts = tp.trace_of(case, 100 + k)
        moves, tables, receipt = ref.planner_trace(layers, experts, top_k, slots, eb, decay, margin, budget, ids, seed_counts, fill=seeded)
        out[f"moves_{k}"] = np.array([m for step in moves for m in step], np.uint32).reshape(-1, 4)
        out[f"counts_{k}"] = np.array([len(s) for s in moves])
        out[f"tables_{k}"] = tables
        out[f"receipt_{k}"] = np.array(list(receipt.values()), np.uint64)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "planner_golden.npz"), **out)
    print("planner_golden.npz:", sum(int(v.sum()) for k, v in out.items() if k.startswith("counts_")), "moves")


if __name__ == "__main__":
    only = [a for a in sys.argv[1:] if a.endswith("-only")]
    if not only:
        main()
    if not only or "--norm-only" in only:
        norm_vectors()
    if not only or "--formats-only" in only:
        format_vectors()
    if not only or "--planner-only" in only:
        planner_vectors()
