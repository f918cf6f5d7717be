#!/usr/bin/env python
"""Benchmark of the block-quantized MoE FFN hot path on B200.

Default workload (`--workload c4`): the large routed layer in decode at a FIXED global batch of 64 rows - hidden 7168, 256
Q4_K routed experts behind a sigmoid + bias, group-limited top-8 router, one Q8_0 shared expert, inter 2048. One GPU holds
every expert (b200moe_ffn); N GPUs run expert parallelism (b200moe_ep_ffn: 256 / N experts and 64 / N home rows per rank),
so the total work is the same at every N ("scaling": "strong"). A step reads the realised distinct experts' bytes - about
2.7 GB, far beyond the 126 MB L2. Other workloads: c1 (Q8_0 decode, batch 1), c2 (Q4_K decode, hidden 2048, batch 1 - 8;
its batch-8 line is repeated under `extra.c2_b8` of the default run), c3 (Q4_K prefill, 4096 tokens), c5 (dense Q4_K block;
tensor parallelism at N > 1). Smaller layers rotate over several layers' worth of distinct weights (over twice the L2).

One JSON line on stdout (rank 0):
  value     whole-job tokens/s with inputs resident in HBM, steps replayed from a CUDA graph (device-timed, max over
            ranks, repeated until the timed region is at least a quarter of a second); `ms_per_step` likewise
  e2e       the same metric through the C ABI with pinned host rows in and the result back on the host every step
  roofline  the dominant kernel (routed Q4_K gate/up GEMV): algorithmic bytes / its CUDA-event duration, against the
            measured HBM copy peak; `traffic` = DRAM bytes per launch (ncu capture, see the note in the line)
  parity    one step against the CPU oracle, outside the timed regions
  cpu_baseline  the reference's own CPU row kernels (oracle/_ref) or the oracle port, on the host cores, bounded sample
`--impl reference` times that CPU arm alone on the same config and prints the same line shape.
"""
import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "strix-halo-engine-lab_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

CONFIGS = {
    # name: hidden, experts, top_k, inter, gate_type, down_type
    "c2": dict(hidden=2048, experts=128, top_k=8, inter=768, gate_type=12, down_type=12,
               desc="MoE decode layer, Q4_K experts: hidden 2048, 128 experts, top-8, inter 768"),
}
CONFIGS["c1"] = dict(hidden=2048, experts=64, top_k=4, inter=1024, gate_type=8, down_type=8, batch=1, parts_form=True,
                     desc="MoE decode layer, Q8_0 experts (the reference's CPU-backend case): hidden 2048, 64 experts, top-4, inter 1024")
CONFIGS["c3"] = dict(CONFIGS["c2"], desc="MoE prefill layer, Q4_K experts: hidden 2048, 128 experts, top-8, inter 768, "
                                           "bf16-rounded activations, Zipf(1.1) expert load", prefill=True)
CONFIGS["c4"] = dict(hidden=7168, experts=256, top_k=8, inter=2048, gate_type=12, down_type=12, large=True,
                     desc="large routed MoE decode layer: hidden 7168, 256 Q4_K experts + 1 Q8_0 shared expert, inter 2048, "
                          "sigmoid + bias router, 8 groups / best 4 / top-8, bf16-rounded activations")
CONFIGS["c5"] = dict(hidden=5120, experts=1, top_k=1, inter=17408, gate_type=12, down_type=12, dense=True,
                     desc="dense SwiGLU FFN block, Q4_K: hidden 5120, inter 17408")
METRIC = "MoE-layer tokens/s (Q4_K decode)"
UNIT = "tokens/s"
L2_BYTES = 126 * 2 ** 20
NCU_TRAFFIC_RATIO = 1.00  # measured dram bytes / algorithmic bytes of the gate/up kernel (ncu, three launches: 0.999 - 1.002)
# The same ratio for the segment-streaming gate/up kernel, from one ncu capture of a REDUCED config-4 layer (64 experts,
# batch 32: 1001.2 MB of DRAM traffic against 972.6 MB algorithmic). Traffic grows with the distinct experts a launch
# touches, as the algorithmic bytes do, so a full launch is quoted as its algorithmic bytes times this ratio.
C4_TRAFFIC_RATIO = 1.03


def metric_of(cfg):
    if cfg.get("dense"):
        return "dense FFN block tokens/s (Q4_K decode)"
    return METRIC if cfg["gate_type"] == 12 else "MoE-layer tokens/s (Q8_0 decode)"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """SM clock and throttle reasons sampled through NVML while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
            while not self.stop_flag:
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                r = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.reasons |= {n for bit, n in names.items() if r & bit}
                time.sleep(0.005)
        except Exception as e:  # NVML missing: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_layer(cfg, seed):
    from b200moe import synth
    rng = np.random.default_rng(seed)
    g, u, d = synth.expert_tensors(rng, cfg["experts"], cfg["hidden"], cfg["inter"], cfg["gate_type"], cfg["down_type"])
    return g, u, d, synth.router_weight(rng, cfg["experts"], cfg["hidden"])


def expert_bytes(cfg):
    if cfg["gate_type"] == 8:
        return 2 * cfg["inter"] * (cfg["hidden"] // 32 * 34), cfg["hidden"] * (cfg["inter"] // 32 * 34)
    gate_row = cfg["hidden"] // 256 * 144
    down_row = cfg["inter"] // 256 * 144
    return 2 * cfg["inter"] * gate_row, cfg["hidden"] * down_row


def cpu_arm(cfg, batch, target_s, threads=None):
    """Times the reference's own CPU code (oracle/_ref) - or the oracle port when that build is absent - on one
    layer of the workload. Returns (tokens/s, description dict)."""
    from oracle import loader as O
    from b200moe import synth
    g, u, d, rw = make_layer(cfg, 1000)
    x = synth.activations(np.random.default_rng(7), batch, cfg["hidden"])
    threads = threads or os.cpu_count() or 1
    if cfg["gate_type"] == 8:  # the reference's Q8_0 path is scalar and single-threaded (reference_window; no SIMD / threaded table)
        pol = O.softmax_policy(cfg["experts"], cfg["top_k"])
        orc = O.Oracle()
        _, _, ids, wts = orc.router(pol, x=x, w=rw)
        if O.Ref.available():
            ref = O.Ref()
            call = lambda: ref.window_q8_0(g, u, d, cfg["experts"], cfg["hidden"], cfg["inter"], float("inf"), x, ids, wts, None, cfg["experts"] // 2)
            kind = "reference"
        else:
            sh = O.Shape(cfg["hidden"], cfg["inter"], cfg["experts"], cfg["top_k"], 8, 8, float("inf"))
            call = lambda: orc.ffn(sh, pol, g, u, d, rw, x, O.COMBINE_PARTS)
            kind = "port"
        t0 = time.perf_counter()
        call()
        one = time.perf_counter() - t0
        reps = max(1, int(target_s / max(one, 1e-6)))
        t0 = time.perf_counter()
        for _ in range(reps):
            call()
        sec = time.perf_counter() - t0
        value = batch * reps / sec
        return value, {"value": value, "unit": UNIT, "cores": 1, "kind": kind,
                       "sample": f"{reps} reference_window calls of batch {batch} on one layer's weights ({sec:.1f} s, scalar single thread: "
                                 "the reference has no SIMD or threaded Q8_0 kernel; router ids precomputed)"}
    if O.Ref.available():
        ref = O.Ref()
        args = (g, u, d, cfg["experts"], cfg["hidden"], cfg["inter"], cfg["top_k"], rw, x, threads)
        sec, _, _ = ref.time_layer_q4k(*args, 1)
        reps = max(1, min(5000, int(target_s / max(sec, 1e-6))))
        sec, _, _ = ref.time_layer_q4k(*args, reps)
        kind, isa = "reference", ref.isa()
    else:
        orc = O.Oracle()
        sh = O.Shape(cfg["hidden"], cfg["inter"], cfg["experts"], cfg["top_k"], cfg["gate_type"], cfg["down_type"], float("inf"))
        pol = O.softmax_policy(cfg["experts"], cfg["top_k"])
        t0 = time.perf_counter()
        orc.ffn(sh, pol, g, u, d, rw, x, O.COMBINE_FMA_SLOTS)
        one = time.perf_counter() - t0
        reps = max(1, int(target_s / max(one, 1e-6)))
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.ffn(sh, pol, g, u, d, rw, x, O.COMBINE_FMA_SLOTS)
        sec = time.perf_counter() - t0
        kind, isa = "port", "scalar"
    value = batch * reps / sec
    return value, {"value": value, "unit": UNIT, "cores": threads, "kind": kind,
                   "sample": f"{reps} layer calls of batch {batch} on one layer's weights ({sec:.1f} s, isa {isa}, synthetic exp tables)"}


def reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    batch = cfg.get("batch", args.batch) if args.batch == 8 else args.batch
    total = max(1, args.steps + args.warmup)
    value, base = cpu_arm(cfg, batch, target_s=min(60.0, 0.02 * total + 15.0))
    line = {"impl": "reference", "metric": metric_of(cfg), "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * batch / value, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8xint4->int32, fp32 chains", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {cfg['desc']}, batch {batch}", "l2": "host arm"},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def prefill_arm(args, cfg, rank, world, dev):
    """Token-block (prefill) form: a step is one b200moe_ffn call over `--batch` tokens (default 4096) through the
    grouped tensor-core kernels. Each rank is a replica with its own tokens. The roofline is the one the path is quoted
    on - useful FLOP (2 x assignments x 3 x hidden x inter) against the measured dense bf16 rate - although the kernel
    itself is bound by the FP32 work after the integer MMAs; the gate/up kernel is timed with CUDA events."""
    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ops, synth

    K, W, L = args.steps, max(args.warmup, 3), min(args.layers, 2)
    B = args.batch if args.batch != 8 else 4096
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    shape = ops.make_shape(H, I, E, TK, cfg["gate_type"], cfg["down_type"])
    policy = ops.softmax_policy(E, TK)
    layers = []
    for li in range(L):
        g, u, d, rw = make_layer(cfg, 1000 + li + 100 * rank)
        bias = synth.zipf_logit_bias(np.random.default_rng(50 + li), E)
        layers.append(ops.MoeFfn(shape, policy, *(torch.from_numpy(a).to(dev) for a in (g, u, d, rw)), capacity=B,
                                 combine_form=b200moe.COMBINE_FMA_SLOTS, logit_bias=torch.from_numpy(bias).to(dev)))
    rng = np.random.default_rng(7 + rank)
    NX = 2
    xs_host = [torch.from_numpy(synth.bf16_round(synth.activations(rng, B, H))).pin_memory() for _ in range(NX)]
    xs = [x.to(dev) for x in xs_host]
    y = torch.empty((B, H), dtype=torch.float32, device=dev)
    ys_host = torch.empty((B, H), dtype=torch.float32).pin_memory()
    ids = torch.empty((B, TK), dtype=torch.int32, device=dev)
    wts = torch.empty((B, TK), dtype=torch.float32, device=dev)
    lib = b200moe.lib()
    stream = torch.cuda.current_stream()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True),
            torch.cuda.Event(enable_timing=True)) for _ in range(L * NX)]
    for e4 in evs:
        for e in e4:
            e.record()
    torch.cuda.synchronize()
    taps = [ops.MoeFfn.stage_events([None, None, a.cuda_event, b.cuda_event, c.cuda_event, d.cuda_event, None, None]) for a, b, c, d in evs]
    views = [layers[s % L]._view(B, xs[s % NX], y, ids, wts, events=taps[s]) for s in range(L * NX)]
    host_views = [layers[s % L]._view(B, None, None) for s in range(L * NX)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(n):
        for s in range(n):
            b200moe.check(lib.b200moe_ffn(C.byref(views[s % len(views)]), stream.cuda_stream))

    def run_host(n):
        for s in range(n):
            b200moe.check(lib.b200moe_ffn_host(C.byref(host_views[s % len(host_views)]), xs_host[s % NX].data_ptr(), ys_host.data_ptr(),
                                               stream.cuda_stream))

    run(W)
    barrier()
    counts = np.bincount(ids.cpu().numpy().reshape(-1), minlength=E)
    launches0 = b200moe.launch_count()
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gu_ms, dn_ms, done = [], [], 0
    barrier()
    e0.record()
    while done < K:
        n = min(K - done, len(views))
        run(n)
        torch.cuda.synchronize()
        gu_ms += [evs[s][0].elapsed_time(evs[s][1]) for s in range(n)]
        dn_ms += [evs[s][2].elapsed_time(evs[s][3]) for s in range(n)]
        done += n
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = b200moe.launch_count() - launches0
    run_host(min(W, 3))
    barrier()
    t0 = time.perf_counter()
    run_host(K)
    barrier()
    host_ms = 1000.0 * (time.perf_counter() - t0)
    sampler.stop_flag = True
    sampler.join(timeout=2)
    t = torch.tensor([dev_ms, host_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, host_ms = (float(v) for v in t.cpu())
    tokens = B * K * world
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak_tf, kind = (float(json.load(open(path))["bf16_tflops_sustained"]), "measured sustained") if os.path.exists(path) else (1400.0, "fallback")
    gu_flop = 2.0 * B * TK * 2 * I * H          # gate + up
    achieved = gu_flop / (float(np.mean(gu_ms)) * 1e-3) / 1e12
    line = {
        "metric": "MoE-layer tokens/s (Q4_K prefill)", "value": tokens / (dev_ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8xint4->int32 (tcgen05 kind::i8), fp32 chains", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}, {B} tokens per step", "parallelism": f"replicas x{world}" if world > 1 else "1 gpu",
                   "l2": f"{L} layers of distinct expert weights rotated ({L * 340} MB > 2 x 126 MiB L2)", "launch": "per-step launches",
                   "expert_load": {"max_rows": int(counts.max()), "mean_rows": float(counts.mean()), "empty_experts": int((counts == 0).sum())}},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens / (host_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "ms_per_step": host_ms / K},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "grouped_q4k_kernel<gate/up>", "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                     "frac": achieved / peak_tf, "peak_kind": f"{kind} dense bf16", "traffic": None,
                     "algorithmic_flop_per_launch": gu_flop, "avg_launch_us": float(np.mean(gu_ms)) * 1000.0,
                     "down_avg_launch_us": float(np.mean(dn_ms)) * 1000.0},
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            _, base = cpu_arm(cfg, 256, target_s=12.0)
            base["sample"] = "256 of the step's tokens: " + base["sample"]
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def dense_arm(args, cfg, rank, world, dev):
    """Config 5: the dense Q4_K FFN block (hidden 5120, inter 17408), `--batch` rows (1..8). One GPU holds the whole
    block; N GPUs run tensor parallelism (b200moe.tp): whole-super-block shares of inter per rank, every rank sees the
    same rows, the partial sums are exchanged by the library's peer stores and folded in rank order on every rank
    (b200moe_tp_dense: one C call per step). A step = A8 of x + gate/up + SwiGLU + A8 of h + down (+ exchange + fold).
    Enough distinct layers are rotated that one rotation exceeds twice the L2."""
    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ops, synth, tp

    K, W = args.steps if args.steps != 2000 else 400, max(min(args.warmup, 50), 3)
    B = args.batch
    H, I = cfg["hidden"], cfg["inter"]
    start, size = tp.tp_shares(I, world)[rank]
    shape = ops.make_shape(H, size, 1, 1, 12, 12)
    rank_bytes = 3 * (size // 256) * 144 * H                     # gate + up rows of the share, down K-share of every row
    # shares differ by one super-block when the blocks do not divide: every rank must build the SAME number of layers (each
    # one hands its window round collectively), so the count comes from rank 0's share, the largest
    largest = 3 * (tp.tp_shares(I, world)[0][1] // 256) * 144 * H
    layers = max(2, min(32, -(-2 * L2_BYTES // largest) + 1))
    kernels = []
    for layer in range(layers):
        gate, up, down = synth.expert_tensors(np.random.default_rng(900 + layer), 1, H, I, 12, 12)
        g2, u2, d3 = gate.reshape(I, -1), up.reshape(I, -1), down.reshape(H, I // 256, 144)
        share = (np.ascontiguousarray(g2[start:start + size]).reshape(-1), np.ascontiguousarray(u2[start:start + size]).reshape(-1),
                 np.ascontiguousarray(d3[:, start // 256:(start + size) // 256]).reshape(-1))
        kernels.append(tp.DeviceDenseKernels(shape, *(torch.from_numpy(a).to(dev) for a in share)))
        del gate, up, down, share
    # N > 1: share + exchange + rank-ordered fold behind ONE C call per step (b200moe_tp_dense: peer stores, flag waits)
    ffns = [tp.PeerTpDense(k.shape, k.gate, k.up, k.down, B, payload_bf16=args.tp_payload == "bf16") for k in kernels] if world > 1 else None
    rng = np.random.default_rng(7)                            # the same rows on every rank (x is replicated under TP)
    NX = 4
    xs_host = [torch.from_numpy(synth.activations(rng, B, H)).pin_memory() for _ in range(NX)]
    xs = [x.to(dev) for x in xs_host]
    ys_host = torch.empty((B, H), dtype=torch.float32).pin_memory()

    def step(s, x):
        return ffns[s % layers](x) if world > 1 else kernels[s % layers].partial(x)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for s in range(W):
        step(s, xs[s % NX])
    barrier()
    graph, mode, G = None, "per-step launches", layers * NX // math.gcd(layers, NX)
    if world > 1:
        G *= 2          # every layer's exchange alternates between two window halves: an even number of its steps per graph
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            launches_before = b200moe.launch_count()
            with torch.cuda.graph(g, stream=cap):
                kept = [step(s, xs[s % NX]) for s in range(G)]
            per_graph = b200moe.launch_count() - launches_before
            graph, mode = g, f"CUDA graph replay of {G} steps"
            for _ in range(2):
                graph.replay()
        except Exception as e:  # noqa: BLE001 - any capture problem: measure the eager path and say so
            graph, mode = None, f"per-step launches (graph capture failed: {type(e).__name__})"
    barrier()
    launches0 = b200moe.launch_count()
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    if graph is not None:
        for _ in range(K // G):
            graph.replay()
        for s in range(K % G):
            step(s, xs[s % NX])
    else:
        for s in range(K):
            step(s, xs[s % NX])
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = (b200moe.launch_count() - launches0) + (per_graph * (K // G) if graph is not None else 0)
    t0 = time.perf_counter()
    for s in range(K):
        ys_host.copy_(step(s, xs_host[s % NX].to(dev, non_blocking=True)), non_blocking=True)
    barrier()
    host_ms = 1000.0 * (time.perf_counter() - t0)
    sampler.stop_flag = True
    sampler.join(timeout=2)
    t = torch.tensor([dev_ms, host_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, host_ms = (float(v) for v in t.cpu())
    tokens = B * K                                            # TP: every rank works on the same rows (strong scaling)
    peak, peak_kind = peaks()
    achieved = rank_bytes / (dev_ms / K * 1e-3) / 1e9
    line = {
        "metric": metric_of(cfg), "value": tokens / (dev_ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "int8xint4->int32, fp32 chains", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}, batch {B}",
                   "parallelism": f"tp x{world} (inter share {size} of {I} on rank 0)" if world > 1 else "1 gpu",
                   "l2": f"{layers} distinct layers rotated ({layers * rank_bytes / 2 ** 20:.0f} MB per rank per rotation, L2 is 126 MB)",
                   "launch": mode + (f"; partial sums exchanged by the library's peer stores ({args.tp_payload} payload) with bounded flag waits, "
                                     "folded in rank order on every rank (no collective)" if world > 1 else "")},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens / (host_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "ms_per_step": host_ms / K},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "whole step (the rank's gate + up + down bytes / step time)", "bound": "hbm", "achieved": achieved,
                     "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"{peak_kind} HBM copy", "traffic": None,
                     "algorithmic_bytes_per_step": rank_bytes},
    }
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            _, base = cpu_arm(cfg, B, target_s=10.0)
            line["cpu_baseline"] = base
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---- config 4: the default workload ---------------------------------------------------------------------------------
C4_PARTS = 8          # the fold always has 8 expert ranges: 1 GPU and 8 GPUs give the same bits
C4_GLOBAL_BATCH = 64


def gate_up_kernel_name(cfg, rows, form):
    """The routed gate/up kernel the library picks for a decode window of `rows` rows (csrc/api.cu: pick_decode_form,
    use_q8_wide), or the one --form forces."""
    if cfg["gate_type"] != 12:
        return "q8_wide_kernel<gate/up>" if (form == 2 or (form == 0 and rows >= 8)) else "gate_up_q8_kernel"
    if form == 3:
        return "gate_up_q4k_kernel (per-block form)"
    stream = form == 1 or (form == 0 and rows <= 2 and cfg["hidden"] <= 2048)
    return "gate_up_q4k_stream_kernel" if stream else "q4k_wide_kernel<gate/up>"


def c4_phase(batch):
    """Windows of 128 rows and more are token blocks (the routed experts then take the grouped tensor-core form)."""
    return "prefill" if batch >= 128 else "decode"


def c4_config(cfg, batch, world):
    """The `config` object both arms print (the driver compares them key by key)."""
    return {"workload": f"c4: {cfg['desc']}, {c4_phase(batch)}, global batch {batch}",
            "parallelism": f"ep x{world} ({cfg['experts'] // world} experts and {batch // world} home rows per rank)" if world > 1 else "1 gpu (all 256 experts)",
            "l2": "5.5 GB of distinct routed expert weights per step (far beyond the 126 MB L2)"}


class C4Model:
    """Seeded synthetic config-4 layer. The routed experts are drawn once for one slice of 32 experts (0.8 GB); slice r of
    the 8 is that slice with every tensor rotated by r * 37 weight rows, so the 256 experts differ while a host only
    ever draws one slice. expert_host(e) cuts one expert out of that definition without building the 6.3 GB layer."""

    SHIFT_ROWS = 37

    def __init__(self, cfg):
        from b200moe import synth
        self.cfg = cfg
        H, E, I = cfg["hidden"], cfg["experts"], cfg["inter"]
        self.per = 32
        rng0 = np.random.default_rng(400)
        self.rw = synth.router_weight(rng0, E, H)
        self.bias = (rng0.standard_normal(E) * 0.1).astype(np.float32)
        self.shared = synth.expert_tensors(rng0, 1, H, I, 8, 8)
        self.base = synth.expert_tensors(np.random.default_rng(500), self.per, H, I, 12, 12)
        self.row_bytes = (H // 256 * 144, H // 256 * 144, I // 256 * 144)
        self.rows = (I, I, H)

    def shift(self, t, r):
        return r * self.SHIFT_ROWS * self.row_bytes[t]

    def slice_device(self, r, dev):
        import torch
        return tuple(torch.roll(torch.from_numpy(self.base[t]).to(dev), self.shift(t, r)) for t in range(3))

    def expert_host(self, e):
        r, el = divmod(e, self.per)
        out = []
        for t in range(3):
            n = self.rows[t] * self.row_bytes[t]
            idx = (np.arange(el * n, (el + 1) * n, dtype=np.int64) - self.shift(t, r)) % self.base[t].size
            out.append(self.base[t][idx])
        return out

    def compact(self, ids):
        """Host tensors holding only the experts `ids` name, and the ids renumbered into them (ascending expert id)."""
        used = np.unique(ids)
        parts = [self.expert_host(int(e)) for e in used]
        tensors = tuple(np.concatenate([p[t] for p in parts]) for t in range(3))
        return tensors, np.searchsorted(used, ids).astype(np.uint32), len(used)

    def batches(self, n, batch):
        from b200moe import synth
        rng = np.random.default_rng(7)
        return [synth.bf16_round(synth.activations(rng, batch, self.cfg["hidden"])) for _ in range(n)]


def c4_oracle_rows(model, x):
    """The CPU oracle's y for the rows x (config-4 layer: group-limited router, routed Q4_K experts over the experts the
    rows select, Q8_0 shared expert, 8-range fold). Returns (y, ids)."""
    from oracle import loader as O
    cfg = model.cfg
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    orc = O.Oracle()
    _, _, ids, wts = orc.router(O.sigmoid_group_policy(E, TK, 8, 4), x=x, w=model.rw, bias=model.bias)
    codes, deltas, sums = orc.quantize_a8(x)
    (g, u, d), local, n_used = model.compact(ids)
    raw = orc.experts(O.Shape(H, I, n_used, TK, 12, 12, float("inf")), g, u, d, local, codes, deltas, sums)["raw"]
    sg, su, sd = model.shared
    shared = orc.experts(O.Shape(H, I, 1, 1, 8, 8, float("inf")), sg, su, sd, np.zeros((x.shape[0], 1), np.uint32), codes, deltas, sums)["raw"]
    y = orc.combine(O.COMBINE_PARTS, raw, wts, ids, shared=shared, parts=C4_PARTS, part_experts=E // C4_PARTS)
    return y, ids


def c4_cpu_arm(model, x, target_s):
    """The reference's CPU code on a bounded sample of the step: its routed-expert row kernels (AVX2 / AVX-VNNI table,
    all host threads) on the sample's routes, its Q8_0 x A8 product for the shared expert's three matrices (rows split
    over the threads), and the group-limited router, which the reference does not have, from the CPU oracle.
    Returns (tokens/s, description)."""
    from oracle import loader as O
    cfg = model.cfg
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    threads = os.cpu_count() or 1
    orc = O.Oracle()
    pol = O.sigmoid_group_policy(E, TK, 8, 4)
    _, _, ids, _ = orc.router(pol, x=x, w=model.rw, bias=model.bias)
    (g, u, d), local, _ = model.compact(ids)
    codes, deltas, _ = orc.quantize_a8(x)
    sg, su, sd = model.shared
    have_ref = O.Ref.available()
    ref = O.Ref() if have_ref else None

    def once(reps):
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.router(pol, x=x, w=model.rw, bias=model.bias)
        t_router = time.perf_counter() - t0
        if have_ref:
            t_experts, _ = ref.time_experts_q4k(g, u, d, H, I, TK, x, local, threads, reps)
            t_shared = sum(ref.time_gemv_q8_0_a8(w, width, c, dl, threads, reps)[0]
                           for w, width, c, dl in ((sg, H, codes, deltas), (su, H, codes, deltas),
                                                   (sd, I, np.ascontiguousarray(codes[:, :I]), np.ascontiguousarray(deltas[:, :I // 32]))))
        else:
            t0 = time.perf_counter()
            for _ in range(reps):
                c4_oracle_rows(model, x)
            t_experts, t_shared = time.perf_counter() - t0 - t_router, 0.0
        return t_router + t_experts + t_shared

    one = once(1)
    reps = max(1, min(200, int(target_s / max(one, 1e-6))))
    sec = once(reps)
    value = x.shape[0] * reps / sec
    kind = "reference" if have_ref else "port"
    what = (f"{reps} x {x.shape[0]} tokens of one step ({sec:.1f} s): reference row kernels (isa {ref.isa()}) for the routed experts on the sample's routes + "
            "reference gemv_q8_0_a8 for the shared expert, own threaded driver with a kept pool; group-limited router from the CPU oracle "
            "(the reference has none)") if have_ref else f"{reps} x {x.shape[0]} tokens of one step through the CPU oracle port ({sec:.1f} s)"
    base = {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": what}
    if have_ref:
        # what the arm streamed per second (the sample's distinct experts + the shared expert, once per repetition) beside the
        # host's pure-read ceiling over the same tensors
        streamed = (g.nbytes + u.nbytes + d.nbytes + sum(a.nbytes for a in model.shared)) * reps
        base["weights_gbs"] = streamed / sec / 1e9
        base["host_read_gbs"] = ref.host_read_gbs(g, threads)
    return value, base


def c4_reference_arm(args, cfg, rank, world):
    if rank != 0:
        return
    model = C4Model(cfg)
    x = model.batches(1, C4_GLOBAL_BATCH)[0][:8]
    total = max(1, args.steps + args.warmup)
    value, base = c4_cpu_arm(model, x, target_s=min(45.0, 0.05 * total + 15.0))
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1000.0 * C4_GLOBAL_BATCH / value, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8xint4->int32, fp32 chains", "data": "synthetic", "config": c4_config(cfg, C4_GLOBAL_BATCH, world),
            "cpu_baseline": base, "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def large_arm(args, cfg, rank, world, dev):
    """Config 4, decode at a FIXED global batch of 64 rows per step (strong scaling): 256 routed Q4_K experts behind a
    sigmoid + bias, group-limited router plus one Q8_0 shared expert. One GPU holds every expert (b200moe_ffn, the fold
    over 8 expert ranges); N GPUs run expert parallelism through b200moe_ep_ffn: experts / N and 64 / N home rows per rank,
    dispatch and return by the library's peer-store kernels with flag waits, no collective on the data path. Same kernels
    and the same total work at every N. A step = shared expert + routed experts + fold for the 64 rows."""
    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ep, ops

    K, W = args.steps if args.steps != 2000 else 40, max(min(args.warmup, 20), 3)
    B = args.batch if args.batch != 8 else C4_GLOBAL_BATCH
    if args.experts:
        assert args.experts % 32 == 0 and world == 1, "--experts: a multiple of 32, one GPU"
        cfg = dict(cfg, experts=args.experts, desc=cfg["desc"].replace("256 Q4_K experts", f"{args.experts} Q4_K experts (REDUCED layer for a profiler capture)"))
    assert B % world == 0 and cfg["experts"] % world == 0, "the global batch and the experts must split over the ranks"
    R = B // world
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    per = E // world
    model = C4Model(cfg)
    shape = ops.make_shape(H, I, E, TK, 12, 12)
    sh_shape = ops.make_shape(H, I, 1, 1, 8, 8)
    policy = ops.sigmoid_group_policy(E, TK, 8, 4)
    rw, bias = torch.from_numpy(model.rw).to(dev), torch.from_numpy(model.bias).to(dev)
    sg, su, sd = (torch.from_numpy(a).to(dev) for a in model.shared)
    n_slices = cfg["experts"] // model.per
    slices = range(n_slices) if world == 1 else range(rank * C4_PARTS // world, (rank + 1) * C4_PARTS // world)
    parts = [model.slice_device(r, dev) for r in slices]
    gate, up, down = (torch.cat([p[t] for p in parts]) for t in range(3))
    del parts
    NX = 4
    batches = model.batches(NX, B)
    xs_host = [torch.from_numpy(np.ascontiguousarray(x[rank * R:(rank + 1) * R])).pin_memory() for x in batches]
    xs = [x.to(dev) for x in xs_host]
    ys_host = torch.empty((R, H), dtype=torch.float32).pin_memory()
    ys = [torch.empty((R, H), dtype=torch.float32, device=dev) for _ in range(NX)]
    summary = torch.zeros(1, dtype=torch.int32, device=dev)
    if world > 1:
        layer = ep.PeerEpFfn(shape, policy, rw, gate, up, down, R, select_bias=bias, fold_parts=C4_PARTS)
        routed = lambda x, shared, y, ev=None: b200moe.check(b200moe.lib().b200moe_ep_ffn(layer.handle, C.byref(layer.view(x, y, shared, summary, ev)), b200moe.stream_ptr()))
    else:
        ffn = ops.MoeFfn(shape, policy, gate, up, down, rw, capacity=B, combine_form=b200moe.COMBINE_PARTS, parts=C4_PARTS, select_bias=bias)  # part_experts = E / 8
        routed = lambda x, shared, y, ev=None: b200moe.check(b200moe.lib().b200moe_ffn(C.byref(ffn._view(R, x, y, shared=shared, events=ev, summary=summary)), b200moe.stream_ptr()))

    def step(s, x=None, ev=None):
        x = xs[s % NX] if x is None else x
        shared = ops.enqueue_dense_ffn(sh_shape, sg, su, sd, ops.enqueue_quantize_a8(x))
        routed(x, shared, ys[s % NX], ev)
        return ys[s % NX]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for s in range(W):
        step(s)
    barrier()
    assert int(summary.item()) == 0, f"job summary {int(summary.item()):#x} after the warm-up"

    # ---- parity of one step against the CPU oracle, outside every timed region ------------------------------------
    parity = None
    y0 = step(0)                                              # every rank: the exchange needs all of them in every step
    barrier()
    if rank == 0 and not args.no_check:
        n = min(R, 8)
        y0 = y0.cpu().numpy()[:n]
        want, _ = c4_oracle_rows(model, batches[0][:n])
        err = float(np.max(np.abs(y0 - want).max(axis=-1) / np.maximum(np.abs(want).max(axis=-1), 1e-30)))
        parity = {"rows_checked": n, "bits_equal": bool(np.array_equal(y0.view(np.uint32), want.view(np.uint32))), "max_rel": err,
                  "against": "CPU oracle (oracle/), same seeded inputs, outside the timed regions"}
    barrier()

    # ---- distinct experts and entries per step on this rank: the algorithmic bytes of the routed GEMVs -----------
    gate_up_bytes, down_bytes = expert_bytes(cfg)
    uniq, entries = [], []
    for x in batches:
        _, _, ids, _ = ops.enqueue_router(policy, x=torch.from_numpy(x).to(dev), weight=rw, bias=bias)
        ids = ids.cpu().numpy()
        mine = ids[(ids >= rank * per) & (ids < (rank + 1) * per)]
        uniq.append(len(np.unique(mine)))
        entries.append(mine.size)
    uniq, entries = np.array(uniq, np.float64), np.array(entries, np.float64)

    # ---- timed region 1: the K-step block, replayed from a CUDA graph, repeated until the region is >= 0.25 s ------
    graph, mode, per_graph = None, "per-step launches", 0
    if not args.no_graph:
        try:
            cap = torch.cuda.Stream()
            cap.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            launches_before = b200moe.launch_count()
            with torch.cuda.graph(g, stream=cap):
                for s in range(NX):
                    step(s)
            per_graph = b200moe.launch_count() - launches_before
            graph, mode = g, f"CUDA graph replay of {NX} steps"
        except Exception as e:  # noqa: BLE001 - any capture problem: measure the eager path and say so
            graph, mode = None, f"per-step launches (graph capture failed: {type(e).__name__})"
    ok = torch.tensor([1 if graph is not None else 0], dtype=torch.int32, device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if not int(ok.item()):
        graph = None
        mode = mode if mode.startswith("per-step") else "per-step launches (a peer's capture failed)"

    def run_block(k):
        if graph is not None:
            for _ in range(k // NX):
                graph.replay()
            for s in range(k % NX):
                step(s)
        else:
            for s in range(k):
                step(s)

    run_block(K)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_block(K)
    e1.record()
    barrier()
    pilot = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(pilot, op=dist.ReduceOp.MAX)
    reps = max(1, int(math.ceil(250.0 / max(float(pilot.item()), 1e-3))))
    launches0 = b200moe.launch_count()
    sampler = ClockSampler(dev.index)
    sampler.start()
    barrier()
    e0.record()
    for _ in range(reps):
        run_block(K)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    eager = b200moe.launch_count() - launches0
    launches_per_step = (eager + (per_graph * (K // NX) * reps if graph is not None else 0)) / (K * reps)

    # ---- timed region 2: the same steps launched one by one, CUDA events around the routed gate/up kernel -----------
    evs = []
    for s in range(NX):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    taps = [ops.MoeFfn.stage_events([None, None, a.cuda_event, b.cuda_event, None, None, None, None]) for a, b in evs]
    kern_ms = []
    for _ in range(max(2, min(10, K // NX))):
        for s in range(NX):
            step(s, ev=taps[s])
        torch.cuda.synchronize()
        kern_ms += [evs[s][0].elapsed_time(evs[s][1]) for s in range(NX)]
    kern_ms = np.array(kern_ms).reshape(-1, NX)
    barrier()

    # ---- timed region 3: end to end, pinned host rows in, pinned host y out, every step ---------------------------
    def run_host(k):
        for s in range(k):
            ys_host.copy_(step(s, x=xs_host[s % NX].to(dev, non_blocking=True)), non_blocking=True)
        torch.cuda.synchronize()

    run_host(NX)
    barrier()
    t0 = time.perf_counter()
    run_host(K)
    barrier()
    host_ms = 1000.0 * (time.perf_counter() - t0)
    sampler.stop_flag = True
    sampler.join(timeout=2)
    assert int(summary.item()) == 0, f"job summary {int(summary.item()):#x}: a bounded wait ran out during the timed steps"

    algo = uniq * gate_up_bytes + entries * (H * 1.25)              # per batch: distinct local experts + the entries' A8 rows
    stats = torch.tensor([dev_ms, host_ms, float(kern_ms.mean()), float((algo / (kern_ms.mean(axis=0) * 1e-3)).mean() / 1e9), float(algo.mean()),
                          float(uniq.mean())], dtype=torch.float64, device=dev)
    if world > 1:
        allr = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(allr, stats)
        allr = torch.stack(allr).cpu().numpy()
    else:
        allr = stats.cpu().numpy()[None]
    dev_ms, host_ms = float(allr[:, 0].max()), float(allr[:, 1].max())
    slow = int(np.argmax(allr[:, 2]))                                # the rank whose gate/up launches take longest
    tokens = B * K * reps
    peak, peak_kind = peaks()
    achieved = float(allr[slow, 3])
    line = {
        "metric": METRIC.replace("decode", c4_phase(B)), "value": tokens / (dev_ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / (K * reps), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8xint4->int32, fp32 chains", "data": "synthetic", "config": c4_config(cfg, B, world),
        "clocks": sampler.summary(),
        "e2e": {"value": B * K / (host_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "ms_per_step": host_ms / K},
        "gpu_launches": int(round(launches_per_step * K)),
        "roofline": {"kernel": "q4k_wide_kernel<gate/up> (routed experts, segment-streaming GEMV)" if B < 128 else
                               "grouped_q4k_kernel<gate/up> (routed experts over a token block, tcgen05; quoted against HBM on its distinct-expert bytes)",
                     "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"{peak_kind} HBM copy", "frac_of_nominal_8tbs": achieved / 8000.0,
                     "traffic": float(allr[slow, 4]) * C4_TRAFFIC_RATIO,
                     "traffic_note": "scaled by distinct experts from the ncu capture of a reduced layer (x 1.03 algorithmic): profiles/wide_kernels_c4_decode.md",
                     "algorithmic_bytes_per_launch": float(allr[slow, 4]), "avg_launch_us": float(allr[slow, 2]) * 1000.0,
                     "distinct_experts_per_step_on_that_rank": float(allr[slow, 5]), "rank": slow},
        "extra": {"timed_steps": K * reps, "timed_region_s": dev_ms / 1000.0, "launch": mode + (
                      "; dispatch and return by the library's peer-store kernels with bounded flag waits (CUDA IPC windows, no collective)" if world > 1 else ""),
                  "launches_per_step": launches_per_step, "rows_per_rank": R,
                  "step_hbm_gbs_per_rank": float(np.mean(uniq) * (gate_up_bytes + down_bytes) / (dev_ms / (K * reps) * 1e-3) / 1e9)},
    }
    if parity is not None:
        line["parity"] = parity
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            _, base = c4_cpu_arm(model, batches[0][:8], target_s=10.0)
            line["cpu_baseline"] = base
        if world == 1 and not args.no_extra:
            line["extra"]["c2_b8"] = c2_summary(args, dev)
        print(json.dumps(line), flush=True)
    if world > 1:
        layer.close()
        dist.destroy_process_group()


def ep_arm(args, cfg, rank, world, dev):
    """Expert parallelism: every rank holds experts / world experts of each layer and `batch` local token rows; a step is
    one EpMoeFfn call (route, all-gather, local experts over the global window, all-to-all, combine). Timed on the device,
    max over ranks; e2e adds the pinned-host copies of x and y every step."""
    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ep, ops, synth

    K, W, B, L = args.steps, max(args.warmup, 3), args.batch, args.layers
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    per = E // world
    shape = ops.make_shape(H, I, E, TK, cfg["gate_type"], cfg["down_type"])
    policy = ops.softmax_policy(E, TK)
    gate_up_bytes, down_bytes = expert_bytes(cfg)
    layers = []
    for li in range(L):
        g, u, d, rw = make_layer(cfg, 1000 + li)          # same seed on every rank: one model, sliced by expert range
        gb, db = g.size // E, d.size // E
        sl = lambda t, b: torch.from_numpy(np.ascontiguousarray(t.reshape(-1)[rank * per * b:(rank + 1) * per * b])).to(dev)
        k = ep.DeviceKernels(shape, policy, torch.from_numpy(rw).to(dev), sl(g, gb), sl(u, gb), sl(d, db), world * B,
                             b200moe.COMBINE_FMA_SLOTS, world, rank)
        layers.append(ep.EpMoeFfn(k, B, TK, H, b200moe.COMBINE_FMA_SLOTS))
    rng = np.random.default_rng(7 + rank)
    NX = 16
    xs_host = [torch.from_numpy(synth.activations(rng, B, H)).pin_memory() for _ in range(NX)]
    xs = [x.to(dev) for x in xs_host]
    ys_host = torch.empty((B, H), dtype=torch.float32).pin_memory()

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def run(n):
        for s in range(n):
            layers[s % L](xs[s % NX])

    def run_host(n):
        for s in range(n):
            ys_host.copy_(layers[s % L](xs_host[s % NX].to(dev, non_blocking=True)), non_blocking=True)
        torch.cuda.synchronize()

    run(W)
    barrier()
    launches0 = b200moe.launch_count()
    sampler = ClockSampler(dev.index)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    run(K)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = b200moe.launch_count() - launches0
    run_host(min(W, 50))
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    h0.record()
    run_host(K)
    h1.record()
    barrier()
    host_ms = max(h0.elapsed_time(h1), 1000.0 * (time.perf_counter() - t0))
    sampler.stop_flag = True
    sampler.join(timeout=2)
    t = torch.tensor([dev_ms, host_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, host_ms = (float(v) for v in t.cpu())
    tokens = B * K * world
    peak, peak_kind = peaks()
    rank_bytes = per * (gate_up_bytes + down_bytes)       # at most: every local expert hit once per step
    achieved = rank_bytes / (dev_ms / K * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": tokens / (dev_ms / 1000.0), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8xint4->int32, fp32 chains", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}, batch {B} per rank", "parallelism": f"ep x{world} ({per} experts per rank)",
                   "l2": f"rotating {L} layers of distinct expert weights", "launch": "per-step launches + NCCL (no graph)"},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens / (host_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "ms_per_step": host_ms / K},
        "gpu_launches": int(launches),
        "roofline": {"kernel": "whole EP step (local expert weights / step time)", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"{peak_kind} HBM copy", "traffic": None},
    }
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


def decode_arm(args, cfg, rank, world, dev):
    """Configs 1 and 2: one MoE decode layer on every GPU (replicas at N > 1), rotating over several layers of distinct
    weights. Returns the JSON line as a dict."""
    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ops, synth

    local = dev.index
    K, W, L = args.steps, max(args.warmup, 3), args.layers
    B = cfg.get("batch", args.batch) if args.batch == 8 else args.batch
    H, E, TK, I = cfg["hidden"], cfg["experts"], cfg["top_k"], cfg["inter"]
    shape = ops.make_shape(H, I, E, TK, cfg["gate_type"], cfg["down_type"])
    policy = ops.softmax_policy(E, TK)
    form = b200moe.COMBINE_PARTS if cfg.get("parts_form") else b200moe.COMBINE_FMA_SLOTS
    layers = []
    for li in range(L):
        g, u, d, rw = make_layer(cfg, 1000 + li + 100 * rank)
        layers.append(ops.MoeFfn(shape, policy, *(torch.from_numpy(a).to(dev) for a in (g, u, d, rw)), capacity=B, combine_form=form))
    rng = np.random.default_rng(7 + rank)
    NX = 16
    xs_host = [torch.from_numpy(synth.activations(rng, B, H)).pin_memory() for _ in range(NX)]
    xs = [x.to(dev) for x in xs_host]
    y = torch.empty((B, H), dtype=torch.float32, device=dev)
    ys_host = torch.empty((B, H), dtype=torch.float32).pin_memory()
    ids = torch.empty((B, TK), dtype=torch.int32, device=dev)
    wts = torch.empty((B, TK), dtype=torch.float32, device=dev)
    lib = b200moe.lib()

    def views(events=None):
        return [layers[s % L]._view(B, xs[s % NX], y, ids, wts, events=events[s] if events else None) for s in range(L * NX)]

    plain = views()
    stream = torch.cuda.current_stream()

    def run_plain(n, vs, first=0):
        sp = stream.cuda_stream
        for s in range(n):
            rc = lib.b200moe_ffn(C.byref(vs[(first + s) % len(vs)]), sp)
            if rc:
                b200moe.check(rc)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    run_plain(W, plain)
    torch.cuda.synchronize()
    # distinct experts per step (realised routing) -> algorithmic bytes of the gate/up kernel
    gate_up_bytes, down_bytes = expert_bytes(cfg)
    uniq = []
    for s in range(L * NX):
        run_plain(1, plain, s)
        torch.cuda.synchronize()
        uniq.append(len(np.unique(ids.cpu().numpy())))
    uniq = np.array(uniq, dtype=np.float64)

    # ---- timed region 1: K steps replayed from CUDA graphs (value) ---------------------------------------------
    G = min(K, L * NX)
    cap_stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    launches0 = b200moe.launch_count()
    with torch.cuda.graph(graph, stream=cap_stream):
        sp = torch.cuda.current_stream().cuda_stream
        for s in range(G):
            rc = lib.b200moe_ffn(C.byref(plain[s]), sp)
            if rc:
                b200moe.check(rc)
    launches_per_step = (b200moe.launch_count() - launches0) / G
    replays, rest = divmod(K, G)
    for _ in range(3):
        graph.replay()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(replays):
        graph.replay()
    run_plain(rest, plain)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)

    # ---- timed region 2: the same K steps launched one by one, CUDA events around the gate/up kernel -------------
    evs = []
    for s in range(L * NX):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    taps = [ops.MoeFfn.stage_events([None, None, a.cuda_event, b.cuda_event, None, None, None, None]) for a, b in evs]
    tapped = views(taps)
    kern_ms, plain_ms_total, done = [], 0.0, 0
    while done < K:
        n = min(K - done, L * NX)
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        run_plain(n, tapped)
        p1.record()
        torch.cuda.synchronize()
        plain_ms_total += p0.elapsed_time(p1)
        kern_ms += [evs[s][0].elapsed_time(evs[s][1]) for s in range(n)]
        done += n
    kern_ms = np.array(kern_ms)
    steps_uniq = np.array([uniq[s % (L * NX)] for s in range(K)])

    # ---- timed region 3: end to end through the host-buffer call -------------------------------------------------
    host_views = [layers[s % L]._view(B, None, None) for s in range(L * NX)]

    def run_host(n):
        sp = stream.cuda_stream
        for s in range(n):
            rc = lib.b200moe_ffn_host(C.byref(host_views[s % len(host_views)]), xs_host[s % NX].data_ptr(), ys_host.data_ptr(), sp)
            if rc:
                b200moe.check(rc)

    run_host(min(W, 50))
    barrier()
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    h0.record()
    run_host(K)
    h1.record()
    barrier()
    host_ms = max(h0.elapsed_time(h1), 1000.0 * (time.perf_counter() - t0))
    sampler.stop_flag = True
    sampler.join(timeout=2)

    t = torch.tensor([dev_ms, host_ms, plain_ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, host_ms, plain_ms_total = (float(v) for v in t.cpu())
    tokens = B * K * world
    value = tokens / (dev_ms / 1000.0)
    peak, peak_kind = peaks()
    algo_bytes = float(np.mean(steps_uniq)) * gate_up_bytes + B * H * 1.25  # weights of the distinct experts + the A8 rows
    achieved = algo_bytes / (float(np.mean(kern_ms)) * 1e-3) / 1e9
    step_bytes = float(np.mean(steps_uniq)) * (gate_up_bytes + down_bytes) + E * H * 4
    line = {
        "metric": METRIC if cfg["gate_type"] == 12 else "MoE-layer tokens/s (Q8_0 decode)", "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8xint4->int32, fp32 chains" if cfg["gate_type"] == 12 else "int8xint8->int32, fp32 lane classes", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {cfg['desc']}, batch {B}", "parallelism": f"replicas x{world}" if world > 1 else "1 gpu",
                   "l2": f"rotating {L} layers of distinct expert weights ({L * E * (gate_up_bytes + down_bytes) / 2**20:.0f} MiB) > 2 x {L2_BYTES // 2**20} MiB L2",
                   "launch": "CUDA graph replay of the per-step kernel sequence"},
        "clocks": sampler.summary(),
        "e2e": {"value": tokens / (host_ms / 1000.0), "unit": UNIT, "h2d_bytes_per_step": B * H * 4, "d2h_bytes_per_step": B * H * 4,
                "ms_per_step": host_ms / K},
        "gpu_launches": int(round(launches_per_step * K)),
        "roofline": {"kernel": gate_up_kernel_name(cfg, B, args.form), "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": f"{peak_kind} HBM copy",
                     # dram read + write per launch from an ncu capture of this kernel on this workload: 1.00 of the algorithmic bytes
                     "traffic": algo_bytes * NCU_TRAFFIC_RATIO if cfg["gate_type"] == 12 else None,
                     "traffic_source": "profiles/stream_kernels_c2_decode_b8_dram.md" if cfg["gate_type"] == 12 else None,
                     "algorithmic_bytes_per_launch": algo_bytes, "avg_launch_us": float(np.mean(kern_ms)) * 1000.0,
                     "distinct_experts_per_step": float(np.mean(steps_uniq))},
        "extra": {"step_hbm_gbs_graph": step_bytes / (dev_ms / K * 1e-3) / 1e9, "ms_per_step_no_graph": plain_ms_total / K,
                  "tokens_per_s_no_graph": tokens / (plain_ms_total / 1000.0), "launches_per_step": launches_per_step},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        _, base = cpu_arm(cfg, B, target_s=12.0)
        line["cpu_baseline"] = base
    return line




def c2_summary(args, dev):
    """Config 2 at batch 8 measured in the same run (the headline of earlier reports): value and the gate/up roofline."""
    import copy
    a = copy.copy(args)
    a.steps, a.warmup, a.batch, a.layers, a.no_cpu_baseline, a.workload = 400, 50, 8, 4, True, "c2"
    line = decode_arm(a, CONFIGS["c2"], 0, 1, dev)
    return {"workload": line["config"]["workload"], "value": line["value"], "ms_per_step": line["ms_per_step"], "e2e": line["e2e"]["value"],
            "gate_up_kernel": line["roofline"]["kernel"], "gate_up_frac": line["roofline"]["frac"], "gate_up_us": line["roofline"]["avg_launch_us"]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c4", choices=sorted(CONFIGS))
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=4, help="distinct layers of weights rotated between steps")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--experts", type=int, default=0,
                    help="config 4: a reduced layer of this many routed experts (a multiple of 32; 0 = the config's 256) for profiler captures, "
                         "which must hold only a few GB on the device; the line then says so in config.workload")
    ap.add_argument("--no-check", action="store_true", help="skip the comparison of one step with the CPU oracle (the `parity` key)")
    ap.add_argument("--no-extra", action="store_true", help="config 4 on one GPU: skip the config 2 batch 8 figures under extra.c2_b8")
    ap.add_argument("--no-graph", action="store_true", help="config 4 arm: launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-peer-return", action="store_true",
                    help="expert parallelism, PARTS form: return the partial sums with an NCCL all-to-all instead of the combine kernel's peer stores")
    ap.add_argument("--tp-payload", default="bf16", choices=["bf16", "fp32"], help="config 5, N > 1: what the partial sums cross NVLink as")
    ap.add_argument("--form", type=int, default=0, choices=[0, 1, 2, 3],
                    help="Q4_K decode GEMV form: 0 = by plan, 1 = row streaming, 2 = segment streaming, 3 = per block (measurement hook)")
    ap.add_argument("--parallelism", default="replicas", choices=["replicas", "ep"],
                    help="N > 1: independent replicas (rows sharded, weights replicated, no collective) or expert parallelism "
                         "(experts / N per rank, all-gather dispatch + all-to-all return over NCCL)")
    args = ap.parse_args()
    cfg = CONFIGS[args.workload]
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        return c4_reference_arm(args, cfg, rank, world) if cfg.get("large") else reference_arm(args, cfg, rank, world)

    import torch
    import torch.distributed as dist
    import b200moe
    from b200moe import ops, synth

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU path)"
    if args.form:
        b200moe.debug_set(b200moe.DEBUG_DECODE_FORM, args.form)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if cfg.get("prefill"):
        return prefill_arm(args, cfg, rank, world, dev)
    if cfg.get("dense"):
        return dense_arm(args, cfg, rank, world, dev)
    if cfg.get("large"):
        return large_arm(args, cfg, rank, world, dev)
    if world > 1 and args.parallelism == "ep":
        return ep_arm(args, cfg, rank, world, dev)
    line = decode_arm(args, cfg, rank, world, dev)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
