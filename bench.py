"""Benchmark of the B200 fused-MoE hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1: the INT4 decode configuration (M=64, K=7168, N=4096, E=48, top_k=8, group 32) — a
"step" is one ``fused_moe_int4_w4a16`` call (align + grouped GEMM + top-k combine).
N > 1 (under torchrun): the expert-parallel configuration (E=256 sharded evenly, K=7168,
N=2048, top_k=8, 4096 tokens per GPU) with NCCL all-to-all dispatch and combine.

One JSON line is printed by rank 0.  ``value`` is tokens/s over all ranks with inputs
resident in HBM; ``e2e`` is the same through the public Python API with pinned-host
activations/routing copied in and the result copied out inside the timed region (the expert
weights are model state and stay resident); ``roofline`` is the grouped-GEMM kernel's
algorithmic bytes (or flops) per launch over its CUDA-event duration, against the measured
peak in MEASURED_PEAKS.json; ``cpu_baseline`` is the CPU oracle port timed on the host cores.
``--impl reference`` times that CPU port alone on the same configuration.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi sampled every 100 ms while the timed region runs (read-only query)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# --------------------------------------------------------------------------------------
# CPU baseline (oracle port) — also the --impl reference arm
# --------------------------------------------------------------------------------------
def cpu_int4_sample(cfg, seed: int, n_rows: int, repeats: int = 1):
    """Time the CPU port of the reference algorithm (oracle/moe_oracle.py:moe_w4a16, the grouped
    restatement of ops/moe/reference.py) on an N-slice of the configuration: all M tokens, all E
    experts, ``n_rows`` of the N weight rows.  Work is linear in N, so the time scales by N/n_rows."""
    from oracle import moe_oracle as oracle
    from xkernels_b200 import synth

    A = synth.activations(cfg.M, cfg.K, seed=seed)
    packed, scale = synth.int4_weights(cfg.E, n_rows, cfg.K, cfg.group_size, seed=seed + 1)
    ids, w = synth.routing(cfg.M, cfg.E, cfg.top_k, seed=seed + 3, expert_bias_std=cfg.expert_bias_std,
                           zipf_scale=cfg.zipf_scale)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        oracle.moe_w4a16(A, packed, scale, ids, w, cfg.group_size)
        times.append(time.perf_counter() - t0)
    return min(times) * (cfg.N / n_rows), times


def cpu_baseline_block(cfg, n_rows: int):
    t_full, _ = cpu_int4_sample(cfg, 1729, n_rows)
    return {
        "value": cfg.M / t_full, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
        "sample": f"oracle.moe_w4a16 (CPU torch, fp32) on all {cfg.M} tokens x {cfg.E} experts x "
                  f"{n_rows}/{cfg.N} weight rows, time scaled by {cfg.N // n_rows}",
        "seconds_per_call_scaled": t_full,
    }


def run_reference_arm(args, world: int, rank: int):
    """--impl reference: the CPU port with all host threads; rank 0 only."""
    if rank != 0:
        return
    from xkernels_b200 import synth

    cfg = synth.CONFIGS["int4_decode" if world == 1 else "int4_ep"]
    M_total = cfg.M * world
    if world > 1:
        cfg = synth.Int4Config(cfg.name, M=M_total, K=cfg.K, N=cfg.N, E=cfg.E, top_k=cfg.top_k,
                               zipf_scale=cfg.zipf_scale)
    # size the per-step sample so that the whole run stays within about two minutes
    t_probe, _ = cpu_int4_sample(cfg, 1, 8)           # seconds for the FULL N, scaled from 8 rows
    budget = 120.0 / max(args.steps + min(args.warmup, 1), 1)
    n_rows = 8
    while n_rows * 2 <= min(512, cfg.N) and t_probe * (n_rows * 2 / cfg.N) <= budget:
        n_rows *= 2
    for _ in range(min(args.warmup, 1)):
        cpu_int4_sample(cfg, 1, n_rows)
    per_step = []
    for s in range(args.steps):
        t, _ = cpu_int4_sample(cfg, 1729 + s, n_rows)
        per_step.append(t)
    t_mean = sum(per_step) / len(per_step)
    value = cfg.M / t_mean
    sample = (f"each step: oracle.moe_w4a16 on all {cfg.M} tokens x {cfg.E} experts x {n_rows}/{cfg.N} "
              f"weight rows, time scaled by {cfg.N // n_rows}")
    line = {
        "impl": "reference", "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg, world),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg, world: int):
    if world == 1:
        name = (f"int4_w4a16 decode: M={cfg.M} K={cfg.K} N={cfg.N} E={cfg.E} top_k={cfg.top_k} "
                f"group={cfg.group_size}")
        return {"workload": name, "l2": "weights (794 MB) exceed the 126 MB L2, no flush needed",
                "parallelism": "single GPU"}
    return {"workload": (f"int4_w4a16 expert-parallel: E={cfg.E} over {world} GPUs, K={cfg.K} N={cfg.N} "
                         f"top_k={cfg.top_k}, {cfg.M // world} tokens per GPU, zipf(1.1)*2.0 expert bias"),
            "expert_placement": "see the ep key",
            "l2": "per-rank weights exceed the 126 MB L2, no flush needed",
            "parallelism": f"ep{world} (E/W experts per rank, NCCL all-to-all dispatch/combine)"}


# --------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------
def timed_loop(fn, steps: int, sync, barrier):
    """barrier + synchronize, K steps between two CUDA events on the current stream, barrier +
    synchronize.  Returns milliseconds for all K steps."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sync()
    start.record()
    for i in range(steps):
        fn(i)
    stop.record()
    sync()
    barrier()
    return start.elapsed_time(stop)


def run_single_gpu(args):
    import xkernels_b200 as xkb
    from xkernels_b200 import _lib, ops, synth

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peaks = load_peaks()
    cfg = synth.CONFIGS["int4_decode"]
    d = synth.make_int4(cfg, seed=1729, device=dev)
    n_active = int(torch.unique(d["topk_ids"]).numel())
    alg_bytes = synth.int4_algorithmic_bytes(cfg, n_active)

    def step(_i):
        return xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"],
                                        group_size=cfg.group_size)

    sync = torch.cuda.synchronize
    for i in range(max(args.warmup, 3)):
        step(i)
    ops.check_status(dev)

    # ---- device-resident throughput + live GEMM-kernel timing ---------------------------
    _lib.gemm_timer_enable(args.steps)
    launches0 = _lib.launch_count()
    with ClockSampler(0) as clocks:
        ms = timed_loop(step, args.steps, sync, lambda: None)
    launches = _lib.launch_count() - launches0
    gemm_ms = _lib.gemm_timer_read()
    _lib.gemm_timer_enable(0)
    ops.check_status(dev)
    ms_per_step = ms / args.steps
    value = cfg.M / (ms_per_step * 1e-3)
    gemm_avg_ms = sum(gemm_ms) / max(len(gemm_ms), 1)
    achieved = alg_bytes / (gemm_avg_ms * 1e-3) / 1e9
    # DRAM traffic per launch from the ncu capture of the 16-expert relative of this workload
    # (profiles/moe_tc_kernel_int4_decode_small.md: 273.9 MB read+write for 264.2 MB of weights and
    # scales); traffic grows with the experts touched, so it is scaled by n_active / 16.
    traffic = 273.9e6 * n_active / 16.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                "kernel": "moe_tc_kernel<16, int4>", "kernel_us": gemm_avg_ms * 1e3,
                "algorithmic_bytes": alg_bytes, "peak_source": peaks["source"],
                "whole_call_frac": (alg_bytes / (ms_per_step * 1e-3) / 1e9) / peaks["hbm_gbs"]}

    # ---- end to end: pinned host inputs in, result out, through the public API -----------
    hA = d["A"].cpu().pin_memory()
    hI = d["topk_ids"].cpu().pin_memory()
    hW = d["topk_w"].cpu().pin_memory()
    hO = torch.empty((cfg.M, cfg.N), dtype=torch.bfloat16).pin_memory()
    dA, dI, dW = torch.empty_like(d["A"]), torch.empty_like(d["topk_ids"]), torch.empty_like(d["topk_w"])

    def e2e_step(_i):
        dA.copy_(hA, non_blocking=True)
        dI.copy_(hI, non_blocking=True)
        dW.copy_(hW, non_blocking=True)
        out = xkb.fused_moe_int4_w4a16(dA, d["packed"], d["scale"], dI, dW, group_size=cfg.group_size)
        hO.copy_(out, non_blocking=True)

    for i in range(3):
        e2e_step(i)
    sync()
    t0 = time.perf_counter()
    e2e_ms_events = timed_loop(e2e_step, args.steps, sync, lambda: None)
    e2e_wall = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(e2e_ms_events, 0.0)
    e2e = {"value": cfg.M / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
           "h2d_bytes_per_step": hA.numel() * 2 + hI.numel() * 4 + hW.numel() * 4,
           "d2h_bytes_per_step": hO.numel() * 2, "us_per_call": e2e_ms / args.steps * 1e3,
           "wall_us_per_call": e2e_wall / args.steps * 1e3,
           "note": "expert weights stay resident in HBM (model state); per-step inputs A/topk_ids/topk_w "
                   "come from pinned host memory, the bf16 result goes back to pinned host memory"}

    line = {
        "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "us_per_call": ms_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(cfg, 1), "clocks": clocks.summary(), "e2e": e2e,
        "gpu_launches": int(launches), "roofline": roofline,
    }
    if not args.no_extras:
        line["other_configs"] = extras(dev, peaks)
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_block(cfg, 256)
    print(json.dumps(line), flush=True)


def time_call(fn, warmup: int, steps: int):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def extras(dev, peaks):
    """The other single-GPU configurations, timed briefly (whole call and GEMM kernel)."""
    import xkernels_b200 as xkb
    from xkernels_b200 import _lib, ops, synth

    out = {}
    try:
        cfg = synth.CONFIGS["int4_prefill"]
        d = synth.make_int4(cfg, seed=1729, device=dev)
        fn = lambda: xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])  # noqa: E731
        _lib.gemm_timer_enable(5)
        ms = time_call(fn, 2, 5)
        g = _lib.gemm_timer_read()[-5:]
        _lib.gemm_timer_enable(0)
        ops.check_status(dev)
        gm = sum(g) / len(g)
        tf = synth.int4_flops(cfg) / (gm * 1e-3) / 1e12
        al = time_call(lambda: xkb.moe_align_block_size(d["topk_ids"], 16, cfg.E, truncate=False), 3, 20)
        out["int4_prefill"] = {"ms_per_call": ms, "tokens_per_s": cfg.M / (ms * 1e-3), "gemm_kernel_ms": gm,
                               "gemm_tflops": tf, "frac_of_bf16_peak": tf / peaks["bf16_tflops"],
                               "align_block16_us": al * 1e3}
        del d
    except Exception as exc:  # noqa: BLE001
        out["int4_prefill"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    try:
        cfg = synth.CONFIGS["mxfp4_decode"]
        d = synth.make_mxfp4(cfg, seed=1729, device=dev)
        n_active = int(torch.unique(d["topk_ids"]).numel())
        fn = lambda: xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"],  # noqa: E731
                                         d["topk_ids"], d["topk_w"])
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        _lib.gemm_timer_enable(64)          # two GEMM kernels (gate_up, down) per call
        ms = time_call(fn, 0, 20)
        g = _lib.gemm_timer_read()
        _lib.gemm_timer_enable(0)
        ops.check_status(dev)
        gm = sum(g) / 20
        b = synth.mxfp4_algorithmic_bytes(cfg, n_active)
        out["mxfp4_decode"] = {"us_per_call": ms * 1e3, "gemm_kernels_us": gm * 1e3, "active_experts": n_active,
                               "algorithmic_bytes": b, "gemm_gbs": b / (gm * 1e-3) / 1e9,
                               "frac_of_hbm_peak": b / (gm * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        del d
    except Exception as exc:  # noqa: BLE001
        out["mxfp4_decode"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    try:
        # the decode call captured in a CUDA graph (the call is stream-ordered end to end): launch
        # overhead of its four kernels collapses into one graph launch
        cfg = synth.CONFIGS["int4_decode"]
        d = synth.make_int4(cfg, seed=1729, device=dev)
        fn = lambda: xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"],  # noqa: E731
                                              group_size=cfg.group_size)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        ms = time_call(graph.replay, 3, 50)
        out["int4_decode_cuda_graph"] = {"us_per_call": ms * 1e3, "tokens_per_s": cfg.M / (ms * 1e-3)}
        del d, graph
    except Exception as exc:  # noqa: BLE001
        out["int4_decode_cuda_graph"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    try:
        M, E, top_k = 16384, 256, 8          # the router in front of the prefill configuration
        logits = torch.randn(M, E, device=dev).to(torch.bfloat16)
        ms = time_call(lambda: xkb.topk_softmax(logits, top_k, True), 3, 20)
        b = M * E * 2 + M * top_k * 8
        out["topk_softmax_16384x256_top8_bf16"] = {"us_per_call": ms * 1e3, "gbs": b / (ms * 1e-3) / 1e9,
                                                   "frac_of_hbm_peak": b / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                                   "note": "8.9 MB per call: fits in L2, launch-latency sized"}
    except Exception as exc:  # noqa: BLE001
        out["topk_softmax_16384x256_top8_bf16"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    try:
        M, top_k, H = 8192, 8, 7168
        y = torch.randn(M, top_k, H, device=dev, dtype=torch.bfloat16)
        w = torch.rand(M, top_k, device=dev)
        ms = time_call(lambda: xkb.moe_sum_reduce(y, w), 3, 20)
        b = M * top_k * H * 2 + M * top_k * 4 + M * H * 2
        out["moe_sum_reduce_8192x8x7168_bf16"] = {"us_per_call": ms * 1e3, "gbs": b / (ms * 1e-3) / 1e9,
                                                  "frac_of_hbm_peak": b / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    except Exception as exc:  # noqa: BLE001
        out["moe_sum_reduce_8192x8x7168_bf16"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    return out


def run_multi_gpu(args, world: int, rank: int, local_rank: int):
    import torch.distributed as dist

    from xkernels_b200 import _lib, ep, ops, synth

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    cfg = synth.CONFIGS["int4_ep"]
    e_local = cfg.E // world
    # every rank: its own tokens/routing (seeded by rank) and its experts.  Weights are synthetic, so
    # each rank simply draws E/W experts; which GLOBAL ids they stand for is fixed by the placement.
    A = synth.activations(cfg.M, cfg.K, seed=1729 + 100 * rank, device=dev)
    ids, w = synth.routing(cfg.M, cfg.E, cfg.top_k, seed=1732 + 100 * rank, device=dev, zipf_scale=cfg.zipf_scale)
    packed, scale = synth.int4_weights(e_local, cfg.N, cfg.K, cfg.group_size, seed=1730 + 7 * rank, device=dev)
    layer = ep.ExpertParallelInt4(packed, scale, num_global_experts=cfg.E, group=dist.group.WORLD,
                                  group_size=cfg.group_size, placement=args.ep_placement, chunks=args.ep_chunks,
                                  sm_margin=args.ep_sm_margin)

    # reference point for scaling: the SAME configuration on one GPU (all 256 experts local, 4096
    # tokens, no exchange), timed on rank 0 before the group run
    single = None
    if rank == 0:
        import xkernels_b200 as xkb
        pk1, sc1 = synth.int4_weights(cfg.E, cfg.N, cfg.K, cfg.group_size, seed=99, device=dev)
        t1 = time_call(lambda: xkb.fused_moe_int4_w4a16(A, pk1, sc1, ids, w, group_size=cfg.group_size), 3, 10)
        single = {"tokens_per_s": cfg.M / (t1 * 1e-3), "ms_per_step": t1}
        del pk1, sc1
        torch.cuda.empty_cache()
    dist.barrier()

    def step(_i):
        return layer(A, ids, w)

    def sync():
        torch.cuda.synchronize(dev)

    for i in range(max(args.warmup, 3)):
        step(i)
    ops.check_status(dev)
    _lib.gemm_timer_enable(args.steps)
    launches0 = _lib.launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.__enter__()
    ms = timed_loop(step, args.steps, sync, dist.barrier)
    if sampler:
        sampler.__exit__()
    launches = _lib.launch_count() - launches0
    gemm_ms = _lib.gemm_timer_read()
    _lib.gemm_timer_enable(0)
    t = torch.tensor([ms, sum(gemm_ms) / max(len(gemm_ms), 1), float(layer.count_recv_slots()),
                      float(layer.last_recv_rows)], device=dev, dtype=torch.float64)
    gathered = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    ms_max = max(float(g[0]) for g in gathered)
    gemm_max = max(float(g[1]) for g in gathered)
    slots = [int(g[2]) for g in gathered]
    rows_in = [int(g[3]) for g in gathered]

    # end to end: pinned host activations/routing in, result out
    hA, hI, hW = A.cpu().pin_memory(), ids.cpu().pin_memory(), w.cpu().pin_memory()
    hO = torch.empty((cfg.M, cfg.N), dtype=torch.bfloat16).pin_memory()
    dA, dI, dW = torch.empty_like(A), torch.empty_like(ids), torch.empty_like(w)

    def e2e_step(_i):
        dA.copy_(hA, non_blocking=True)
        dI.copy_(hI, non_blocking=True)
        dW.copy_(hW, non_blocking=True)
        hO.copy_(layer(dA, dI, dW), non_blocking=True)

    for i in range(2):
        e2e_step(i)
    e2e_ms = timed_loop(e2e_step, args.steps, sync, dist.barrier)
    te = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
    dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_ms = float(te[0])

    if rank == 0:
        ms_per_step = ms_max / args.steps
        tokens = cfg.M * world
        max_slots = max(slots)
        flops = 2.0 * max_slots * cfg.N * cfg.K  # the busiest rank bounds the step
        tf = flops / (gemm_max * 1e-3) / 1e12
        line = {
            "metric": "fused_moe_tokens_per_s", "value": tokens / (ms_per_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(synth.Int4Config(cfg.name, M=tokens, K=cfg.K, N=cfg.N, E=cfg.E,
                                                       top_k=cfg.top_k), world),
            "clocks": sampler.summary() if sampler else None,
            "e2e": {"value": tokens / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": world * (hA.numel() * 2 + hI.numel() * 4 + hW.numel() * 4),
                    "d2h_bytes_per_step": world * hO.numel() * 2},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops_sustained"], "traffic": None,
                         "kernel": "moe_tc_kernel (busiest rank)", "kernel_ms": gemm_max,
                         "peak_source": peaks["source"] + " (sustained)"},
            "slots_received_per_rank": slots,
            "rows_received_per_rank": rows_in,   # one activation row per (token, rank) pair crosses the wire
            "ep": {"placement": args.ep_placement, "chunks": args.ep_chunks, "sm_margin": args.ep_sm_margin,
                   "same_config_on_one_gpu": single},
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


PROFILE_CASES = {
    # small relatives of the benchmark configurations (weights still exceed the 126 MB L2) for
    # ncu captures: few launches, a few hundred MB on the device
    "int4_decode_small": ("int4", dict(M=22, K=7168, N=4096, E=16, top_k=8)),
    "int4_prefill_small": ("int4", dict(M=2048, K=7168, N=4096, E=16, top_k=8, expert_bias_std=0.5)),
    "mxfp4_decode_small": ("mxfp4", dict(M=12, hidden=4096, ispp=512, E=64, top_k=6)),
}


def run_profile_case(args):
    """One small case, a handful of calls, no extras: the command ncu wraps."""
    import xkernels_b200 as xkb
    from xkernels_b200 import ops, synth

    dev = torch.device("cuda", 0)
    kind, kw = PROFILE_CASES[args.case]
    if kind == "int4":
        cfg = synth.Int4Config(args.case, **kw)
        d = synth.make_int4(cfg, seed=1729, device=dev)
        fn = lambda: xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])  # noqa: E731
    else:
        cfg = synth.Mxfp4Config(args.case, **kw)
        d = synth.make_mxfp4(cfg, seed=1729, device=dev)
        fn = lambda: xkb.fused_moe_mxfp4(d["A"], d["w13"], d["w13_scale"], d["w2"], d["w2_scale"],  # noqa: E731
                                         d["topk_ids"], d["topk_w"])
    ms = time_call(fn, args.warmup, args.steps)
    ops.check_status(dev)
    print(json.dumps({"case": args.case, "config": kw, "us_per_call": ms * 1e3, "steps": args.steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the other single-GPU configurations")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--ep-placement", default="round_robin", choices=["contiguous", "round_robin", "snake"],
                    help="expert -> rank assignment of the expert-parallel run")
    ap.add_argument("--ep-chunks", type=int, default=1, help="token chunks pipelined through the exchanges")
    ap.add_argument("--ep-sm-margin", type=int, default=16,
                    help="SMs the GEMM kernels leave to the exchange kernels when chunks > 1")
    ap.add_argument("--case", default=None, choices=sorted(PROFILE_CASES),
                    help="run one small profiling case instead of the benchmark")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.case is not None:
        if args.steps == 200:
            args.steps = 3
        run_profile_case(args)
        return
    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 3
        run_reference_arm(args, max(world, args.gpus), rank)
        return
    if world == 1 and args.gpus == 1:
        run_single_gpu(args)
    else:
        if args.steps == 200:
            args.steps = 20
        run_multi_gpu(args, world, rank, local_rank)


if __name__ == "__main__":
    main()
