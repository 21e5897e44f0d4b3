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
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0,
               "window": "the timed steps plus an untimed continuation of the same loop (about 0.45 s; "
                         "the timed steps alone are shorter than one sampling period)"}
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
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm),
                       sm_mhz_first_sample=sm[0])
        return out


# --------------------------------------------------------------------------------------
# CPU baseline and the --impl reference arm
# --------------------------------------------------------------------------------------
def host_threads() -> int:
    """Use every host core, also under torchrun (which exports OMP_NUM_THREADS=1)."""
    n = os.cpu_count() or 1
    if torch.get_num_threads() != n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def reference_cpu_callable():
    """The reference's own CPU implementation of the path, ``moe_w4a16_ref``
    (src/xkernels/ops/moe/reference.py:22-70), from the unmodified package installed under
    ``baseline/_ref``; None where that package is not there.  Nothing of this repo is on its path."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "xkernels" / "__init__.py").exists():
        return None
    if str(ref_dir) not in sys.path:
        sys.path.insert(0, str(ref_dir))
    try:
        from xkernels.ops.moe.reference import moe_w4a16_ref
        return moe_w4a16_ref
    except Exception:
        return None


def cpu_int4_sample(cfg, seed: int, n_rows: int, fn=None):
    """One bounded CPU sample of the configuration: all M tokens, all E experts, ``n_rows`` of the N
    weight rows (a column slice of the output), through ``fn`` = the reference's ``moe_w4a16_ref``
    or, without the reference package, the oracle port of it.  Returns (seconds, kind)."""
    from xkernels_b200 import synth

    kind = "reference"
    if fn is None:
        fn = reference_cpu_callable()
    if fn is None:
        from oracle import moe_oracle as oracle
        fn, kind = oracle.moe_w4a16, "port"
    A = synth.activations(cfg.M, cfg.K, seed=seed)
    packed, scale = synth.int4_weights(cfg.E, n_rows, cfg.K, cfg.group_size, seed=seed + 1)
    ids, w = synth.routing(cfg.M, cfg.E, cfg.top_k, seed=seed + 3, expert_bias_std=cfg.expert_bias_std,
                           zipf_scale=cfg.zipf_scale)
    t0 = time.perf_counter()
    fn(A, packed, scale, ids, w, cfg.group_size)
    return time.perf_counter() - t0, kind


def cpu_baseline_block(cfg, n_rows: int, verbatim: bool):
    """``cpu_baseline`` of the N=1 line: the reference's CPU code on an N-slice of the workload
    (work is linear in N) and, once, the same function verbatim on the WHOLE configuration."""
    cores = host_threads()
    t, kind = cpu_int4_sample(cfg, 1729, n_rows)
    frac = n_rows / cfg.N
    out = {
        "value": cfg.M * frac / t, "unit": "tokens/s", "cores": cores, "kind": kind,
        "sample": (f"{'xkernels moe_w4a16_ref (baseline/_ref, unmodified)' if kind == 'reference' else 'oracle.moe_w4a16'}"
                   f" on CPU torch: all {cfg.M} tokens x {cfg.E} experts x {n_rows}/{cfg.N} weight rows in {t:.2f} s; "
                   f"value = tokens x {n_rows}/{cfg.N} / seconds"),
        "seconds_per_sample": t,
    }
    fn = reference_cpu_callable() if verbatim else None
    if fn is not None:
        try:
            import psutil
            room = psutil.virtual_memory().available > 48 * 2 ** 30     # the reference materialises every expert
        except Exception:
            room = False
        if room:
            from xkernels_b200 import synth
            d = synth.make_int4(cfg, seed=1729)
            t0 = time.perf_counter()
            fn(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"], cfg.group_size)
            out["reference_verbatim_s"] = time.perf_counter() - t0
            out["reference_verbatim_tokens_per_s"] = cfg.M / out["reference_verbatim_s"]
    return out


def run_reference_arm(args, world: int, rank: int):
    """--impl reference: the reference's own CPU implementation with all host threads; rank 0 only.
    A step is a bounded sample of the workload (an N-slice sized so that the whole run takes about
    two minutes); ``ms_per_step`` is the measured time of a step, ``value`` counts the tokens of a
    step weighted by the fraction of the N rows it computed."""
    if rank != 0:
        return
    from xkernels_b200 import synth

    cores = host_threads()
    cfg = synth.CONFIGS["int4_decode" if world == 1 else "int4_ep"]
    if world > 1:
        cfg = synth.Int4Config(cfg.name, M=cfg.M * world, K=cfg.K, N=cfg.N, E=cfg.E, top_k=cfg.top_k,
                               zipf_scale=cfg.zipf_scale)
    fn = reference_cpu_callable()
    # the reference loops over M * top_k slots in Python, which does not shrink with the N-slice;
    # at the expert-parallel size that loop alone is minutes, so there the per-expert port stands in
    if fn is not None and cfg.M * cfg.top_k > 4096:
        fn = None
    # the largest N-slice (up to 512 rows) for which steps + warm-up stay within about two minutes
    n_steps = max(args.steps + args.warmup, 1)
    n_rows = min(512, cfg.N)
    while True:
        t_probe, kind = cpu_int4_sample(cfg, 1, n_rows, fn)
        if t_probe * n_steps <= 120.0 or n_rows <= 8:
            break
        n_rows //= 2
    for _ in range(args.warmup):
        cpu_int4_sample(cfg, 1, n_rows, fn)
    per_step = [cpu_int4_sample(cfg, 1729 + s, n_rows, fn)[0] for s in range(args.steps)]
    t_mean = sum(per_step) / len(per_step)
    value = cfg.M * (n_rows / cfg.N) / t_mean
    name = "xkernels moe_w4a16_ref (baseline/_ref, unmodified)" if kind == "reference" else \
        "oracle.moe_w4a16 (per-expert port of moe_w4a16_ref)"
    sample = (f"each step: {name} on all {cfg.M} tokens x {cfg.E} experts x {n_rows}/{cfg.N} weight rows; "
              f"value = tokens x {n_rows}/{cfg.N} / seconds per step")
    line = {
        "impl": "reference", "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_mean * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(cfg, world),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": sample},
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
def keep_loaded(fn, sync, total_ms: float, steps: int, seconds: float = 0.45, cap: int = 4000):
    """Untimed continuation of the timed loop, run while the clock sampler is still on: the K timed
    steps of a decode-sized call last a few milliseconds, less than one nvidia-smi sampling period, so
    the clocks and throttle reasons are read while the SAME loop goes on for about `seconds` more.
    The number of extra steps depends only on the arguments (every rank passes the same ones)."""
    per_step = max(total_ms / max(steps, 1), 1e-3)
    n = int(min(cap, max(1, seconds * 1e3 / per_step)))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(n):
        fn(i)
    stop.record()
    sync()
    return n, start.elapsed_time(stop)


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


class StagedInputs:
    """Per-step inputs of the fused op in one pinned host buffer and one device buffer of the same
    layout (256-byte aligned sections), so that a step's host-to-device traffic is a single copy."""

    def __init__(self, A, topk_ids, topk_w, dev):
        parts = [A.cpu().contiguous(), topk_ids.cpu().contiguous(), topk_w.cpu().contiguous()]
        offs, off = [], 0
        for t in parts:
            offs.append(off)
            off += -(-t.numel() * t.element_size() // 256) * 256
        self.nbytes = off
        self.host = torch.empty(off, dtype=torch.uint8).pin_memory()
        self.dev = torch.empty(off, dtype=torch.uint8, device=dev)
        self.views = []
        for t, o in zip(parts, offs):
            n = t.numel() * t.element_size()
            self.host[o:o + n].view(t.dtype).view(t.shape).copy_(t)
            self.views.append(self.dev[o:o + n].view(t.dtype).view(t.shape))

    def upload(self):
        self.dev.copy_(self.host, non_blocking=True)
        return self.views


def int4_parity(out, d, cfg, n0: int, n_cols: int, tokens=None):
    """Compare ``out[tokens, n0:n0+n_cols]`` with the CPU oracle on the same inputs (the oracle is the
    checker only; tolerance of the op spec: |a-e| <= 1e-2 + 2e-2|e|)."""
    from oracle import moe_oracle as oracle

    sel = slice(None) if tokens is None else tokens
    want = oracle.moe_w4a16(d["A"][sel].cpu(), d["packed"][:, n0:n0 + n_cols].cpu(), d["scale"][:, n0:n0 + n_cols].cpu(),
                            d["topk_ids"][sel].cpu(), d["topk_w"][sel].cpu(), cfg.group_size)
    got = out[sel][:, n0:n0 + n_cols].cpu()
    return {"violations": int(oracle.count_violations(got, want, 2e-2, 1e-2)), "elements_checked": int(want.numel()),
            "checked": f"{want.shape[0]} tokens x columns [{n0}, {n0 + n_cols}) against oracle.moe_w4a16",
            "rtol": 2e-2, "atol": 1e-2}


def int4_parity_global(out, d, cfg, n0: int, n_cols: int, tokens):
    """As :func:`int4_parity`, for weights that are already a column slice on the CPU."""
    from oracle import moe_oracle as oracle

    want = oracle.moe_w4a16(d["A"][tokens.to(d["A"].device)].cpu(), d["packed"], d["scale"],
                            d["topk_ids"][tokens.to(d["topk_ids"].device)].cpu(),
                            d["topk_w"][tokens.to(d["topk_w"].device)].cpu(), cfg.group_size)
    got = out[tokens.to(out.device)][:, n0:n0 + n_cols].cpu()
    return {"violations": int(oracle.count_violations(got, want, 2e-2, 1e-2)), "elements_checked": int(want.numel()),
            "checked": f"{want.shape[0]} tokens per rank x columns [{n0}, {n0 + n_cols}) against oracle.moe_w4a16 "
                       "on the global expert set"}


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

    # ---- device-resident throughput: exactly K steps, nothing else on the stream ----------
    launches0 = _lib.launch_count()
    with ClockSampler(0) as clocks:
        ms = timed_loop(step, args.steps, sync, lambda: None)
        launches = _lib.launch_count() - launches0
        n_more, ms_more = keep_loaded(step, sync, ms, args.steps)
    ops.check_status(dev)
    # ---- the GEMM kernel's own duration, live, in a second pass of K steps: the event pairs the
    # library records around that launch sit between the kernels of a call and would keep them from
    # overlapping their launch latency (programmatic dependent launch), so they stay out of the pass
    # that `value` is taken from
    _lib.gemm_timer_enable(args.steps)
    timed_loop(step, args.steps, sync, lambda: None)
    gemm_ms = _lib.gemm_timer_read()
    _lib.gemm_timer_enable(0)
    ops.check_status(dev)
    ms_per_step = ms / args.steps
    value = cfg.M / (ms_per_step * 1e-3)
    gemm_avg_ms = sum(gemm_ms) / max(len(gemm_ms), 1)
    achieved = alg_bytes / (gemm_avg_ms * 1e-3) / 1e9
    # DRAM traffic per launch from the ncu capture of the 16-expert relative of this workload
    # (--case int4_decode_small: 273.9 MB read+write for 264.2 MB of weights and scales); traffic
    # grows with the experts touched, so it is scaled by n_active / 16.
    traffic = 273.9e6 * n_active / 16.0
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                "traffic_source": "estimated: ncu dram bytes of a 16-expert capture scaled by experts touched",
                "kernel": "moe_tc_kernel<16, int4>", "kernel_us": gemm_avg_ms * 1e3,
                "algorithmic_bytes": alg_bytes, "peak_source": peaks["source"],
                "whole_call_frac": (alg_bytes / (ms_per_step * 1e-3) / 1e9) / peaks["hbm_gbs"]}

    # ---- parity of this very output, outside the timed region --------------------------------
    parity = int4_parity(step(0), d, cfg, n0=1024, n_cols=256)

    # ---- end to end: pinned host inputs in, result out, through the public API -----------
    # A | topk_ids | topk_w are staged in ONE pinned buffer and cross in one copy; the op reads views
    # of the device copy.
    stage = StagedInputs(d["A"], d["topk_ids"], d["topk_w"], dev)
    hO = torch.empty((cfg.M, cfg.N), dtype=torch.bfloat16).pin_memory()

    def e2e_step(_i):
        dA, dI, dW = stage.upload()
        out = xkb.fused_moe_int4_w4a16(dA, d["packed"], d["scale"], dI, dW, group_size=cfg.group_size)
        hO.copy_(out, non_blocking=True)

    for i in range(3):
        e2e_step(i)
    sync()
    assert torch.equal(hO, step(0).cpu()), "end-to-end result differs from the device-resident one"
    t0 = time.perf_counter()
    e2e_ms_events = timed_loop(e2e_step, args.steps, sync, lambda: None)
    e2e_wall = (time.perf_counter() - t0) * 1e3
    e2e_ms = max(e2e_ms_events, 0.0)
    e2e = {"value": cfg.M / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
           "h2d_bytes_per_step": stage.nbytes,
           "d2h_bytes_per_step": hO.numel() * 2, "us_per_call": e2e_ms / args.steps * 1e3,
           "wall_us_per_call": e2e_wall / args.steps * 1e3,
           "note": "expert weights stay resident in HBM (model state); per-step inputs A/topk_ids/topk_w "
                   "come from one pinned host buffer in one copy, the bf16 result goes back to pinned host memory"}

    line = {
        "metric": "fused_moe_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "us_per_call": ms_per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(cfg, 1), "clocks": clocks.summary(), "e2e": e2e,
        "sustained": {"tokens_per_s": cfg.M * n_more / (ms_more * 1e-3), "ms_per_step": ms_more / n_more, "steps": n_more,
                      "note": "the untimed continuation of the timed loop during which the clocks were sampled "
                              "(long enough for the power cap to act)"},
        "gpu_launches": int(launches), "roofline": roofline, "parity": parity,
    }
    if not args.no_extras:
        line["other_configs"] = extras(dev, peaks)
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline_block(cfg, 512, verbatim=not args.no_verbatim)
    if args.write_cards:
        line["cards_written"] = write_cards(args, line)
    print(json.dumps(line), flush=True)


def write_cards(args, line):
    """--write-cards DIR: append this run's numbers to the cards' ``perf.measured`` through the
    reference's own record_measurement (needs the reference package under baseline/_ref)."""
    if reference_cpu_callable() is None:
        return {"error": "the reference package is not installed under baseline/_ref"}
    from xkernels_b200 import plugin

    gpu = torch.cuda.get_device_name(0)
    src = (f"python bench.py --gpus 1 --steps {args.steps} --warmup {args.warmup} on {gpu}, CUDA events, "
           f"SM clock {line['clocks'].get('sm_mhz')} MHz, throttle reasons {line['clocks'].get('reasons')}, "
           f"{time.strftime('%Y-%m-%dT%H:%M:%SZ', time.gmtime())}")
    done = []
    r = line["roofline"]
    plugin.write_back("moe_int4_w4a16.cuda@1.0.0", shape={"M": 64, "K": 7168, "N": 4096, "E": 48, "top_k": 8}, dtype="bf16",
                      source=src, ms=round(line["ms_per_step"], 5), achieved_bw_pct=round(100 * r["whole_call_frac"], 2),
                      cards_dir=args.write_cards)
    done.append("moe_int4_w4a16.cuda@1.0.0 decode")
    oc = line.get("other_configs", {})
    if "ms_per_call" in oc.get("int4_prefill", {}):
        p = oc["int4_prefill"]
        plugin.write_back("moe_int4_w4a16.cuda@1.0.0", shape={"M": 16384, "K": 7168, "N": 4096, "E": 48, "top_k": 8},
                          dtype="bf16", source=src, ms=round(p["ms_per_call"], 4),
                          tflops=round(2.0 * 16384 * 8 * 4096 * 7168 / (p["ms_per_call"] * 1e-3) / 1e12, 1),
                          cards_dir=args.write_cards)
        plugin.write_back("moe_align_block_size.cuda@1.0.0", shape={"M": 16384, "top_k": 8, "num_experts": 48, "block_size": 16},
                          dtype="i32", source=src, ms=round(p["align_block16_us"] * 1e-3, 5), cards_dir=args.write_cards)
        done += ["moe_int4_w4a16.cuda@1.0.0 prefill", "moe_align_block_size.cuda@1.0.0"]
    if "us_per_call" in oc.get("mxfp4_decode", {}):
        m = oc["mxfp4_decode"]
        plugin.write_back("moe_mxfp4.cuda@1.0.0", shape={"M": 48, "hidden": 4096, "ispp": 512, "E": 256, "top_k": 6},
                          dtype="bf16", source=src, ms=round(m["us_per_call"] * 1e-3, 5),
                          achieved_bw_pct=round(100 * m["algorithmic_bytes"] / (m["us_per_call"] * 1e-6) / 1e9 / load_peaks()["hbm_gbs"], 2),
                          cards_dir=args.write_cards)
        done.append("moe_mxfp4.cuda@1.0.0")
    if "us_per_call" in oc.get("moe_sum_reduce_8192x8x7168_bf16", {}):
        m = oc["moe_sum_reduce_8192x8x7168_bf16"]
        plugin.write_back("moe_sum_reduce.cuda@1.1.0", shape={"M": 8192, "top_k": 8, "H": 7168}, dtype="bf16", source=src,
                          ms=round(m["us_per_call"] * 1e-3, 5), achieved_bw_pct=round(100 * m["frac_of_hbm_peak"], 2),
                          cards_dir=args.write_cards)
        done.append("moe_sum_reduce.cuda@1.1.0")
    if "us_per_call" in oc.get("topk_softmax_16384x256_top8_bf16", {}):
        m = oc["topk_softmax_16384x256_top8_bf16"]
        plugin.write_back("topk_softmax.cuda@1.0.0", shape={"M": 16384, "E": 256, "topk": 8}, dtype="bf16", source=src,
                          ms=round(m["us_per_call"] * 1e-3, 5), cards_dir=args.write_cards)
        done.append("topk_softmax.cuda@1.0.0")
    return done


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
    def settle():
        # a long tensor-bound run leaves the SM clock under the power cap for a while; the short
        # configurations are timed first and every block starts from an idle, synchronised device
        torch.cuda.synchronize()
        time.sleep(0.5)

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
    settle()
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
    settle()
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
    settle()
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
    settle()
    try:
        # The two expert-GEMM shapes of the reference's own INT4 benchmark (E=48, top_k=8, group 32;
        # meta/benchmarks/bench_moe_int4_w4a16.py:3-12,88-91): gate_up N=4096 K=7168 and the
        # down projection N=7168 K=2048, at decode and prefill batch sizes.  Small batches are
        # weight-stream bound (fraction of the measured HBM peak), large ones tensor bound.
        table = {}
        for name, (N, K) in {"gate_up_N4096_K7168": (4096, 7168), "down_N7168_K2048": (7168, 2048)}.items():
            packed, scale = synth.int4_weights(48, N, K, 32, seed=11, device=dev)
            rows = {}
            settle()
            for M in (1, 16, 64, 512, 4096):
                cfg = synth.Int4Config(name, M=M, K=K, N=N, E=48, top_k=8)
                A = synth.activations(M, K, seed=M, device=dev)
                ids, w = synth.routing(M, 48, 8, seed=M + 3, device=dev)
                fn = lambda: xkb.fused_moe_int4_w4a16(A, packed, scale, ids, w)  # noqa: E731
                for _ in range(3):
                    fn()
                torch.cuda.synchronize()
                n = 20 if M <= 512 else 5
                _lib.gemm_timer_enable(n)
                ms = time_call(fn, 0, n)
                g = _lib.gemm_timer_read()
                _lib.gemm_timer_enable(0)
                gm = sum(g) / len(g)
                b = synth.int4_algorithmic_bytes(cfg, int(torch.unique(ids).numel()))
                fl = synth.int4_flops(cfg)
                rows[f"M={M}"] = {"us_per_call": ms * 1e3, "gemm_kernel_us": gm * 1e3,
                                  "kernel_frac_of_hbm_peak": b / (gm * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                  "kernel_frac_of_bf16_peak": fl / (gm * 1e-3) / 1e12 / peaks["bf16_tflops"]}
            ops.check_status(dev)
            table[name] = rows
            del packed, scale
        out["int4_kimi_shapes"] = table
    except Exception as exc:  # noqa: BLE001
        out["int4_kimi_shapes"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    settle()
    try:
        # the two GEMMs above as ONE expert layer: gate_up (2*inter = 4096 rows) -> SwiGLU -> down, one call
        hidden, inter, E, top_k = 7168, 2048, 48, 8
        w13, s13 = synth.int4_weights(E, 2 * inter, hidden, 32, seed=21, device=dev)
        w2, s2 = synth.int4_weights(E, hidden, inter, 32, seed=22, device=dev)
        rows = {}
        for M in (16, 64):
            A = synth.activations(M, hidden, seed=M + 1, device=dev)
            ids, w = synth.routing(M, E, top_k, seed=M + 4, device=dev)
            fn = lambda: xkb.fused_moe_int4_ffn(A, w13, s13, w2, s2, ids, w)  # noqa: E731
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            ms = time_call(fn, 0, 20)           # the call, kernels overlapping as in use
            _lib.gemm_timer_enable(20)
            time_call(fn, 0, 20)
            g = _lib.gemm_timer_read()
            _lib.gemm_timer_enable(0)
            gm = sum(g) / 20
            n_act = int(torch.unique(ids).numel())
            b = n_act * (2 * inter * hidden + hidden * inter) * (0.5 + 2.0 / 32)      # packed nibbles + bf16 group scales
            rows[f"M={M}"] = {"us_per_call": ms * 1e3, "gemm_kernels_us": gm * 1e3, "active_experts": n_act,
                              "weight_bytes": b, "kernels_frac_of_hbm_peak": b / (gm * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        ops.check_status(dev)
        out["int4_ffn_hidden7168_inter2048"] = rows
        del w13, s13, w2, s2
    except Exception as exc:  # noqa: BLE001
        out["int4_ffn_hidden7168_inter2048"] = {"error": repr(exc)[:300]}
    torch.cuda.empty_cache()
    settle()
    try:
        cfg = synth.CONFIGS["int4_prefill"]
        d = synth.make_int4(cfg, seed=1729, device=dev)
        fn = lambda: xkb.fused_moe_int4_w4a16(d["A"], d["packed"], d["scale"], d["topk_ids"], d["topk_w"])  # noqa: E731
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        _lib.gemm_timer_enable(5)           # armed after the warm-up: five timed launches, five pairs
        ms = time_call(fn, 0, 5)
        g = _lib.gemm_timer_read()
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
                                  sm_margin=args.ep_sm_margin, local_first=bool(args.ep_local_first))
    # model set-up, outside the timed region: the most popular experts (measured on this batch's
    # routing) are copied to every rank; their slots are then served where the token lives
    hot = layer.rebalance(ids, args.ep_replicas) if args.ep_replicas > 0 else []

    # reference point for scaling: the SAME configuration on one GPU (all 256 experts local, 4096
    # tokens, no exchange), timed on rank 0 before the group run
    single = None
    if rank == 0:
        import xkernels_b200 as xkb
        pk1, sc1 = synth.int4_weights(cfg.E, cfg.N, cfg.K, cfg.group_size, seed=99, device=dev)
        t1 = time_call(lambda: xkb.fused_moe_int4_w4a16(A, pk1, sc1, ids, w, group_size=cfg.group_size),
                       max(args.warmup, 3), args.steps)
        single = {"tokens_per_s": cfg.M / (t1 * 1e-3), "ms_per_step": t1, "steps": args.steps,
                  "warmup": max(args.warmup, 3)}
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
    launches0 = _lib.launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.__enter__()
    ms = timed_loop(step, args.steps, sync, dist.barrier)
    launches = _lib.launch_count() - launches0
    # same number of extra steps on every rank (the steps are collective): from the slowest rank's time
    t_all = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t_all, op=dist.ReduceOp.MAX)
    n_more, ms_more = keep_loaded(step, sync, float(t_all), args.steps, cap=400)
    dist.barrier()
    if sampler:
        sampler.__exit__()
    _lib.gemm_timer_enable(4 * args.steps)      # kernel durations in a second pass (see run_single_gpu);
    timed_loop(step, args.steps, sync, dist.barrier)   # a step may launch more than one GEMM (local pass, chunks)
    gemm_ms = _lib.gemm_timer_read()
    _lib.gemm_timer_enable(0)
    t = torch.tensor([ms, sum(gemm_ms) / args.steps, float(layer.count_recv_slots()),
                      float(layer.last_recv_rows)], device=dev, dtype=torch.float64)
    gathered = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    ms_max = max(float(g[0]) for g in gathered)
    gemm_max = max(float(g[1]) for g in gathered)
    slots = [int(g[2]) for g in gathered]
    rows_in = [int(g[3]) for g in gathered]

    # parity of this rank's output, outside the timed region: 64 of its tokens x 256 columns against
    # the CPU oracle on the GLOBAL expert set (every rank's column slice of the weights is gathered
    # and put in global-id order), so that a wrong exchange, placement or combine shows on any rank
    n0, n_cols = 512, 256
    loc_p = packed[:, n0:n0 + n_cols].contiguous()
    loc_s = scale[:, n0:n0 + n_cols].contiguous()
    all_p = torch.empty((world,) + tuple(loc_p.shape), dtype=loc_p.dtype, device=dev)
    all_s = torch.empty((world,) + tuple(loc_s.shape), dtype=loc_s.dtype, device=dev)
    dist.all_gather_into_tensor(all_p, loc_p)
    dist.all_gather_into_tensor(all_s, loc_s)
    glob_p = torch.empty((cfg.E,) + tuple(loc_p.shape[1:]), dtype=loc_p.dtype)
    glob_s = torch.empty((cfg.E,) + tuple(loc_s.shape[1:]), dtype=loc_s.dtype)
    for r in range(world):
        gids = torch.tensor(ep.local_expert_ids(r, e_local, world, args.ep_placement))
        glob_p[gids] = all_p[r].cpu()
        glob_s[gids] = all_s[r].cpu()
    del all_p, all_s
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    tokens = torch.arange(0, cfg.M, cfg.M // 64)[:64]
    out_now = layer(A, ids, w)
    dsl = {"A": A, "packed": glob_p, "scale": glob_s, "topk_ids": ids, "topk_w": w}
    par = int4_parity_global(out_now, dsl, cfg, n0, n_cols, tokens)
    pv = torch.tensor([par["violations"], par["elements_checked"]], device=dev, dtype=torch.float64)
    pg = [torch.zeros_like(pv) for _ in range(world)]
    dist.all_gather(pg, pv)

    # end to end: pinned host activations/routing in (one staged copy), result out
    stage = StagedInputs(A, ids, w, dev)
    hO = torch.empty((cfg.M, cfg.N), dtype=torch.bfloat16).pin_memory()

    def e2e_step(_i):
        dA, dI, dW = stage.upload()
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
            "sustained": {"tokens_per_s": world * cfg.M * n_more / (ms_more * 1e-3), "ms_per_step": ms_more / n_more,
                          "steps": n_more, "note": "rank 0's untimed continuation of the timed loop during which "
                                                   "the clocks were sampled"},
            "e2e": {"value": tokens / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": world * stage.nbytes,
                    "d2h_bytes_per_step": world * hO.numel() * 2},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops_sustained"],
                         "unit": "TFLOP/s", "frac": tf / peaks["bf16_tflops_sustained"], "traffic": None,
                         "kernel": "moe_tc_kernel (busiest rank)", "kernel_ms": gemm_max,
                         "peak_source": peaks["source"] + " (sustained)"},
            "slots_received_per_rank": slots,
            "rows_received_per_rank": rows_in,   # one activation row per (token, rank) pair crosses the wire
            "ep": {"placement": args.ep_placement, "chunks": args.ep_chunks, "sm_margin": args.ep_sm_margin, "local_first": layer.local_first,
                   "replicated_experts": hot,
                   "same_config_on_one_gpu": single,
                   # weak scaling against the SAME configuration on one GPU (the N=1 line of this
                   # benchmark is the decode workload, a different one)
                   "weak_scaling_efficiency": (tokens / (ms_per_step * 1e-3)) / (world * single["tokens_per_s"])},
            "parity": {"violations_per_rank": [int(g[0]) for g in pg], "elements_checked_per_rank": int(pg[0][1]),
                       "tokens_checked": 64, "checked": par["checked"], "rtol": 2e-2, "atol": 1e-2},
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
    ap.add_argument("--no-verbatim", action="store_true",
                    help="skip the one full-size run of the reference's CPU function (about 15 s, 24 GB of host memory)")
    ap.add_argument("--write-cards", default=None, metavar="DIR",
                    help="append this run's numbers to the cards' perf.measured (through the reference's "
                         "record_measurement) and write the updated card files to DIR")
    ap.add_argument("--ep-placement", default="round_robin", choices=["contiguous", "round_robin", "snake"],
                    help="expert -> rank assignment of the expert-parallel run")
    ap.add_argument("--ep-chunks", type=int, default=1, help="token chunks pipelined through the exchanges")
    ap.add_argument("--ep-replicas", type=int, default=4,
                    help="most popular experts copied to every rank (their slots stay on the token's rank)")
    ap.add_argument("--ep-local-first", type=int, default=0, choices=[0, 1],
                    help="compute the slots of a rank's own experts beside the exchange instead of sending them to itself")
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
