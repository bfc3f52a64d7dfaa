"""Benchmark of the packed groupwise GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1]

Workload (default "c2"): packed INT4 GEMV, M=4, K=4096, N=11008, group 128, 32 exact fp16
outlier columns (41 requested, snapped as the reference constructor does), rank-8 residual,
heavy-tailed (lognormal channel scale) fp16 activations.  "c1" is the INT2 M=1 4096x4096 g64 case.

One step = one pass over a ring of RING distinct weight sets (each its own packed / scales /
outlier / residual tensors, > 2x the 126 MB L2 in total), i.e. RING fused GEMVs that all read
cold weights.  `value` is algorithmic bytes per second over all ranks with every operand
resident in HBM (the step is replayed from a CUDA graph).  `e2e` is the same quantity through
the public module API with HOST activations: pinned-memory H2D copy of x, forward, D2H copy of
y, every GEMV, inside the timed region.  With N > 1 each rank owns its own ring (row shards of
a larger layer need no collective), so scaling is weak.

`--impl reference` times the CPU restatement of the reference's dequantise-then-matmul path
(oracle/qgemv_ref.c, OpenMP over all host cores) on the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

RING = 16
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0

WORKLOADS = {
    "c2": dict(bits=4, m=4, n=11008, k=4096, group=128, outliers=32, rank=8,
               name="int4_gemv_M4_K4096_N11008_g128_oc32_r8"),
    "c1": dict(bits=2, m=1, n=4096, k=4096, group=64, outliers=0, rank=0,
               name="int2_gemv_M1_K4096_N4096_g64"),
    # variants used to attribute time (not headline workloads)
    "c2_plain": dict(bits=4, m=4, n=11008, k=4096, group=128, outliers=0, rank=0,
                     name="int4_gemv_M4_K4096_N11008_g128_plain"),
    "int2_big": dict(bits=2, m=1, n=14336, k=4096, group=128, outliers=32, rank=8,
                     name="int2_gemv_M1_K4096_N14336_g128_oc32_r8"),
    "int2_tp": dict(bits=2, m=1, n=3584, k=8192, group=128, outliers=64, rank=8,
                    name="int2_gemv_M1_K8192_N3584_g128_oc64_r8"),
    "int2_kv": dict(bits=2, m=1, n=1024, k=4096, group=128, outliers=32, rank=8,
                    name="int2_gemv_M1_K4096_N1024_g128_oc32_r8"),
    "int2_q": dict(bits=2, m=1, n=4096, k=4096, group=128, outliers=32, rank=8,
                   name="int2_gemv_M1_K4096_N4096_g128_oc32_r8"),
    "int2_down": dict(bits=2, m=1, n=4096, k=14336, group=128, outliers=64, rank=8,
                      name="int2_gemv_M1_K14336_N4096_g128_oc64_r8"),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (None until a capture exists for that workload).
NCU_TRAFFIC_BYTES = {"c2": 24303360, "c1": 4776192, "c2_plain": 23340544}


def algorithmic_bytes(w) -> int:
    """Every operand counted once: packed codes + scales + outlier weights/indices + residual
    factors + activations + output (bytes)."""
    n, k, m = w["n"], w["k"], w["m"]
    b = n * k * w["bits"] // 8 + n * (k // w["group"]) * 2
    if w["outliers"]:
        b += n * w["outliers"] * 2 + w["outliers"] * 4
    if w["rank"]:
        b += n * w["rank"] * 2 + w["rank"] * k * 2
    return b + m * k * 2 + m * n * 2


def make_weight_set(w, seed):
    """Random packed tensors of the workload's shapes (uniform codes, positive fp16 scales):
    throughput does not depend on the values, and quantising RING real matrices on the host
    would take minutes.  Activations are N(0,1) x lognormal(0,1) channel scales as configured."""
    rng = np.random.default_rng(seed)
    n, k = w["n"], w["k"]
    d = dict(
        packed=rng.integers(0, 256, size=(n, k * w["bits"] // 8), dtype=np.uint8),
        scales=(rng.random((n, k // w["group"]), dtype=np.float32) * 0.01 + 0.002).astype(np.float16),
    )
    if w["outliers"]:
        d["outlier_idx"] = rng.choice(k, size=w["outliers"], replace=False).astype(np.int32)
        d["outlier_weight"] = (rng.standard_normal((n, w["outliers"]), dtype=np.float32) * 0.02).astype(np.float16)
    if w["rank"]:
        d["res_u"] = (rng.standard_normal((n, w["rank"]), dtype=np.float32) * 0.01).astype(np.float16)
        d["res_v"] = (rng.standard_normal((w["rank"], k), dtype=np.float32) * 0.01).astype(np.float16)
    return d


def make_x(w, seed):
    rng = np.random.default_rng(1000 + seed)
    c = np.exp(rng.standard_normal(w["k"], dtype=np.float32))
    return (rng.standard_normal((w["m"], w["k"]), dtype=np.float32) * c).astype(np.float16)


# ----------------------------------------------------------------------------------------------
# CPU arm: the C restatement of the reference's CPU path
# ----------------------------------------------------------------------------------------------
def load_c_oracle():
    lib = ROOT / "oracle" / "libqgemv_oracle.so"
    src = ROOT / "oracle" / "qgemv_ref.c"
    if not lib.exists() or lib.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    l = ctypes.CDLL(str(lib))
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    l.qref_forward.argtypes = [vp, i64, ci, ci, vp, vp, i64, i64, i64, ci, ci, vp, vp, vp, ci, vp, vp, ci, ci, vp, vp]
    l.qref_forward.restype = None
    l.qref_num_threads.restype = ci
    l.qref_set_threads.argtypes = [ci]
    l.qref_set_threads.restype = None
    try:                                         # all host cores this process may use, whatever OMP_NUM_THREADS says
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    l.qref_set_threads(cores)
    return l


def cpu_gemv_seconds(lib, w, ws, x, reps):
    """Time `reps` forward passes of the CPU restatement on one weight set; returns (seconds, y)."""
    n, k, m = w["n"], w["k"], w["m"]
    wbuf = np.empty((n, k), dtype=np.float32)
    y = np.empty((m, n), dtype=np.float32)
    p = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)
    args = (p(x.view(np.uint16)), k, 0, m, p(ws["packed"]), p(ws["scales"]), n, k, k, w["group"], w["bits"], None,
            p(ws.get("outlier_idx")), p(ws.get("outlier_weight")), w["outliers"],
            p(ws.get("res_u")), p(ws.get("res_v")), w["rank"], 0, p(wbuf), p(y))
    lib.qref_forward(*args)                      # warm-up: page in the scratch matrix
    t0 = time.perf_counter()
    for _ in range(reps):
        lib.qref_forward(*args)
    return time.perf_counter() - t0, y


def cpu_baseline(w, budget_s=12.0):
    lib = load_c_oracle()
    ws, x = make_weight_set(w, 0), make_x(w, 0)
    t1, _ = cpu_gemv_seconds(lib, w, ws, x, 1)
    reps = max(1, min(200, int(budget_s / max(t1, 1e-4))))
    t, _ = cpu_gemv_seconds(lib, w, ws, x, reps)
    per = t / reps
    return dict(value=algorithmic_bytes(w) / per / 1e9, unit="GB/s", cores=int(lib.qref_num_threads()), kind="port",
                sample=f"{reps} GEMVs of one weight set of the workload ({per * 1e3:.2f} ms each; "
                       f"dequantise whole matrix to fp32, then matmul, OpenMP)",
                ms_per_gemv=per * 1e3)


def run_reference_arm(args, w):
    """`--impl reference`: rank 0 times the CPU path; other ranks exit."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    lib = load_c_oracle()
    ws, x = make_weight_set(w, 0), make_x(w, 0)
    t1, _ = cpu_gemv_seconds(lib, w, ws, x, 1)
    # one step = a bounded sample of the ring: at most RING GEMVs, fewer when the whole run
    # (steps + warm-up) would otherwise exceed about 90 s of host time
    per_step = max(1, min(RING - 1, int(90.0 / (args.steps + args.warmup) / max(t1, 1e-4)) - 1))
    for _ in range(args.warmup):
        cpu_gemv_seconds(lib, w, ws, x, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_gemv_seconds(lib, w, ws, x, per_step)
    # cpu_gemv_seconds runs one extra warm-up pass per call; account for it
    elapsed = time.perf_counter() - t0
    gemvs = args.steps * (per_step + 1)
    per = elapsed / gemvs
    val = algorithmic_bytes(w) / per / 1e9
    cores = int(lib.qref_num_threads())
    line = dict(metric="packed_gemv_algorithmic_GBps", value=val, unit="GB/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=elapsed / args.steps * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(workload=w["name"], gemvs_per_step=per_step + 1, l2="host run: not applicable"),
                us_per_gemv=per * 1e6,
                cpu_baseline=dict(value=val, unit="GB/s", cores=cores, kind="port",
                                  sample=f"{gemvs} GEMVs on one weight set, dequantise-then-matmul in C/OpenMP"),
                e2e=dict(value=val, unit="GB/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        self.stop_flag.set()
        self.join(timeout=6)
        if not self.samples:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["unavailable"])
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return dict(sm_mhz=mhz[len(mhz) // 2], sm_max_mhz=float(self.samples[0][1]), reasons=reasons,
                    samples=len(self.samples))


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def run_gpu_arm(args, w):
    import torch
    import torch.distributed as dist
    from ai_accel_studio_b200 import _cabi, ops
    from ai_accel_studio_b200.optimize._hybrid_base import HybridPackedLinear

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the packed GEMV has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _cabi.lib()                                   # fail loudly if the CUDA library is missing

    bits, m, n, k = w["bits"], w["m"], w["n"], w["k"]
    sets = []
    for i in range(RING):
        h = make_weight_set(w, rank * RING + i)
        sets.append({key: torch.from_numpy(v).to(dev) for key, v in h.items()})
    xs_host = [torch.from_numpy(make_x(w, rank * RING + i)).pin_memory() for i in range(RING)]
    xs_dev = [x.to(dev) for x in xs_host]
    ys_host = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _ in range(RING)]
    ops.ensure_workspace(dev)
    kernel = _cabi.KERNEL[args.kernel] | (args.debug << 8)

    def gemv(i, x):
        s = sets[i]
        return ops.gemv(x, s["packed"], s["scales"], None, s.get("outlier_idx"), s.get("outlier_weight"),
                        s.get("res_u"), s.get("res_v"), bits, w["group"], k, 0, kernel)

    # Public-API modules for the end-to-end leg: the drop-in Linear wrapper around each weight set.
    class _Layer(HybridPackedLinear):
        def __init__(self, s):
            super().__init__()
            self.bits = bits
            for key in ("outlier_idx", "outlier_weight", "packed", "scales"):
                if key in s:
                    self.register_buffer(key, s[key])
            if "outlier_idx" not in s:
                self.register_buffer("outlier_idx", torch.empty(0, dtype=torch.int32, device=dev))
                self.register_buffer("outlier_weight", torch.empty((n, 0), dtype=torch.float16, device=dev))
            self.original_k = self.padded_k = self.in_features = k
            self.group_size, self.out_features, self.graph_safe, self.kernel = w["group"], n, True, args.kernel
            self.debug = args.debug
            self.bias = None
            self.residual_rank = w["rank"]
            self.res_u, self.res_v = s.get("res_u"), s.get("res_v")
    layers = [_Layer(s) for s in sets]

    # ---- device-resident leg: one step captured as a CUDA graph --------------------------
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(RING):
            gemv(i, xs_dev[i])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = [gemv(i, xs_dev[i]) for i in range(RING)]
    s0 = sets[0]
    launches_per_gemv = ops.plan_launches(xs_dev[0], s0["packed"], s0["scales"], bits, w["group"], k, s0.get("outlier_idx"),
                                          s0.get("outlier_weight"), s0.get("res_u"), s0.get("res_v"), kernel=args.kernel)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        graph.replay()
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)

    # ---- end-to-end leg: host activations in, host results out, every GEMV ----------------
    # The step (pinned-host x -> device, module forward, result -> pinned host, for each of the
    # RING layers) is captured once and replayed, as a serving loop would do; the copies are
    # memcpy nodes of the graph and run inside the timed region.
    # Host activations arrive on one stream, the GEMVs run on the current stream and the results
    # leave on a third, tied together with events (captured as parallel branches of the graph):
    # layer i+1's input copy and layer i-1's result copy overlap layer i's kernel.  Each layer has
    # its own device input / output buffer, written with forward_into.  --e2e-mode serial puts
    # all three on one stream instead.
    xd_bufs = [torch.empty_like(x, device=dev) for x in xs_host]
    yd_bufs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(RING)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        cur = torch.cuda.current_stream()
        if args.e2e_mode == "serial":
            for i in range(RING):
                xd_bufs[i].copy_(xs_host[i], non_blocking=True)
                layers[i].forward_into(xd_bufs[i], yd_bufs[i])
                ys_host[i].copy_(yd_bufs[i], non_blocking=True)
            return
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        for i in range(RING):
            with torch.cuda.stream(s_in):
                xd_bufs[i].copy_(xs_host[i], non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            cur.wait_event(ready)
            layers[i].forward_into(xd_bufs[i], yd_bufs[i])
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                ys_host[i].copy_(yd_bufs[i], non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
    side2 = torch.cuda.Stream()
    side2.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side2):
        for _ in range(2):
            e2e_step()
    torch.cuda.current_stream().wait_stream(side2)
    torch.cuda.synchronize()
    e2e_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(e2e_graph):
        e2e_step()
    for _ in range(max(args.warmup, 3)):
        e2e_graph.replay()
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        e2e_graph.replay()
    f1.record()
    barrier()
    # the replayed graph wrote real results to the host buffers
    torch.cuda.synchronize()
    assert bool(torch.isfinite(ys_host[0].float()).all()) and float(ys_host[0].float().abs().sum()) > 0
    for i in (0, RING - 1):                      # ... and they are the device-resident leg's results, bit for bit
        assert torch.equal(ys_host[i], outs[i].cpu()), "end-to-end result differs from the device-resident result"
    ms_e2e = f0.elapsed_time(f1)
    clocks = sampler.summary() if sampler else None

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        ab = algorithmic_bytes(w)
        gemvs = RING * args.steps
        us = ms * 1e3 / gemvs
        value = ab * world / (us * 1e-6) / 1e9
        us_e2e = ms_e2e * 1e3 / gemvs
        peak, peak_kind = measured_peak()
        per_gpu = ab / (us * 1e-6) / 1e9
        with torch.cuda.device(dev):
            prob_name = ops.plan_name(xs_dev[0], sets[0]["packed"], sets[0]["scales"], bits, w["group"], k,
                                      kernel=args.kernel)
        line = dict(
            metric="packed_gemv_algorithmic_GBps", value=value, unit="GB/s", n_gpus=world, steps=args.steps,
            warmup=max(args.warmup, 3), ms_per_step=ms / args.steps, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="f32", data="synthetic",
            config=dict(workload=w["name"], gemvs_per_step=RING, kernel=prob_name,
                        l2=f"ring of {RING} distinct weight sets ({RING * ab / 1e6:.0f} MB) larger than 2x L2; no flush needed",
                        timing="CUDA events around graph replays on the launching stream, max over ranks"),
            us_per_gemv=us, pct_of_nominal_8000=100.0 * per_gpu / NOMINAL_HBM_GBS,
            pct_of_measured_copy=100.0 * per_gpu / peak,
            e2e=dict(value=ab * world / (us_e2e * 1e-6) / 1e9, unit="GB/s", us_per_gemv=us_e2e,
                     h2d_bytes_per_step=RING * m * k * 2, d2h_bytes_per_step=RING * m * n * 2,
                     api="pinned host x -> device, HybridPackedLinear.forward_into, result -> pinned host y, per GEMV; "
                         + ("copies on their own streams overlap the kernels" if args.e2e_mode == "overlap" else "one stream")
                         + "; step replayed from a CUDA graph"),
            gpu_launches=gemvs * launches_per_gemv * 2,     # device-resident leg + end-to-end leg
            roofline=dict(bound="hbm", achieved=per_gpu, peak=peak, unit="GB/s", frac=per_gpu / peak,
                          traffic=NCU_TRAFFIC_BYTES.get(args.workload), peak_source=f"{peak_kind} copy bandwidth",
                          algorithmic_bytes_per_launch=ab,
                          note="launch duration = event time of the timed region / GEMVs (includes inter-kernel gaps; "
                               f"{launches_per_gemv} launch(es) per GEMV)"),
            clocks=clocks,
        )
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma", "mma_phased"])
    ap.add_argument("--debug", type=lambda v: int(v, 0), default=0,
                    help="qgemv_problem.debug bits (tuning aids of the pipelined kernel; see include/qgemv_b200.h)")
    ap.add_argument("--e2e-mode", choices=["overlap", "serial"], default="overlap",
                    help="end-to-end leg: copies on their own streams overlapping the kernels, or everything on one stream")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
