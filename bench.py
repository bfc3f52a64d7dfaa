"""Benchmark of the packed groupwise GEMV hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1]

Headline workload (default "c2"): packed INT4 GEMV, M=4, K=4096, N=11008, group 128, 32 exact fp16
outlier columns (41 requested, snapped as the reference constructor does), rank-8 residual,
heavy-tailed (lognormal channel scale) fp16 activations.  "c1" is the INT2 M=1 4096x4096 g64 case.

One step = PASSES passes over a ring of RING distinct weight sets (each its own packed / scales /
outlier / residual tensors, > 2x the 126 MB L2 in total), i.e. PASSES x RING fused GEMVs that all
read cold weights; a pass is one CUDA graph of RING kernel nodes.  `value` is algorithmic bytes per
second over all ranks with every operand resident in HBM.  `e2e` is the same quantity through the
public module API with HOST activations: pinned-memory H2D copy of x, forward, D2H copy of y, every
GEMV, inside the timed region (`e2e_serial`: the same on one stream, nothing overlapping).  With
N > 1 each rank owns its own ring (row shards of a larger layer need no collective), so `value`
scales weakly.

The same JSON line also carries `c1` (the INT2 configuration, device-resident) and `decode`: whole-
model greedy decode of the benchmark's decoder shapes through the packed modules and through fp16
cuBLAS -- on one GPU the 8B shape (batch 1 and 4) and the 70B shape, on N > 1 GPUs the 70B shape
tensor parallel (q/k/v/gate/up split by rows, o/down by K with an all-reduce inside the captured
graph, lm_head by vocabulary rows) -- with the per-token time split into packed GEMVs, all-reduces
and everything else.

`--impl reference` times the CPU restatement of the reference's dequantise-then-matmul path
(oracle/qgemv_ref.c, OpenMP over all host cores) on the same workload; its value does not grow with
--gpus (one host process).
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

RING = 16          # weight sets per pass of the headline workload (389 MB)
PASSES = 32        # passes per step: 512 GEMVs, a few milliseconds, so that 20 steps span > 50 ms
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
NCU_TRAFFIC_BYTES = {"c2": 24303616, "c1": 4776192, "c2_plain": 23340544}


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


def workload_config(w):
    """The `config` object, identical in both arms: the two lines describe one workload."""
    ab = algorithmic_bytes(w)
    return dict(workload=w["name"], gemvs_per_step=RING * PASSES,
                l2=f"GPU arm: ring of {RING} distinct weight sets ({RING * ab / 1e6:.0f} MB) larger than 2x L2, no flush needed; "
                   "CPU arm: host run, not applicable")


def run_reference_arm(args, w):
    """`--impl reference`: rank 0 times the CPU path; other ranks exit.  One host process, whatever
    --gpus says: its value does not scale with N."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    lib = load_c_oracle()
    ws, x = make_weight_set(w, 0), make_x(w, 0)
    t1, _ = cpu_gemv_seconds(lib, w, ws, x, 1)
    # one step = a bounded sample of the GPU arm's step: at most RING GEMVs, fewer when the whole run
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
    cfg = workload_config(w)
    line = dict(metric="packed_gemv_algorithmic_GBps", value=val, unit="GB/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=elapsed / args.steps * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic", impl="reference", config=cfg,
                us_per_gemv=per * 1e6, sampled_gemvs_per_step=per_step + 1,
                note="one host process on rank 0: the value does not grow with --gpus; each step is a bounded sample "
                     f"({per_step + 1} GEMVs) of the GPU arm's step",
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


def time_resident_ring(w, ring, passes, steps, warmup, kernel, dev, rank, world, barrier, hints=True):
    """Device-resident leg for one workload: `ring` weight sets, one CUDA graph per pass, `passes`
    replays per step.  Returns (ms of the timed region, launches per GEMV, plan description, outputs, tensors)."""
    import torch
    from ai_accel_studio_b200 import ops
    bits, k = w["bits"], w["k"]
    sets = []
    for i in range(ring):
        h = make_weight_set(w, rank * ring + i)
        sets.append({key: torch.from_numpy(v).to(dev) for key, v in h.items()})
    xs_host = [torch.from_numpy(make_x(w, rank * ring + i)).pin_memory() for i in range(ring)]
    xs_dev = [x.to(dev) for x in xs_host]

    def gemv(i, x):
        s = sets[i]
        # the hint a chain of layers gives: while set i streams, set i+1's packed codes are announced to L2
        return ops.gemv(x, s["packed"], s["scales"], None, s.get("outlier_idx"), s.get("outlier_weight"),
                        s.get("res_u"), s.get("res_v"), bits, w["group"], k, 0, kernel,
                        sets[(i + 1) % ring]["packed"] if hints else None)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(ring):
            gemv(i, xs_dev[i])
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = [gemv(i, xs_dev[i]) for i in range(ring)]
    s0 = sets[0]
    info = ops.plan_describe(xs_dev[0], s0["packed"], s0["scales"], bits, w["group"], k, s0.get("outlier_idx"),
                             s0.get("outlier_weight"), s0.get("res_u"), s0.get("res_v"), kernel=kernel)
    for _ in range(max(warmup, 3)):
        graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps * passes):
        graph.replay()
    e1.record()
    barrier()
    return e0.elapsed_time(e1), info, outs, dict(sets=sets, xs_host=xs_host, xs_dev=xs_dev)


def decode_legs(args, dev, rank, world):
    """Whole-model greedy decode of the benchmark's decoder shapes (mixed-bit packed modules and the
    fp16 cuBLAS model), one record per (shape, batch).  Bounded by --decode-budget-s."""
    import gc
    import torch
    import torch.distributed as dist
    from ai_accel_studio_b200 import model_tools as mt
    if world == 1:
        legs = [("llama-3-8b", 1, 512, 128, (0.6, 0.3, 0.1)), ("llama-3-8b", 4, 512, 128, (0.6, 0.3, 0.1)),
                ("llama-3-70b", 1, 1024, 128, (0.7, 0.3, 0.0))]
    else:
        legs = [("llama-3-8b", 1, 512, 128, (0.6, 0.3, 0.1)), ("llama-3-70b", 1, 1024, 128, (0.7, 0.3, 0.0))]
    records, t_start = [], time.perf_counter()
    for shape, batch, prompt, new, probs in legs:
        rec = dict(shape=shape, batch=batch, prompt_tokens=prompt, new_tokens=new, tensor_parallel=world,
                   plan="seeded P(INT2), P(INT4), P(FP16) = %s, group 128, 1%% outliers, rank-8 residual" % (probs,),
                   layers=mt.SHAPES[shape]["layers"])
        for variant in ("mixed", "fp16"):
            spent = time.perf_counter() - t_start
            over = torch.tensor([1.0 if spent > args.decode_budget_s else 0.0], device=dev)
            if world > 1:
                dist.all_reduce(over, op=dist.ReduceOp.MAX)       # every rank takes the same decision
            if float(over[0]) > 0:
                rec[variant] = dict(skipped=f"decode time budget of {args.decode_budget_s:.0f} s spent")
                continue
            if variant == "fp16":
                need = mt.fp16_weight_bytes(shape, world) * 1.08 + (6 << 30)
                free = torch.cuda.mem_get_info(dev)[0]
                if need > free:
                    rec[variant] = dict(skipped=f"{need / 1e9:.0f} GB of fp16 weights and buffers do not fit {free / 1e9:.0f} GB free")
                    continue
            t0 = time.perf_counter()
            try:
                res = mt.decode_benchmark(shape, dev, batch, prompt, new, probs, variant == "mixed", world,
                                          split=True, shard_vocab=True, fuse_siblings=True)
            except torch.cuda.OutOfMemoryError:
                rec[variant] = dict(skipped="out of device memory")
                gc.collect()
                torch.cuda.empty_cache()
                continue
            tps = torch.tensor([res["aggregate_decode_tokens_s"]], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(tps, op=dist.ReduceOp.MIN)        # the slowest rank sets the pace
            rec[variant] = dict(decode_tokens_s=float(tps[0]), ttft_ms=res["ttft_ms"],
                                ms_per_token=res["decode_ms_per_token"], weight_bytes_per_rank=res["total"],
                                all_reduces_per_token=res["all_reduces_per_token"],
                                packed_gemvs_per_token=res["packed_gemvs_per_token"],
                                lm_head_rows_per_rank=res["lm_head_rows_per_rank"],
                                split_ms_per_token=res.get("split_ms_per_token"),
                                all_reduce_impl=res.get("all_reduce_impl"), one_shot_status=res.get("one_shot_status"),
                                decode_step=res.get("decode_step"), fused_sibling_groups=res.get("fused_sibling_groups"),
                                build_and_run_s=time.perf_counter() - t0)
            del res
            gc.collect()
            torch.cuda.empty_cache()
        if "decode_tokens_s" in rec.get("mixed", {}) and "decode_tokens_s" in rec.get("fp16", {}):
            rec["mixed_over_fp16"] = rec["mixed"]["decode_tokens_s"] / rec["fp16"]["decode_tokens_s"]
        records.append(rec)
    return records


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
    ops.ensure_workspace(dev)
    kernel = _cabi.KERNEL[args.kernel] | (args.debug << 8)
    bits, m, n, k = w["bits"], w["m"], w["n"], w["k"]
    passes = args.passes

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident leg: the headline number ------------------------------------------------
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    ms, info, outs, t = time_resident_ring(w, RING, passes, args.steps, args.warmup, kernel, dev, rank, world, barrier,
                                           hints=args.prefetch_hints)
    sets, xs_host = t["sets"], t["xs_host"]

    # ---- end-to-end leg: host activations in, host results out, every GEMV ----------------------
    # The pass (pinned-host x -> device, module forward, result -> pinned host, for each of the RING
    # layers) is captured once and replayed, as a serving loop would do; the copies are memcpy nodes
    # of the graph and run inside the timed region.  "overlap": host activations arrive on one
    # stream, the GEMVs run on the current stream and the results leave on a third, tied together with
    # events (parallel branches of the graph), so layer i+1's input copy and layer i-1's result copy
    # overlap layer i's kernel -- right for independent requests.  "serial": everything on one
    # stream, nothing overlaps -- what a dependent chain of layers sees.
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
            self.prefetch_next = None
            self.residual_rank = w["rank"]
            self.res_u, self.res_v = s.get("res_u"), s.get("res_v")
    layers = [_Layer(s) for s in sets]
    if args.prefetch_hints:
        for i, layer in enumerate(layers):
            layer.prefetch_next = sets[(i + 1) % RING]["packed"]
    ys_host = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _ in range(RING)]
    xd_bufs = [torch.empty_like(x, device=dev) for x in xs_host]
    yd_bufs = [torch.empty((m, n), dtype=torch.float16, device=dev) for _ in range(RING)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_pass(mode):
        cur = torch.cuda.current_stream()
        if mode == "serial":
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

    def time_e2e(mode):
        side2 = torch.cuda.Stream()
        side2.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side2):
            for _ in range(2):
                e2e_pass(mode)
        torch.cuda.current_stream().wait_stream(side2)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            e2e_pass(mode)
        for _ in range(max(args.warmup, 3)):
            g.replay()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.steps * passes):
            g.replay()
        f1.record()
        barrier()
        torch.cuda.synchronize()
        # the replayed graph wrote real results to the host buffers: the device-resident leg's, bit for bit
        assert bool(torch.isfinite(ys_host[0].float()).all()) and float(ys_host[0].float().abs().sum()) > 0
        for i in (0, RING - 1):
            assert torch.equal(ys_host[i], outs[i].cpu()), "end-to-end result differs from the device-resident result"
        return f0.elapsed_time(f1)
    ms_e2e = time_e2e("overlap")
    ms_e2e_serial = time_e2e("serial")
    clocks = sampler.summary() if sampler else None
    status = ops.workspace_status(dev)
    del layers, xd_bufs, yd_bufs, outs, t, sets
    torch.cuda.empty_cache()

    # ---- configuration 1 (INT2, M = 1, 4096 x 4096, group 64), device-resident -------------------
    c1 = None
    if args.workload != "c1" and not args.no_c1:
        w1 = WORKLOADS["c1"]
        ring1 = 64                                   # 64 x 4.7 MB = 303 MB > 2x L2
        passes1 = max(1, passes // 4)
        ms1, info1, _, t1 = time_resident_ring(w1, ring1, passes1, args.steps, args.warmup, kernel, dev, rank, world, barrier,
                                               hints=args.prefetch_hints)
        del t1
        torch.cuda.empty_cache()
        if world > 1:
            tt = torch.tensor([ms1], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms1 = float(tt[0])
        us1 = ms1 * 1e3 / (args.steps * passes1 * ring1)
        c1 = dict(workload=w1["name"], us_per_gemv=us1, gemvs_per_step=passes1 * ring1, kernel=info1["name"],
                  algorithmic_bytes_per_launch=algorithmic_bytes(w1),
                  per_gpu_GBps=algorithmic_bytes(w1) / (us1 * 1e-6) / 1e9)

    if world > 1:
        tt = torch.tensor([ms, ms_e2e, ms_e2e_serial], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, ms_e2e, ms_e2e_serial = float(tt[0]), float(tt[1]), float(tt[2])

    decode = None
    if not args.no_decode:
        decode = decode_legs(args, dev, rank, world)

    if rank == 0:
        ab = algorithmic_bytes(w)
        gemvs = RING * passes * args.steps
        us = ms * 1e3 / gemvs
        value = ab * world / (us * 1e-6) / 1e9
        us_e2e, us_ser = ms_e2e * 1e3 / gemvs, ms_e2e_serial * 1e3 / gemvs
        peak, peak_kind = measured_peak()
        per_gpu = ab / (us * 1e-6) / 1e9
        cfg = workload_config(w)
        cfg["gemvs_per_step"] = RING * passes
        plan = dict(kernel=info["name"], **{key: info[key] for key in ("variant", "grid", "warps", "stages", "smem_bytes",
                                                                        "ctas_per_sm", "chunk_bytes", "launches")})
        if c1 is not None:
            c1.update(frac_of_measured_peak=c1["per_gpu_GBps"] / peak, pct_of_nominal_8000=100.0 * c1["per_gpu_GBps"] / NOMINAL_HBM_GBS)
        line = dict(
            metric="packed_gemv_algorithmic_GBps", value=value, unit="GB/s", n_gpus=world, steps=args.steps,
            warmup=max(args.warmup, 3), ms_per_step=ms / args.steps, higher_is_better=True, scaling="weak",
            vs_baseline=None, dtype="f32", data="synthetic", config=cfg, kernel_plan=plan,
            timing="CUDA events around graph replays on the launching stream, max over ranks",
            us_per_gemv=us, pct_of_nominal_8000=100.0 * per_gpu / NOMINAL_HBM_GBS,
            pct_of_measured_copy=100.0 * per_gpu / peak,
            e2e=dict(value=ab * world / (us_e2e * 1e-6) / 1e9, unit="GB/s", us_per_gemv=us_e2e,
                     h2d_bytes_per_step=RING * passes * m * k * 2, d2h_bytes_per_step=RING * passes * m * n * 2,
                     api="pinned host x -> device, HybridPackedLinear.forward_into, result -> pinned host y, per GEMV; "
                         "copies on their own streams overlap the kernels; pass replayed from a CUDA graph"),
            e2e_serial=dict(value=ab * world / (us_ser * 1e-6) / 1e9, unit="GB/s", us_per_gemv=us_ser,
                            api="the same on one stream: copy in, GEMV, copy out, nothing overlapping"),
            gpu_launches=gemvs * info["launches"] * 3,      # device-resident leg + the two end-to-end legs
            roofline=dict(bound="hbm", achieved=per_gpu, peak=peak, unit="GB/s", frac=per_gpu / peak,
                          traffic=NCU_TRAFFIC_BYTES.get(args.workload), peak_source=f"{peak_kind} copy bandwidth",
                          algorithmic_bytes_per_launch=ab,
                          note="launch duration = event time of the timed region / GEMVs (includes inter-kernel gaps; "
                               f"{info['launches']} launch(es) per GEMV)"),
            clocks=clocks, kernel_wait_status=status, c1=c1, decode=decode,
        )
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--passes", type=int, default=PASSES, help="passes over the ring of weight sets per step")
    ap.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma", "mma_pipe"])
    ap.add_argument("--debug", type=lambda v: int(v, 0), default=0,
                    help="qgemv_problem.debug bits (tuning aids of the pipelined kernel; see include/qgemv_b200.h)")
    ap.add_argument("--prefetch-hints", action="store_true",
                    help="pass the next weight set's packed codes as the L2 prefetch hint of each GEMV (honoured by --kernel mma_pipe only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-c1", action="store_true", help="skip the INT2 configuration leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the whole-model decode legs")
    ap.add_argument("--decode-budget-s", type=float, default=420.0,
                    help="stop starting new decode legs once this much wall time has gone into them")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
