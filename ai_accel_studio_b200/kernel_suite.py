"""Kernel micro-benchmark rows for the packed decode GEMVs.

Mirrors the hot-path rows of ``ai_accel_lab/kernel_suite.py`` (:35-100): ``torch-fp16`` (:58-59),
``decode-int2-v4`` (:63-64) and ``decode-int4-v5`` (:65-67) on the same synthetic problem
(seed 3, x ~ N(0,1) fp16, W ~ N(0,1)/sqrt(K), bias ~ N(0, 0.01)), with the reference's error
metrics against the dense result.  Timing uses CUDA events around the repetitions (the reference
uses host wall-clock); like the reference it re-runs the same buffers, so for matrices smaller
than L2 these are warm-cache latencies -- ``bench.py`` measures the cold, HBM-bound case.

    python -m ai_accel_studio_b200.kernel_suite --m 1 --n 4096 --k 4096 --group-size 64
    python -m ai_accel_studio_b200.kernel_suite --dequant          # the M > 4 path's dequantisation kernel
    python -m ai_accel_studio_b200.kernel_suite --sweep            # cold-cache size sweep, 4.7 - 117 MB of weights
"""
from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F

from .kernels.decode_int2 import decode_int2_linear
from .kernels.groupwise_int2 import pack_groupwise_int2
from .kernels.groupwise_int4 import decode_int4_linear, pack_groupwise_int4


def _metrics(ref, y):
    ref, y = ref.float(), y.float()
    err = y - ref
    return dict(mse_vs_dense=float(err.square().mean()), mae_vs_dense=float(err.abs().mean()),
                nmse_vs_dense=float(err.square().sum() / ref.square().sum().clamp_min(1e-12)),
                cosine_vs_dense=float(F.cosine_similarity(y.reshape(1, -1), ref.reshape(1, -1)).item()))


def _bench(fn, repeats=100, warmup=10):
    for _ in range(warmup):
        y = fn()
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(repeats):
        y = fn()
    en.record()
    en.synchronize()
    return y, float(st.elapsed_time(en)) / repeats


def run_kernel_suite(m=1, n=4096, k=4096, group_size=128, repeats=100, methods=None):
    if not torch.cuda.is_available():
        raise RuntimeError("the kernel suite requires an NVIDIA CUDA GPU")
    if m > 4:
        raise ValueError("the packed decode rows are defined for M <= 4")
    methods = methods or ["torch-fp16", "decode-int2-v4", "decode-int4-v5"]
    torch.manual_seed(3)
    x = torch.randn(m, k, device="cuda", dtype=torch.float16)
    w = torch.randn(n, k, device="cuda", dtype=torch.float16) / (k ** 0.5)
    b = torch.randn(n, device="cuda", dtype=torch.float16) * 0.01
    ref = F.linear(x, w, b)
    rows = []

    def add(name, fn, weight_bytes, note=""):
        y, ms = _bench(fn, repeats)
        rows.append(dict(method=name, latency_ms=ms, speedup=None, weight_mb=weight_bytes / 1024 ** 2, note=note,
                         **_metrics(ref, y)))

    if "torch-fp16" in methods:
        add("torch-fp16", lambda: F.linear(x, w, b), w.numel() * 2)
    if "decode-int2-v4" in methods:
        pw = pack_groupwise_int2(w, group_size)
        add("decode-int2-v4", lambda: decode_int2_linear(x, pw, b), pw.packed.numel() + pw.scales.numel() * 2,
            "M<=4 packed INT2 decode GEMV (sm_100a)")
    if "decode-int4-v5" in methods:
        p4 = pack_groupwise_int4(w, group_size)
        add("decode-int4-v5", lambda: decode_int4_linear(x, p4, b), p4.packed.numel() + p4.scales.numel() * 2,
            "M<=4 packed INT4 decode GEMV (sm_100a)")
    base = next((r["latency_ms"] for r in rows if r["method"] == "torch-fp16"), None)
    if base:
        for r in rows:
            r["speedup"] = base / r["latency_ms"]
    return rows


def run_dequant_suite(shapes=((11008, 4096), (4096, 14336), (28672, 8192)), group_size=128, repeats=20):
    """Microseconds and GB/s (packed bytes read + dense bytes written) of the dequantisation kernel that
    feeds the M > 4 path, per bit width and output type.  Four output buffers are written in turn, so
    the destination is never L2-resident."""
    from . import ops
    if not torch.cuda.is_available():
        raise RuntimeError("the dequantisation suite requires an NVIDIA CUDA GPU")
    rows = []
    for n, k in shapes:
        for bits in (2, 4):
            packed = torch.randint(0, 256, (4, n, k * bits // 8), dtype=torch.uint8, device="cuda")
            scales = (torch.rand((4, n, k // group_size), device="cuda") * 0.01 + 0.002).half()
            for name in ("float16", "float32"):
                def once(i):
                    return ops.dequant(packed[i % 4], scales[i % 4], bits, group_size, k, name)
                for i in range(4):
                    once(i)
                torch.cuda.synchronize()
                st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                st.record()
                for i in range(repeats):
                    once(i)
                en.record()
                en.synchronize()
                us = float(st.elapsed_time(en)) * 1e3 / repeats
                moved = n * k * bits // 8 + n * (k // group_size) * 2 + n * k * (2 if name == "float16" else 4)
                rows.append(dict(kernel="dequant", bits=bits, n=n, k=k, out=name, us=us, bytes=moved, GBps=moved / us / 1e3))
    return rows


SWEEP_SHAPES = (
    # bits, m, n, k, group, outlier columns, residual rank: decoder Linear shapes from 4.7 to 117 MB of weights
    (2, 1, 4096, 4096, 64, 0, 0), (2, 1, 1024, 4096, 128, 32, 8), (2, 1, 4096, 4096, 128, 32, 8), (4, 1, 4096, 4096, 128, 32, 8),
    (2, 1, 14336, 4096, 128, 32, 8), (4, 4, 11008, 4096, 128, 32, 8), (4, 1, 14336, 4096, 128, 32, 8), (2, 1, 4096, 14336, 128, 64, 8),
    (4, 1, 4096, 14336, 128, 64, 8), (2, 1, 28672, 8192, 128, 64, 8), (4, 1, 28672, 8192, 128, 64, 8), (4, 1, 8192, 28672, 128, 64, 8),
)


def algorithmic_bytes(bits, m, n, k, group, oc, rank, bias=False) -> int:
    """Every operand of one fused GEMV counted once."""
    b = n * k * bits // 8 + n * (k // group) * 2 + m * k * 2 + m * n * 2
    if oc:
        b += n * oc * 2 + oc * 4
    if rank:
        b += n * rank * 2 + rank * k * 2
    return b + (n * 2 if bias else 0)


def run_size_sweep(shapes=SWEEP_SHAPES, kernel="auto", peak_gbs=6532.2, ring_bytes=320 << 20, replays=20):
    """Cold-cache microseconds per fused GEMV over decoder Linear shapes of growing size: for every
    shape a ring of distinct weight sets larger than 2 x L2 is run back to back from one CUDA graph
    (the protocol of bench.py), so every launch streams its weights from HBM.  Random codes and scales:
    timing only.  ``frac`` = algorithmic bytes / time / ``peak_gbs`` (the measured copy bandwidth)."""
    from . import _cabi, ops
    if not torch.cuda.is_available():
        raise RuntimeError("the size sweep requires an NVIDIA CUDA GPU")
    rows, kern = [], _cabi.KERNEL[kernel]
    g = torch.Generator(device="cuda").manual_seed(0)
    for bits, m, n, k, group, oc, rank in shapes:
        alg = algorithmic_bytes(bits, m, n, k, group, oc, rank)
        ring = max(4, min(64, -(-ring_bytes // alg)))
        sets = []
        for _ in range(ring):
            sets.append(dict(
                packed=torch.randint(0, 256, (n, k * bits // 8), dtype=torch.uint8, device="cuda", generator=g),
                scales=(torch.rand((n, k // group), device="cuda", generator=g) * 0.01 + 0.002).half(),
                oidx=torch.randperm(k, device="cuda", generator=g)[:oc].to(torch.int32) if oc else None,
                ow=(torch.randn((n, oc), device="cuda", generator=g) * 0.02).half() if oc else None,
                ru=(torch.randn((n, rank), device="cuda", generator=g) * 0.02).half() if rank else None,
                rv=(torch.randn((rank, k), device="cuda", generator=g) * 0.02).half() if rank else None))
        x = torch.randn((m, k), device="cuda", generator=g).half()

        def one_pass():
            out = None
            for w in sets:
                out = ops.gemv(x, w["packed"], w["scales"], None, w["oidx"], w["ow"], w["ru"], w["rv"], bits, group, k, 0, kern)
            return out
        w0 = sets[0]
        try:
            plan = ops.plan_describe(x, w0["packed"], w0["scales"], bits, group, k, w0["oidx"], w0["ow"], w0["ru"], w0["rv"], kernel=kern)
        except _cabi.QgemvError as e:          # a forced kernel this shape cannot use
            rows.append(dict(bits=bits, m=m, n=n, k=k, group=group, outliers=oc, rank=rank, weight_mb=alg / 1e6, skipped=str(e)))
            del sets
            torch.cuda.empty_cache()
            continue
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                one_pass()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        st.record()
        for _ in range(replays):
            graph.replay()
        en.record()
        en.synchronize()
        us = float(st.elapsed_time(en)) * 1e3 / (replays * ring)
        rows.append(dict(bits=bits, m=m, n=n, k=k, group=group, outliers=oc, rank=rank, weight_mb=alg / 1e6, ring=ring,
                         us_per_gemv=us, GBps=alg / us / 1e3, frac_of_measured_peak=alg / us / 1e3 / peak_gbs,
                         kernel=plan.get("name"), grid=plan.get("grid"), tile_aligned=plan.get("tile_aligned")))
        del sets, graph
        torch.cuda.empty_cache()
    return rows


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dequant", action="store_true", help="time the dequantisation kernel instead of the decode rows")
    ap.add_argument("--sweep", action="store_true", help="cold-cache size sweep over decoder Linear shapes (4.7 - 117 MB of weights)")
    ap.add_argument("--kernel", default="auto", choices=["auto", "simt", "mma", "mma_pipe"])
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--repeats", type=int, default=500)
    a = ap.parse_args()
    if a.sweep:
        rows = run_size_sweep(kernel=a.kernel)
    elif a.dequant:
        rows = run_dequant_suite(group_size=a.group_size)
    else:
        rows = run_kernel_suite(a.m, a.n, a.k, a.group_size, a.repeats)
    for row in rows:
        print(json.dumps(row))
