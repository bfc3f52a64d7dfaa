"""Kernel micro-benchmark rows for the packed decode GEMVs.

Mirrors the hot-path rows of ``ai_accel_lab/kernel_suite.py`` (:35-100): ``torch-fp16`` (:58-59),
``decode-int2-v4`` (:63-64) and ``decode-int4-v5`` (:65-67) on the same synthetic problem
(seed 3, x ~ N(0,1) fp16, W ~ N(0,1)/sqrt(K), bias ~ N(0, 0.01)), with the reference's error
metrics against the dense result.  Timing uses CUDA events around the repetitions (the reference
uses host wall-clock); like the reference it re-runs the same buffers, so for matrices smaller
than L2 these are warm-cache latencies -- ``bench.py`` measures the cold, HBM-bound case.

    python -m ai_accel_studio_b200.kernel_suite --m 1 --n 4096 --k 4096 --group-size 64
    python -m ai_accel_studio_b200.kernel_suite --dequant          # the M > 4 path's dequantisation kernel
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


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dequant", action="store_true", help="time the dequantisation kernel instead of the decode rows")
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--group-size", type=int, default=128)
    ap.add_argument("--repeats", type=int, default=500)
    a = ap.parse_args()
    rows = run_dequant_suite(group_size=a.group_size) if a.dequant else run_kernel_suite(a.m, a.n, a.k, a.group_size, a.repeats)
    for row in rows:
        print(json.dumps(row))
