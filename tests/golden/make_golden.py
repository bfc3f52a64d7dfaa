"""Generate the golden fixtures in this directory by RUNNING the reference project's own code.

Usage (only where a checkout of the reference project is available; it is imported
read-only and nothing is copied from it):

    python tests/golden/make_golden.py --reference /path/to/ai_accel_studio

The fixtures pin the CPU oracle (oracle/qgemv_oracle.py) and the package's own
quantisers to what the reference computes on the same seeded inputs:

  small_cases.npz ....... every tensor of a set of small shapes: packed codes, scales,
                          float32 / float16 dequantised matrices, CPU forward results of
                          the reference modules (float16) and hybrid-module buffers.
  full_size.npz ......... SHA-256 digests of the reference's packed/scales tensors for the
                          two benchmark shapes (INT2 4096x4096 g64, seeds 0-4; INT4
                          11008x4096 g128 with activation-aware scales and outliers, seed 0)
                          together with the reference's float16 CPU results for them.
  snap_table.json ....... requested -> actual outlier-column count for a grid of (K, request).

The reference publishes no golden vectors of its own for this path; its tests only
assert shapes and inequalities (tests/test_groupwise_int2.py, tests/test_v4_hybrid.py,
tests/test_v5_mixedbit.py in the reference).  Those structural facts are re-asserted in
tests/test_host_logic.py.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def sha(t) -> str:
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()


def npy(t):
    return t.detach().cpu().contiguous().numpy()


def seeded_c1(seed):
    """INT2 benchmark shape: W ~ N(0, 0.02) fp16 [4096,4096], x ~ N(0,1) fp16 [1,4096]."""
    torch.manual_seed(seed)
    w = (torch.randn(4096, 4096) * 0.02).half()
    x = torch.randn(1, 4096).half()
    return w, x


def seeded_c2(seed):
    """INT4 benchmark shape with lognormal channel scales, a 256-row calibration batch,
    given rank-8 factors and a 4-row activation."""
    torch.manual_seed(seed)
    w = torch.randn(11008, 4096) * 0.02
    c = torch.exp(torch.randn(4096))
    xc = torch.randn(256, 4096) * c
    arms = xc.square().mean(0).sqrt()
    u = (torch.randn(11008, 8) * 0.01).half()
    v = (torch.randn(8, 4096) * 0.01).half()
    x = (torch.randn(4, 4096) * c).half()
    return w, arms, u, v, x


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (ai_accel_lab on its path)")
    ap.add_argument("--skip-full", action="store_true")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    torch.set_num_threads(8)
    from torch import nn
    import torch.nn.functional as F
    from ai_accel_lab.kernels import groupwise_int2 as g2, groupwise_int4 as g4
    from ai_accel_lab.kernels.decode_int2 import reference_hybrid_linear
    from ai_accel_lab.optimize.hybrid_int2 import HybridInt2Linear
    from ai_accel_lab.optimize.hybrid_int4 import HybridInt4Linear

    out = {}

    def put(name, t):
        out[name] = npy(t) if isinstance(t, torch.Tensor) else np.asarray(t)

    # ---- plain pack / unpack / reference_linear cases ----------------------------------
    pack_cases = [
        # name, bits, n, k, group, activation-aware, m, seed
        ("i2_n17_k130_g64", 2, 17, 130, 64, False, 3, 11),
        ("i2_n17_k130_g64_act", 2, 17, 130, 64, True, 2, 12),
        ("i2_n64_k256_g64", 2, 64, 256, 64, False, 1, 13),
        ("i2_n40_k512_g128_act", 2, 40, 512, 128, True, 4, 14),
        ("i2_n9_k64_g32", 2, 9, 64, 32, False, 4, 15),
        ("i2_n5_k20_g4", 2, 5, 20, 4, False, 2, 16),
        ("i4_n24_k200_g32", 4, 24, 200, 32, False, 3, 21),
        ("i4_n96_k512_g128_act", 4, 96, 512, 128, True, 4, 22),
        ("i4_n33_k256_g64", 4, 33, 256, 64, False, 1, 23),
        ("i4_n7_k30_g2", 4, 7, 30, 2, True, 2, 24),
    ]
    meta = {"pack_cases": []}
    for name, bits, n, k, g, aware, m, seed in pack_cases:
        torch.manual_seed(seed)
        w = torch.randn(n, k) * 0.05
        arms = (torch.rand(k) * 2 + 0.05) if aware else None
        x = torch.randn(m, k).half()
        bias = (torch.randn(n) * 0.01).half()
        if bits == 2:
            pw = g2.pack_groupwise_int2(w, g, arms)
            d32 = g2.unpack_groupwise_int2(pw, torch.float32)
            d16 = g2.unpack_groupwise_int2(pw, torch.float16)
            y16 = g2.reference_linear(x, pw, bias)
        else:
            pw = g4.pack_groupwise_int4(w, g, arms)
            d32 = g4.unpack_groupwise_int4(pw, torch.float32)
            d16 = g4.unpack_groupwise_int4(pw, torch.float16)
            y16 = g4.reference_linear(x, pw, bias)
        put(name + ".w", w)
        if aware:
            put(name + ".arms", arms)
        put(name + ".x", x)
        put(name + ".bias", bias)
        put(name + ".packed", pw.packed)
        put(name + ".scales", pw.scales)
        put(name + ".deq32", d32)
        put(name + ".deq16", d16)
        put(name + ".y16", y16)
        meta["pack_cases"].append(dict(name=name, bits=bits, n=n, k=k, group=g, aware=aware, m=m,
                                       padded_k=int(pw.padded_k), original_k=int(pw.original_k)))

    # ---- hybrid modules -------------------------------------------------------------------
    hyb_cases = [
        # name, bits, n, k, group, aware, requested outliers, rank, bias, seed
        ("h2_32x64_g32_o8", 2, 32, 64, 32, False, 8, 0, False, 31),       # reference test shape
        ("h2_48x256_g64_o5_r4_b", 2, 48, 256, 64, True, 5, 4, True, 32),
        ("h2_20x130_g64_o0_r2", 2, 20, 130, 64, False, 0, 2, True, 33),
        ("h4_32x64_g32_o8", 4, 32, 64, 32, False, 8, 0, False, 34),
        ("h4_56x384_g128_o11_b", 4, 56, 384, 128, True, 11, 0, True, 35),
        ("h4_19x96_g32_o0", 4, 19, 96, 32, False, 0, 0, True, 36),
    ]
    meta["hybrid_cases"] = []
    for name, bits, n, k, g, aware, oc, rank, has_bias, seed in hyb_cases:
        torch.manual_seed(seed)
        lin = nn.Linear(k, n, bias=has_bias)
        with torch.no_grad():
            lin.weight.normal_(0, 0.05)
            lin.weight[:, ::7] *= 3.0          # some heavy columns so that outlier choice is unambiguous
            if has_bias:
                lin.bias.normal_(0, 0.02)
        arms = (torch.rand(k) * 2 + 0.05) if aware else None
        if bits == 2:
            mod = HybridInt2Linear(lin, g, arms, oc, rank)
        else:
            mod = HybridInt4Linear(lin, g, arms, oc)
        put(name + ".w", lin.weight)
        if has_bias:
            put(name + ".srcbias", lin.bias)
        if aware:
            put(name + ".arms", arms)
        for b in ("packed", "scales", "outlier_idx", "outlier_weight"):
            put(name + "." + b, getattr(mod, b))
        if mod.bias is not None:
            put(name + ".bias", mod.bias)
        if bits == 2 and mod.residual_rank:
            put(name + ".res_u", mod.res_u)
            put(name + ".res_v", mod.res_v)
        for m in (1, 2, 3, 4, 6):
            x = torch.randn(m, k).half()
            with torch.no_grad():
                y = mod(x)                      # CPU tensors -> dequant + F.linear branch
            put(f"{name}.x{m}", x)
            put(f"{name}.y{m}", y)
        x3 = torch.randn(2, 2, k).half()
        with torch.no_grad():
            put(name + ".x3d", x3)
            put(name + ".y3d", mod(x3))
        meta["hybrid_cases"].append(dict(name=name, bits=bits, n=n, k=k, group=g, aware=aware, requested=oc,
                                         outliers=int(mod.outlier_idx.numel()), rank=rank, bias=has_bias,
                                         padded_k=int(mod.padded_k)))
    out["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "small_cases.npz", **out)

    # ---- outlier-count snapping -----------------------------------------------------------
    snap = {}
    for k in (3, 6, 64, 896, 4096, 4864, 8192, 11008, 14336, 28672):
        for req in (0, 1, 3, 5, 6, 7, 12, 24, 41, 48, 49, 64, 82, 143, 286, 100000):
            lin = nn.Linear(k, 2, bias=False)
            snap[f"{k}:{req}"] = int(HybridInt4Linear(lin, 2, None, req).outlier_idx.numel())
    (HERE / "snap_table.json").write_text(json.dumps(snap, indent=0, sort_keys=True))

    if args.skip_full:
        return
    # ---- full benchmark shapes: digests + reference CPU results -----------------------
    full = {}
    fmeta = {"c1": [], "c2": []}
    for seed in range(5):
        w, x = seeded_c1(seed)
        pw = g2.pack_groupwise_int2(w, 64)
        y16 = g2.reference_linear(x, pw)
        y32 = x.float() @ g2.unpack_groupwise_int2(pw, torch.float32).double().float().t()
        full[f"c1.s{seed}.y16"] = npy(y16)
        full[f"c1.s{seed}.y32"] = npy(y32)
        fmeta["c1"].append(dict(seed=seed, w=sha(w), x=sha(x), packed=sha(pw.packed), scales=sha(pw.scales)))
        print("c1 seed", seed, "done", flush=True)
    for seed in (0,):
        w, arms, u, v, x = seeded_c2(seed)
        lin = nn.Linear(4096, 11008, bias=False)
        with torch.no_grad():
            lin.weight.copy_(w)
        mod = HybridInt4Linear(lin, 128, arms, outlier_columns=41)
        with torch.no_grad():
            y16 = mod(x)                                                     # stock module: no residual
            y16r = y16 + F.linear(F.linear(x, v), u).to(y16.dtype)           # + residual, INT2 module's formula
        full[f"c2.s{seed}.y16"] = npy(y16)
        full[f"c2.s{seed}.y16_res"] = npy(y16r)
        full[f"c2.s{seed}.outlier_idx"] = npy(mod.outlier_idx)
        fmeta["c2"].append(dict(seed=seed, w=sha(w), x=sha(x), arms=sha(arms), u=sha(u), v=sha(v),
                                packed=sha(mod.packed), scales=sha(mod.scales),
                                outlier_idx=sha(mod.outlier_idx), outlier_weight=sha(mod.outlier_weight),
                                outliers=int(mod.outlier_idx.numel())))
        print("c2 seed", seed, "done", flush=True)
    full["meta"] = np.frombuffer(json.dumps(fmeta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "full_size.npz", **full)


if __name__ == "__main__":
    main()
