"""Parity of the fused GEMV (through the C ABI) with the CPU oracle and the reference fixtures."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import qgemv_oracle as O
from conftest import c_forward, assert_within_tolerance
from ai_accel_studio_b200 import _cabi, ops
from ai_accel_studio_b200.kernels.groupwise_int2 import GroupwiseInt2Weight, pack_groupwise_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import GroupwiseInt4Weight, pack_groupwise_int4, decode_int4_linear
from ai_accel_studio_b200.kernels.decode_int2 import decode_int2_linear

pytestmark = pytest.mark.gpu

KERNELS = ("simt", "auto", "mma_pipe")     # CUDA-core kernel, planner's choice, barrier-free tensor-core kernel


def _dev(pw):
    return type(pw)(pw.packed.cuda(), pw.scales.cuda(), pw.original_k, pw.padded_k, pw.group_size)


def _run(bits, x, pw, **kw):
    fn = decode_int2_linear if bits == 2 else decode_int4_linear
    if kw.get("kernel") == "mma_pipe":
        # shapes outside the tensor-core family (odd groups, unaligned rows) or whose balance needs shared
        # tiles have no barrier-free variant
        try:
            return fn(x, pw, **kw)
        except _cabi.QgemvError as e:
            if e.code != -2:
                raise
            kw = dict(kw, kernel="auto")
    return fn(x, pw, **kw)


def _pad(x, kp):
    return x if x.shape[1] == kp else torch.nn.functional.pad(x, (0, kp - x.shape[1]))


def test_reference_fixture_cases(small_cases):
    z, meta = small_cases
    for c in meta["pack_cases"]:
        nm = c["name"]
        cls = GroupwiseInt2Weight if c["bits"] == 2 else GroupwiseInt4Weight
        pw = cls(torch.from_numpy(z[nm + ".packed"]).cuda(), torch.from_numpy(z[nm + ".scales"]).cuda(),
                 c["original_k"], c["padded_k"], c["group"])
        host = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["original_k"], c["padded_k"], c["group"])
        x = torch.from_numpy(z[nm + ".x"])
        bias = torch.from_numpy(z[nm + ".bias"])
        ref = O.gemv_f32(x.numpy(), host, bias.numpy())
        for kern in KERNELS:
            y = _run(c["bits"], _pad(x, c["padded_k"]).cuda(), pw, bias=bias.cuda(), kernel=kern)
            assert y.dtype == torch.float16 and tuple(y.shape) == (c["m"], c["n"])
            assert_within_tolerance(y.float().cpu().numpy(), ref, f"{nm}/{kern}")
            # the reference's own fp16 CPU result is a looser witness: agree to fp16 rounding of both
            assert np.abs(y.float().cpu().numpy() - z[nm + ".y16"].astype(np.float32)).max() < 5e-3, nm


def test_hybrid_fixture_cases(small_cases):
    z, meta = small_cases
    for c in meta["hybrid_cases"]:
        nm = c["name"]
        cls = GroupwiseInt2Weight if c["bits"] == 2 else GroupwiseInt4Weight
        pw = cls(torch.from_numpy(z[nm + ".packed"]).cuda(), torch.from_numpy(z[nm + ".scales"]).cuda(),
                 c["k"], c["padded_k"], c["group"])
        host = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["k"], c["padded_k"], c["group"])
        kw_h = dict(bias=z[nm + ".bias"] if c["bias"] else None, outlier_idx=z[nm + ".outlier_idx"],
                    outlier_weight=z[nm + ".outlier_weight"],
                    res_u=z[nm + ".res_u"] if c["rank"] else None, res_v=z[nm + ".res_v"] if c["rank"] else None)
        kw_d = {k: (None if v is None else torch.from_numpy(v).cuda()) for k, v in kw_h.items()}
        for m in (1, 2, 3, 4):
            x = torch.from_numpy(z[f"{nm}.x{m}"])
            ref = O.gemv_f32(x.numpy(), host, **kw_h)
            for kern in KERNELS:
                y = _run(c["bits"], _pad(x, c["padded_k"]).cuda(), pw, kernel=kern, **kw_d)
                assert_within_tolerance(y.float().cpu().numpy(), ref, f"{nm} m={m} {kern}")
                assert np.abs(y.float().cpu().numpy() - z[f"{nm}.y{m}"].astype(np.float32)).max() < 8e-3, (nm, m)


GRID = [
    # bits, n, k, group, oc, rank, bias
    (2, 128, 256, 64, 0, 0, False),
    (2, 130, 512, 128, 4, 0, True),
    (2, 17, 130, 64, 3, 2, True),        # odd N, padded K, odd outlier count
    (2, 64, 64, 32, 8, 0, False),        # group 32: 8-byte groups
    (2, 33, 40, 4, 0, 0, True),          # tiny groups: byte-wise path
    (2, 1, 4096, 4096, 0, 0, False),     # one group per row = per-output-channel scale
    (2, 300, 1792, 128, 41, 8, True),
    (2, 96, 8192, 128, 64, 8, False),
    (4, 128, 256, 128, 0, 0, False),
    (4, 77, 384, 64, 5, 0, True),
    (4, 24, 200, 32, 8, 3, True),
    (4, 19, 30, 2, 0, 0, False),
    (4, 260, 2048, 128, 41, 8, True),
    (4, 48, 14336, 128, 64, 8, False),
    (4, 512, 896, 128, 8, 8, True),
]


@pytest.mark.parametrize("bits,n,k,group,oc,rank,has_bias", GRID)
def test_grid_against_oracle(bits, n, k, group, oc, rank, has_bias, coracle):
    g = torch.Generator().manual_seed(n * 7 + k)
    w = torch.randn(n, k, generator=g) * 0.05
    pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, group)
    dev = _dev(pw)
    bias = (torch.randn(n, generator=g) * 0.1).half() if has_bias else None
    oidx = torch.randperm(k, generator=g)[:oc].to(torch.int32) if oc else None
    ow = (torch.randn(n, oc, generator=g) * 0.05).half() if oc else None
    ru = (torch.randn(n, rank, generator=g) * 0.05).half() if rank else None
    rv = (torch.randn(rank, k, generator=g) * 0.05).half() if rank else None
    np_ = lambda t: None if t is None else t.numpy()
    cu = lambda t: None if t is None else t.cuda()
    for m in (1, 2, 3, 4):
        x = torch.randn(m, k, generator=g).half()
        xp = _pad(x, pw.padded_k)
        ref = c_forward(coracle, xp.numpy(), bits, pw.packed.numpy(), pw.scales.numpy(), k, group,
                        np_(bias), np_(oidx), np_(ow), np_(ru), np_(rv))
        for kern in KERNELS:
            y = _run(bits, xp.cuda(), dev, bias=cu(bias), outlier_idx=cu(oidx), outlier_weight=cu(ow),
                     res_u=cu(ru), res_v=cu(rv), kernel=kern)
            assert_within_tolerance(y.float().cpu().numpy(), ref, f"m={m} {kern}")


@pytest.mark.parametrize("bits", [2, 4])
def test_bf16_activations_and_strided_x(bits, coracle):
    g = torch.Generator().manual_seed(91 + bits)
    n, k, group = 200, 1024, 128
    w = torch.randn(n, k, generator=g) * 0.05
    pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, group)
    dev = _dev(pw)
    big = torch.randn(4, 3 * k, generator=g).bfloat16()
    x = big[:, k:2 * k]                                    # row stride 3k, unit inner stride
    ref = c_forward(coracle, x.contiguous().view(torch.int16).numpy().view(np.uint16), bits, pw.packed.numpy(),
                    pw.scales.numpy(), k, group, x_is_bf16=True)
    for kern in KERNELS:
        y = _run(bits, big.cuda()[:, k:2 * k], dev, kernel=kern)
        assert y.dtype == torch.bfloat16
        # bf16 output rounding (2^-9 relative) dominates: compare with a matching bound
        yf, r = y.float().cpu().numpy(), ref
        assert np.abs(yf - r).max() <= 1e-2 + 4e-3 * np.abs(r).max()
        assert np.linalg.norm(yf - r) <= 4e-3 * np.linalg.norm(r)


def test_activations(coracle):
    g = torch.Generator().manual_seed(5)
    w = torch.randn(96, 512, generator=g) * 0.05
    pw = pack_groupwise_int2(w, 64)
    x = torch.randn(2, 512, generator=g).half()
    for name, code in (("relu", 1), ("silu", 2), ("swish", 2)):
        ref = c_forward(coracle, x.numpy(), 2, pw.packed.numpy(), pw.scales.numpy(), 512, 64, act=code)
        for kern in KERNELS:
            y = decode_int2_linear(x.cuda(), _dev(pw), activation=name, kernel=kern)
            assert_within_tolerance(y.float().cpu().numpy(), ref, name)
    with pytest.raises(ValueError):
        decode_int2_linear(x.cuda(), _dev(pw), activation="gelu")


def test_lognormal_channel_scales(coracle):
    """Heavy-tailed activations as in the INT4 benchmark configuration (|x| reaches 50+)."""
    g = torch.Generator().manual_seed(77)
    n, k = 512, 4096
    w = torch.randn(n, k, generator=g) * 0.02
    c = torch.exp(torch.randn(k, generator=g))
    for bits, pack in ((2, pack_groupwise_int2), (4, pack_groupwise_int4)):
        pw = pack(w, 128)
        x = (torch.randn(4, k, generator=g) * c).half()
        ref = c_forward(coracle, x.numpy(), bits, pw.packed.numpy(), pw.scales.numpy(), k, 128)
        for kern in KERNELS:
            y = _run(bits, x.cuda(), _dev(pw), kernel=kern)
            assert_within_tolerance(y.float().cpu().numpy(), ref, f"bits={bits} {kern}")


def test_extreme_activation_magnitudes(coracle):
    """Very large and very small activations: the result must not depend on the scale of x."""
    g = torch.Generator().manual_seed(3)
    n, k = 256, 1024
    w = torch.randn(n, k, generator=g) * 0.05
    for bits, pack in ((2, pack_groupwise_int2), (4, pack_groupwise_int4)):
        pw = pack(w, 128)
        base = torch.randn(2, k, generator=g)
        for scale in (2000.0, 1.0, 2e-4):
            x = (base * scale).half()
            ref = c_forward(coracle, x.numpy(), bits, pw.packed.numpy(), pw.scales.numpy(), k, 128)
            for kern in KERNELS:
                y = _run(bits, x.cuda(), _dev(pw), kernel=kern).float().cpu().numpy()
                if not np.isfinite(ref).all() or np.abs(ref).max() > 6e4:
                    continue
                s = max(np.abs(ref).max(), 1e-30)
                assert np.abs(y - ref).max() <= 2e-3 * s, (bits, scale, kern)
                assert np.linalg.norm(y - ref) <= 1e-3 * np.linalg.norm(ref), (bits, scale, kern)


def test_full_size_int2_benchmark_shape_all_seeds(full_size, coracle):
    """INT2 4096x4096 g64 M=1, seeds 0-4: GPU result vs the C oracle, vs the reference's fp32-accumulate
    result and vs its fp16 CPU result (fixtures made by running the reference)."""
    import hashlib
    z, meta = full_size
    sha = lambda t: hashlib.sha256(t.numpy().tobytes()).hexdigest()
    for seed in range(5):
        rec = meta["c1"][seed]
        torch.manual_seed(seed)
        w = (torch.randn(4096, 4096) * 0.02).half()
        x = torch.randn(1, 4096).half()
        pw = pack_groupwise_int2(w, 64)
        same_stream = sha(w) == rec["w"] and sha(x) == rec["x"]
        if same_stream:
            assert sha(pw.packed) == rec["packed"] and sha(pw.scales) == rec["scales"]
        ref = c_forward(coracle, x.numpy(), 2, pw.packed.numpy(), pw.scales.numpy(), 4096, 64)
        for kern in KERNELS:
            y = decode_int2_linear(x.cuda(), _dev(pw), kernel=kern).float().cpu().numpy()
            assert_within_tolerance(y, ref, f"int2 4096x4096 seed {seed} {kern}")
            if same_stream:
                assert_within_tolerance(y, z[f"c1.s{seed}.y32"], f"seed {seed} {kern} vs the reference's fp32 result")
                assert np.abs(y - z[f"c1.s{seed}.y16"].astype(np.float32)).max() < 8e-3


def test_full_size_int4_benchmark_configuration(full_size, coracle):
    """The INT4 benchmark configuration exactly as specified: 11008x4096, group 128, activation-aware
    scales from a 256-row calibration batch with lognormal channel scales, 41 requested outlier
    columns (the constructor keeps 32), given rank-8 factors, M=4 heavy-tailed activations.  The
    module must pick the reference's outlier columns and pack the reference's bytes; the fused GEMV
    must match the oracle and the reference's own fp16 CPU results."""
    import hashlib
    from torch import nn
    from ai_accel_studio_b200.optimize import HybridInt4Linear
    z, meta = full_size
    sha = lambda t: hashlib.sha256(t.detach().cpu().contiguous().numpy().tobytes()).hexdigest()
    rec = meta["c2"][0]
    torch.manual_seed(0)
    w = torch.randn(11008, 4096) * 0.02
    c = torch.exp(torch.randn(4096))
    xc = torch.randn(256, 4096) * c
    arms = xc.square().mean(0).sqrt()
    u = (torch.randn(11008, 8) * 0.01).half()
    v = (torch.randn(8, 4096) * 0.01).half()
    x = (torch.randn(4, 4096) * c).half()
    same_stream = sha(w) == rec["w"] and sha(x) == rec["x"] and sha(arms) == rec["arms"]
    lin = nn.Linear(4096, 11008, bias=False)
    with torch.no_grad():
        lin.weight.copy_(w)
    plain = HybridInt4Linear(lin, 128, arms, 41)
    assert plain.outlier_idx.numel() == 32 == rec["outliers"]
    if same_stream:
        assert np.array_equal(plain.outlier_idx.numpy(), z["c2.s0.outlier_idx"])
        assert sha(plain.packed) == rec["packed"] and sha(plain.scales) == rec["scales"]
        assert sha(plain.outlier_weight) == rec["outlier_weight"]
    withres = HybridInt4Linear.from_buffers(plain.packed, plain.scales, 4096, 128, plain.outlier_idx, plain.outlier_weight,
                                            None, u, v)
    host = dict(packed=plain.packed.numpy(), scales=plain.scales.numpy(), oidx=plain.outlier_idx.numpy(),
                ow=plain.outlier_weight.numpy())
    ref_plain = c_forward(coracle, x.numpy(), 4, host["packed"], host["scales"], 4096, 128, None, host["oidx"], host["ow"])
    ref_res = c_forward(coracle, x.numpy(), 4, host["packed"], host["scales"], 4096, 128, None, host["oidx"], host["ow"],
                        u.numpy(), v.numpy())
    plain, withres = plain.cuda(), withres.cuda()
    for kern in KERNELS:
        plain.kernel = withres.kernel = kern
        y0 = plain(x.cuda()).float().cpu().numpy()
        y1 = withres(x.cuda()).float().cpu().numpy()
        assert_within_tolerance(y0, ref_plain, f"int4 11008x4096 without residual, {kern}")
        assert_within_tolerance(y1, ref_res, f"int4 11008x4096 with residual, {kern}")
        if same_stream:
            # the reference's fp16 CPU results round every term to fp16: agree to a few fp16 ulps of the largest output
            tol = 4 * 2.0 ** -11 * float(np.abs(ref_res).max()) + 1e-2
            assert np.abs(y0 - z["c2.s0.y16"].astype(np.float32)).max() < tol
            assert np.abs(y1 - z["c2.s0.y16_res"].astype(np.float32)).max() < tol


def test_linearity_and_repeatability():
    """Size-independent properties at a model-sized shape: y(a*x) == a*y(x) for a power of two,
    and two launches give bit-identical results (fixed reduction order)."""
    g = torch.Generator().manual_seed(9)
    w = torch.randn(1024, 14336, generator=g) * 0.02
    for bits, pack in ((2, pack_groupwise_int2), (4, pack_groupwise_int4)):
        dev = _dev(pack(w, 128))
        x = torch.randn(3, 14336, generator=g).half().cuda()
        for kern in KERNELS:
            y1 = _run(bits, x, dev, kernel=kern)
            y2 = _run(bits, x, dev, kernel=kern)
            assert torch.equal(y1, y2)
            y4 = _run(bits, x * 4, dev, kernel=kern)
            assert torch.equal(y4, y1 * 4)


def test_argument_errors():
    pw = _dev(pack_groupwise_int2(torch.randn(32, 128), 64))
    x = torch.randn(1, 128).half().cuda()
    with pytest.raises(ValueError):
        decode_int2_linear(torch.randn(5, 128).half().cuda(), pw)       # M > 4
    with pytest.raises(ValueError):
        decode_int2_linear(torch.randn(1, 100).half().cuda(), pw)       # not padded
    with pytest.raises(RuntimeError):
        decode_int2_linear(x.float(), pw)                               # dtype
    with pytest.raises(ValueError):
        decode_int2_linear(x[0], pw)                                    # ndim


def test_direct_c_abi_call_and_plan_name():
    """Raw pointers through ctypes, the way a non-torch host would call the library."""
    w = torch.randn(64, 256) * 0.05
    pw = pack_groupwise_int4(w, 64)
    packed, scales = pw.packed.cuda(), pw.scales.cuda()
    x = torch.randn(2, 256).half().cuda()
    y = torch.zeros(2, 64, dtype=torch.float16, device="cuda")
    ws = torch.zeros(_cabi.workspace_bytes(4, 2, 64, 256, 64, 0), dtype=torch.uint8, device="cuda")
    p = _cabi.Problem()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = 4, 2, 64, 256, 256, 64
    p.x, p.ldx, p.packed, p.ldp, p.scales, p.lds = x.data_ptr(), 256, packed.data_ptr(), 128, scales.data_ptr(), 4
    p.y, p.ldy, p.workspace, p.workspace_bytes = y.data_ptr(), 64, ws.data_ptr(), ws.numel()
    assert _cabi.plan_name(p) is not None
    stream = torch.cuda.current_stream().cuda_stream
    assert _cabi.lib().qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0
    torch.cuda.synchronize()
    host = O.PackedWeight(4, pw.packed.numpy(), pw.scales.numpy(), 256, 256, 64)
    assert_within_tolerance(y.float().cpu().numpy(), O.gemv_f32(x.cpu().numpy(), host), "direct C ABI")
    assert not ws[1024:1024 + 4 * 16384].any()            # scratch invariant: arrival counters back to zero
    p.kernel = _cabi.KERNEL["simt"]
    assert _cabi.plan_name(p).startswith("simt_int4")


def test_reference_selftest_probes_pass():
    """The hot-path probes of the reference's self test (its inputs, its comparison, its thresholds)."""
    from ai_accel_studio_b200.selftest import run_selftest
    torch.manual_seed(0)
    report = run_selftest()
    assert report["ok"], report
    by = {p["name"]: p for p in report["probes"]}
    assert by["decode-int2-v4"]["max_abs_error"] < 0.5 and by["decode-int4-v5"]["max_abs_error"] < 0.35
    assert by["decode-int2-v4"]["cosine"] > 0.999 and by["decode-int4-v5"]["cosine"] > 0.999 and by["cuda-graph"]["ok"]
