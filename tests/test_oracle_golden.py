"""The CPU oracle against fixtures produced by running the reference project's own code
(tests/golden/make_golden.py), and the C restatement against the numpy one."""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import qgemv_oracle as O
from conftest import GOLDEN, c_forward, assert_within_tolerance


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def test_linspace_matches_torch():
    for lo, hi, n in ((0.55, 1.15, 13), (0.72, 1.18, 11), (0.1, 0.9, 7)):
        assert np.array_equal(O.torch_linspace_f32(lo, hi, n), torch.linspace(lo, hi, n).numpy())


def test_pack_unpack_cases(small_cases):
    z, meta = small_cases
    for c in meta["pack_cases"]:
        nm = c["name"]
        arms = z[nm + ".arms"] if c["aware"] else None
        pw = (O.pack_int2 if c["bits"] == 2 else O.pack_int4)(z[nm + ".w"], c["group"], arms)
        assert pw.padded_k == c["padded_k"] and pw.original_k == c["original_k"]
        assert np.array_equal(pw.packed, z[nm + ".packed"]), nm
        assert np.array_equal(_bits(pw.scales), _bits(z[nm + ".scales"])), nm
        assert np.array_equal(_bits(O.dequant(pw, np.float32)), _bits(z[nm + ".deq32"])), nm
        assert np.array_equal(_bits(O.dequant(pw, np.float16)), _bits(z[nm + ".deq16"])), nm


def test_reference_linear_cases(small_cases):
    z, meta = small_cases
    for c in meta["pack_cases"]:
        nm = c["name"]
        pw = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["original_k"], c["padded_k"], c["group"])
        y16 = O.reference_forward_f16(z[nm + ".x"], pw, z[nm + ".bias"])
        ref = z[nm + ".y16"].astype(np.float32)
        # the fp16 restatement differs from torch's half GEMM by at most one fp16 rounding
        assert np.abs(y16.astype(np.float32) - ref).max() <= 2 ** -10 * max(1.0, np.abs(ref).max()), nm
        # and the reference's fp16 result sits within the path's tolerance of the fp32 target
        assert_within_tolerance(ref, O.gemv_f32(z[nm + ".x"], pw, z[nm + ".bias"]), nm)


def test_hybrid_construction_and_forward(small_cases):
    z, meta = small_cases
    for c in meta["hybrid_cases"]:
        nm = c["name"]
        arms = z[nm + ".arms"] if c["aware"] else None
        bias = z[nm + ".srcbias"] if c["bias"] else None
        h = O.build_hybrid(z[nm + ".w"], c["bits"], c["group"], arms, c["requested"], c["rank"], bias)
        assert h.outlier_idx.size == c["outliers"]
        assert np.array_equal(h.pw.packed, z[nm + ".packed"]), nm
        assert np.array_equal(_bits(h.pw.scales), _bits(z[nm + ".scales"])), nm
        assert np.array_equal(h.outlier_idx, z[nm + ".outlier_idx"]), nm
        assert np.array_equal(_bits(h.outlier_weight), _bits(z[nm + ".outlier_weight"])), nm
        ru = rv = None
        if c["rank"]:
            # SVD factors are unique only up to sign; the product is what the forward uses
            ru, rv = z[nm + ".res_u"], z[nm + ".res_v"]
            mine = h.res_u.astype(np.float32) @ h.res_v.astype(np.float32)
            theirs = ru.astype(np.float32) @ rv.astype(np.float32)
            assert np.abs(mine - theirs).max() < 1e-3, nm
        b16 = z[nm + ".bias"] if c["bias"] else None
        pw = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["k"], c["padded_k"], c["group"])
        for m in (1, 2, 3, 4, 6):
            x = z[f"{nm}.x{m}"]
            ref16 = z[f"{nm}.y{m}"].astype(np.float32)
            y16 = O.reference_forward_f16(x, pw, b16, z[nm + ".outlier_idx"], z[nm + ".outlier_weight"], ru, rv)
            assert np.abs(y16.astype(np.float32) - ref16).max() <= 2 ** -10 * max(1.0, np.abs(ref16).max()), (nm, m)
            y32 = O.gemv_f32(x, pw, b16, z[nm + ".outlier_idx"], z[nm + ".outlier_weight"], ru, rv)
            assert_within_tolerance(ref16, y32, f"{nm} m={m}")


def test_outlier_snap_table():
    snap = json.loads((GOLDEN / "snap_table.json").read_text())
    for key, want in snap.items():
        k, req = (int(v) for v in key.split(":"))
        assert O.snap_outlier_count(req, k) == want, key


def test_c_restatement_matches_numpy(small_cases, coracle):
    z, meta = small_cases
    for c in meta["hybrid_cases"]:
        nm = c["name"]
        pw = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["k"], c["padded_k"], c["group"])
        ru = z[nm + ".res_u"] if c["rank"] else None
        rv = z[nm + ".res_v"] if c["rank"] else None
        b16 = z[nm + ".bias"] if c["bias"] else None
        for m in (1, 4):
            x = z[f"{nm}.x{m}"]
            xp = np.zeros((m, c["padded_k"]), dtype=np.float16)
            xp[:, :c["k"]] = x
            for act, name in ((0, "none"), (1, "relu"), (2, "silu")):
                yc = c_forward(coracle, xp, c["bits"], pw.packed, pw.scales, c["k"], c["group"], b16,
                               z[nm + ".outlier_idx"], z[nm + ".outlier_weight"], ru, rv, act)
                yn = O.gemv_f32(x, pw, b16, z[nm + ".outlier_idx"], z[nm + ".outlier_weight"], ru, rv, name)
                assert np.abs(yc - yn).max() <= 2e-6 * max(1.0, np.abs(yn).max()), (nm, m, name)


def test_full_size_int2_digests(full_size):
    """INT2 4096x4096 g64 (the M=1 benchmark shape), seed 0: the oracle's pack is byte-identical
    to the reference's, and the reference's fp16 result is within tolerance of the oracle."""
    z, meta = full_size
    rec = meta["c1"][0]
    torch.manual_seed(rec["seed"])
    w = (torch.randn(4096, 4096) * 0.02).half()
    x = torch.randn(1, 4096).half()
    if _sha(w.numpy()) != rec["w"]:
        pytest.skip("torch's CPU random stream differs from the one the fixture was made with")
    pw = O.pack_int2(w.numpy(), 64)
    assert _sha(pw.packed) == rec["packed"]
    assert _sha(pw.scales) == rec["scales"]
    ref = O.gemv_f32(x.numpy(), pw)
    assert_within_tolerance(z["c1.s0.y16"].astype(np.float32), ref, "c1 seed 0")


def test_full_size_c_oracle(full_size, coracle):
    z, meta = full_size
    rec = meta["c1"][1]
    torch.manual_seed(rec["seed"])
    w = (torch.randn(4096, 4096) * 0.02).half()
    x = torch.randn(1, 4096).half()
    if _sha(w.numpy()) != rec["w"]:
        pytest.skip("torch's CPU random stream differs from the one the fixture was made with")
    pw = O.pack_int2(w.numpy(), 64)
    assert _sha(pw.packed) == rec["packed"] and _sha(pw.scales) == rec["scales"]
    yc = c_forward(coracle, x.numpy(), 2, pw.packed, pw.scales, 4096, 64)
    assert_within_tolerance(z["c1.s1.y16"].astype(np.float32), yc, "c1 seed 1 (C oracle)")
