"""CPU-side checks: the package's quantisers and modules against the reference-made fixtures,
the structural facts the reference's own tests assert, error behaviour, and that the C-ABI
library loads and exports everything the header declares (no kernel is launched here)."""
import ctypes
import hashlib
import re

import numpy as np
import pytest
import torch
from torch import nn

from conftest import ROOT
from ai_accel_studio_b200 import _cabi, build as build_mod
from ai_accel_studio_b200.kernels.groupwise_int2 import GroupwiseInt2Weight, pack_groupwise_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import pack_groupwise_int4
from ai_accel_studio_b200.kernels.decode_int2 import decode_int2_linear
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.optimize._hybrid_base import snap_outlier_count


def _sha(t):
    return hashlib.sha256(np.ascontiguousarray(t.numpy() if isinstance(t, torch.Tensor) else t).tobytes()).hexdigest()


def test_pack_matches_reference_fixtures(small_cases):
    z, meta = small_cases
    for c in meta["pack_cases"]:
        nm = c["name"]
        arms = torch.from_numpy(z[nm + ".arms"]) if c["aware"] else None
        pack = pack_groupwise_int2 if c["bits"] == 2 else pack_groupwise_int4
        pw = pack(torch.from_numpy(z[nm + ".w"]), c["group"], arms)
        assert (pw.padded_k, pw.original_k, pw.group_size) == (c["padded_k"], c["original_k"], c["group"])
        assert pw.activation_aware == c["aware"]
        assert np.array_equal(pw.packed.numpy(), z[nm + ".packed"]), nm
        assert np.array_equal(pw.scales.numpy().view(np.uint16), z[nm + ".scales"].view(np.uint16)), nm


def test_pack_is_chunk_invariant(monkeypatch):
    from ai_accel_studio_b200.kernels import groupwise_int2 as g2, groupwise_int4 as g4
    torch.manual_seed(5)
    w = torch.randn(37, 256) * 0.1
    arms = torch.rand(256) + 0.1
    a2, a4 = g2.pack_groupwise_int2(w, 64, arms), g4.pack_groupwise_int4(w, 64, arms)
    monkeypatch.setattr(g2, "_ROW_CHUNK_ELEMS", 256 * 5)
    monkeypatch.setattr(g4, "_ROW_CHUNK_ELEMS", 256 * 3)
    b2, b4 = g2.pack_groupwise_int2(w, 64, arms), g4.pack_groupwise_int4(w, 64, arms)
    assert torch.equal(a2.packed, b2.packed) and torch.equal(a2.scales, b2.scales)
    assert torch.equal(a4.packed, b4.packed) and torch.equal(a4.scales, b4.scales)


def test_structure_facts_of_the_reference_tests():
    # N=17, K=130, group 64 -> padded 192, packed (17,48), scales (17,3)
    pw = pack_groupwise_int2(torch.randn(17, 130), 64)
    assert pw.padded_k == 192 and tuple(pw.packed.shape) == (17, 48) and tuple(pw.scales.shape) == (17, 3)
    assert pw.packed.dtype == torch.uint8 and pw.scales.dtype == torch.float16
    assert torch.isfinite(pw.scales.float()).all()
    assert pack_groupwise_int2(torch.randn(17, 130), 64, torch.rand(130) + 0.1).activation_aware
    # HybridInt2Linear(64 -> 32, group 32, 8 outliers): 8 outlier columns, no dense [N,K] tensor kept, smaller than fp16
    mod = HybridInt2Linear(nn.Linear(64, 32), 32, None, 8)
    assert mod.outlier_idx.numel() == 8 and mod.outlier_idx.dtype == torch.int32
    assert not any(tuple(t.shape) == (32, 64) for t in list(mod.parameters()) + list(mod.buffers()))
    info = mod.optimization_info()
    assert info.optimized_bytes < info.original_bytes and info.method == "hybrid-int2"
    # INT4 round trip error (host dequantisation) below 0.1 ||w||^2
    w = torch.randn(48, 256)
    p4 = pack_groupwise_int4(w, 64)
    codes = torch.stack([p4.packed & 15, p4.packed >> 4], -1).reshape(48, -1).to(torch.int16)
    deq = (codes - 8).float() * p4.scales.float().repeat_interleave(64, 1)
    assert (deq - w).square().mean() < 0.1 * w.square().mean()
    with pytest.raises(ValueError):
        pack_groupwise_int2(torch.randn(4, 8), 6)
    with pytest.raises(ValueError):
        pack_groupwise_int4(torch.randn(4, 8), 3)
    with pytest.raises(ValueError):
        pack_groupwise_int2(torch.randn(4, 64), 32, torch.rand(10))


def test_modules_match_reference_fixtures(small_cases):
    z, meta = small_cases
    for c in meta["hybrid_cases"]:
        nm = c["name"]
        lin = nn.Linear(c["k"], c["n"], bias=c["bias"])
        with torch.no_grad():
            lin.weight.copy_(torch.from_numpy(z[nm + ".w"]))
            if c["bias"]:
                lin.bias.copy_(torch.from_numpy(z[nm + ".srcbias"]))
        arms = torch.from_numpy(z[nm + ".arms"]) if c["aware"] else None
        if c["bits"] == 2:
            mod = HybridInt2Linear(lin, c["group"], arms, c["requested"], c["rank"])
        else:
            mod = HybridInt4Linear(lin, c["group"], arms, c["requested"])
        want = {"packed", "scales", "outlier_idx", "outlier_weight"}
        if c["bias"]:
            want.add("bias")
        if c["rank"]:
            want |= {"res_u", "res_v"}
        sd = mod.state_dict()
        assert set(sd) == want, nm
        for key in want:
            got, ref = sd[key].numpy(), z[f"{nm}.{key}"]
            assert got.dtype == ref.dtype and got.shape == ref.shape, (nm, key)
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), (nm, key)
        assert (mod.in_features, mod.out_features, mod.padded_k) == (c["k"], c["n"], c["padded_k"])
        assert mod.graph_safe is False
        # round trip through a state dict into a freshly built module (bundle load path)
        lin2 = nn.Linear(c["k"], c["n"], bias=c["bias"])
        other = HybridInt2Linear(lin2, c["group"], None, c["requested"], c["rank"]) if c["bits"] == 2 \
            else HybridInt4Linear(lin2, c["group"], None, c["requested"])
        missing, unexpected = other.load_state_dict(sd, strict=False)
        assert not missing and not unexpected
        assert torch.equal(other.packed, mod.packed)


def test_outlier_snapping():
    import json
    from conftest import GOLDEN
    for key, want in json.loads((GOLDEN / "snap_table.json").read_text()).items():
        k, req = (int(v) for v in key.split(":"))
        assert snap_outlier_count(req, k) == want, key
    assert HybridInt4Linear(nn.Linear(4096, 8), 128, None, 41).outlier_idx.numel() == 32


def test_full_size_pack_digests(full_size):
    """The package's quantisers reproduce the reference's bytes at the benchmark shapes."""
    z, meta = full_size
    rec = meta["c1"][2]
    torch.manual_seed(rec["seed"])
    w = (torch.randn(4096, 4096) * 0.02).half()
    if _sha(w) != rec["w"]:
        pytest.skip("torch's CPU random stream differs from the one the fixture was made with")
    pw = pack_groupwise_int2(w, 64)
    assert _sha(pw.packed) == rec["packed"] and _sha(pw.scales) == rec["scales"]


def test_cpu_tensors_raise():
    mod = HybridInt2Linear(nn.Linear(64, 32), 32, None, 4, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        mod(torch.randn(1, 64).half())
    with pytest.raises(RuntimeError, match="CUDA"):
        HybridInt4Linear(nn.Linear(64, 32), 32)(torch.randn(6, 64).half())
    pw = pack_groupwise_int2(torch.randn(8, 64), 32)
    with pytest.raises(RuntimeError, match="CUDA"):
        decode_int2_linear(torch.randn(1, 64).half(), pw)


def test_library_builds_loads_and_exports_header_symbols():
    lib_path = build_mod.build()
    assert lib_path.exists()
    header = "\n".join(p.read_text() for p in sorted((ROOT / "include").glob("*.h")))
    declared = set(re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(q[a-z_0-9]+)\s*\(", header, flags=re.M))
    declared = {d for d in declared if d.startswith(("qgemv_", "qdequant", "qunpack", "qcomm_", "qdec_"))}
    assert {"qgemv_run", "qgemv_run_static", "qgemv_workspace_bytes", "qgemv_plan_name", "qgemv_plan_describe",
            "qgemv_workspace_status", "qdequant", "qunpack_codes", "qgemv_error_string", "qgemv_abi_version",
            "qcomm_allreduce", "qcomm_status", "qcomm_alloc", "qcomm_ipc_export", "qcomm_ipc_open",
            "qdec_rmsnorm", "qdec_rope_append", "qdec_attention", "qdec_attention_workspace_bytes", "qdec_silu_mul"} <= declared
    raw = ctypes.CDLL(str(lib_path))
    for name in declared:
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"
    assert set(_cabi.EXPORTS) <= declared
    l = _cabi.lib()
    assert l.qgemv_abi_version() == _cabi.ABI_VERSION
    assert _cabi.workspace_bytes(2, 1, 4096, 4096, 64, 0) >= 17408
    assert ctypes.sizeof(_cabi.Problem) == l.qgemv_sizeof_problem() == 12 * 4 + 20 * 8


def test_c_abi_rejects_bad_problems_without_launching():
    l = _cabi.lib()
    assert l.qgemv_run(None, None) == -1
    p = _cabi.Problem()
    p.bits = 3
    assert l.qgemv_run(ctypes.byref(p), None) == -1
    assert "bits" in _cabi.last_error()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = 2, 5, 8, 64, 64, 32
    assert l.qgemv_run(ctypes.byref(p), None) == -1 and "M must be" in _cabi.last_error()
    p.m = 1
    p.x = p.packed = p.scales = p.y = 256          # never dereferenced: validation fails first
    p.ldx, p.ldp, p.lds, p.ldy = 64, 16, 2, 8
    p.group = 6
    assert l.qgemv_run(ctypes.byref(p), None) == -2
    p.group = 32
    assert l.qgemv_run(ctypes.byref(p), None) == -4  # no workspace
    assert l.qdequant(2, None, 0, None, 0, 1, 4, 4, 4, None, 4, 0, None) == -1
    assert l.qunpack_codes(5, 256, 1, 1, 4, 256, 4, None) == -1


def test_selftest_reports_a_missing_device_instead_of_falling_back():
    from ai_accel_studio_b200.selftest import run_selftest
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    report = run_selftest()
    assert report["ok"] is False and report["probes"][0]["name"] == "cuda" and "no CPU implementation" in report["probes"][0]["error"]
