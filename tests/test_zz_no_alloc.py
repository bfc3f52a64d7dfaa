"""qgemv_run_static: the entry point for hosts that are not allowed to allocate device memory
(fixed start-up memory budget, plugin hooks without an allocator): it must give the same answer
as qgemv_run with a caller-owned workspace, on back-to-back calls that share the built-in scratch.

Collected last on purpose: a failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

from ai_accel_studio_b200 import _cabi
from ai_accel_studio_b200.kernels.groupwise_int2 import pack_groupwise_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import pack_groupwise_int4

pytestmark = pytest.mark.gpu


def _problem(bits, m, n, k, group, oc, rank, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.05
    pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, group)
    t = dict(packed=pw.packed.cuda(), scales=pw.scales.cuda(), x=torch.randn(m, k, generator=g).half().cuda(),
             bias=(torch.randn(n, generator=g) * 0.1).half().cuda())
    if oc:
        t["oidx"] = torch.randperm(k, generator=g)[:oc].to(torch.int32).cuda()
        t["ow"] = (torch.randn(n, oc, generator=g) * 0.05).half().cuda()
    if rank:
        t["ru"] = (torch.randn(n, rank, generator=g) * 0.05).half().cuda()
        t["rv"] = (torch.randn(rank, k, generator=g) * 0.05).half().cuda()
    p = _cabi.Problem()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = bits, m, n, k, k, group
    p.x, p.ldx = t["x"].data_ptr(), k
    p.packed, p.ldp = t["packed"].data_ptr(), t["packed"].stride(0)
    p.scales, p.lds = t["scales"].data_ptr(), t["scales"].stride(0)
    p.bias = t["bias"].data_ptr()
    p.outliers, p.rank = oc, rank
    if oc:
        p.outlier_idx, p.outlier_w, p.ldow = t["oidx"].data_ptr(), t["ow"].data_ptr(), oc
    if rank:
        p.res_u, p.ldu, p.res_v, p.ldv = t["ru"].data_ptr(), rank, t["rv"].data_ptr(), k
    return p, t


# Shapes that exercise the scratch: residual projections passed between CTAs through it (rank > 0,
# pipelined and phased kernels), the separate projection kernel of the general path (last case), and
# one whose tiles are shared between CTAs (partial sums and arrival counters live in the scratch).
CASES = [(4, 4, 2048, 4096, 128, 32, 8), (2, 1, 96, 8192, 128, 8, 8), (2, 3, 4096, 1024, 64, 0, 0),
         (4, 1, 2400, 14336, 128, 64, 8), (4, 2, 50, 200, 8, 5, 3)]
SHARED_TILE_CASE = 3


def test_static_scratch_matches_workspace_entry_point_twice(coracle):
    from conftest import c_forward, assert_within_tolerance
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(_cabi.workspace_bytes(4, 4, 1, 256, 128, 8), dtype=torch.uint8, device="cuda")
    for rep in range(2):                       # two rounds in a row over the same built-in scratch
        for i, (bits, m, n, k, group, oc, rank) in enumerate(CASES):
            p, keep = _problem(bits, m, n, k, group, oc, rank, seed=100 * rep + i)
            y_ref = torch.zeros(m, n, dtype=torch.float16, device="cuda")
            y_sta = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
            p.y, p.ldy = y_ref.data_ptr(), n
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
            if i == SHARED_TILE_CASE:
                assert _cabi.plan_describe(p).tile_aligned == 0
            assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
            p.y = y_sta.data_ptr()
            p.workspace, p.workspace_bytes = None, 0          # ignored by the static entry point
            assert lib.qgemv_run_static(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
            torch.cuda.synchronize()
            # same kernels, same fixed summation order: the tolerance of the parity tests is met trivially
            diff = (y_sta.float() - y_ref.float()).abs()
            assert torch.isfinite(y_sta.float()).all()
            assert float(diff.max()) <= 1e-2 + 1e-3 * float(y_ref.float().abs().max()), (rep, i, float(diff.max()))
            assert torch.equal(y_sta, y_ref), (rep, i)
            if rep == 0:                       # ... and on its own feet: against the CPU oracle
                h = {k_: v.cpu().numpy() for k_, v in keep.items()}
                ref = c_forward(coracle, h["x"], bits, h["packed"], h["scales"], k, group, h["bias"], h.get("oidx"),
                                h.get("ow"), h.get("ru"), h.get("rv"))
                assert_within_tolerance(y_sta.float().cpu().numpy(), ref, f"static scratch case {i}")
            del keep


def test_static_scratch_rejects_oversized_problems():
    lib = _cabi.lib()
    p, keep = _problem(2, 1, 64, 256, 64, 0, 0, seed=1)
    y = torch.zeros(1, 64, dtype=torch.float16, device="cuda")
    p.y, p.ldy = y.data_ptr(), 1 << 20
    p.n = 262128 + 16                                          # beyond QGEMV_STATIC_MAX_N; nothing is launched
    assert lib.qgemv_run_static(ctypes.byref(p), None) == -6
    assert "limit" in _cabi.last_error()
    p.n, p.rank = 64, 65
    assert lib.qgemv_run_static(ctypes.byref(p), None) == -6
