"""Every code path of the tensor-core-assisted kernels is reached on purpose and asserted through
qgemv_plan_describe, so that a later change of the planner cannot silently stop testing one:

* the barrier-phased kernel's tiles shared between CTAs (partial sums and arrival counters in the
  workspace, last arriver adds in CTA order),
* the pipelined kernel's ring geometries (128 / 256-byte slots), forced warp / slot counts and its L2 announcements,
* chains of dependent launches (each kernel starts before its predecessor has finished and must
  wait for it before it reads x),
* GEMVs that overlap on two streams with a workspace each,
* the bounded wait for the residual projections running out (made by a test-only flag on the host
  side; nothing faults), reported through qgemv_workspace_status.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import c_forward, assert_within_tolerance
from ai_accel_studio_b200 import _cabi, ops
from ai_accel_studio_b200.kernels.groupwise_int2 import pack_groupwise_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import pack_groupwise_int4

pytestmark = pytest.mark.gpu

COUNTER_OFF, COUNTERS = 1024, 16384          # workspace layout: arrival counters follow 1024 bytes of projections


def _case(bits, m, n, k, group, oc, rank, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.05
    pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, group)
    h = dict(packed=pw.packed, scales=pw.scales, x=torch.randn(m, k, generator=g).half())
    h["bias"] = (torch.randn(n, generator=g) * 0.1).half() if bias else None
    h["oidx"] = torch.randperm(k, generator=g)[:oc].to(torch.int32) if oc else None
    h["ow"] = (torch.randn(n, oc, generator=g) * 0.05).half() if oc else None
    h["ru"] = (torch.randn(n, rank, generator=g) * 0.05).half() if rank else None
    h["rv"] = (torch.randn(rank, k, generator=g) * 0.05).half() if rank else None
    d = {key: (None if v is None else v.cuda()) for key, v in h.items()}
    return h, d


def _problem(bits, m, n, k, group, oc, rank, d, y, ws, kernel="auto", debug=0):
    p = _cabi.Problem()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = bits, m, n, k, k, group
    p.kernel, p.debug = _cabi.KERNEL[kernel], debug
    p.x, p.ldx = d["x"].data_ptr(), d["x"].stride(0)
    p.packed, p.ldp = d["packed"].data_ptr(), d["packed"].stride(0)
    p.scales, p.lds = d["scales"].data_ptr(), d["scales"].stride(0)
    p.bias = d["bias"].data_ptr() if d["bias"] is not None else None
    p.outliers, p.rank = oc, rank
    if oc:
        p.outlier_idx, p.outlier_w, p.ldow = d["oidx"].data_ptr(), d["ow"].data_ptr(), oc
    if rank:
        p.res_u, p.ldu, p.res_v, p.ldv = d["ru"].data_ptr(), rank, d["rv"].data_ptr(), k
    p.y, p.ldy = y.data_ptr(), y.stride(0)
    if ws is not None:
        p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    return p


def _oracle(coracle, bits, k, group, h):
    np_ = lambda t: None if t is None else t.numpy()
    return c_forward(coracle, h["x"].numpy(), bits, h["packed"].numpy(), h["scales"].numpy(), k, group,
                     np_(h["bias"]), np_(h["oidx"]), np_(h["ow"]), np_(h["ru"]), np_(h["rv"]))


def _workspace():
    return torch.zeros(_cabi.workspace_bytes(4, 4, 1, 256, 128, 8), dtype=torch.uint8, device="cuda")


def _tile_counters(ws):
    return ws[COUNTER_OFF:COUNTER_OFF + 4 * (COUNTERS - 4)]     # the last four words are bookkeeping, not counters


# bits, m, n, k, group, oc, rank: shapes whose balance needs tiles shared between CTAs
SHARED_TILE_CASES = [
    (4, 1, 2400, 14336, 128, 64, 8),     # 150 tiles, two for the busiest CTA, > 160 KB each
    (4, 4, 2400, 14336, 128, 64, 8),
    (4, 1, 1024, 28672, 128, 0, 0),      # fewer tiles than SMs, > 160 KB per tile
    (2, 3, 2560, 28672, 128, 32, 8),     # only 4 warps fit beside 172 KB of staged activations
]


@pytest.mark.parametrize("bits,m,n,k,group,oc,rank", SHARED_TILE_CASES)
def test_tiles_shared_between_ctas(bits, m, n, k, group, oc, rank, coracle):
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    h, d = _case(bits, m, n, k, group, oc, rank, seed=n + k + m)
    ws = _workspace()
    y = [torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda") for _ in range(3)]
    p = _problem(bits, m, n, k, group, oc, rank, d, y[0], ws)
    info = _cabi.plan_describe(p)
    assert info.family == _cabi.KERNEL["mma"] and info.variant == 1 and info.tile_aligned == 0, \
        "this shape no longer reaches the shared-tile path: pick another one"
    assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
    p.y = y[1].data_ptr()
    assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
    p.y = y[2].data_ptr()
    p.workspace, p.workspace_bytes = None, 0
    assert lib.qgemv_run_static(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert_within_tolerance(y[0].float().cpu().numpy(), _oracle(coracle, bits, k, group, h), "shared tiles")
    assert torch.equal(y[0], y[1]) and torch.equal(y[0], y[2])          # fixed summation order, both scratch areas
    assert not _tile_counters(ws).any()                                   # arrival counters back at zero
    out = ctypes.c_int32(-1)
    assert lib.qgemv_workspace_status(ws.data_ptr(), ctypes.c_void_p(stream), ctypes.byref(out)) == 0
    torch.cuda.synchronize()
    assert out.value == 0


PIPE_CASES = [
    # bits, m, n, k, group, oc, rank
    (4, 4, 2048, 4096, 128, 32, 8),
    (4, 1, 4096, 2048, 64, 16, 8),
    (4, 3, 1000, 1024, 32, 8, 0),        # ragged N, 16-byte groups
    (2, 1, 4096, 4096, 64, 0, 0),
    (2, 2, 3000, 8192, 128, 64, 8),
    (2, 4, 640, 14336, 256, 40, 16),
    (2, 1, 128, 896, 128, 8, 8),         # one chunk per tile: a single warp per CTA has work
]
# debug bits: 2 no L2 announcements, 4 / 32 force 128 / 256-byte ring slots, 8 late release of the next launch;
# bits 8.. force the warps per CTA, bits 16.. the ring depth
PIPE_VARIANTS = [0, 2, 4, 4 | 2, 32, 8, (3 << 8) | (2 << 16), 4 | (5 << 8) | (3 << 16), (8 << 8) | (2 << 16),
                 32 | (12 << 8) | (2 << 16), 4 | (16 << 8) | (2 << 16)]


@pytest.mark.parametrize("bits,m,n,k,group,oc,rank", PIPE_CASES)
def test_pipelined_kernel_variants(bits, m, n, k, group, oc, rank, coracle):
    """Ring geometry (128 / 256-byte slots), L2 announcements on / off, forced warp and slot counts:
    all give the oracle's answer, and the same bits as each other where the run structure agrees."""
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    h, d = _case(bits, m, n, k, group, oc, rank, seed=3 * n + k + m)
    ref = _oracle(coracle, bits, k, group, h)
    ws = _workspace()
    seen = {}
    for dbg in PIPE_VARIANTS:
        y = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        p = _problem(bits, m, n, k, group, oc, rank, d, y, ws, kernel="mma_pipe", debug=dbg)
        try:
            info = _cabi.plan_describe(p)
        except _cabi.QgemvError as e:
            assert e.code == -2 and (dbg >> 8 or dbg & (4 | 32)), (dbg, e)
            continue                        # a forced warp count or slot size this shape cannot use
        assert info.variant == 2 and info.tile_aligned == 1, (dbg, info.variant)
        for _ in range(2):
            assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
        torch.cuda.synchronize()
        assert_within_tolerance(y.float().cpu().numpy(), ref, f"pipelined kernel, debug bits {dbg:#x}")
        key = (info.chunk_bytes, info.run_chunks, info.warps, info.projection_parts, info.launches)   # same summation order
        if key in seen:
            assert torch.equal(y, seen[key]), f"debug bits {dbg:#x}"
        seen[key] = y
    out = ctypes.c_int32(-1)
    assert lib.qgemv_workspace_status(ws.data_ptr(), ctypes.c_void_p(stream), ctypes.byref(out)) == 0
    torch.cuda.synchronize()
    assert out.value == 0


def test_planner_takes_the_barrier_free_kernel_for_very_long_rows(coracle):
    """M = 1 and 14 KB of codes per row (INT4, K = 28672): the one shape class where the barrier-free kernel
    measured faster, so the planner picks it; checked against the oracle like every other path."""
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    bits, m, n, k, group, oc, rank = 4, 1, 4096, 28672, 128, 64, 8
    h, d = _case(bits, m, n, k, group, oc, rank, seed=5)
    ws = _workspace()
    y = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    p = _problem(bits, m, n, k, group, oc, rank, d, y, ws)
    info = _cabi.plan_describe(p)
    assert info.variant == 2 and info.warps == 16
    for _ in range(2):
        assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert_within_tolerance(y.float().cpu().numpy(), _oracle(coracle, bits, k, group, h), "barrier-free kernel by the planner's choice")
    p2 = _problem(bits, 2, n, k, group, oc, rank, d, y, ws)                  # two rows: the phased kernel
    p2.x = torch.zeros((2, k), dtype=torch.float16, device="cuda").data_ptr()
    assert _cabi.plan_describe(p2).variant == 1
    out = ctypes.c_int32(-1)
    assert lib.qgemv_workspace_status(ws.data_ptr(), ctypes.c_void_p(stream), ctypes.byref(out)) == 0
    torch.cuda.synchronize()
    assert out.value == 0


@pytest.mark.parametrize("kernel", ["auto", "mma_pipe", "simt"])
def test_chain_of_dependent_launches(kernel):
    """x_{i+1} = y_i through 12 square GEMVs issued back to back: every launch is allowed to start
    (and to fetch its weights) while the previous one runs, and must still see the previous result.
    Compared with the same GEMVs issued one at a time with a device synchronisation in between."""
    torch.manual_seed(11)
    n = 2048
    layers = []
    for i in range(12):
        bits = 2 if i % 2 else 4
        w = torch.randn(n, n) * (0.9 / n ** 0.5)
        pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(w, 128)
        layers.append((bits, pw.packed.cuda(), pw.scales.cuda(), torch.randperm(n)[:16].to(torch.int32).cuda(),
                       (torch.randn(n, 16) * 0.01).half().cuda(), (torch.randn(n, 8) * 0.01).half().cuda(),
                       (torch.randn(8, n) * 0.01).half().cuda()))
    kern = _cabi.KERNEL[kernel]

    def step(i, x):
        bits, packed, scales, oidx, ow, ru, rv = layers[i]
        return ops.gemv(x, packed, scales, None, oidx, ow, ru, rv, bits, 128, n, 0, kern)
    for m in (1, 4):
        x0 = torch.randn(m, n).half().cuda()
        want = x0
        for i in range(12):
            want = step(i, want)
            torch.cuda.synchronize()
        got = x0
        for i in range(12):
            got = step(i, got)
        torch.cuda.synchronize()
        assert torch.isfinite(want.float()).all() and float(want.float().abs().max()) > 0
        assert torch.equal(got, want), kernel
        # the same chain replayed from a CUDA graph (programmatic edges between the kernel nodes)
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        static_x = x0.clone()
        with torch.cuda.stream(s):
            t = static_x
            for i in range(12):
                t = step(i, t)
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            t = static_x
            for i in range(12):
                t = step(i, t)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(t, want), kernel
    assert ops.workspace_status("cuda") == 0


def test_two_streams_overlap_with_a_workspace_each():
    """GEMVs with in-kernel residual projections issued concurrently on two streams: each stream has
    its own scratch buffer, so the results equal the serial ones."""
    torch.manual_seed(5)
    n, k = 4096, 4096
    mods = []
    for bits in (2, 4):
        pw = (pack_groupwise_int2 if bits == 2 else pack_groupwise_int4)(torch.randn(n, k) * 0.02, 128)
        mods.append((bits, pw.packed.cuda(), pw.scales.cuda(), torch.randperm(k)[:32].to(torch.int32).cuda(),
                     (torch.randn(n, 32) * 0.02).half().cuda(), (torch.randn(n, 8) * 0.02).half().cuda(),
                     (torch.randn(8, k) * 0.02).half().cuda()))
    xs = [torch.randn(2, k).half().cuda() for _ in range(2)]

    def run(i):
        bits, packed, scales, oidx, ow, ru, rv = mods[i]
        return ops.gemv(xs[i], packed, scales, None, oidx, ow, ru, rv, bits, 128, k, 0, 0)
    serial = [run(0), run(1)]
    torch.cuda.synchronize()
    s = [torch.cuda.Stream(), torch.cuda.Stream()]
    assert ops.ensure_workspace("cuda", s[0]).data_ptr() != ops.ensure_workspace("cuda", s[1]).data_ptr()
    outs = [[], []]
    for rep in range(50):
        for i in range(2):
            with torch.cuda.stream(s[i]):
                outs[i].append(run(i))
    torch.cuda.synchronize()
    for i in range(2):
        for o in outs[i]:
            assert torch.equal(o, serial[i])
        assert ops.workspace_status("cuda", s[i]) == 0


@pytest.mark.parametrize("kernel", ["auto", "mma_pipe"])
def test_projection_wait_runs_out_and_is_reported(kernel, coracle):
    """QGEMV_DEBUG_DROP_PROJECTIONS: the CTAs that compute the residual projections keep them to
    themselves and the readers' wait is cut to a few microseconds.  The launch must end by itself,
    raise the workspace's status word, and leave the workspace and the device usable."""
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    bits, m, n, k, group, oc, rank = 4, 2, 4096, 4096, 128, 16, 8
    h, d = _case(bits, m, n, k, group, oc, rank, seed=77)
    ws = _workspace()
    out = ctypes.c_int32(-1)

    def status():
        assert lib.qgemv_workspace_status(ws.data_ptr(), ctypes.c_void_p(stream), ctypes.byref(out)) == 0
        torch.cuda.synchronize()
        return out.value
    y = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    p = _problem(bits, m, n, k, group, oc, rank, d, y, ws, kernel=kernel)
    info = _cabi.plan_describe(p)
    assert info.variant == (2 if kernel == "mma_pipe" else 1) and info.inline_projections == 1
    assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0      # a normal launch first
    torch.cuda.synchronize()
    ref = _oracle(coracle, bits, k, group, h)
    assert_within_tolerance(y.float().cpu().numpy(), ref, "before")
    assert status() == 0
    p.debug = _cabi.DEBUG_DROP_PROJECTIONS
    y_bad = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    p.y = y_bad.data_ptr()
    assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0
    torch.cuda.synchronize()                                                  # the launch ends by itself
    assert status() == 1                                                      # ... and says what happened
    assert status() == 0                                                      # the query cleared the word
    p.debug = 0
    y2 = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    p.y = y2.data_ptr()
    assert lib.qgemv_run(ctypes.byref(p), ctypes.c_void_p(stream)) == 0      # same workspace, next launch is fine
    torch.cuda.synchronize()
    assert torch.equal(y2, y)
    assert status() == 0
