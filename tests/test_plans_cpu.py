"""The planner behind qgemv_plan_describe, on the CPU (nothing is launched, the pointers are made up): invariants of
the geometry it hands the kernels for a grid of decoder and tensor-parallel shard shapes, and the rules by which
QGEMV_KERNEL_AUTO picks a kernel."""
import itertools

import pytest

from ai_accel_studio_b200 import _cabi

MAX_SMEM = 232448          # 227 KB per CTA on sm_100
SMS = 148                  # what the library assumes when no device is present


def _problem(bits, m, n, k, group, oc, rank, kernel="auto", act=0, misalign=0):
    p = _cabi.Problem()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = bits, m, n, k, k, group
    p.kernel, p.act = _cabi.KERNEL[kernel], act
    p.x, p.ldx = 0x10000 + misalign, k
    p.packed, p.ldp = 0x1000000, k * bits // 8
    p.scales, p.lds = 0x20000000, k // group
    p.outliers, p.rank = oc, rank
    if oc:
        p.outlier_idx, p.outlier_w, p.ldow = 0x30000000, 0x40000000, oc
    if rank:
        p.res_u, p.ldu, p.res_v, p.ldv = 0x50000000, rank, 0x60000000, k
    p.y, p.ldy = 0x70000000, n
    p.workspace, p.workspace_bytes = 0x80000000, _cabi.workspace_bytes(4, 4, 1, 256, 128, 8)
    return p


def _describe(*a, **kw):
    info = _cabi.plan_describe(_problem(*a, **kw))
    return {name: int(getattr(info, name)) for name, _ in _cabi.PlanInfo._fields_}


SHAPES = [(n, k) for n, k in itertools.product((128, 1024, 3584, 4096, 11008, 14336, 28672), (896, 4096, 8192, 14336, 28672))]


@pytest.mark.parametrize("bits,group", [(2, 64), (2, 128), (2, 256), (4, 32), (4, 64), (4, 128)])
def test_tensor_core_plans_respect_the_machine(bits, group):
    for (n, k), m, (oc, rank) in itertools.product(SHAPES, (1, 4), ((0, 0), (32, 8), (64, 16))):
        if k % group:
            continue
        d = _describe(bits, m, n, k, group, oc, rank)
        if d["family"] != _cabi.KERNEL["mma"]:
            continue                                   # activations too large for shared memory: the CUDA-core kernel
        assert 1 <= d["grid"] <= SMS and 1 <= d["warps"] <= 16 and d["stages"] >= 2, (bits, group, m, n, k, d)
        assert d["smem_bytes"] <= MAX_SMEM and d["ctas_per_sm"] == 1
        assert d["chunk_bytes"] in (128, 256) and d["run_chunks"] >= 1 and d["runs_per_tile"] >= 1
        assert d["launches"] == (1 if (rank == 0 or d["inline_projections"]) else 2)
        tiles = -(-n // 16)
        if tiles <= d["grid"] and d["tile_aligned"]:
            assert d["grid"] == min(tiles, SMS)        # fewer tiles than SMs: one CTA per tile
        if d["variant"] == 2:                          # the barrier-free kernel: only where AUTO's rule says so
            assert m == 1 and k * bits // 8 >= 14336 and d["tile_aligned"] == 1


def test_kernel_selection_rules():
    mma, simt = _cabi.KERNEL["mma"], _cabi.KERNEL["simt"]
    assert _describe(4, 4, 11008, 4096, 128, 32, 8)["variant"] == 1                       # the benchmark shape: phased kernel
    assert _describe(4, 1, 8192, 28672, 128, 64, 8)["variant"] == 2                       # 14 KB rows, one activation row
    assert _describe(4, 2, 8192, 28672, 128, 64, 8)["variant"] == 1
    assert _describe(2, 1, 8192, 28672, 128, 64, 8)["variant"] == 1                       # INT2: 7 KB rows
    assert _describe(4, 1, 8192, 28672, 128, 64, 8, kernel="mma")["variant"] == 1         # forced
    assert _describe(4, 4, 11008, 4096, 128, 32, 8, kernel="mma_pipe")["variant"] == 2
    assert _describe(4, 1, 1024, 28672, 128, 0, 0)["tile_aligned"] == 0                   # big tiles, fewer than SMs: shared
    assert _describe(4, 1, 4096, 4096, 8, 0, 0)["family"] == simt                         # 4-byte groups: CUDA cores
    assert _describe(4, 1, 4096, 4096, 128, 0, 0, misalign=2)["family"] == simt           # x not 16-byte aligned
    assert _describe(4, 1, 4096, 4096, 128, 300, 0)["family"] == simt                     # more than 256 outlier columns
    assert _describe(4, 1, 4096, 4096, 128, 0, 0, kernel="simt")["family"] == simt
    for bad in (dict(kernel="mma", group=8), dict(kernel="mma_pipe", group=8), dict(kernel="simt", act=3), dict(act=3, group=8)):
        kw = dict(kernel="auto", act=0, group=128)
        kw.update(bad)
        with pytest.raises(_cabi.QgemvError) as e:
            _describe(4, 1, 4096, 4096, kw["group"], 0, 0, kernel=kw["kernel"], act=kw["act"])
        assert e.value.code == -2
    with pytest.raises(_cabi.QgemvError) as e:                                            # gated pairs need whole 16-row blocks
        _cabi.plan_describe(_problem(4, 1, 4104, 4096, 128, 0, 0, act=3))
    assert e.value.code == -2
    assert _describe(4, 1, 4096, 4096, 128, 0, 0, act=3)["family"] == mma
