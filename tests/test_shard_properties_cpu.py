"""Property tests (hypothesis) of the tensor-parallel shard algebra on random packed modules: for any
world size, width, group size and outlier placement, the shards' reconstructed weights reassemble the
unsharded module's -- rows concatenated for row shards, K ranges concatenated for column shards --
outlier columns land in exactly one column shard, and the bias stays on rank 0."""
import torch
from hypothesis import given, settings, strategies as st

from ai_accel_studio_b200 import tp
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear


def _random_module(bits, n, k, group, oc, rank, bias, seed):
    g = torch.Generator().manual_seed(seed)
    cls = HybridInt2Linear if bits == 2 else HybridInt4Linear
    packed = torch.randint(0, 256, (n, k * bits // 8), dtype=torch.uint8, generator=g)
    scales = (torch.rand((n, k // group), generator=g) * 0.05 + 0.01).half()
    idx = torch.randperm(k, generator=g)[:oc].sort().values.to(torch.int32) if oc else None
    ow = (torch.randn((n, oc), generator=g) * 0.1).half() if oc else None
    ru = (torch.randn((n, rank), generator=g) * 0.1).half() if rank else None
    rv = (torch.randn((rank, k), generator=g) * 0.1).half() if rank else None
    b = (torch.randn(n, generator=g) * 0.1).half() if bias else None
    return cls.from_buffers(packed, scales, k, group, idx, ow, b, ru, rv)


@settings(max_examples=40, deadline=None)
@given(bits=st.sampled_from([2, 4]), world=st.sampled_from([2, 4, 8]), rows_per_rank=st.integers(1, 5),
       groups_per_rank=st.integers(1, 3), group=st.sampled_from([8, 32, 64]), oc=st.integers(0, 12),
       rank=st.sampled_from([0, 3, 8]), bias=st.booleans(), seed=st.integers(0, 10 ** 6))
def test_shards_reassemble_the_module(bits, world, rows_per_rank, groups_per_rank, group, oc, rank, bias, seed):
    n, k = world * rows_per_rank, world * groups_per_rank * group
    full = _random_module(bits, n, k, group, min(oc, k), rank, bias, seed)
    w_full = full.effective_weight()
    rows = [tp.shard_rows(full, r, world) for r in range(world)]
    assert torch.allclose(torch.cat([m.effective_weight() for m in rows], 0), w_full, atol=1e-6)
    for r, m in enumerate(rows):
        assert m.out_features == rows_per_rank and m.in_features == k
        if bias:
            assert torch.equal(m.bias, full.bias[r * rows_per_rank:(r + 1) * rows_per_rank])
    cols = [tp.shard_cols(full, r, world) for r in range(world)]
    assert torch.allclose(torch.cat([m.effective_weight() for m in cols], 1), w_full, atol=1e-6)
    counts = {int(m.outlier_idx.numel()) for m in cols}
    assert len(counts) == 1                                   # padded to a common count: every rank launches the same shape
    live = sum(int((m.outlier_weight.abs().sum(0) > 0).sum()) for m in cols)
    assert live <= min(oc, k)                                 # each outlier column lives in exactly one K range
    for r, m in enumerate(cols):
        assert m.in_features == k // world and m.out_features == n
        assert (m.bias is not None) == (bias and r == 0)
        if m.outlier_idx.numel():
            assert int(m.outlier_idx.max()) < k // world and int(m.outlier_idx.min()) >= 0
