"""Tensor-parallel sharding on the CPU: shard algebra against the oracle, a 2-rank gloo
all-reduce of K-split partial results, and host-made failure cases.  No GPU involved."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from oracle import qgemv_oracle as O
from ai_accel_studio_b200 import tp
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear


def _module(bits, n=48, k=512, group=64, oc=8, rank=4, bias=True, seed=0):
    torch.manual_seed(seed)
    lin = nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.normal_(0, 0.05)
        lin.weight[:, ::37] *= 4
    if bits == 2:
        return HybridInt2Linear(lin, group, None, oc, rank)
    return HybridInt4Linear(lin, group, None, oc, residual_rank=rank)


def _oracle_forward(mod, x):
    npy = lambda t: None if t is None else t.numpy()
    pw = O.PackedWeight(mod.bits, mod.packed.numpy(), mod.scales.numpy(), mod.original_k, mod.padded_k, mod.group_size)
    return O.gemv_f32(x.numpy(), pw, npy(mod.bias), npy(mod.outlier_idx), npy(mod.outlier_weight),
                      npy(mod.res_u) if mod.residual_rank else None, npy(mod.res_v) if mod.residual_rank else None)


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_and_column_shards_recompose(bits, world):
    mod = _module(bits)
    x = torch.randn(3, 512).half()
    full = _oracle_forward(mod, x)
    rows = [_oracle_forward(tp.shard_rows(mod, r, world), x) for r in range(world)]
    assert np.allclose(np.concatenate(rows, 1), full, rtol=0, atol=1e-9)
    ks = 512 // world
    parts = [_oracle_forward(tp.shard_cols(mod, r, world), x[:, r * ks:(r + 1) * ks].contiguous()) for r in range(world)]
    assert np.allclose(sum(parts), full, rtol=1e-9, atol=1e-9)
    shards = [tp.shard_cols(mod, r, world) for r in range(world)]
    assert len({int(s.outlier_idx.numel()) for s in shards}) == 1          # common padded outlier count
    assert sum(s.bias is not None for s in shards) == 1                    # bias on one rank only
    assert all(s.padded_k == ks and s.in_features == ks for s in shards)


def test_host_side_failures():
    mod = _module(2, n=50, k=512, group=64, oc=0, rank=0, bias=False)
    with pytest.raises(ValueError, match="divisible"):
        tp.shard_rows(mod, 0, 4)                      # 50 rows / 4
    with pytest.raises(ValueError, match="multiple of the group"):
        tp.shard_cols(_module(4, k=512, group=128), 0, 8)      # 512/8 = 64 < group 128
    padded = HybridInt2Linear(nn.Linear(130, 16), 64)
    with pytest.raises(ValueError, match="padded"):
        tp.shard_cols(padded, 0, 2)


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mod = _module(4, seed=3)                      # same seed on every rank -> same unsharded module
        g = torch.Generator().manual_seed(11)
        x = torch.randn(2, 512, generator=g).half()
        ks = 512 // world
        shard = tp.shard_cols(mod, rank, world)
        part = torch.from_numpy(_oracle_forward(shard, x[:, rank * ks:(rank + 1) * ks].contiguous()))
        wrapped = tp.AllReduceLinear(nn.Identity())   # exercises the collective the GPU path uses
        total = wrapped(part.clone())
        full = torch.from_numpy(_oracle_forward(mod, x))
        ret[rank] = float((total - full).abs().max())
        # a rank that brings a wrongly shaped shard is caught on the host before any collective
        shapes = [None] * world
        dist.all_gather_object(shapes, tuple(shard.packed.shape))
        assert len(set(shapes)) == 1
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_all_reduce():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_rank_main, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world and max(ret.values()) < 1e-9
