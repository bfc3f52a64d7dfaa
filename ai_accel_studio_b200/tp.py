"""Tensor-parallel sharding of the packed Linear modules (one process per GPU).

The reference has no multi-GPU path; this follows the usual Megatron split for a decoder layer:

  q/k/v_proj, gate/up_proj   split by output rows (N): no communication, x is replicated
  o_proj, down_proj          split by input columns (K): every rank produces a partial
                             ``[M, hidden]`` and one all-reduce(sum) completes it

Shards are cut from an unsharded module's buffers (the on-disk bundle format does not change):

* row shard: rows ``[r*N/T, (r+1)*N/T)`` of ``packed``, ``scales``, ``outlier_weight``, ``bias``,
  ``res_u``; ``outlier_idx`` and ``res_v`` are replicated.
* column shard: K/T must be a multiple of the group size (so byte and scale columns split
  cleanly).  ``packed[:, bytes of the K range]``, ``scales[:, groups of the K range]``,
  ``res_v[:, K range]`` (``res_u`` replicated: U·(V_t x_t) sums linearly over ranks), the outlier
  columns that fall into the range re-based to local indices (padded to a common count with
  zero-weight columns so every rank launches the same kernel shape), bias kept on rank 0 only.

The all-reduce is ``torch.distributed.all_reduce`` (NCCL over NVLink on GPUs, gloo in the CPU
tests); it is captured into each rank's CUDA graph together with the GEMVs.
"""
from __future__ import annotations

import torch
from torch import nn

from .optimize._hybrid_base import HybridPackedLinear


def _buffers(mod: HybridPackedLinear) -> dict:
    return dict(packed=mod.packed, scales=mod.scales, outlier_idx=mod.outlier_idx, outlier_weight=mod.outlier_weight,
                bias=mod.bias, res_u=mod.res_u if mod.residual_rank else None,
                res_v=mod.res_v if mod.residual_rank else None)


def row_shard_buffers(b: dict, rank: int, world: int) -> dict:
    """Rows ``[rank*N/world, (rank+1)*N/world)`` of every per-row tensor."""
    n = b["packed"].shape[0]
    if n % world:
        raise ValueError(f"N={n} is not divisible by the tensor-parallel size {world}")
    lo, hi = rank * n // world, (rank + 1) * n // world
    cut = lambda t: None if t is None else t[lo:hi].contiguous()
    return dict(packed=cut(b["packed"]), scales=cut(b["scales"]), outlier_idx=b["outlier_idx"],
                outlier_weight=cut(b["outlier_weight"]), bias=cut(b["bias"]), res_u=cut(b["res_u"]), res_v=b["res_v"])


def col_shard_buffers(b: dict, rank: int, world: int, bits: int, group: int, k: int, pad_outliers_to: int | None = None) -> dict:
    """Input columns ``[rank*K/world, (rank+1)*K/world)``; ``k`` is the unpadded K (must equal the
    padded K: a padded tail cannot be split)."""
    kp = b["packed"].shape[1] * (8 // bits)
    if kp != k:
        raise ValueError("column sharding needs K to be a multiple of the group size (no padded tail)")
    if k % world or (k // world) % group:
        raise ValueError(f"K/T = {k}/{world} must be a multiple of the group size {group}")
    ks = k // world
    lo, hi = rank * ks, (rank + 1) * ks
    bpc = 8 // bits
    out = dict(packed=b["packed"][:, lo // bpc:hi // bpc].contiguous(),
               scales=b["scales"][:, lo // group:hi // group].contiguous(),
               bias=b["bias"] if rank == 0 else None,
               res_u=b["res_u"], res_v=None if b["res_v"] is None else b["res_v"][:, lo:hi].contiguous())
    idx, ow = b["outlier_idx"], b["outlier_weight"]
    if idx is not None and idx.numel():
        keep = ((idx >= lo) & (idx < hi)).nonzero().flatten()
        lidx = (idx[keep] - lo).to(torch.int32)
        low = ow[:, keep]
        want = pad_outliers_to if pad_outliers_to is not None else int(keep.numel())
        if want < keep.numel():
            raise ValueError("pad_outliers_to is smaller than the number of outlier columns of this shard")
        if want > keep.numel():            # zero-weight columns pointing at local column 0
            extra = want - int(keep.numel())
            lidx = torch.cat([lidx, torch.zeros(extra, dtype=torch.int32, device=lidx.device)])
            low = torch.cat([low, torch.zeros((low.shape[0], extra), dtype=low.dtype, device=low.device)], 1)
        out.update(outlier_idx=lidx.contiguous(), outlier_weight=low.contiguous())
    else:
        out.update(outlier_idx=None, outlier_weight=None)
    return out


def max_outliers_per_col_shard(outlier_idx: torch.Tensor, k: int, world: int) -> int:
    """Largest number of outlier columns any K-range of size K/world holds (the common padded count)."""
    if outlier_idx is None or outlier_idx.numel() == 0:
        return 0
    ks = k // world
    return int(torch.bincount((outlier_idx.long() // ks), minlength=world).max().item())


def _rebuild(mod: HybridPackedLinear, b: dict, k_local: int) -> HybridPackedLinear:
    return type(mod).from_buffers(b["packed"], b["scales"], k_local, mod.group_size, b["outlier_idx"], b["outlier_weight"],
                                  b["bias"], b["res_u"], b["res_v"])


def shard_rows(mod: HybridPackedLinear, rank: int, world: int) -> HybridPackedLinear:
    """N-split shard of a packed Linear (q/k/v/gate/up)."""
    return _rebuild(mod, row_shard_buffers(_buffers(mod), rank, world), mod.in_features)


def shard_cols(mod: HybridPackedLinear, rank: int, world: int) -> HybridPackedLinear:
    """K-split shard of a packed Linear (o/down); its output must be all-reduced."""
    pad = max_outliers_per_col_shard(mod.outlier_idx, mod.in_features, world)
    b = col_shard_buffers(_buffers(mod), rank, world, mod.bits, mod.group_size, mod.in_features, pad)
    return _rebuild(mod, b, mod.in_features // world)


class AllReduceLinear(nn.Module):
    """A K-split shard followed by the all-reduce that completes its output.

    ``AllReduceLinear.skip_collective = True`` leaves the collective out (the output is then this
    rank's partial sum): a measurement aid that attributes decode time to the all-reduces by
    replaying the same step without them."""

    skip_collective = False
    one_shot = None          # a comm.OneShotAllReduce: used for the tensors it fits, NCCL for the rest

    def __init__(self, inner: nn.Module, group=None):
        super().__init__()
        self.inner = inner
        self.group = group

    def forward(self, x):
        y = self.inner(x)
        if AllReduceLinear.skip_collective:
            return y
        if torch.distributed.is_available() and torch.distributed.is_initialized() and \
                torch.distributed.get_world_size(self.group) > 1:
            comm = AllReduceLinear.one_shot
            if comm is not None and comm.fits(y):
                comm(y)
            else:
                torch.distributed.all_reduce(y, group=self.group)
        return y
