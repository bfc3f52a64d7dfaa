"""``HybridInt4Linear``: packed groupwise INT4 base + exact fp16 outlier columns, with the
constructor, buffers and forward contract of the reference's module
(ai_accel_lab/optimize/hybrid_int4.py:7-38).

Extension: ``residual_rank`` / ``residual_factors`` (keyword-only, default off) attach a
rank-r correction ``res_u [N,r]``, ``res_v [r,K]`` that the fused kernel adds in its epilogue.
The reference's INT4 module has no residual; with the defaults this class behaves like it.
"""
from __future__ import annotations

import torch
from torch import nn

from ..kernels.groupwise_int4 import GroupwiseInt4Weight, pack_groupwise_int4
from ._hybrid_base import HybridPackedLinear, select_outliers


class HybridInt4Linear(HybridPackedLinear):
    """Packed INT4 layer; no dense copy of the source weight is kept."""

    bits = 4

    def __init__(self, source: nn.Linear, group_size=128, activation_rms=None, outlier_columns=0, *,
                 residual_rank: int = 0, residual_factors=None):
        super().__init__()
        w = source.weight.detach()
        n, k = w.shape
        base = select_outliers(self, w, activation_rms, outlier_columns)
        pw = pack_groupwise_int4(base, group_size, activation_rms)
        self._finish_init(pw, k, n, source.bias)
        self.residual_rank = 0
        self.res_u = None
        self.res_v = None
        if residual_factors is not None:
            u, v = residual_factors
            self.set_residual(u, v)
        elif residual_rank:
            rank = max(0, min(int(residual_rank), min(w.shape)))
            p = pw.packed
            codes = torch.stack([p & 15, p >> 4], -1).reshape(n, -1).to(torch.int16)
            q = ((codes - 8).float() * pw.scales.float().repeat_interleave(pw.group_size, dim=1))[:, :k]
            if self.outlier_idx.numel():
                q[:, self.outlier_idx.long()] += self.outlier_weight.float()
            uu, s, vh = torch.linalg.svd(w.float() - q, full_matrices=False)
            self.set_residual((uu[:, :rank] * s[:rank]), vh[:rank, :])

    def packed_weight(self) -> GroupwiseInt4Weight:
        return GroupwiseInt4Weight(self.packed, self.scales, self.original_k, self.padded_k, self.group_size, True)
