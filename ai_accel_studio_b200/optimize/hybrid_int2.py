"""``HybridInt2Linear``: packed groupwise INT2 base + exact fp16 outlier columns + optional
low-rank residual, with the constructor, buffers and forward contract of the reference's
module (ai_accel_lab/optimize/hybrid_int2.py:21-116).

State-dict keys: ``packed`` uint8 [N, Kpad/4], ``scales`` fp16 [N, Kpad/g], ``outlier_idx``
int32 [oc], ``outlier_weight`` fp16 [N, oc], ``bias`` fp16 [N] (only when the source had one),
``res_u`` fp16 [N, r] and ``res_v`` fp16 [r, K] (only when r > 0).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ..kernels.groupwise_int2 import GroupwiseInt2Weight, INT2_LEVELS, pack_groupwise_int2
from ._hybrid_base import HybridPackedLinear, select_outliers


@dataclass
class HybridInfo:
    method: str
    group_size: int
    outlier_columns: int
    residual_rank: int
    original_bytes: int
    optimized_bytes: int
    compression: float


def _dequant_host(pw: GroupwiseInt2Weight) -> torch.Tensor:
    """float32 dequantisation with torch ops, for construction-time error analysis only
    (runs wherever the source weight lives, possibly the CPU)."""
    p = pw.packed
    codes = torch.stack([(p >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).reshape(p.shape[0], -1).long()
    lv = torch.tensor(INT2_LEVELS, device=p.device, dtype=torch.float32)
    s = pw.scales.float().repeat_interleave(pw.group_size, dim=1)
    return (lv[codes] * s)[:, :pw.original_k]


class HybridInt2Linear(HybridPackedLinear):
    """Runtime-only INT2 layer; no dense copy of the source weight is kept."""

    bits = 2

    def __init__(self, source: nn.Linear, group_size=128, activation_rms=None,
                 outlier_columns: int = 0, residual_rank: int = 0, backend="auto"):
        super().__init__()
        w = source.weight.detach()
        n, k = w.shape
        base = select_outliers(self, w, activation_rms, outlier_columns)
        pw = pack_groupwise_int2(base, group_size=group_size, activation_rms=activation_rms)
        self._finish_init(pw, k, n, source.bias)
        self.backend = backend       # accepted for signature compatibility; there is one backend

        rank = max(0, min(int(residual_rank), min(w.shape)))
        self.residual_rank = rank
        if rank:
            q = _dequant_host(pw)
            if self.outlier_idx.numel():
                q[:, self.outlier_idx.long()] += self.outlier_weight.float()
            u, s, vh = torch.linalg.svd(w.float() - q, full_matrices=False)
            self.register_buffer("res_u", (u[:, :rank] * s[:rank]).to(torch.float16).contiguous())
            self.register_buffer("res_v", vh[:rank, :].to(torch.float16).contiguous())
        else:
            self.res_u = None
            self.res_v = None

    def packed_weight(self) -> GroupwiseInt2Weight:
        return GroupwiseInt2Weight(self.packed, self.scales, self.original_k, self.padded_k, self.group_size, True)

    def optimization_info(self) -> HybridInfo:
        def nbytes(t):
            return 0 if t is None else t.numel() * t.element_size()
        orig = self.out_features * self.in_features * 2 + (0 if self.bias is None else self.out_features * 2)
        opt = sum(nbytes(t) for t in (self.packed, self.scales, self.outlier_idx, self.outlier_weight, self.bias))
        if self.residual_rank:
            opt += nbytes(self.res_u) + nbytes(self.res_v)
        return HybridInfo("hybrid-int2", self.group_size, int(self.outlier_idx.numel()), self.residual_rank,
                          orig, opt, orig / max(1, opt))
