"""Shared construction and forward logic of the hybrid packed Linear modules."""
from __future__ import annotations

import torch
from torch import nn
import torch.nn.functional as F

OUTLIER_COUNTS = (4, 8, 16, 32, 64)


def snap_outlier_count(requested: int, k: int) -> int:
    """Clamp to [0, K], then snap to the nearest of 4/8/16/32/64 (ties go to the smaller
    count), as both reference constructors do (ai_accel_lab/optimize/hybrid_int2.py:34-38,
    hybrid_int4.py:14-15).  The kernels accept any count; the snapping is kept so that modules
    built here hold exactly the columns the reference would pick."""
    oc = max(0, min(int(requested), k))
    if oc and oc not in OUTLIER_COUNTS:
        oc = min(OUTLIER_COUNTS, key=lambda v: abs(v - oc))
        oc = min(oc, k)
    return oc


def select_outliers(module: nn.Module, w: torch.Tensor, activation_rms, outlier_columns: int) -> torch.Tensor:
    """Register ``outlier_idx`` / ``outlier_weight`` and return the weight with those columns zeroed.

    Score = column RMS of W (times the activation RMS when given); the top columns are kept
    exactly in fp16 and removed from the quantised base so the two terms never double count."""
    n, k = w.shape
    oc = snap_outlier_count(outlier_columns, k)
    if not oc:
        module.register_buffer("outlier_idx", torch.empty(0, device=w.device, dtype=torch.int32))
        module.register_buffer("outlier_weight", torch.empty((n, 0), device=w.device, dtype=torch.float16))
        return w
    score = w.float().square().mean(0).sqrt()
    if activation_rms is not None:
        score = score * activation_rms.detach().float().to(w.device)[:k]
    idx = torch.topk(score, k=oc, largest=True, sorted=True).indices
    module.register_buffer("outlier_idx", idx.to(torch.int32))
    module.register_buffer("outlier_weight", w[:, idx].to(torch.float16).contiguous())
    base = w.clone()
    base[:, idx] = 0
    return base


class HybridPackedLinear(nn.Module):
    """Common forward: M <= 4 -> one fused GEMV launch; larger M -> CUDA dequantisation into the
    activation dtype + library GEMMs for the base, outlier and residual terms."""

    bits: int = 0
    residual_rank: int = 0

    def _finish_init(self, pw, k: int, n: int, source_bias):
        self.register_buffer("packed", pw.packed)
        self.register_buffer("scales", pw.scales)
        self.original_k = pw.original_k
        self.padded_k = pw.padded_k
        self.group_size = pw.group_size
        self.in_features = k
        self.out_features = n
        self.graph_safe = False      # toggled by runtime_v5.prepare_static_compile; this build is always graph safe
        self.kernel = "auto"         # "auto" | "simt" | "mma": kernel family for the fused path
        if source_bias is None:
            self.bias = None
        else:
            self.register_buffer("bias", source_bias.detach().to(torch.float16))

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        if self.packed.is_cuda:
            from .. import ops
            ops.ensure_workspace(self.packed.device)   # outside any graph capture, pointer-stable afterwards
        return out

    def _fused(self, xp: torch.Tensor) -> torch.Tensor:
        from .. import _cabi, ops
        return ops.gemv(xp, self.packed, self.scales, self.bias, self.outlier_idx if self.outlier_idx.numel() else None,
                        self.outlier_weight if self.outlier_idx.numel() else None,
                        self.res_u if self.residual_rank else None, self.res_v if self.residual_rank else None,
                        self.bits, self.group_size, self.original_k, 0, _cabi.KERNEL[self.kernel])

    def _dense(self, xflat: torch.Tensor) -> torch.Tensor:
        from .. import ops
        name = str(xflat.dtype).split(".")[-1]
        w = ops.dequant(self.packed, self.scales, self.bits, self.group_size, self.original_k, name)
        y = F.linear(xflat, w, None if self.bias is None else self.bias.to(xflat.dtype))
        if self.outlier_idx.numel():
            y = y + F.linear(xflat[:, self.outlier_idx.long()], self.outlier_weight.to(xflat.dtype))
        if self.residual_rank:
            y = y + F.linear(F.linear(xflat.to(self.res_v.dtype), self.res_v), self.res_u).to(y.dtype)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError(f"{type(self).__name__} computes on CUDA only (no CPU fallback); got a {x.device} tensor")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("fp16/bf16 activations required")
        shape = x.shape
        xflat = x.reshape(-1, shape[-1])
        if xflat.shape[0] <= 4:
            xp = xflat if self.padded_k == self.original_k else F.pad(xflat, (0, self.padded_k - self.original_k))
            if xp.stride(1) != 1:
                xp = xp.contiguous()
            y = self._fused(xp)
        else:
            y = self._dense(xflat)
        return y.reshape(*shape[:-1], self.out_features)
