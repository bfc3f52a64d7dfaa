"""Groupwise INT4 weight format: 2 codes per byte (even column in the low nibble), one fp16
scale per (row, group), value ``(code - 8) * scale``.

Mirrors ``ai_accel_lab/kernels/groupwise_int4.py`` of the reference project:
``GroupwiseInt4Weight`` (:16-28), ``pack_groupwise_int4`` (:40-60), ``unpack_groupwise_int4``
(:63-69), ``reference_linear`` (:72-73) and ``decode_int4_linear`` (:110-127).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .groupwise_int2 import _activation_weights, _dtype_name, _padded_float, _ROW_CHUNK_ELEMS


@dataclass
class GroupwiseInt4Weight:
    packed: torch.Tensor       # uint8 [N, Kpad/2]; byte b = c(2b) | c(2b+1) << 4
    scales: torch.Tensor       # fp16 [N, Kpad/group_size]
    original_k: int
    padded_k: int
    group_size: int
    activation_aware: bool = False

    @property
    def n(self) -> int:
        return int(self.packed.shape[0])

    @property
    def compression_bits_per_weight(self) -> float:
        return 4.0 + 16.0 / self.group_size


def pack_groupwise_int4(weight: torch.Tensor, group_size: int = 128, activation_rms=None,
                        refine_steps: int = 11) -> GroupwiseInt4Weight:
    """Symmetric round-to-nearest-even INT4 with scale ``max|w| / 7`` per group; with
    ``activation_rms`` the scale is picked among 11 factors in [0.72, 1.18] by the smallest
    activation-energy-weighted squared error.  Row-chunked; chunking does not change the result."""
    w, original_k, kp = _padded_float(weight, group_size, 2)
    n = w.shape[0]
    ng = kp // group_size
    aw = None if activation_rms is None else _activation_weights(activation_rms.to(w.device), original_k, kp, ng, group_size)
    factors = torch.linspace(0.72, 1.18, refine_steps, device=w.device)
    packed = torch.empty((n, kp // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, ng), dtype=torch.float16, device=w.device)
    rows_per_chunk = max(1, _ROW_CHUNK_ELEMS // kp)
    for r0 in range(0, n, rows_per_chunk):
        wg = w[r0:r0 + rows_per_chunk].view(-1, ng, group_size)
        base = (wg.abs().amax(-1) / 7.0).clamp_min(1e-8)
        if aw is None:
            chosen = base
        else:
            best_err = None
            chosen = None
            for f in factors:
                cand = base * f
                q = torch.round(wg / cand.unsqueeze(-1)).clamp(-8, 7)
                err = ((q * cand.unsqueeze(-1) - wg).square() * aw).sum(-1)
                if best_err is None:
                    best_err, chosen = err, cand
                else:
                    better = err < best_err
                    best_err = torch.where(better, err, best_err)
                    chosen = torch.where(better, cand, chosen)
        q = (torch.round(wg / chosen.unsqueeze(-1)).clamp(-8, 7).to(torch.int16) + 8).to(torch.uint8)
        q = q.view(q.shape[0], kp // 2, 2)
        packed[r0:r0 + rows_per_chunk] = q[..., 0] | (q[..., 1] << 4)
        scales[r0:r0 + rows_per_chunk] = chosen.to(torch.float16)
    return GroupwiseInt4Weight(packed, scales, original_k, kp, group_size, activation_rms is not None)


def unpack_groupwise_int4(pw: GroupwiseInt4Weight, dtype=torch.float32) -> torch.Tensor:
    """Dense ``[N, original_k]`` matrix in ``dtype`` (CUDA kernel, bit-identical to the reference)."""
    from .. import ops
    return ops.dequant(pw.packed, pw.scales, 4, pw.group_size, pw.original_k, _dtype_name(dtype))


def unpack_codes_int4(pw: GroupwiseInt4Weight) -> torch.Tensor:
    """uint8 ``[N, padded_k]`` codes in 0..15 (CUDA kernel)."""
    from .. import ops
    return ops.unpack_codes(pw.packed, 4)


def reference_linear(x, pw: GroupwiseInt4Weight, bias=None):
    return F.linear(x[..., :pw.original_k], unpack_groupwise_int4(pw, x.dtype), bias)


def decode_int4_linear(x: torch.Tensor, pw: GroupwiseInt4Weight, bias=None, outlier_idx=None,
                       outlier_weight=None, res_u=None, res_v=None, kernel: str = "auto") -> torch.Tensor:
    """Fused INT4 GEMV for ``x [M, padded_k]``, M <= 4, fp16/bf16, on CUDA.

    Same contract as the reference's ``decode_int4_linear`` (groupwise_int4.py:110-127) with two
    extensions: any number of outlier columns is accepted, and an optional rank-r residual
    ``res_u [N,r]``, ``res_v [r,K]`` is folded into the same launch.
    """
    from .decode_int2 import _fused
    return _fused(4, x, pw, bias, outlier_idx, outlier_weight, res_u, res_v, "none", kernel)
