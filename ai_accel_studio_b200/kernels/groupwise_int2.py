"""Groupwise INT2 weight format: 4 codes per byte, one fp16 scale per (row, group), fixed
symmetric levels (-1, -1/3, +1/3, +1) -- there is no zero-point.

Mirrors ``ai_accel_lab/kernels/groupwise_int2.py`` of the reference project:
``GroupwiseInt2Weight`` (:21-37), ``pack_groupwise_int2`` (:66-119), ``unpack_groupwise_int2``
(:122-130), ``reference_linear`` (:133-135) and ``triton_groupwise_int2_linear`` (:194-226).
The quantiser is host logic written with torch ops (it runs where the weight lives, CPU or
CUDA) and is bit-identical to the reference's; everything that touches packed data at run
time is a CUDA kernel of ``libqgemv_b200.so`` and therefore needs CUDA tensors.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

INT2_LEVELS = (-1.0, -1.0 / 3.0, 1.0 / 3.0, 1.0)
_ROW_CHUNK_ELEMS = 1 << 22   # bound the temporaries of the scale search to ~13 * 4 * 4 bytes per element


@dataclass
class GroupwiseInt2Weight:
    packed: torch.Tensor       # uint8 [N, Kpad/4]; byte b = c(4b) | c(4b+1)<<2 | c(4b+2)<<4 | c(4b+3)<<6
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
        return 2.0 + 16.0 / self.group_size


def _padded_float(weight: torch.Tensor, group_size: int, codes_per_byte: int):
    if weight.ndim != 2:
        raise ValueError("weight must be [N,K]")
    if group_size % codes_per_byte:
        raise ValueError(f"group_size must be divisible by {codes_per_byte}")
    w = weight.detach().float()
    k = w.shape[1]
    kp = -(-k // group_size) * group_size
    if kp != k:
        w = F.pad(w, (0, kp - k))
    return w, k, kp


def _activation_weights(activation_rms: torch.Tensor, original_k: int, kp: int, ng: int, group_size: int):
    ar = activation_rms.detach().float().flatten()
    if ar.numel() < original_k:
        raise ValueError("activation_rms is shorter than K")
    ar = F.pad(ar[:original_k], (0, kp - original_k)) if kp > original_k else ar[:kp]
    return ar.view(1, ng, group_size).square().clamp_min(1e-8)


def _levels(ref: torch.Tensor) -> torch.Tensor:
    return torch.tensor(INT2_LEVELS, device=ref.device, dtype=ref.dtype)


def _closest_level(x: torch.Tensor, levels: torch.Tensor) -> torch.Tensor:
    # index of the nearest level; argmin keeps the first index on exact ties
    return (x.unsqueeze(-1) - levels).abs().argmin(-1)


def pack_groupwise_int2(weight: torch.Tensor, group_size: int = 128,
                        activation_rms: torch.Tensor | None = None,
                        refine_steps: int = 13) -> GroupwiseInt2Weight:
    """Quantise ``weight [N,K]`` to packed INT2 codes with a per-group fp16 scale.

    Without ``activation_rms`` the scale of a group is its largest magnitude.  With it, 13
    shrink/grow factors in [0.55, 1.15] are tried per group and the one with the smallest
    activation-energy-weighted squared error wins.  Rows are independent, so they are
    processed in chunks; the result does not depend on the chunking.
    """
    w, original_k, kp = _padded_float(weight, group_size, 4)
    n = w.shape[0]
    ng = kp // group_size
    levels = _levels(w)
    aw = None if activation_rms is None else _activation_weights(activation_rms.to(w.device), original_k, kp, ng, group_size)
    factors = torch.linspace(0.55, 1.15, refine_steps, device=w.device)
    packed = torch.empty((n, kp // 4), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, ng), dtype=torch.float16, device=w.device)
    rows_per_chunk = max(1, _ROW_CHUNK_ELEMS // kp)
    for r0 in range(0, n, rows_per_chunk):
        wg = w[r0:r0 + rows_per_chunk].view(-1, ng, group_size)
        peak = wg.abs().amax(-1).clamp_min(1e-8)
        if aw is None:
            chosen = peak
        else:
            best_err = None
            chosen = None
            for f in factors:
                cand = peak * f
                code = _closest_level(wg / cand.unsqueeze(-1).clamp_min(1e-8), levels)
                q = levels[code] * cand.unsqueeze(-1)
                err = ((q - wg).square() * aw).sum(-1)
                if best_err is None:
                    best_err, chosen = err, cand
                else:
                    better = err < best_err          # strict: the first of equal candidates wins, as argmin does
                    best_err = torch.where(better, err, best_err)
                    chosen = torch.where(better, cand, chosen)
        code = _closest_level((wg / chosen.unsqueeze(-1)).clamp(-1, 1), levels).to(torch.uint8)
        c = code.view(code.shape[0], kp // 4, 4)
        packed[r0:r0 + rows_per_chunk] = c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)
        scales[r0:r0 + rows_per_chunk] = chosen.to(torch.float16)
    return GroupwiseInt2Weight(packed, scales, original_k, kp, group_size, activation_rms is not None)


def _dtype_name(dtype: torch.dtype) -> str:
    if dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError("dequantisation supports float32, float16 and bfloat16")
    return str(dtype).split(".")[-1]


def unpack_groupwise_int2(pw: GroupwiseInt2Weight, dtype=torch.float32) -> torch.Tensor:
    """Dense ``[N, original_k]`` matrix in ``dtype`` (CUDA kernel; bit-identical to the
    reference's ``levels.to(dtype)[codes] * scales.to(dtype)[:, k // group]``)."""
    from .. import ops
    return ops.dequant(pw.packed, pw.scales, 2, pw.group_size, pw.original_k, _dtype_name(dtype))


def unpack_codes_int2(pw: GroupwiseInt2Weight) -> torch.Tensor:
    """uint8 ``[N, padded_k]`` codes in 0..3 (CUDA kernel)."""
    from .. import ops
    return ops.unpack_codes(pw.packed, 2)


def groupwise_int2_linear(x: torch.Tensor, pw: GroupwiseInt2Weight, bias=None) -> torch.Tensor:
    """Any-M linear on packed INT2 weights: the fused GEMV for M <= 4, otherwise CUDA
    dequantisation into ``x.dtype`` followed by a library GEMM.  ``x`` is ``[M, padded_k]``."""
    from .decode_int2 import decode_int2_linear
    if x.ndim != 2 or x.shape[1] != pw.padded_k:
        raise ValueError("x must be [M, padded K]")
    if x.shape[0] <= 4:
        return decode_int2_linear(x, pw, bias)
    w = unpack_groupwise_int2(pw, x.dtype)
    return F.linear(x[:, :pw.original_k], w, None if bias is None else bias.to(x.dtype))


# Names kept from the reference for callers that import them.
triton_groupwise_int2_linear = groupwise_int2_linear


def reference_linear(x: torch.Tensor, pw: GroupwiseInt2Weight, bias=None) -> torch.Tensor:
    """Dequantise-then-matmul in ``x.dtype`` (CUDA dequantisation kernel + library GEMM)."""
    w = unpack_groupwise_int2(pw, dtype=x.dtype)
    return F.linear(x[..., :pw.original_k], w, bias)
