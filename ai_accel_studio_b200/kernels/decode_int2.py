"""Decode-specialised (M <= 4) fused GEMV on packed groupwise weights.

Mirrors ``ai_accel_lab/kernels/decode_int2.py`` of the reference project:
``decode_int2_linear`` (:99-144) and ``reference_hybrid_linear`` (:147-151).  Unpack,
group-scale dequantisation, exact-fp16 outlier columns, low-rank residual, bias and activation
all happen in one launch of the sm_100a kernel; weights are streamed once for all M rows.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _cabi
from .groupwise_int2 import GroupwiseInt2Weight, reference_linear


_CALLS: dict = {}        # prepared launches of the functional interface (eager calls), see _fused
_MAX_CALLS = 64


def _as_half(t, device):
    if t is None:
        return None
    if t.dtype != torch.float16 or t.device != device:
        t = t.to(device=device, dtype=torch.float16)
    return t if t.stride(-1) == 1 or t.numel() == 0 else t.contiguous()


def _fused(bits, x, pw, bias, outlier_idx, outlier_weight, res_u, res_v, activation, kernel):
    from .. import ops
    if not x.is_cuda:
        raise RuntimeError("CUDA is required: the packed decode path has no CPU implementation")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("decode path requires fp16/bf16 activations")
    if x.ndim != 2 or x.shape[0] > 4:
        raise ValueError("decode-specialized path is for [M,K] with M<=4")
    if x.shape[1] != pw.padded_k:
        raise ValueError("input must already be padded to packed K")
    act = _cabi.ACT.get(activation)
    if act is None:
        raise ValueError(activation)
    if kernel not in _cabi.KERNEL:
        raise ValueError(kernel)
    dev = x.device
    if outlier_idx is None or outlier_weight is None or outlier_idx.numel() == 0:
        oi = ow = None
    else:
        oi = outlier_idx if (outlier_idx.dtype == torch.int32 and outlier_idx.device == dev) \
            else outlier_idx.to(device=dev, dtype=torch.int32)
        oi = oi.contiguous()
        ow = _as_half(outlier_weight, dev)
    if res_u is None or res_v is None or res_u.numel() == 0:
        ru = rv = None
    else:
        ru, rv = _as_half(res_u, dev), _as_half(res_v, dev)
    if x.stride(1) != 1:
        x = x.contiguous()
    b16 = _as_half(bias, dev)
    if torch.compiler.is_compiling():          # the registered operator only where a tracer needs it
        return ops.gemv(x, pw.packed, pw.scales, b16, oi, ow, ru, rv, bits, pw.group_size, pw.original_k, act,
                        _cabi.KERNEL[kernel])
    # Eager: reuse the prepared launch for these operands.  Keyed by the addresses AND shapes of the tensors of THIS
    # call, so a hit means the struct's pointers are exactly the ones passed now (the cache holds no tensor alive, and
    # a recycled address with other dimensions never meets a stale struct).
    ptr = lambda t: 0 if t is None else t.data_ptr()
    key = (bits, x.shape[0], x.dtype, x.stride(0), dev, pw.packed.data_ptr(), tuple(pw.packed.shape), pw.packed.stride(0),
           pw.scales.data_ptr(), tuple(pw.scales.shape), pw.group_size, pw.original_k, ptr(b16), ptr(oi), ptr(ow),
           0 if oi is None else oi.numel(), ptr(ru), ptr(rv), 0 if ru is None else ru.shape[1], act, kernel)
    call = _CALLS.get(key)
    if call is None:
        if len(_CALLS) >= _MAX_CALLS:
            _CALLS.clear()
        call = _CALLS[key] = ops.prepare_call(x, pw.packed, pw.scales, b16, oi, ow, ru, rv, bits, pw.group_size,
                                              pw.original_k, act, _cabi.KERNEL[kernel], None, key)
    return call.run(x)


def decode_int2_linear(x: torch.Tensor, pw: GroupwiseInt2Weight, bias: torch.Tensor | None = None,
                       outlier_idx: torch.Tensor | None = None, outlier_weight: torch.Tensor | None = None,
                       activation: str = "none", res_u: torch.Tensor | None = None,
                       res_v: torch.Tensor | None = None, kernel: str = "auto") -> torch.Tensor:
    """Fused INT2 GEMV for ``x [M, padded_k]``, M <= 4, fp16/bf16, on CUDA.

    Arguments up to ``activation`` are the reference's; ``res_u``/``res_v`` add the low-rank
    residual to the same launch and ``kernel`` ("auto" | "simt" | "mma") pins a kernel family.
    Unlike the reference, the outlier count is not restricted to 4/8/16/32/64.
    Bias, outlier weights and residual factors are read as fp16 whatever the type of ``x``.
    """
    return _fused(2, x, pw, bias, outlier_idx, outlier_weight, res_u, res_v, activation, kernel)


def reference_hybrid_linear(x, pw, bias=None, outlier_idx=None, outlier_weight=None):
    """Unfused formulation: dequantise + matmul, then the outlier matmul (library GEMMs)."""
    y = reference_linear(x, pw, bias)
    if outlier_idx is not None and outlier_weight is not None and outlier_idx.numel():
        y = y + F.linear(x[..., outlier_idx.long()], outlier_weight.to(x.dtype))
    return y
