"""CPU oracle for the packed groupwise INT2 / INT4 small-M GEMV path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain numpy, the arithmetic
of the reference project's (ai_accel_lab v5.0.0) groupwise quantisers, unpackers
and its torch "dequant + matmul" CPU path.  It exists so that the CUDA kernels can
be checked against an independent implementation.  Only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may import it; the product
package never does and has no CPU fallback.

Parity pin: every function here is checked in ``tests/test_oracle_golden.py``
against fixtures under ``tests/golden/`` that were produced by importing and
running the reference's own Python code (``tests/golden/make_golden.py``).

Reference locations restated here (paths inside the reference project):
  * INT2 codebook ................ ai_accel_lab/kernels/groupwise_int2.py:18
  * zero padding of K ............ ai_accel_lab/kernels/groupwise_int2.py:40-51
  * INT2 quantise + pack ......... ai_accel_lab/kernels/groupwise_int2.py:66-119
  * INT2 unpack .................. ai_accel_lab/kernels/groupwise_int2.py:122-130
  * INT4 quantise + pack ......... ai_accel_lab/kernels/groupwise_int4.py:40-60
  * INT4 unpack .................. ai_accel_lab/kernels/groupwise_int4.py:63-69
  * dequant + matmul ............. ai_accel_lab/kernels/groupwise_int2.py:133-135,
                                   ai_accel_lab/kernels/groupwise_int4.py:72-73
  * outlier-column term .......... ai_accel_lab/kernels/decode_int2.py:147-151
  * hybrid module construction ... ai_accel_lab/optimize/hybrid_int2.py:29-75,
                                   ai_accel_lab/optimize/hybrid_int4.py:12-27
  * hybrid forward (CPU branch) .. ai_accel_lab/optimize/hybrid_int2.py:80-107,
                                   ai_accel_lab/optimize/hybrid_int4.py:29-38
  * fused-kernel epilogue order .. ai_accel_lab/kernels/decode_int2.py:79-96
"""
from __future__ import annotations

from dataclasses import dataclass
import math

import numpy as np

F32 = np.float32
F16 = np.float16

# groupwise_int2.py:18 -- the four symmetric levels, as float32 constants.
INT2_LEVELS_F32 = np.array([-1.0, -1.0 / 3.0, 1.0 / 3.0, 1.0], dtype=F32)
OUTLIER_COUNTS = (4, 8, 16, 32, 64)  # hybrid_int2.py:35-38


@dataclass
class PackedWeight:
    """Packed groupwise weight: uint8 codes and one fp16 scale per (row, group)."""
    bits: int                 # 2 or 4
    packed: np.ndarray        # uint8 [N, Kpad*bits/8]
    scales: np.ndarray        # float16 [N, Kpad/group]
    original_k: int
    padded_k: int
    group_size: int

    @property
    def n(self) -> int:
        return int(self.packed.shape[0])


# --------------------------------------------------------------------------- #
# helpers
# --------------------------------------------------------------------------- #
def torch_linspace_f32(start: float, end: float, steps: int) -> np.ndarray:
    """float32 linspace with the two-sided, fused-multiply-add formula torch uses on CPU.

    ``step`` is computed in float32; the first half is ``fma(step, i, start)`` and the
    second half ``fma(-step, steps-1-i, end)``.  A float64 product of a float32 by a small
    integer is exact, so one rounding of the float64 sum reproduces the fused operation.
    (numpy's own linspace rounds differently in the last bit.)
    """
    start32, end32 = F32(start), F32(end)
    step = F32((end32 - start32) / F32(steps - 1))
    out = np.empty(steps, dtype=F32)
    half = steps // 2
    for i in range(steps):
        if i < half:
            out[i] = F32(np.float64(start32) + np.float64(step) * i)
        else:
            out[i] = F32(np.float64(end32) - np.float64(step) * (steps - 1 - i))
    return out


def pad_k(weight: np.ndarray, group_size: int, bits: int):
    """groupwise_int2.py:40-51 / groupwise_int4.py:31-37: zero-pad K up to a multiple of the group."""
    if weight.ndim != 2:
        raise ValueError("weight must be [N,K]")
    if group_size % (8 // bits):
        raise ValueError("group_size must be divisible by the codes per byte")
    n, k = weight.shape
    kp = math.ceil(k / group_size) * group_size
    w = np.zeros((n, kp), dtype=F32)
    w[:, :k] = weight.astype(F32)
    return w, k


def _nearest_int2(x: np.ndarray) -> np.ndarray:
    """groupwise_int2.py:54-56: index of the closest level, first index on ties."""
    d = np.abs(x[..., None] - INT2_LEVELS_F32)
    return d.argmin(-1).astype(np.uint8)


def _act_weights(activation_rms, original_k, kp, ng, group_size):
    ar = np.asarray(activation_rms, dtype=F32).reshape(-1)
    if ar.size < original_k:
        raise ValueError("activation_rms is shorter than K")
    if kp > original_k:
        ar = np.concatenate([ar[:original_k], np.zeros(kp - original_k, dtype=F32)])
    else:
        ar = ar[:kp]
    return np.maximum(np.square(ar.reshape(1, ng, group_size)), F32(1e-8)).astype(F32)


def _rowsum_f32(a: np.ndarray) -> np.ndarray:
    # float32 accumulation over the last axis (numpy uses pairwise summation,
    # torch a vectorised cascade; both are float32 and differ only in the last
    # ulp, which matters solely for exact ties between candidate scales).
    return a.sum(-1, dtype=F32)


# --------------------------------------------------------------------------- #
# INT2
# --------------------------------------------------------------------------- #
def pack_int2(weight, group_size=128, activation_rms=None, refine_steps=13, row_chunk=256) -> PackedWeight:
    """groupwise_int2.py:66-119.  Rows are independent, so the work is chunked by rows."""
    w, original_k = pad_k(np.asarray(weight), group_size, 2)
    n, kp = w.shape
    ng = kp // group_size
    packed = np.empty((n, kp // 4), dtype=np.uint8)
    scales16 = np.empty((n, ng), dtype=F16)
    aw = None if activation_rms is None else _act_weights(activation_rms, original_k, kp, ng, group_size)
    factors = torch_linspace_f32(0.55, 1.15, refine_steps)
    for r0 in range(0, n, row_chunk):
        wg = w[r0:r0 + row_chunk].reshape(-1, ng, group_size)
        base = np.maximum(np.abs(wg).max(-1), F32(1e-8)).astype(F32)          # :82
        if aw is not None:                                                    # :85-105
            errs = []
            cands = []
            for f in factors:
                cand = (base * f).astype(F32)
                x = wg / np.maximum(cand, F32(1e-8))[..., None]
                code = np.abs(x[..., None] - INT2_LEVELS_F32).argmin(-1)
                q = INT2_LEVELS_F32[code] * cand[..., None]
                errs.append(_rowsum_f32(np.square(q - wg) * aw))
                cands.append(cand)
            best = np.stack(errs, 0).argmin(0)
            scales = np.take_along_axis(np.stack(cands, -1), best[..., None], -1)[..., 0]
        else:
            scales = base
        q = _nearest_int2(np.clip(wg / scales[..., None], F32(-1), F32(1)))    # :109
        q = q.reshape(q.shape[0], kp // 4, 4)
        packed[r0:r0 + row_chunk] = q[..., 0] | (q[..., 1] << 2) | (q[..., 2] << 4) | (q[..., 3] << 6)  # :110-111
        scales16[r0:r0 + row_chunk] = scales.astype(F16)                       # :114
    return PackedWeight(2, packed, scales16, original_k, kp, group_size)


def unpack_codes_int2(packed: np.ndarray) -> np.ndarray:
    """groupwise_int2.py:123-124: code of column 4b+i sits in bits 2i..2i+1 of byte b."""
    p = packed.astype(np.uint8)
    return np.stack([(p >> (2 * i)) & 3 for i in range(4)], -1).reshape(p.shape[0], -1)


# --------------------------------------------------------------------------- #
# INT4
# --------------------------------------------------------------------------- #
def pack_int4(weight, group_size=128, activation_rms=None, refine_steps=11, row_chunk=256) -> PackedWeight:
    """groupwise_int4.py:40-60."""
    w, original_k = pad_k(np.asarray(weight), group_size, 4)
    n, kp = w.shape
    ng = kp // group_size
    packed = np.empty((n, kp // 2), dtype=np.uint8)
    scales16 = np.empty((n, ng), dtype=F16)
    aw = None if activation_rms is None else _act_weights(activation_rms, original_k, kp, ng, group_size)
    factors = torch_linspace_f32(0.72, 1.18, refine_steps)
    for r0 in range(0, n, row_chunk):
        wg = w[r0:r0 + row_chunk].reshape(-1, ng, group_size)
        base = np.maximum((np.abs(wg).max(-1) / F32(7.0)).astype(F32), F32(1e-8))   # :43
        if aw is not None:                                                          # :45-55
            errs = []
            cands = []
            for f in factors:
                cand = (base * f).astype(F32)
                q = np.clip(np.rint(wg / cand[..., None]), -8, 7).astype(F32)
                errs.append(_rowsum_f32(np.square(q * cand[..., None] - wg) * aw))
                cands.append(cand)
            best = np.stack(errs, 0).argmin(0)
            scales = np.take_along_axis(np.stack(cands, -1), best[..., None], -1)[..., 0]
        else:
            scales = base
        q = (np.clip(np.rint(wg / scales[..., None]), -8, 7).astype(np.int16) + 8).astype(np.uint8)  # :57
        q = q.reshape(q.shape[0], kp // 2, 2)
        packed[r0:r0 + row_chunk] = q[..., 0] | (q[..., 1] << 4)                     # :58-59
        scales16[r0:r0 + row_chunk] = scales.astype(F16)
    return PackedWeight(4, packed, scales16, original_k, kp, group_size)


def unpack_codes_int4(packed: np.ndarray) -> np.ndarray:
    """groupwise_int4.py:64-65: even column in the low nibble."""
    p = packed.astype(np.uint8)
    return np.stack([p & 15, (p >> 4) & 15], -1).reshape(p.shape[0], -1)


def unpack_codes(pw: PackedWeight) -> np.ndarray:
    return unpack_codes_int2(pw.packed) if pw.bits == 2 else unpack_codes_int4(pw.packed)


# --------------------------------------------------------------------------- #
# dequantisation
# --------------------------------------------------------------------------- #
def dequant(pw: PackedWeight, dtype=F32) -> np.ndarray:
    """unpack_groupwise_int2 / unpack_groupwise_int4 in ``dtype`` (float32 or float16).

    float32: ``level_f32 * float32(scale_f16)`` -- one rounding.
    float16: the level is first rounded to float16, then the float16 product is
    rounded once more (what torch does for ``vals * scales`` in half precision).
    """
    codes = unpack_codes(pw).astype(np.int64)
    if pw.bits == 2:
        vals = INT2_LEVELS_F32.astype(dtype)[codes]
    else:
        vals = (codes - 8).astype(dtype)
    gids = np.arange(pw.padded_k) // pw.group_size
    s = pw.scales.astype(dtype)[:, gids]
    out = (vals * s).astype(dtype)
    return out[:, :pw.original_k]


# --------------------------------------------------------------------------- #
# linear / hybrid forward
# --------------------------------------------------------------------------- #
def _act(y, activation):
    if activation in (None, "none"):
        return y
    if activation == "relu":
        return np.maximum(y, 0)
    if activation in ("silu", "swish"):
        return y / (1.0 + np.exp(-y))
    raise ValueError(activation)


def gemv_f32(x, pw: PackedWeight, bias=None, outlier_idx=None, outlier_weight=None,
             res_u=None, res_v=None, activation="none", acc=np.float64) -> np.ndarray:
    """The tolerance target: every term in exact-ish arithmetic on float32 dequant.

    y = x[:, :K] . dequant_f32(W)^T  + x[:, idx] . OW^T + (x[:, :K] . V^T) . U^T + bias, then
    activation.  Products are formed from the fp16/bf16 inputs widened to ``acc``
    (float64 by default, so the summation order does not matter).  The epilogue
    order (base, outliers, bias, activation) follows decode_int2.py:79-96; the
    residual follows hybrid_int2.py:104-106 and is added before the activation
    only because the module never combines the two.
    Returns float64/float32 [M, N]; the caller compares the kernel's fp16 result to it.
    """
    x = np.asarray(x)
    xf = x.astype(acc)
    k = pw.original_k
    w = dequant(pw, F32).astype(acc)
    y = xf[:, :k] @ w.T
    if outlier_idx is not None and outlier_weight is not None and np.size(outlier_idx):
        idx = np.asarray(outlier_idx).astype(np.int64)
        y = y + xf[:, idx] @ np.asarray(outlier_weight).astype(acc).T
    if res_u is not None and res_v is not None and np.size(res_u):
        kv = np.asarray(res_v).shape[1]
        t = xf[:, :kv] @ np.asarray(res_v).astype(acc).T
        y = y + t @ np.asarray(res_u).astype(acc).T
    if bias is not None:
        y = y + np.asarray(bias).astype(acc)
    return _act(y, activation)


def _half_matmul(a16: np.ndarray, b16_t: np.ndarray) -> np.ndarray:
    """fp16 x fp16 -> fp16 matmul the way torch's CPU half GEMM behaves: float32
    accumulation of exact products, one rounding of the result to float16."""
    return (a16.astype(F32) @ b16_t.astype(F32).T).astype(F16)


def reference_forward_f16(x16, pw: PackedWeight, bias=None, outlier_idx=None, outlier_weight=None,
                          res_u=None, res_v=None) -> np.ndarray:
    """The reference modules' CPU branch in float16, step for step.

    hybrid_int2.py:100-106 / hybrid_int4.py:36-37: dequantise the whole matrix to
    x.dtype, ``F.linear`` (bias added inside), ``+ F.linear(x[:, idx], outlier_weight)``,
    ``+ F.linear(F.linear(x, V), U)`` -- each op rounding its result to float16.
    """
    x16 = np.asarray(x16, dtype=F16)
    k = pw.original_k
    w16 = dequant(pw, F16)
    acc = x16[:, :k].astype(F32) @ w16.astype(F32).T
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=F16).astype(F32)
    y = acc.astype(F16)
    if outlier_idx is not None and np.size(outlier_idx):
        idx = np.asarray(outlier_idx).astype(np.int64)
        y = (y.astype(F32) + _half_matmul(x16[:, idx], np.asarray(outlier_weight, dtype=F16)).astype(F32)).astype(F16)
    if res_u is not None and np.size(res_u):
        t = _half_matmul(x16[:, :k], np.asarray(res_v, dtype=F16))
        corr = _half_matmul(t, np.asarray(res_u, dtype=F16))
        y = (y.astype(F32) + corr.astype(F32)).astype(F16)
    return y


# --------------------------------------------------------------------------- #
# hybrid module construction
# --------------------------------------------------------------------------- #
def snap_outlier_count(requested: int, k: int) -> int:
    """hybrid_int2.py:34-38: clamp to [0,K]; snap to the nearest of 4/8/16/32/64, ties to the smaller."""
    oc = max(0, min(int(requested), k))
    if oc and oc not in OUTLIER_COUNTS:
        oc = min(OUTLIER_COUNTS, key=lambda v: abs(v - oc))
        oc = min(oc, k)
    return oc


@dataclass
class HybridLayer:
    bits: int
    pw: PackedWeight
    outlier_idx: np.ndarray      # int32 [oc]
    outlier_weight: np.ndarray   # float16 [N, oc]
    bias: np.ndarray | None      # float16 [N]
    res_u: np.ndarray | None     # float16 [N, r]
    res_v: np.ndarray | None     # float16 [r, K]


def build_hybrid(weight, bits, group_size=128, activation_rms=None, outlier_columns=0,
                 residual_rank=0, bias=None) -> HybridLayer:
    """hybrid_int2.py:29-75 (bits=2) and hybrid_int4.py:12-27 (bits=4; no residual there)."""
    w = np.asarray(weight)
    n, k = w.shape
    oc = snap_outlier_count(outlier_columns, k)
    wf = w.astype(F32)
    if oc:
        wrms = np.sqrt(np.mean(np.square(wf), axis=0, dtype=F32)).astype(F32)
        score = wrms if activation_rms is None else wrms * np.asarray(activation_rms, dtype=F32)[:k]
        # topk(largest, sorted): descending score; stable so equal scores keep the lower index first
        idx = np.argsort(-score, kind="stable")[:oc]
        exact = w[:, idx].astype(F16)
        base = w.copy()
        base[:, idx] = 0
        oidx = idx.astype(np.int32)
    else:
        base = w
        oidx = np.empty(0, dtype=np.int32)
        exact = np.empty((n, 0), dtype=F16)
    pw = (pack_int2 if bits == 2 else pack_int4)(base, group_size, activation_rms)
    b16 = None if bias is None else np.asarray(bias).astype(F16)
    rank = max(0, min(int(residual_rank), min(w.shape)))
    ru = rv = None
    if rank:
        q = dequant(pw, F32).copy()
        if oc:
            q[:, oidx.astype(np.int64)] += exact.astype(F32)
        err = wf - q
        u, s, vh = np.linalg.svd(err, full_matrices=False)
        ru = (u[:, :rank] * s[:rank]).astype(F16)
        rv = vh[:rank, :].astype(F16)
    return HybridLayer(bits, pw, oidx, exact, b16, ru, rv)


def algorithmic_bytes(m, n, kpad, k, bits, group, oc=0, rank=0, has_bias=False) -> int:
    """Bytes one GEMV must move if every operand is touched exactly once."""
    b = n * kpad * bits // 8 + n * (kpad // group) * 2
    if oc:
        b += n * oc * 2 + oc * 4
    if rank:
        b += n * rank * 2 + rank * k * 2
    if has_bias:
        b += n * 2
    b += m * kpad * 2 + m * n * 2
    return b
