"""The v5 plan record and the measured decode-speed gate, on the packed modules of this package.

Mirrors the parts of ``ai_accel_lab/optimize/planner_v5.py`` that touch the hot path:
``LayerDecisionV5`` (:10-25, the record a v5 bundle's manifest stores per Linear) and the timed
M = 1 gate ``_runtime_speedups`` (:36-52: 3 warm-ups, 24 CUDA-event repetitions of the dense fp16
Linear against the packed candidate, a small-prefill pair with 12 repetitions, and the projected
speed-up for a given number of decode tokens).  The reference's quality search around the gate
(candidate enumeration, NMSE / cosine limits) is outside this package's scope; ``gate_passes``
is the acceptance rule of ``decide_linear_v5`` (:68, :90).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
import torch.nn.functional as F


@dataclass
class LayerDecisionV5:
    name: str
    method: str
    bits: int
    group_size: int
    outlier_columns: int
    residual_rank: int
    nmse: float
    cosine: float
    compression: float
    decode_speedup: float | None
    prefill_speedup: float | None
    projected_speedup: float | None
    reason: str

    def to_dict(self):
        return asdict(self)


def _cuda_ms(fn, repeats):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    st, en = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    st.record()
    for _ in range(repeats):
        fn()
    en.record()
    en.synchronize()
    return float(st.elapsed_time(en)) / repeats


def runtime_speedups(layer, candidate, x, expected_decode_tokens=64):
    """(decode, prefill, projected) speed-ups of ``candidate`` over the dense ``layer``; ``(None,)*3``
    when the layer is not on a CUDA device (the reference's convention)."""
    if layer.weight.device.type != "cuda":
        return None, None, None
    bias = None if layer.bias is None else layer.bias.to(x.dtype)
    x1 = x[:1].contiguous()
    xp = x[:min(32, x.shape[0])].contiguous()
    w = layer.weight.to(x.dtype)
    d1 = _cuda_ms(lambda: F.linear(x1, w, bias), 24)
    q1 = _cuda_ms(lambda: candidate(x1), 24)
    dp = _cuda_ms(lambda: F.linear(xp, w, bias), 12)
    qp = _cuda_ms(lambda: candidate(xp), 12)
    decode, prefill = d1 / max(q1, 1e-9), dp / max(qp, 1e-9)
    projected = (dp + d1 * expected_decode_tokens) / max(qp + q1 * expected_decode_tokens, 1e-9)
    return decode, prefill, projected


def gate_passes(decode, projected, min_decode_speedup=1.0, min_projected_speedup=1.02) -> bool:
    """A candidate is kept if it could not be timed, or is at least as fast as fp16 for M = 1 and
    at least 2 % faster over prefill + the expected decode tokens."""
    return decode is None or (decode >= min_decode_speedup and projected >= min_projected_speedup)
