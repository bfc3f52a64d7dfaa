"""The v5 per-layer planner on the packed modules of this package.

Mirrors ``ai_accel_lab/optimize/planner_v5.py`` and the INT2 search it builds on
(``ai_accel_lab/optimize/planner_v4.py``):

* ``quality`` (planner_v4.py:22-25): normalised MSE and mean row cosine of a candidate's output.
* ``decide_linear_v4`` (planner_v4.py:27-71): INT2 candidates over group sizes x outlier counts without a
  residual; the passing candidate with the highest compression wins (ties: lower NMSE, higher
  cosine); if none passes, the two most accurate ones are retried with each residual rank and the
  first that passes is taken; otherwise the layer stays fp16.
* ``LayerDecisionV5`` (planner_v5.py:10-25), the record a v5 bundle's manifest stores per Linear.
* ``runtime_speedups`` (planner_v5.py:36-52): the timed gate -- 3 warm-ups, 24 CUDA-event
  repetitions of the dense fp16 Linear against the packed candidate at M = 1, a small-prefill pair
  with 12 repetitions, and the projected speed-up for a number of decode tokens.
* ``decide_linear_v5`` (planner_v5.py:55-106): INT2 first (quality search, then the gate); a layer
  whose INT2 candidate fails quality or the gate is tried as INT4 (group sizes x outlier counts,
  best compression first, each timed until one passes); otherwise fp16.
* ``build_plan_v5`` (planner_v5.py:109-117).

Differences from the reference, all forced by this package having a CUDA-only forward: the
quality of a candidate held on the CPU is measured through its reconstructed float32 weight
(``HybridPackedLinear.effective_weight``) instead of a CPU forward; on a CUDA device the module's
own forward is used, as in the reference.  A candidate whose construction raises is skipped, as
there.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
import torch.nn.functional as F
from torch import nn

from .hybrid_int2 import HybridInt2Linear
from .hybrid_int4 import HybridInt4Linear


@dataclass
class LayerDecisionV4:
    name: str
    method: str
    group_size: int
    outlier_columns: int
    residual_rank: int
    nmse: float
    cosine: float
    compression: float
    reason: str

    def to_dict(self):
        return asdict(self)


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


@dataclass
class _Trial:
    nmse: float
    cosine: float
    compression: float
    group_size: int
    outlier_columns: int
    residual_rank: int

    def passes(self, nmse_limit, cosine_limit, min_compression) -> bool:
        return self.nmse <= nmse_limit and self.cosine >= cosine_limit and self.compression >= min_compression

    @property
    def preference(self):
        """Sort key of the reference: compression first, then accuracy."""
        return (self.compression, -self.nmse, self.cosine)


def quality(ref: torch.Tensor, cand: torch.Tensor):
    """(normalised mean squared error, mean cosine similarity of rows) of ``cand`` against ``ref``."""
    ref32, cand32 = ref.float(), cand.float()
    nmse = (cand32 - ref32).square().mean().item() / (ref32.square().mean().item() + 1e-12)
    rows = ref32.shape[0]
    cosine = F.cosine_similarity(ref32.reshape(rows, -1), cand32.reshape(rows, -1), dim=-1).mean().item()
    return nmse, cosine


def _output(candidate, x: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        if x.is_cuda:
            return candidate(x)
        bias = None if candidate.bias is None else candidate.bias.to(x.dtype)
        return F.linear(x, candidate.effective_weight().to(x.dtype), bias)


def _compression(layer: nn.Linear, cand) -> float:
    def nbytes(t):
        return 0 if t is None else t.numel() * t.element_size()
    orig = layer.weight.numel() * 2 + (0 if layer.bias is None else layer.bias.numel() * 2)
    opt = sum(nbytes(t) for t in (cand.packed, cand.scales, cand.outlier_idx, cand.outlier_weight, cand.bias))
    if getattr(cand, "residual_rank", 0):
        opt += nbytes(cand.res_u) + nbytes(cand.res_v)
    return orig / max(1, opt)


def _sample(layer: nn.Linear, sample_x: torch.Tensor):
    dev = layer.weight.device
    dt = torch.float16 if dev.type == "cuda" else torch.float32
    x = sample_x.to(dev, dtype=dt)
    rms = sample_x.float().square().mean(0).sqrt().to(dev)
    with torch.no_grad():
        ref = F.linear(x, layer.weight.to(dt), None if layer.bias is None else layer.bias.to(dt))
    return x, rms, ref


def _grid(make, layer, x, ref, group_sizes, outliers):
    """Every (group size, outlier count) candidate that can be built, measured."""
    trials = []
    for g in group_sizes:
        if layer.in_features < g:
            continue
        for oc in outliers:
            if oc >= layer.in_features:
                continue
            try:
                cand = make(g, oc, 0)
                nm, co = quality(ref, _output(cand, x))
                trials.append(_Trial(nm, co, _compression(layer, cand), g, oc, 0))
                del cand
            except Exception:
                continue
    return trials


def decide_linear_v4(name, layer, sample_x, group_sizes=(128, 64, 32), outliers=(0, 8, 16, 32), residual_ranks=(0, 4, 8),
                     nmse_limit=.06, cosine_limit=.96, min_compression=1.5) -> LayerDecisionV4:
    dev = layer.weight.device
    x, rms, ref = _sample(layer, sample_x)
    limits = (nmse_limit, cosine_limit, min_compression)

    def make(g, oc, rank):
        return HybridInt2Linear(layer, g, rms, oc, rank, "auto").to(dev)

    trials = _grid(make, layer, x, ref, group_sizes, outliers)
    good = [t for t in trials if t.passes(*limits)]
    if good:
        b = max(good, key=lambda t: t.preference)
        return LayerDecisionV4(name, "int2-outlier" if b.outlier_columns else "int2", b.group_size, b.outlier_columns, 0,
                               b.nmse, b.cosine, b.compression, "passes local guard")
    # the SVD is expensive: only the two most accurate rank-0 candidates get a residual
    for seed in sorted(trials, key=lambda t: (t.nmse, -t.cosine))[:2]:
        for rank in (r for r in residual_ranks if r > 0):
            try:
                cand = make(seed.group_size, seed.outlier_columns, rank)
                nm, co = quality(ref, _output(cand, x))
                t = _Trial(nm, co, _compression(layer, cand), seed.group_size, seed.outlier_columns, rank)
                del cand
            except Exception:
                continue
            trials.append(t)
            if t.passes(*limits):
                return LayerDecisionV4(name, "int2-outlier-residual", t.group_size, t.outlier_columns, rank, t.nmse, t.cosine,
                                       t.compression, "passes local guard with residual")
    if not trials:
        return LayerDecisionV4(name, "fp16", 128, 0, 0, float("inf"), 0.0, 1.0, "no viable quantized candidate")
    b = min(trials, key=lambda t: t.nmse)
    return LayerDecisionV4(name, "fp16", b.group_size, b.outlier_columns, b.residual_rank, b.nmse, b.cosine, 1.0,
                           "kept dense: local guard failed")


def build_plan_v4(model, captures, group_sizes=(128, 64, 32), outliers=(0, 8, 16, 32), residual_ranks=(0, 4, 8),
                  nmse_limit=.06, cosine_limit=.96, min_compression=1.5):
    """One ``LayerDecisionV4`` per captured ``nn.Linear`` (``ai_accel_lab/optimize/planner_v4.py:73-81``)."""
    mods = dict(model.named_modules())
    return [decide_linear_v4(name, mods[name], x, group_sizes, outliers, residual_ranks, nmse_limit, cosine_limit, min_compression)
            for name, x in captures.items() if isinstance(mods.get(name), nn.Linear)]


GATE_WARMUPS, GATE_DECODE_REPEATS, GATE_PREFILL_REPEATS, GATE_PREFILL_ROWS = 3, 24, 12, 32   # the reference's protocol


def _mean_ms(call, repeats: int, warmups: int = GATE_WARMUPS) -> float:
    """Mean milliseconds of ``call`` over ``repeats`` eager invocations between two CUDA events."""
    for _ in range(warmups):
        call()
    torch.cuda.synchronize()
    begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
    begin.record()
    for _ in range(repeats):
        call()
    end.record()
    end.synchronize()
    return begin.elapsed_time(end) / repeats


@dataclass
class GateTiming:
    """Eager milliseconds of the dense layer and of the packed candidate for one decode row and for a small prefill."""
    dense_decode: float
    packed_decode: float
    dense_prefill: float
    packed_prefill: float

    def speedups(self, expected_decode_tokens: int):
        """(decode, prefill, projected over one prefill + ``expected_decode_tokens`` decode steps)."""
        tiny = 1e-9
        dense_total = self.dense_prefill + expected_decode_tokens * self.dense_decode
        packed_total = self.packed_prefill + expected_decode_tokens * self.packed_decode
        return (self.dense_decode / max(self.packed_decode, tiny), self.dense_prefill / max(self.packed_prefill, tiny),
                dense_total / max(packed_total, tiny))


def time_gate(layer, candidate, x) -> GateTiming:
    """Time ``candidate`` against ``F.linear`` with the dense layer's weight on the first row and on the first
    ``GATE_PREFILL_ROWS`` rows of ``x`` (``ai_accel_lab/optimize/planner_v5.py:36-52``)."""
    weight = layer.weight.to(x.dtype)
    bias = None if layer.bias is None else layer.bias.to(x.dtype)
    timings = {}
    for label, rows, repeats in (("decode", 1, GATE_DECODE_REPEATS), ("prefill", min(GATE_PREFILL_ROWS, x.shape[0]), GATE_PREFILL_REPEATS)):
        sample = x[:rows].contiguous()
        timings["dense_" + label] = _mean_ms(lambda: F.linear(sample, weight, bias), repeats)
        timings["packed_" + label] = _mean_ms(lambda: candidate(sample), repeats)
    return GateTiming(**timings)


def runtime_speedups(layer, candidate, x, expected_decode_tokens=64):
    """(decode, prefill, projected) speed-ups of ``candidate`` over the dense ``layer``; ``(None,)*3``
    when the layer is not on a CUDA device (the reference's convention)."""
    if layer.weight.device.type != "cuda":
        return None, None, None
    return time_gate(layer, candidate, x).speedups(expected_decode_tokens)


def gate_passes(decode, projected, min_decode_speedup=1.0, min_projected_speedup=1.02) -> bool:
    """A candidate is kept if it could not be timed, or is at least as fast as fp16 for M = 1 and
    at least 2 % faster over prefill + the expected decode tokens."""
    return decode is None or (decode >= min_decode_speedup and projected >= min_projected_speedup)


def _timed(make, layer, x, expected_decode_tokens):
    try:
        cand = make()
        out = runtime_speedups(layer, cand, x, expected_decode_tokens)
        del cand
        return out
    except Exception:
        return None, None, None


def decide_linear_v5(name, layer, sample_x, group_sizes=(128, 64, 32), outliers=(0, 8, 16, 32), residual_ranks=(0, 4, 8),
                     nmse_limit=.06, cosine_limit=.96, min_compression=1.45, min_decode_speedup=1.0,
                     min_projected_speedup=1.02, expected_decode_tokens=64) -> LayerDecisionV5:
    dev = layer.weight.device
    x, rms, ref = _sample(layer, sample_x)

    d2 = decide_linear_v4(name, layer, sample_x, group_sizes, outliers, residual_ranks, nmse_limit, cosine_limit, min_compression)
    int2_too_slow = False
    if d2.method != "fp16":
        sp, ps, proj = _timed(lambda: HybridInt2Linear(layer, d2.group_size, rms, d2.outlier_columns, d2.residual_rank, "auto").to(dev),
                              layer, x, expected_decode_tokens)
        if gate_passes(sp, proj, min_decode_speedup, min_projected_speedup):
            return LayerDecisionV5(name, d2.method, 2, d2.group_size, d2.outlier_columns, d2.residual_rank, d2.nmse, d2.cosine,
                                   d2.compression, sp, ps, proj, "INT2 passes quality + measured decode/projected-runtime guard")
        int2_too_slow = True

    def make4(g, oc, _rank=0):
        return HybridInt4Linear(layer, g, rms, oc).to(dev)

    trials = _grid(make4, layer, x, ref, group_sizes, outliers)
    good = [t for t in trials if t.passes(nmse_limit, cosine_limit, min_compression)]
    for b in sorted(good, key=lambda t: t.preference, reverse=True):
        sp, ps, proj = _timed(lambda: make4(b.group_size, b.outlier_columns), layer, x, expected_decode_tokens)
        if gate_passes(sp, proj, min_decode_speedup, min_projected_speedup):
            reason = ("INT2 was slower than FP16; INT4 passes measured decode-speed guard" if int2_too_slow else
                      "INT4 promoted fallback passes quality and measured decode-speed guard")
            return LayerDecisionV5(name, "int4-outlier" if b.outlier_columns else "int4", 4, b.group_size, b.outlier_columns, 0,
                                   b.nmse, b.cosine, b.compression, sp, ps, proj, reason)
    if trials:
        b = min(trials, key=lambda t: t.nmse)
        return LayerDecisionV5(name, "fp16", 16, b.group_size, b.outlier_columns, 0, b.nmse, b.cosine, 1.0, 1.0, 1.0, 1.0,
                               "kept FP16: no packed candidate passed quality + measured decode speed")
    return LayerDecisionV5(name, "fp16", 16, 128, 0, 0, float("inf"), 0.0, 1.0, 1.0, 1.0, 1.0, "no viable packed candidate")


def build_plan_v5(model, captures, group_sizes=(128, 64, 32), outliers=(0, 8, 16, 32), residual_ranks=(0, 4, 8),
                  nmse_limit=.06, cosine_limit=.96, min_compression=1.45, min_decode_speedup=1.0, min_projected_speedup=1.02,
                  expected_decode_tokens=64):
    """One ``LayerDecisionV5`` per captured ``nn.Linear`` of ``model`` (``captures``: module name -> sample inputs)."""
    mods = dict(model.named_modules())
    return [decide_linear_v5(name, mods[name], x, group_sizes, outliers, residual_ranks, nmse_limit, cosine_limit,
                             min_compression, min_decode_speedup, min_projected_speedup, expected_decode_tokens)
            for name, x in captures.items() if isinstance(mods.get(name), nn.Linear)]


def collect_linear_inputs(model: nn.Module, input_ids_batches, device, max_rows=128, target_tokens=None):
    """Sample inputs of the model's Linear layers (``ai_accel_lab/optimize/planner.py:32-54``): up to four
    forward calls' worth per layer, at most ``max_rows`` rows each, float32 on the CPU.  Takes token-id
    tensors instead of texts + tokenizer (no tokenizer is needed for synthetic benchmarks)."""
    captures, hooks = {}, []
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear) and (target_tokens is None or any(t in name for t in target_tokens)):
            captures[name] = []

            def hook(mod, args, key=name):
                if len(captures[key]) < 4:
                    a = args[0].detach()
                    captures[key].append(a.reshape(-1, a.shape[-1])[:max_rows].float().cpu())
            hooks.append(module.register_forward_pre_hook(hook))
    model.eval()
    with torch.no_grad():
        for ids in input_ids_batches:
            model(input_ids=ids.to(device), use_cache=False)
    for h in hooks:
        h.remove()
    return {k: torch.cat(v, 0)[:max_rows] for k, v in captures.items() if v}


def _demo():
    """Decisions of the planner, timed gate included, for seeded random layers of decoder shapes on the current
    CUDA device: one JSON line per layer (python -m ai_accel_studio_b200.optimize.planner_v5)."""
    import argparse
    import json
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", nargs="+", default=["4096x4096", "14336x4096", "4096x14336"], help="N x K of each layer")
    ap.add_argument("--rows", type=int, default=64, help="calibration rows")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("the timed gate needs a CUDA device")
    for i, shape in enumerate(a.shapes):
        n, k = (int(v) for v in shape.lower().split("x"))
        g = torch.Generator().manual_seed(100 + i)
        layer = nn.Linear(k, n, bias=False)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(n, k, generator=g) * 0.02)
        layer = layer.half().cuda()
        x = torch.randn(a.rows, k, generator=g) * torch.exp(0.5 * torch.randn(k, generator=g))
        d = decide_linear_v5(f"layer{i}_{n}x{k}", layer, x)
        print(json.dumps(d.to_dict()), flush=True)
        del layer
        torch.cuda.empty_cache()


if __name__ == "__main__":
    _demo()
