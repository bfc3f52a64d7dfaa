"""The per-layer planner (candidate search, tie-breaking, fallbacks) against the decisions the
reference planner took on the same seeded layers (tests/golden/planner_decisions.json, written by
tests/golden/make_planner_golden.py).  CPU only: the timed gate reports "not measured" there, in
the reference as here."""
import json
import math
import sys
from pathlib import Path

import pytest
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN))
import planner_cases as pc                                              # noqa: E402

from ai_accel_studio_b200.optimize import planner_v5 as pl             # noqa: E402

WANT = json.loads((GOLDEN / "planner_decisions.json").read_text())
V4_KEYS = ("group_sizes", "outliers", "residual_ranks", "nmse_limit", "cosine_limit")


def _same(got: dict, want: dict):
    for key in ("name", "method", "group_size", "outlier_columns", "residual_rank", "reason"):
        assert got[key] == want[key], (key, got, want)
    if "bits" in want:
        assert got["bits"] == want["bits"]
        for key in ("decode_speedup", "prefill_speedup", "projected_speedup"):
            assert got[key] == want[key]
    assert got["compression"] == pytest.approx(want["compression"], rel=1e-12)
    if math.isinf(want["nmse"]):
        assert math.isinf(got["nmse"])
    else:   # the reference measures through a float32 CPU forward, this package through the reconstructed weight
        assert got["nmse"] == pytest.approx(want["nmse"], rel=2e-3, abs=1e-9)
        assert got["cosine"] == pytest.approx(want["cosine"], abs=1e-5)


@pytest.mark.parametrize("name", pc.CASES)
def test_decisions_match_the_reference_planner(name):
    layer, x, kw = pc.make_case(name)
    v4 = pl.decide_linear_v4(name, layer, x, **{k: v for k, v in kw.items() if k in V4_KEYS})
    _same(v4.to_dict(), WANT[name]["v4"])
    v5 = pl.decide_linear_v5(name, layer, x, **kw)
    _same(v5.to_dict(), WANT[name]["v5"])


def test_gate_rejects_slow_candidates(monkeypatch):
    """An INT2 candidate that passes quality but is timed slower than fp16 gives way to INT4, and a
    layer whose every candidate is slow stays fp16 (timings injected on the host)."""
    layer, x, kw = pc.make_case("on_levels")
    calls = []

    def fake(layer_, cand, x_, tokens=64):
        calls.append(cand.bits)
        return (0.8, 1.0, 0.9) if cand.bits == 2 else (1.3, 0.9, 1.25)
    monkeypatch.setattr(pl, "runtime_speedups", fake)
    d = pl.decide_linear_v5("l", layer, x, **kw)
    assert d.bits == 4 and d.reason.startswith("INT2 was slower than FP16") and d.decode_speedup == 1.3
    assert calls[0] == 2 and set(calls[1:]) == {4}
    monkeypatch.setattr(pl, "runtime_speedups", lambda *a, **k: (0.9, 0.9, 0.9))
    d = pl.decide_linear_v5("l", layer, x, **kw)
    assert d.method == "fp16" and d.bits == 16 and d.reason.startswith("kept FP16")


def test_build_plan_and_capture():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(128, 64), torch.nn.ReLU(), torch.nn.Linear(64, 32))
    caps = {"0": torch.randn(16, 128), "2": torch.randn(16, 64), "1": torch.randn(16, 64)}
    plan = pl.build_plan_v5(model, caps)
    assert [d.name for d in plan] == ["0", "2"]                         # the ReLU is not a Linear
    assert all(isinstance(d, pl.LayerDecisionV5) for d in plan)


def test_capture_then_plan_on_a_decoder(monkeypatch):
    """collect_linear_inputs on a tiny decoder (token ids instead of texts), then both planners over the captures."""
    from ai_accel_studio_b200 import model_tools as mt
    monkeypatch.setitem(mt.SHAPES, "tiny", dict(family="llama", layers=1, hidden=128, inter=256, heads=2, kv_heads=1,
                                                head_dim=64, vocab=96, qkv_bias=False))
    model = mt.build_fp16_model("tiny", "cpu").float()
    ids = [torch.randint(0, 96, (2, 12), generator=torch.Generator().manual_seed(i)) for i in range(6)]
    caps = pl.collect_linear_inputs(model, ids, "cpu", max_rows=40, target_tokens=("q_proj", "down_proj"))
    assert set(caps) == {"model.layers.0.self_attn.q_proj", "model.layers.0.mlp.down_proj"}
    assert caps["model.layers.0.self_attn.q_proj"].shape == (40, 128)        # four forward calls of 24 rows, cut to 40
    assert caps["model.layers.0.mlp.down_proj"].shape == (40, 256) and caps["model.layers.0.mlp.down_proj"].dtype == torch.float32
    p5 = pl.build_plan_v5(model, caps, group_sizes=(64,), outliers=(0, 8))
    p4 = pl.build_plan_v4(model, caps, group_sizes=(64,), outliers=(0, 8))
    assert [d.name for d in p5] == [d.name for d in p4] == list(caps)
    assert all(d.decode_speedup is None or d.method == "fp16" for d in p5)    # CPU: the gate reports "not measured"


def test_gate_arithmetic():
    t = pl.GateTiming(dense_decode=0.016, packed_decode=0.013, dense_prefill=0.016, packed_prefill=0.045)
    decode, prefill, projected = t.speedups(64)
    assert decode == pytest.approx(16 / 13) and prefill == pytest.approx(16 / 45)
    assert projected == pytest.approx((0.016 + 64 * 0.016) / (0.045 + 64 * 0.013))
    assert pl.gate_passes(decode, projected) and not pl.gate_passes(*pl.GateTiming(1.0, 1.1, 1.0, 1.0).speedups(64)[::2])
    layer = torch.nn.Linear(8, 8)
    assert pl.runtime_speedups(layer, layer, torch.randn(4, 8)) == (None, None, None)      # CPU: not measured
