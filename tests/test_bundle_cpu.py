"""v5 bundle round trip on the CPU: manifest format, state-dict keys, and loading straight from the
bundle's buffers into a dense skeleton (no re-quantisation)."""
import json

import torch
from torch import nn

from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.optimize.bundle import FORMAT, load_bundle, save_bundle
from ai_accel_studio_b200.optimize.planner_v5 import LayerDecisionV5, gate_passes


class Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.q_proj = nn.Linear(128, 64, bias=True)
        self.down_proj = nn.Linear(128, 32, bias=False)
        self.lm_head = nn.Linear(128, 16, bias=False)


def _decision(name, bits, oc, rank):
    return LayerDecisionV5(name, "hybrid-int2" if bits == 2 else "int4-outlier", bits, 64, oc, rank, 0.01, 0.99, 5.0,
                           1.3, 0.9, 1.2, "test")


def test_bundle_round_trip(tmp_path):
    torch.manual_seed(0)
    m = Toy()
    m.q_proj = HybridInt2Linear(m.q_proj, 64, None, 8, 4)
    m.down_proj = HybridInt4Linear(m.down_proj, 64, None, 4)
    decisions = [_decision("q_proj", 2, 8, 4), _decision("down_proj", 4, 4, 0),
                 LayerDecisionV5("lm_head", "fp16", 16, 128, 0, 0, 0.0, 1.0, 1.0, 1.0, 1.0, 1.0, "kept")]
    out = save_bundle(m, None, "toy/model", decisions, tmp_path / "b")
    manifest = json.loads((out / "accel_manifest.json").read_text())
    assert manifest["format"] == FORMAT == "ai-accel-studio-bundle-v5" and manifest["source_model"] == "toy/model"
    assert set(manifest["layers"][0]) == {"name", "method", "bits", "group_size", "outlier_columns", "residual_rank",
                                          "nmse", "cosine", "compression", "decode_speedup", "prefill_speedup",
                                          "projected_speedup", "reason"}
    state = torch.load(out / "optimized_state.pt", weights_only=True)
    assert {"q_proj.packed", "q_proj.scales", "q_proj.outlier_idx", "q_proj.outlier_weight", "q_proj.bias",
            "q_proj.res_u", "q_proj.res_v", "down_proj.packed", "down_proj.scales", "lm_head.weight"} <= set(state)
    assert "q_proj.weight" not in state

    skeleton = Toy()
    loaded, man, missing, unexpected = load_bundle(out, skeleton)
    assert not missing and not unexpected
    assert isinstance(loaded.q_proj, HybridInt2Linear) and isinstance(loaded.down_proj, HybridInt4Linear)
    assert loaded.q_proj.residual_rank == 4 and loaded.q_proj.group_size == 64 and loaded.q_proj.in_features == 128
    for k, v in m.state_dict().items():
        assert torch.equal(loaded.state_dict()[k], v), k


def test_gate_rule():
    assert gate_passes(None, None)
    assert gate_passes(1.0, 1.02) and not gate_passes(0.99, 1.5) and not gate_passes(1.2, 1.01)
