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


class Block(nn.Module):
    """Linear names of one decoder layer; sizes divided by ``world`` where tensor parallelism splits them."""

    def __init__(self, hidden=128, inter=256, world=1, wrap=False):
        super().__init__()
        from ai_accel_studio_b200.tp import AllReduceLinear
        self.q_proj = nn.Linear(hidden, hidden // world, bias=True)
        self.up_proj = nn.Linear(hidden, inter // world, bias=False)
        self.gate_proj = nn.Linear(hidden, inter // world, bias=True)        # stays fp16 in the plan below
        o, down = nn.Linear(hidden // world, hidden, bias=True), nn.Linear(inter // world, hidden, bias=False)
        self.o_proj = AllReduceLinear(o) if wrap else o
        self.down_proj = AllReduceLinear(down) if wrap else down
        self.norm = nn.LayerNorm(hidden)


def test_bundle_loads_one_tensor_parallel_shard(tmp_path):
    """Every rank's shard loaded straight from the unsharded bundle equals the shard cut from the
    loaded full module, dense layers are sliced the same way, and the shards' effective weights
    reassemble the full matrices (rows concatenated, K ranges concatenated)."""
    from ai_accel_studio_b200.tp import AllReduceLinear, shard_cols, shard_rows
    torch.manual_seed(1)
    full = Block()
    rms = torch.rand(128) + 0.5
    full.q_proj = HybridInt2Linear(full.q_proj, 64, rms, 8, 4)
    full.up_proj = HybridInt4Linear(full.up_proj, 32, None, 0)
    full.o_proj = HybridInt4Linear(full.o_proj, 64, rms, 8)
    full.down_proj = HybridInt2Linear(full.down_proj, 64, None, 16, 4)
    decisions = [_decision("q_proj", 2, 8, 4), _decision("o_proj", 4, 8, 0), _decision("down_proj", 2, 16, 4)]
    decisions.append(LayerDecisionV5("up_proj", "int4", 4, 32, 0, 0, 0.01, 0.99, 3.8, None, None, None, "test"))
    decisions.append(LayerDecisionV5("gate_proj", "fp16", 16, 128, 0, 0, 0.5, 0.5, 1.0, 1.0, 1.0, 1.0, "kept"))
    out = save_bundle(full, None, "toy/block", decisions, tmp_path / "tp")
    world = 2
    parts = []
    for rank in range(world):
        for wrap in (False, True):
            skel = Block(world=world, wrap=wrap)
            loaded, _, missing, unexpected = load_bundle(out, skel, tp=(rank, world))
            assert not missing and not unexpected, (missing, unexpected)
            assert isinstance(loaded.o_proj, AllReduceLinear) and isinstance(loaded.down_proj, AllReduceLinear)
            for name, cut in (("q_proj", shard_rows), ("up_proj", shard_rows), ("o_proj", shard_cols), ("down_proj", shard_cols)):
                got = getattr(loaded, name)
                got = got.inner if isinstance(got, AllReduceLinear) else got
                want = cut(getattr(full, name), rank, world)
                assert type(got) is type(want) and got.in_features == want.in_features and got.group_size == want.group_size
                gs, ws = got.state_dict(), want.state_dict()
                assert set(gs) == set(ws), name
                for k in ws:
                    assert torch.equal(gs[k], ws[k]), (name, k)
            n = full.gate_proj.out_features // world
            assert torch.equal(loaded.gate_proj.weight, full.gate_proj.weight[rank * n:(rank + 1) * n])
            assert torch.equal(loaded.gate_proj.bias, full.gate_proj.bias[rank * n:(rank + 1) * n])
            assert torch.equal(loaded.norm.weight, full.norm.weight)
        parts.append(loaded)
    for name, dim in (("q_proj", 0), ("up_proj", 0), ("o_proj", 1), ("down_proj", 1)):
        mods = [getattr(p, name) for p in parts]
        mods = [m.inner if isinstance(m, AllReduceLinear) else m for m in mods]
        assert torch.allclose(torch.cat([m.effective_weight() for m in mods], dim), getattr(full, name).effective_weight(), atol=1e-6)
    biases = [p.o_proj.inner.bias for p in parts]
    assert torch.equal(biases[0], full.o_proj.bias) and biases[1] is None          # bias on rank 0 only


def test_bundle_shard_rejects_a_wrong_skeleton(tmp_path):
    import pytest
    torch.manual_seed(2)
    full = Block()
    full.q_proj = HybridInt2Linear(full.q_proj, 64, None, 0, 0)
    out = save_bundle(full, None, "toy/block", [_decision("q_proj", 2, 0, 0)], tmp_path / "bad")
    with pytest.raises(ValueError, match="skeleton"):
        load_bundle(out, Block(world=1), tp=(0, 2))                               # full-size skeleton, half-size shard
    with pytest.raises(ValueError, match="tensor-parallel position"):
        load_bundle(out, Block(world=2), tp=(2, 2))
