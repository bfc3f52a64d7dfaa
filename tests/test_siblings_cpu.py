"""Sibling fusion on the CPU: the merged buffers describe the same function as the separate modules
(checked with the oracle in float64), the merge refuses what it cannot express, and the rewiring of
a decoder-shaped module tree calls the fused module once per activation tensor."""
import numpy as np
import pytest
import torch
from torch import nn

from oracle import qgemv_oracle as O
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.optimize.siblings import can_merge, fuse_decoder_siblings, merge_packed


def _oracle(mod, x16):
    pw = O.PackedWeight(mod.bits, mod.packed.numpy(), mod.scales.numpy(), mod.original_k, mod.padded_k, mod.group_size)
    return O.gemv_f32(x16, pw,
                      None if mod.bias is None else mod.bias.numpy(),
                      mod.outlier_idx.numpy() if mod.outlier_idx.numel() else None,
                      mod.outlier_weight.numpy() if mod.outlier_idx.numel() else None,
                      mod.res_u.numpy() if mod.residual_rank else None,
                      mod.res_v.numpy() if mod.residual_rank else None)


@pytest.mark.parametrize("bits", [2, 4])
def test_merged_buffers_equal_separate_modules(bits):
    torch.manual_seed(bits)
    k = 256
    cls = HybridInt2Linear if bits == 2 else HybridInt4Linear
    mods = []
    for n, oc, bias in ((48, 8, True), (16, 4, False), (33, 0, False)):
        lin = nn.Linear(k, n, bias=bias)
        with torch.no_grad():
            lin.weight[:, torch.randperm(k)[:6]] *= 8          # distinct heavy columns per sibling
        m = cls(lin, 64, None, oc)
        if n != 33:
            m.set_residual(torch.randn(n, 8) * 0.05, torch.randn(8, k) * 0.05)
        mods.append(m)
    assert can_merge(mods)
    fused, sizes = merge_packed(mods)
    assert sizes == [48, 16, 33] and fused.out_features == 97 and type(fused) is cls
    assert fused.outlier_idx.numel() % 8 == 0 and fused.residual_rank == 16
    assert fused.bias is not None and torch.equal(fused.bias[48:], torch.zeros(49, dtype=torch.float16))
    x = (torch.randn(3, k) * 2).half().numpy()
    got = _oracle(fused, x)
    want = np.concatenate([_oracle(m, x) for m in mods], axis=1)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-9)


def test_merge_refuses_mismatched_siblings():
    torch.manual_seed(0)
    a = HybridInt2Linear(nn.Linear(128, 16), 64, None, 4)
    assert not can_merge([a])
    assert not can_merge([a, HybridInt4Linear(nn.Linear(128, 16), 64, None, 4)])        # bit width
    assert not can_merge([a, HybridInt2Linear(nn.Linear(128, 16), 32, None, 4)])        # group size
    assert not can_merge([a, HybridInt2Linear(nn.Linear(256, 16), 64, None, 4)])        # K
    assert not can_merge([a, nn.Linear(128, 16)])
    with pytest.raises(ValueError):
        merge_packed([a, nn.Linear(128, 16)])


class _Attn(nn.Module):
    def __init__(self, k):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(k, 32), nn.Linear(k, 8), nn.Linear(k, 8)
        self.o_proj = nn.Linear(32, k)


class _Mlp(nn.Module):
    def __init__(self, k):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = nn.Linear(k, 64), nn.Linear(k, 64), nn.Linear(64, k)


class _Layer(nn.Module):
    def __init__(self, k):
        super().__init__()
        self.self_attn, self.mlp = _Attn(k), _Mlp(k)


def test_rewiring_calls_the_fused_module_once_per_activation():
    torch.manual_seed(1)
    layer = _Layer(128)
    for name in ("q_proj", "k_proj", "v_proj"):
        setattr(layer.self_attn, name, HybridInt4Linear(getattr(layer.self_attn, name), 64, None, 4))
    layer.mlp.gate_proj = HybridInt2Linear(layer.mlp.gate_proj, 64, None, 4)
    layer.mlp.up_proj = HybridInt4Linear(layer.mlp.up_proj, 64, None, 4)            # differs: stays unfused
    assert fuse_decoder_siblings(layer) == 1
    assert isinstance(layer.mlp.gate_proj, HybridInt2Linear) and isinstance(layer.mlp.up_proj, HybridInt4Linear)
    fused = layer.self_attn.q_proj.fused
    assert fused.out_features == 48 and "self_attn.q_proj.fused.packed" in layer.state_dict()
    assert not any(k.startswith("self_attn.k_proj") for k in layer.state_dict())
    calls = []
    fused.forward = lambda x: calls.append(x) or torch.arange(48.0).repeat(x.shape[0], 1)     # stand-in: no GPU here
    x = torch.randn(2, 128)
    q, kk, v = layer.self_attn.q_proj(x), layer.self_attn.k_proj(x), layer.self_attn.v_proj(x)
    assert len(calls) == 1 and q.shape == (2, 32) and kk.shape == (2, 8) and v.shape == (2, 8)
    assert float(kk[0, 0]) == 32.0 and float(v[0, 0]) == 40.0
    x2 = torch.randn(2, 128)
    layer.self_attn.q_proj(x2), layer.self_attn.k_proj(x2), layer.self_attn.v_proj(x2)
    assert len(calls) == 2


@pytest.mark.parametrize("bits", [2, 4])
def test_gate_up_interleave_describes_the_same_rows(bits):
    """merge_gate_up: block b of the fused module holds gate rows 8b..8b+7 then up rows 8b..8b+7, with
    every per-row tensor permuted alike (checked through the oracle on each half)."""
    from ai_accel_studio_b200.optimize.siblings import can_merge_gate_up, merge_gate_up
    torch.manual_seed(10 + bits)
    k, n = 256, 48
    cls = HybridInt2Linear if bits == 2 else HybridInt4Linear
    gate = cls(nn.Linear(k, n, bias=True), 64, None, 8)
    up = cls(nn.Linear(k, n, bias=False), 64, None, 4)
    gate.set_residual(torch.randn(n, 4) * 0.05, torch.randn(4, k) * 0.05)
    assert can_merge_gate_up(gate, up)
    fused = merge_gate_up(gate, up)
    assert fused.gated_pairs and fused.out_features == n and fused.packed.shape[0] == 2 * n and type(fused) is cls
    x = (torch.randn(3, k) * 0.5).half().numpy()
    both = _oracle(fused, x).reshape(3, n // 8, 2, 8)
    np.testing.assert_allclose(both[:, :, 0, :].reshape(3, n), _oracle(gate, x), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(both[:, :, 1, :].reshape(3, n), _oracle(up, x), rtol=1e-5, atol=1e-6)
    assert not can_merge_gate_up(gate, cls(nn.Linear(k, n + 8), 64, None, 0))       # widths differ
    assert not can_merge_gate_up(cls(nn.Linear(k, 12), 64, None, 0), cls(nn.Linear(k, 12), 64, None, 0))   # not whole blocks
    with pytest.raises(ValueError):
        merge_gate_up(gate, (HybridInt4Linear if bits == 2 else HybridInt2Linear)(nn.Linear(k, n), 64, None, 0))


def test_decoder_rewiring_builds_gated_feed_forward():
    from ai_accel_studio_b200.optimize.siblings import GatedFeedForward

    class MLP(nn.Module):
        def __init__(self, act):
            super().__init__()
            self.gate_proj = HybridInt4Linear(nn.Linear(128, 64, bias=False), 64, None, 0)
            self.up_proj = HybridInt4Linear(nn.Linear(128, 64, bias=False), 64, None, 0)
            self.down_proj = nn.Linear(64, 128, bias=False)
            self.act_fn = act

    class Layer(nn.Module):
        def __init__(self, act):
            super().__init__()
            self.mlp = MLP(act)

    torch.manual_seed(3)
    model = nn.ModuleList([Layer(nn.SiLU()), Layer(nn.GELU())])
    assert fuse_decoder_siblings(model) == 2                     # one gated block, one plain gate/up merge
    assert isinstance(model[0].mlp, GatedFeedForward) and model[0].mlp.gate_up.gated_pairs
    assert not isinstance(model[1].mlp, GatedFeedForward)        # another activation: only the launches are merged
    assert fuse_decoder_siblings(nn.ModuleList([Layer(nn.SiLU())]), gated=False) == 1


def test_merge_algebra_holds_for_random_sibling_sets():
    """Property test: for random sibling sets (sizes, outlier sets, residual ranks, biases) the merged module's
    reconstructed weight is the row-wise concatenation of the siblings', and its bias their concatenation."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=25, deadline=None)
    @given(bits=st.sampled_from([2, 4]), sizes=st.lists(st.integers(1, 40), min_size=2, max_size=4),
           ocs=st.lists(st.integers(0, 9), min_size=4, max_size=4), ranks=st.lists(st.sampled_from([0, 2, 5]), min_size=4, max_size=4),
           seed=st.integers(0, 10 ** 6))
    def check(bits, sizes, ocs, ranks, seed):
        torch.manual_seed(seed)
        k = 128
        cls = HybridInt2Linear if bits == 2 else HybridInt4Linear
        mods = []
        for i, n in enumerate(sizes):
            m = cls(nn.Linear(k, n, bias=bool((seed + i) % 2)), 64, None, ocs[i])
            if ranks[i]:
                m.set_residual(torch.randn(n, ranks[i]) * 0.05, torch.randn(ranks[i], k) * 0.05)
            mods.append(m)
        fused, out_sizes = merge_packed(mods)
        assert out_sizes == sizes and fused.out_features == sum(sizes)
        want = torch.cat([m.effective_weight() for m in mods], 0)
        assert torch.allclose(fused.effective_weight(), want, atol=1e-6)
        if fused.bias is not None:
            want_b = torch.cat([m.bias if m.bias is not None else torch.zeros(m.out_features, dtype=torch.float16) for m in mods])
            assert torch.equal(fused.bias, want_b)
        assert fused.outlier_idx.numel() % 8 == 0                   # rows stay 16-byte aligned for the prefetching kernel
    check()
