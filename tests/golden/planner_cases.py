"""Seeded layers for the planner fixtures: shared by the generator (which runs the reference
planner on them) and the test (which runs this package's planner on the same layers)."""
import torch
from torch import nn

from ai_accel_studio_b200.kernels.groupwise_int2 import INT2_LEVELS


def _linear(w, bias=None):
    layer = nn.Linear(w.shape[1], w.shape[0], bias=bias is not None)
    with torch.no_grad():
        layer.weight.copy_(w)
        if bias is not None:
            layer.bias.copy_(bias)
    return layer


def _on_levels(g, n, k, group):
    """A matrix that groupwise INT2 represents exactly: level x per-group scale."""
    lv = torch.tensor(INT2_LEVELS)[torch.randint(0, 4, (n, k), generator=g)]
    lv[:, ::group] = 1.0                                             # every group holds its own maximum
    scale = (torch.rand(n, k // group, generator=g) * 0.05 + 0.01).repeat_interleave(group, dim=1)
    return lv * scale


def make_case(name: str):
    """-> (layer, sample_x, keyword arguments of decide_linear_v5)."""
    g = torch.Generator().manual_seed(sum(map(ord, name)))
    kw = {}
    if name == "gaussian":                     # INT2 too coarse for a normal matrix: promoted to INT4
        layer = _linear(torch.randn(64, 256, generator=g) * 0.02, torch.randn(64, generator=g) * 0.01)
        x = torch.randn(48, 256, generator=g)
    elif name == "on_levels":                  # INT2 is exact
        layer = _linear(_on_levels(g, 48, 256, 128))
        x = torch.randn(32, 256, generator=g)
    elif name == "levels_plus_low_rank":       # INT2 needs the residual
        w = _on_levels(g, 64, 256, 32)
        w = w + 0.6 * (torch.randn(64, 3, generator=g) @ torch.randn(3, 256, generator=g)) * 0.02
        layer = _linear(w)
        x = torch.randn(40, 256, generator=g)
    elif name == "hot_columns":                # a few input channels dominate: outlier columns pay
        w = _on_levels(g, 64, 256, 64)
        hot = torch.randperm(256, generator=g)[:8]
        w[:, hot] = torch.randn(64, 8, generator=g) * 0.3
        layer = _linear(w)
        x = torch.randn(40, 256, generator=g)
        x[:, hot] *= 6.0
    elif name == "narrow":                     # fewer input features than the smallest group
        layer = _linear(torch.randn(32, 16, generator=g) * 0.02)
        x = torch.randn(16, 16, generator=g)
    elif name == "strict":                     # limits nothing packed can meet
        layer = _linear(torch.randn(32, 128, generator=g) * 0.02)
        x = torch.randn(16, 128, generator=g)
        kw = dict(nmse_limit=1e-9, cosine_limit=0.9999999)
    elif name == "heavy_tail":                 # normal / sqrt(uniform) weights, loose limits, small group only
        w = (torch.randn(96, 192, generator=g) / torch.rand(96, 192, generator=g).clamp_min(0.05).sqrt()) * 0.01
        layer = _linear(w)
        x = torch.randn(64, 192, generator=g) * torch.exp(torch.randn(192, generator=g))
        kw = dict(group_sizes=(64, 32), outliers=(0, 8, 16), nmse_limit=0.12, cosine_limit=0.9)
    else:
        raise KeyError(name)
    return layer, x, kw


CASES = ("gaussian", "on_levels", "levels_plus_low_rank", "hot_columns", "narrow", "strict", "heavy_tail")
