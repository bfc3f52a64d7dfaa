"""Sibling fusion: Linears that read the same activations (q/k/v, gate/up) as ONE packed GEMV.

The reference launches one kernel per Linear (``ai_accel_lab/optimize/hybrid_int2.py:80-107`` is
called once per projection by the Hugging Face decoder), and blames launch / runtime overhead for
most of its decode time.  Packed modules that agree on bit width, group size and K can be merged
into one module of the same class with no change to the kernel:

* packed rows, scales, biases: concatenated along N;
* outlier columns: the union of the siblings' column sets, each sibling's weights scattered into
  its rows and zeros elsewhere (a zero weight adds exactly 0);
* low-rank residual: block structure, ``U = diag(U_1, U_2, ...)`` and ``V = [V_1; V_2; ...]``, so row
  block i only sees its own ``U_i (V_i x)``.

Gate / up pairs go one step further (``merge_gate_up``): their rows are interleaved in blocks of 8
(8 gate rows, then the 8 up rows with the same indices), which puts every (gate_j, up_j) pair into
one lane of the kernel's 16-row output tile, so the epilogue computes ``silu(gate) * up`` itself and
stores ``[M, intermediate]`` directly (``QGEMV_ACT_SILU_MUL``): gate projection, up projection,
activation and product become one launch.  Both intermediate results and the activation are rounded
to the activation type exactly where separate operators would round them.

``merge_packed`` does that algebra (any device).  ``fuse_decoder_siblings`` rewires a Hugging Face
Llama / Qwen2 style decoder in place: the first sibling called computes the fused result, the
others take their slice of it.  Per row the quantised term is bit-identical to the unfused module
(same bytes, same activations, same order); outlier and residual terms are summed over a longer
column list, so results agree to fp32 rounding, not bitwise.
"""
from __future__ import annotations

import torch
from torch import nn

from ._hybrid_base import HybridPackedLinear

SIBLING_SETS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))
MAX_FUSED_OUTLIERS = 256      # the fast kernel stages at most this many outlier activations
MAX_FUSED_RANK = 64


def can_merge(mods) -> bool:
    """Same class (bit width), group size, K and padding; all packed modules; limits respected."""
    mods = list(mods)
    if len(mods) < 2 or not all(isinstance(m, HybridPackedLinear) for m in mods):
        return False
    a = mods[0]
    if any(type(m) is not type(a) or m.group_size != a.group_size or m.original_k != a.original_k
           or m.padded_k != a.padded_k or m.packed.device != a.packed.device for m in mods[1:]):
        return False
    cols = set()
    for m in mods:
        cols.update(m.outlier_idx.tolist())
    if len(cols) > MAX_FUSED_OUTLIERS or sum(m.residual_rank for m in mods) > MAX_FUSED_RANK:
        return False
    return True


@torch.no_grad()
def merge_packed(mods):
    """Merge sibling packed modules into one module of the same class.  Returns ``(fused, sizes)``
    where ``sizes`` are the siblings' output widths in order (``fused(x).split(sizes, -1)``)."""
    mods = list(mods)
    if not can_merge(mods):
        raise ValueError("modules cannot be merged (class, group size, K, device or size limits differ)")
    a = mods[0]
    dev = a.packed.device
    sizes = [m.out_features for m in mods]
    n_total = sum(sizes)
    packed = torch.cat([m.packed for m in mods], 0)
    scales = torch.cat([m.scales for m in mods], 0)
    bias = None
    if any(m.bias is not None for m in mods):
        bias = torch.cat([m.bias if m.bias is not None else torch.zeros(m.out_features, dtype=torch.float16, device=dev)
                          for m in mods], 0)
    # union of the outlier columns, padded to a multiple of 8 with repeats of the first column
    # (zero weights) so that the rows stay 16-byte aligned for the prefetching kernel
    union = sorted({int(c) for m in mods for c in m.outlier_idx.tolist()})
    idx = w = None
    if union:
        while len(union) % 8:
            union.append(union[0])
        idx = torch.tensor(union, dtype=torch.int32, device=dev)
        w = torch.zeros((n_total, len(union)), dtype=torch.float16, device=dev)
        pos = {}
        for j, c in enumerate(union):
            pos.setdefault(c, j)                 # first position of every column; padding repeats stay zero
        row = 0
        for m in mods:
            if m.outlier_idx.numel():
                dst = torch.tensor([pos[int(c)] for c in m.outlier_idx.tolist()], dtype=torch.long, device=dev)
                w[row:row + m.out_features, dst] = m.outlier_weight
            row += m.out_features
    # block residual
    rank = sum(m.residual_rank for m in mods)
    res_u = res_v = None
    if rank:
        res_u = torch.zeros((n_total, rank), dtype=torch.float16, device=dev)
        res_v = torch.zeros((rank, a.in_features), dtype=torch.float16, device=dev)
        row = col = 0
        for m in mods:
            r = m.residual_rank
            if r:
                res_u[row:row + m.out_features, col:col + r] = m.res_u
                res_v[col:col + r] = m.res_v
                col += r
            row += m.out_features
    fused = type(a).from_buffers(packed, scales, a.original_k, a.group_size, idx, w, bias, res_u, res_v)
    fused.graph_safe = True
    fused.kernel = a.kernel
    return fused, sizes


def can_merge_gate_up(gate, up) -> bool:
    """Mergeable siblings of equal width whose row count fills whole 8-row blocks, on the tensor-core
    kernels' shapes (16-byte aligned packed rows and a supported group size)."""
    if not can_merge([gate, up]) or gate.out_features != up.out_features or gate.out_features % 8:
        return False
    group_bytes = gate.group_size * gate.bits // 8
    return group_bytes in (16, 32, 64) and gate.packed.shape[1] % 16 == 0 and gate.padded_k % 8 == 0


@torch.no_grad()
def merge_gate_up(gate, up):
    """One packed module computing ``silu(gate(x)) * up(x)``: ``merge_packed`` followed by the 8-row
    interleave of the two halves.  ``out_features`` of the result is the intermediate size."""
    if not can_merge_gate_up(gate, up):
        raise ValueError("gate / up projections cannot be merged into a gated pair")
    fused, sizes = merge_packed([gate, up])
    n = sizes[0]
    rows = torch.arange(n, device=fused.packed.device).view(n // 8, 1, 8)
    perm = torch.cat([rows, rows + n], dim=1).reshape(-1)            # block b: gate rows 8b..8b+7, up rows 8b..8b+7
    for name in ("packed", "scales", "outlier_weight", "bias", "res_u"):
        t = getattr(fused, name, None)
        if t is not None and t.shape[0] == 2 * n:
            fused._buffers[name] = t[perm].contiguous()
    fused.__dict__.pop("_call", None)               # buffers were replaced behind the module's back
    fused.gated_pairs = True
    fused.out_features = n
    return fused


class GatedFeedForward(nn.Module):
    """Stands where a Llama / Qwen2 style feed-forward block stood: ``down(silu(gate(x)) * up(x))`` with
    the part in parentheses computed by one fused packed module."""

    def __init__(self, gate_up: HybridPackedLinear, down_proj: nn.Module):
        super().__init__()
        self.gate_up = gate_up
        self.down_proj = down_proj

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down_proj(self.gate_up(x))


def _is_silu(fn) -> bool:
    return isinstance(fn, nn.SiLU) or fn is torch.nn.functional.silu or type(fn).__name__ in ("SiLUActivation", "SiLU")


class _SiblingSlice(nn.Module):
    """Stands where one sibling Linear stood.  All slices of a group share one fused module; the
    first slice called with a given activation tensor runs it, the others reuse that result."""

    def __init__(self, group: "_SiblingGroup", index: int):
        super().__init__()
        self._group = [group]                     # in a list: not registered as a sub-module of every slice
        self.index = index
        self.out_features = group.sizes[index]
        self.in_features = group.fused.in_features
        if index == 0:
            self.fused = group.fused              # owned (moved, saved, counted) by the first slice only

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._group[0].result(x)[self.index]


class _SiblingGroup:
    def __init__(self, fused: HybridPackedLinear, sizes):
        self.fused, self.sizes = fused, list(sizes)
        self._x = None
        self._parts = None
        self._served = 0

    def result(self, x: torch.Tensor):
        if self._x is not x:                      # a new activation tensor: one fused launch
            self._parts = self.fused(x).split(self.sizes, dim=-1)
            self._x, self._served = x, 0
        parts = self._parts
        self._served += 1
        if self._served == len(self.sizes):       # everyone served: drop the references
            self._x = self._parts = None
        return parts


def fuse_decoder_siblings(model: nn.Module, sets=SIBLING_SETS, gated=True) -> int:
    """Replace mergeable sibling sets (same parent module, see ``SIBLING_SETS``) by slices of one fused
    packed module each.  Returns the number of groups fused.  Siblings that differ in bit width or
    group size, or are not packed modules, are left alone.  With ``gated`` a feed-forward block whose
    gate / up projections merge and whose activation is SiLU becomes a ``GatedFeedForward`` (one launch
    for both projections, the activation and the product)."""
    fused_groups = 0
    if gated:
        for name, parent in list(model.named_modules()):
            for child_name, mlp in list(parent.named_children()):
                g, u, d = (getattr(mlp, n, None) for n in ("gate_proj", "up_proj", "down_proj"))
                if g is None or u is None or d is None or not _is_silu(getattr(mlp, "act_fn", None)):
                    continue
                if isinstance(g, HybridPackedLinear) and isinstance(u, HybridPackedLinear) and can_merge_gate_up(g, u):
                    setattr(parent, child_name, GatedFeedForward(merge_gate_up(g, u), d))
                    fused_groups += 1
    for parent in list(model.modules()):
        for names in sets:
            mods = [getattr(parent, n, None) for n in names]
            if any(m is None for m in mods) or not can_merge(mods):
                continue
            fused, sizes = merge_packed(mods)
            group = _SiblingGroup(fused, sizes)
            for i, n in enumerate(names):
                setattr(parent, n, _SiblingSlice(group, i))
            fused_groups += 1
    if fused_groups and torch.cuda.is_available():
        torch.cuda.empty_cache()
    return fused_groups
