"""v5 bundle files: ``accel_manifest.json`` + ``optimized_state.pt``.

Same on-disk format as ``ai_accel_lab/optimize/bundle.py`` (:15-25 ``save_bundle``, :50-68
``load_bundle``): the manifest lists one ``LayerDecisionV5`` dict per planned Linear under
``format: ai-accel-studio-bundle-v5``; the state file is the model's ``state_dict`` whose packed
layers contribute ``packed / scales / outlier_idx / outlier_weight / bias / res_u / res_v``.

Loading differs in one respect: the reference rebuilds every packed module by quantising the
freshly loaded dense layer (and running an SVD for the residual) only to overwrite all of it with
the bundle's tensors (:34-47).  Here the modules are created directly from the bundle's buffers
(``from_buffers``); nothing is quantised at load time.  The caller supplies the skeleton model
(the reference downloads it by name, which this package does not do).
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
from torch import nn

from .hybrid_int2 import HybridInt2Linear
from .hybrid_int4 import HybridInt4Linear
from .planner_v5 import LayerDecisionV5

FORMAT = "ai-accel-studio-bundle-v5"


def save_bundle(model, tokenizer, source_model_id, decisions, out_dir, extra=None):
    """Same positional order as the reference (ai_accel_lab/optimize/bundle.py:15); ``tokenizer`` may be
    None (random-token benchmarks have none)."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    manifest = {"format": FORMAT, "source_model": source_model_id,
                "layers": [d.to_dict() for d in decisions], "extra": dict(extra or {}, format_version=5)}
    (out / "accel_manifest.json").write_text(json.dumps(manifest, ensure_ascii=False, indent=2), encoding="utf-8")
    torch.save(model.state_dict(), out / "optimized_state.pt")
    if tokenizer is not None:
        try:
            tokenizer.save_pretrained(out / "tokenizer")
        except Exception:
            pass
    return out


def _parent(root, fqn):
    parts = fqn.split(".")
    obj = root
    for p in parts[:-1]:
        obj = getattr(obj, p)
    return obj, parts[-1]


def install_packed_modules(model, decisions, state):
    """Replace every planned Linear of ``model`` by a packed module built straight from ``state``
    (the bundle's state dict).  Returns the names that were replaced."""
    done = []
    for d in decisions:
        if d.bits not in (2, 4):
            continue
        parent, leaf = _parent(model, d.name)
        src = getattr(parent, leaf)
        if not isinstance(src, nn.Linear):
            continue
        g = lambda k: state.get(f"{d.name}.{k}")
        if g("packed") is None or g("scales") is None:
            raise KeyError(f"bundle state has no packed tensors for {d.name}")
        cls = HybridInt2Linear if d.bits == 2 else HybridInt4Linear
        dev = src.weight.device
        mv = lambda t: None if t is None else t.to(dev)
        mod = cls.from_buffers(mv(g("packed")), mv(g("scales")), src.in_features, d.group_size, mv(g("outlier_idx")),
                               mv(g("outlier_weight")), mv(g("bias")), mv(g("res_u")), mv(g("res_v")))
        setattr(parent, leaf, mod)
        done.append(d.name)
    return done


def load_bundle(out_dir, model, device=None):
    """Load a v5 bundle into the skeleton ``model`` (same architecture as the one that was saved,
    dense Linears in place).  Returns ``(model, manifest, missing, unexpected)``."""
    out = Path(out_dir)
    manifest = json.loads((out / "accel_manifest.json").read_text(encoding="utf-8"))
    if not manifest.get("format", "").endswith("v5"):
        raise ValueError(f"unsupported bundle format {manifest.get('format')!r}: only v5 bundles are handled here")
    decisions = [LayerDecisionV5(**x) for x in manifest["layers"]]
    state = torch.load(out / "optimized_state.pt", map_location=device or "cpu", weights_only=True)
    install_packed_modules(model, decisions, state)
    missing, unexpected = model.load_state_dict(state, strict=False)
    model.eval()
    return model, manifest, missing, unexpected
