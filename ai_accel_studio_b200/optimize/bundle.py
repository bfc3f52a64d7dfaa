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

``load_bundle(..., tp=(rank, world))`` loads one tensor-parallel shard straight from the unsharded
bundle: the file format does not change, each rank maps the state file and copies only its rows /
columns to its GPU.
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


def _leaf(name: str) -> str:
    return name.rsplit(".", 1)[-1]


def install_packed_shards(model, decisions, state, rank: int, world: int, column_split=("o_proj", "down_proj"), group=None):
    """Tensor-parallel variant of ``install_packed_modules``: every planned Linear is replaced by THIS
    rank's shard, cut from the bundle's (host-resident, possibly memory-mapped) tensors before anything
    moves to the device, so a rank never holds more than its 1/world of the packed weights.  Layers
    whose leaf name is in ``column_split`` are split by input columns and wrapped in
    ``AllReduceLinear``; all others by output rows.  ``model`` is the rank's skeleton (local sizes)."""
    from ..tp import AllReduceLinear, col_shard_buffers, max_outliers_per_col_shard, row_shard_buffers
    done = []
    for d in decisions:
        if d.bits not in (2, 4):
            continue
        parent, leaf = _parent(model, d.name)
        src = getattr(parent, leaf)
        if isinstance(src, AllReduceLinear):
            src = src.inner
        if not isinstance(src, nn.Linear):
            continue
        g = lambda k: state.get(f"{d.name}.{k}")
        if g("packed") is None or g("scales") is None:
            raise KeyError(f"bundle state has no packed tensors for {d.name}")
        idx, ow = g("outlier_idx"), g("outlier_weight")
        if idx is not None and idx.numel() == 0:
            idx, ow = None, None
        full = dict(packed=g("packed"), scales=g("scales"), outlier_idx=idx, outlier_weight=ow, bias=g("bias"),
                    res_u=g("res_u"), res_v=g("res_v"))
        k_full = full["packed"].shape[1] * (8 // d.bits)
        cols = leaf in column_split
        if cols:
            pad = max_outliers_per_col_shard(idx, k_full, world)
            b = col_shard_buffers(full, rank, world, d.bits, d.group_size, k_full, pad)
            k_local = k_full // world
        else:
            b = row_shard_buffers(full, rank, world)
            k_local = src.in_features
        if k_local != src.in_features or b["packed"].shape[0] != src.out_features:
            raise ValueError(f"{d.name}: the bundle's shard is [{b['packed'].shape[0]}, {k_local}] but the skeleton's Linear "
                             f"is [{src.out_features}, {src.in_features}]")
        dev = src.weight.device
        mv = lambda t: None if t is None else t.to(dev)
        cls = HybridInt2Linear if d.bits == 2 else HybridInt4Linear
        mod = cls.from_buffers(mv(b["packed"]), mv(b["scales"]), k_local, d.group_size, mv(b["outlier_idx"]),
                               mv(b["outlier_weight"]), mv(b["bias"]), mv(b["res_u"]), mv(b["res_v"]))
        setattr(parent, leaf, AllReduceLinear(mod, group) if cols else mod)
        done.append(d.name)
    return done


def _dense_shard_state(model, state, packed_names, rank, world, column_split):
    """The bundle's remaining tensors, cut to this rank's slice where the skeleton's parameter is smaller
    (dense Linears that stayed fp16: rows, or columns for ``column_split`` layers; bias of a column-split
    layer on rank 0 only)."""
    from ..tp import AllReduceLinear
    own = {}
    for name, mod in model.named_modules():
        if isinstance(mod, AllReduceLinear) and isinstance(mod.inner, nn.Linear):
            own[name] = (mod.inner, name + ".inner")
        elif isinstance(mod, nn.Linear) and not name.endswith(".inner"):
            own[name] = (mod, name)
    out = {}
    for key, t in state.items():
        mod_name, _, leaf_key = key.rpartition(".")
        if mod_name in packed_names:
            continue
        if mod_name in own and leaf_key in ("weight", "bias"):
            lin, target = own[mod_name]
            cols = _leaf(mod_name) in column_split
            if leaf_key == "weight" and tuple(t.shape) != tuple(lin.weight.shape):
                n, k = t.shape
                t = t[:, rank * k // world:(rank + 1) * k // world] if cols else t[rank * n // world:(rank + 1) * n // world]
                if tuple(t.shape) != tuple(lin.weight.shape):
                    raise ValueError(f"{key}: shard {tuple(t.shape)} does not match the skeleton {tuple(lin.weight.shape)}")
            elif leaf_key == "bias" and lin.bias is not None:
                if cols:
                    t = t if rank == 0 else torch.zeros_like(t)
                elif t.shape[0] != lin.bias.shape[0]:
                    n = t.shape[0]
                    t = t[rank * n // world:(rank + 1) * n // world]
            out[f"{target}.{leaf_key}"] = t
        else:
            out[key] = t
    return out


def load_bundle(out_dir, model, device=None, tp=None, column_split=("o_proj", "down_proj"), group=None):
    """Load a v5 bundle into the skeleton ``model`` (same architecture as the one that was saved,
    dense Linears in place).  Returns ``(model, manifest, missing, unexpected)``.

    ``tp=(rank, world)`` loads one tensor-parallel shard: ``model`` is then the rank's skeleton (local
    sizes, column-split Linears optionally already wrapped in ``AllReduceLinear``), the state file is
    memory-mapped, and only this rank's rows / columns of every split tensor are copied to the device."""
    out = Path(out_dir)
    manifest = json.loads((out / "accel_manifest.json").read_text(encoding="utf-8"))
    if not manifest.get("format", "").endswith("v5"):
        raise ValueError(f"unsupported bundle format {manifest.get('format')!r}: only v5 bundles are handled here")
    decisions = [LayerDecisionV5(**x) for x in manifest["layers"]]
    if tp is None:
        state = torch.load(out / "optimized_state.pt", map_location=device or "cpu", weights_only=True)
        install_packed_modules(model, decisions, state)
        missing, unexpected = model.load_state_dict(state, strict=False)
    else:
        rank, world = int(tp[0]), int(tp[1])
        if not 0 <= rank < world:
            raise ValueError(f"bad tensor-parallel position {tp}")
        state = torch.load(out / "optimized_state.pt", map_location="cpu", weights_only=True, mmap=True)
        done = set(install_packed_shards(model, decisions, state, rank, world, column_split, group))
        rest = _dense_shard_state(model, state, done, rank, world, column_split)
        missing, unexpected = model.load_state_dict(rest, strict=False)
        missing = [m for m in missing if m.rpartition(".")[0].removesuffix(".inner") not in done]
    model.eval()
    return model, manifest, missing, unexpected
