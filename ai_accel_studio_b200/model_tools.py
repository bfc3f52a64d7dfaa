"""Random-init decoder models with seeded mixed-bit plans, for whole-model decode measurements.

Mirrors what the reference's model benchmark does around the hot path (module swap:
``ai_accel_lab/model_benchmark.py:83-103``; plan application: ``ai_accel_lab/optimize/bundle.py:34-47``)
without checkpoints or tokenizers: the benchmark configurations specify random-init weights
N(0, 0.02), a seeded per-Linear bit-width plan, group 128, 1 % outlier columns and rank-8
residual factors given directly (an SVD per layer of an 8B/70B model is not affordable and not
what is being measured).

Tensor parallelism: every rank builds a *local* model whose attention heads and MLP width are
divided by the world size (row shards of q/k/v/gate/up, column shards of o/down) and wraps
o_proj / down_proj in ``AllReduceLinear``.
"""
from __future__ import annotations

import dataclasses

import torch
from torch import nn

from .optimize import HybridInt2Linear, HybridInt4Linear
from .optimize._hybrid_base import snap_outlier_count
from .kernels.groupwise_int2 import pack_groupwise_int2
from .kernels.groupwise_int4 import pack_groupwise_int4
from .tp import AllReduceLinear

TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
COLUMN_SPLIT = ("o_proj", "down_proj")

SHAPES = {
    "qwen2.5-0.5b": dict(family="qwen2", layers=24, hidden=896, inter=4864, heads=14, kv_heads=2, head_dim=64,
                         vocab=151936, qkv_bias=True),
    "llama-3-8b": dict(family="llama", layers=32, hidden=4096, inter=14336, heads=32, kv_heads=8, head_dim=128,
                       vocab=128256, qkv_bias=False),
    "llama-3-70b": dict(family="llama", layers=80, hidden=8192, inter=28672, heads=64, kv_heads=8, head_dim=128,
                        vocab=128256, qkv_bias=False),
}


def local_config(shape: str, world: int = 1, layers: int | None = None, max_positions: int = 4096):
    """HF config of one rank's slice of the model (world == 1: the whole model)."""
    from transformers import LlamaConfig, Qwen2Config
    s = SHAPES[shape]
    if s["heads"] % world or s["kv_heads"] % world or s["inter"] % world:
        raise ValueError(f"{shape} cannot be split {world} ways (heads {s['heads']}/{s['kv_heads']}, inter {s['inter']})")
    kw = dict(hidden_size=s["hidden"], intermediate_size=s["inter"] // world,
              num_hidden_layers=layers if layers is not None else s["layers"],
              num_attention_heads=s["heads"] // world, num_key_value_heads=s["kv_heads"] // world,
              head_dim=s["head_dim"], vocab_size=s["vocab"], max_position_embeddings=max_positions,
              initializer_range=0.02, tie_word_embeddings=False)
    if s["family"] == "qwen2":
        cfg = Qwen2Config(**kw)
    else:
        cfg = LlamaConfig(attention_bias=False, mlp_bias=False, **kw)
    return cfg


def build_fp16_model(shape: str, device, world: int = 1, layers: int | None = None, seed: int = 0,
                     max_positions: int = 4096):
    """Random-init fp16 model (this rank's slice) on ``device``; o_proj / down_proj all-reduce when world > 1."""
    from transformers import AutoModelForCausalLM
    cfg = local_config(shape, world, layers, max_positions)
    torch.manual_seed(seed)
    with torch.device(device):
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    if world > 1:
        for name, mod in list(model.named_modules()):
            if isinstance(mod, nn.Linear) and name.split(".")[-1] in COLUMN_SPLIT:
                _set(model, name, AllReduceLinear(mod))
    return model


def _set(root, fqn, new):
    parts = fqn.split(".")
    obj = root
    for p in parts[:-1]:
        obj = getattr(obj, p)
    setattr(obj, parts[-1], new)


def target_linears(model):
    """(fqn, module) of every Linear the reference's planners consider (lm_head is not one of them)."""
    out = []
    for name, mod in model.named_modules():
        if name.split(".")[-1] not in TARGETS:
            continue
        if isinstance(mod, nn.Linear):
            out.append((name, mod))
        elif isinstance(mod, AllReduceLinear) and isinstance(mod.inner, nn.Linear):
            out.append((name, mod.inner))
    return out


@dataclasses.dataclass
class PlanEntry:
    name: str
    bits: int            # 2, 4 or 16
    group_size: int
    outlier_columns: int
    residual_rank: int


def seeded_plan(model, probs=(0.6, 0.3, 0.1), seed=0, group_size=128, outlier_frac=0.01, residual_rank=8,
                global_k: dict | None = None):
    """Per-Linear bit width drawn from ``probs`` = P(INT2), P(INT4), P(FP16) with a seeded generator.
    The outlier count is ``int(outlier_frac * K)`` of the *unsharded* layer, snapped as the module
    constructors do (``global_k`` maps a leaf name to the unsharded K when the model is a shard)."""
    g = torch.Generator().manual_seed(seed)
    names = [n for n, _ in target_linears(model)]
    draws = torch.multinomial(torch.tensor(probs, dtype=torch.float), len(names), replacement=True, generator=g)
    mods = dict(model.named_modules())
    plan = []
    for n, d in zip(names, draws.tolist()):
        lin = mods[n].inner if isinstance(mods[n], AllReduceLinear) else mods[n]
        k = lin.in_features
        kg = (global_k or {}).get(n.split(".")[-1], k)
        oc = snap_outlier_count(int(outlier_frac * kg), kg)
        bits = (2, 4, 16)[d]
        plan.append(PlanEntry(n, bits, group_size, min(oc, k), residual_rank if bits != 16 else 0))
    return plan


@torch.no_grad()
def apply_plan(model, plan, seed=0):
    """Swap the planned Linears for packed modules (quantised where the weight lives, GPU or CPU).
    Residual factors are drawn N(0, 0.01) as the benchmark configurations specify."""
    mods = dict(model.named_modules())
    g = torch.Generator(device="cpu").manual_seed(seed + 1)
    for e in plan:
        if e.bits == 16:
            continue
        holder = mods[e.name]
        lin = holder.inner if isinstance(holder, AllReduceLinear) else holder
        cls = HybridInt2Linear if e.bits == 2 else HybridInt4Linear
        new = cls(lin, e.group_size, None, e.outlier_columns)
        if e.residual_rank:
            u = torch.randn(lin.out_features, e.residual_rank, generator=g) * 0.01
            v = torch.randn(e.residual_rank, lin.in_features, generator=g) * 0.01
            new.set_residual(u.to(lin.weight.device), v.to(lin.weight.device))
        new.graph_safe = True
        if isinstance(holder, AllReduceLinear):
            holder.inner = new
        else:
            _set(model, e.name, new)
        lin.weight = None          # drop the dense source
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
    return model


@torch.no_grad()
def build_mixed_model_streaming(shape: str, device, world: int = 1, layers: int | None = None, seed: int = 0,
                                max_positions: int = 4096, probs=(0.6, 0.3, 0.1)):
    """The seeded mixed-bit model (this rank's slice) built without ever holding the dense model: the
    skeleton lives on the meta device, and every Linear is materialised (random N(0, 0.02) fp16),
    quantised where the plan says so and dropped, one at a time.  Peak memory is the packed model plus
    one dense Linear, so the 70B shape (139 GB in fp16, 26 GB packed) builds on a single GPU.
    Returns ``(model, plan)``; same plan and residual factors as ``seeded_plan`` + ``apply_plan``
    (the dense values differ: they are drawn per layer, not in construction order)."""
    from transformers import AutoModelForCausalLM
    cfg = local_config(shape, world, layers, max_positions)
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    model.eval()
    s = SHAPES[shape]
    if world > 1:
        for name, mod in list(model.named_modules()):
            if isinstance(mod, nn.Linear) and name.split(".")[-1] in COLUMN_SPLIT:
                _set(model, name, AllReduceLinear(mod))
    plan = seeded_plan(model, probs, seed, global_k={"o_proj": s["heads"] * s["head_dim"], "down_proj": s["inter"]})
    by_name = {e.name: e for e in plan}
    dev = torch.device(device)
    gen = torch.Generator(device=dev).manual_seed(seed)
    g_res = torch.Generator(device="cpu").manual_seed(seed + 1)

    def dense(meta_lin):
        lin = nn.Linear(meta_lin.in_features, meta_lin.out_features, bias=meta_lin.bias is not None, device=dev, dtype=torch.float16)
        lin.weight.normal_(0, 0.02, generator=gen)
        if lin.bias is not None:
            lin.bias.zero_()
        return lin

    for name, mod in list(model.named_modules()):
        leaf = name.split(".")[-1]
        holder = mod if isinstance(mod, AllReduceLinear) else None
        lin = holder.inner if holder is not None else mod
        if not isinstance(lin, nn.Linear) or (holder is None and isinstance(dict(model.named_modules()).get(name.rsplit(".", 1)[0]), AllReduceLinear)):
            continue
        new = dense(lin)
        e = by_name.get(name)
        if e is not None and e.bits != 16:
            cls = HybridInt2Linear if e.bits == 2 else HybridInt4Linear
            packed = cls(new, e.group_size, None, e.outlier_columns)
            if e.residual_rank:
                u = torch.randn(new.out_features, e.residual_rank, generator=g_res) * 0.01
                v = torch.randn(e.residual_rank, new.in_features, generator=g_res) * 0.01
                packed.set_residual(u.to(dev), v.to(dev))
            packed.graph_safe = True
            new = packed
        if holder is not None:
            holder.inner = new
        else:
            _set(model, name, new)
    # what is still on the meta device: embeddings, norms, rotary tables
    for name, mod in list(model.named_modules()):
        if "rotary" in type(mod).__name__.lower() and any(b.is_meta for b in mod.buffers()):
            _set(model, name, type(mod)(config=cfg, device=dev))
    for name, prm in list(model.named_parameters()):
        if prm.is_meta:
            real = torch.empty(prm.shape, dtype=prm.dtype, device=dev)
            if name.endswith("norm.weight") or "layernorm" in name:
                real.fill_(1.0)
            else:
                real.normal_(0, 0.02, generator=gen)
            parent, leaf = name.rsplit(".", 1)
            setattr(dict(model.named_modules())[parent], leaf, nn.Parameter(real, requires_grad=False))
    assert not any(t.is_meta for t in list(model.parameters()) + list(model.buffers())), "a tensor was left on the meta device"
    if dev.type == "cuda":
        torch.cuda.empty_cache()
    return model, plan


def chain_weight_prefetch(model) -> int:
    """Give every packed module of a decoder the weights of the Linear that runs after it as its L2
    prefetch hint (``HybridPackedLinear.prefetch_next``): while one GEMV streams, the next one's packed
    codes (or fp16 weight) are announced to L2.  Execution order: q, k, v, o, gate, up, down of each
    layer, then the next layer, finally lm_head.  Call after the model is on its device (the hints
    alias the modules' own tensors).  Returns the number of hints set."""
    order = []
    for layer in model.model.layers:
        attn, mlp = layer.self_attn, layer.mlp
        for holder, name in ((attn, "q_proj"), (attn, "k_proj"), (attn, "v_proj"), (attn, "o_proj"),
                             (mlp, "gate_proj"), (mlp, "up_proj"), (mlp, "down_proj")):
            mod = getattr(holder, name, None)
            if mod is not None:
                order.append(mod.inner if isinstance(mod, AllReduceLinear) else mod)
    if getattr(model, "lm_head", None) is not None:
        order.append(model.lm_head)

    def main_tensor(mod):
        if isinstance(mod, (HybridInt2Linear, HybridInt4Linear)):
            return mod.packed
        return getattr(mod, "weight", None)
    n = 0
    for cur, nxt in zip(order, order[1:]):
        if isinstance(cur, (HybridInt2Linear, HybridInt4Linear)):
            t = main_tensor(nxt)
            if t is not None and not t.is_meta:
                cur.__dict__["prefetch_next"] = t.detach()      # a plain attribute: never a parameter or buffer
                n += 1
    return n


def fp16_weight_bytes(shape: str, world: int = 1) -> int:
    """Bytes of the fp16 model's weights on one rank (Linear layers split ``world`` ways, embeddings
    replicated, lm_head split by vocabulary rows)."""
    s = SHAPES[shape]
    h, i, v = s["hidden"], s["inter"], s["vocab"]
    qkv = h * (s["heads"] + 2 * s["kv_heads"]) * s["head_dim"]
    per_layer = (qkv + s["heads"] * s["head_dim"] * h + 3 * h * i) // world
    return 2 * (s["layers"] * per_layer + v * h + v * h // world)


def linear_weight_bytes(model) -> dict:
    """Bytes of Linear-layer weights one decoded token must read (packed + fp16, lm_head included)."""
    packed = dense = 0
    for _, mod in model.named_modules():
        if isinstance(mod, (HybridInt2Linear, HybridInt4Linear)):
            for t in (mod.packed, mod.scales, mod.outlier_weight, mod.res_u, mod.res_v, mod.bias):
                if t is not None:
                    packed += t.numel() * t.element_size()
        elif isinstance(mod, nn.Linear) and mod.weight is not None:
            dense += mod.weight.numel() * mod.weight.element_size()
    return dict(packed_bytes=packed, fp16_bytes=dense, total=packed + dense)


def shard_lm_head(model, world: int):
    """Replace ``lm_head`` by this rank's ``vocab / world`` rows (random-init models: the rows are
    simply drawn at the smaller size).  The decoder finds the greedy token with an all-gather of
    (best logit, index) pairs (``StaticGraphDecoder(vocab_shard=...)``)."""
    head = model.lm_head
    v = head.out_features
    if world <= 1:
        return model
    if v % world:
        raise ValueError(f"vocabulary {v} is not divisible by the tensor-parallel size {world}")
    dev = head.weight.device if not head.weight.is_meta else None
    new = nn.Linear(head.in_features, v // world, bias=False, device=dev if dev is not None else "meta", dtype=torch.float16)
    if dev is not None:
        with torch.no_grad():
            new.weight.normal_(0, 0.02)
    model.lm_head = new
    return model


def _timed_decode(dec, ids, new_tokens):
    """Prefill, then ``new_tokens - 1`` graph replays timed with CUDA events: (ms per decoded token, tokens)."""
    first = dec.prefill(ids)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    rest = dec.decode(new_tokens - 1)
    e1.record()
    e1.synchronize()
    return float(e0.elapsed_time(e1)) / max(1, new_tokens - 1), torch.cat([first, rest], 1)


def decode_benchmark(shape: str, device, batch=1, prompt_len=128, new_tokens=64, probs=(0.6, 0.3, 0.1),
                     mixed=True, world=1, layers=None, seed=0, use_cuda_graph=True, compile_layers=False,
                     fuse_siblings=False, split=False, shard_vocab=True, prefetch_hints=False, one_shot=True, native_step=None):
    """Build (this rank's slice of) the model, optionally with the seeded mixed-bit plan, and run the
    fixed-length greedy decode benchmark.  Returns the runtime's result dict plus weight-byte counts.

    ``split=True`` also replays the captured decode step without the all-reduces and without the
    packed GEMVs and reports the per-token milliseconds each of them accounts for
    (``split_ms_per_token``: ``packed_gemv``, ``all_reduce``, ``other``).  ``one_shot`` (world > 1, CUDA)
    routes the K-split projections' all-reduces through the peer-memory kernel of ``comm.OneShotAllReduce``
    instead of NCCL; ``all_reduce_impl`` in the result says which ran."""
    from .runtime_v5 import generate_static_benchmark, StaticGraphDecoder
    from .optimize._hybrid_base import HybridPackedLinear
    max_pos = prompt_len + new_tokens + 16
    if mixed:
        model, _ = build_mixed_model_streaming(shape, device, world, layers, seed, max_pos, probs)
    else:
        model = build_fp16_model(shape, device, world, layers, seed, max_positions=max_pos)
    vocab_shard = None
    if world > 1 and shard_vocab:
        shard_lm_head(model, world)
        if model.lm_head.weight.is_meta:
            raise RuntimeError("lm_head was left on the meta device")
        vocab_shard = (int(torch.distributed.get_rank()), world)
    fused_groups = 0
    if mixed and fuse_siblings:
        from .optimize.siblings import fuse_decoder_siblings
        fused_groups = fuse_decoder_siblings(model)
    if mixed and prefetch_hints and not fuse_siblings:
        chain_weight_prefetch(model)
    g = torch.Generator().manual_seed(seed + 7)
    ids = torch.randint(0, SHAPES[shape]["vocab"], (batch, prompt_len), generator=g)
    comm = None
    if world > 1 and one_shot and torch.device(device).type == "cuda":
        from .comm import OneShotAllReduce
        # decode steps reduce [batch, hidden]; prefill reduces [batch * prompt_len, hidden] and stays with NCCL
        comm = OneShotAllReduce(max_elems=-(-batch * SHAPES[shape]["hidden"] // 8) * 8, device=device)
        AllReduceLinear.one_shot = comm
    try:
        res = _decode_benchmark_body(model, ids, shape, device, batch, prompt_len, new_tokens, mixed, world,
                                     use_cuda_graph, compile_layers, vocab_shard, fused_groups, split, native_step)
        res["all_reduce_impl"] = "none" if world <= 1 else ("one_shot_peer_memory" if comm is not None else "nccl")
        if comm is not None:
            res["one_shot_status"] = comm.status()
    finally:
        if comm is not None:
            AllReduceLinear.one_shot = None
            comm.close()
    return res


def _decode_benchmark_body(model, ids, shape, device, batch, prompt_len, new_tokens, mixed, world, use_cuda_graph,
                           compile_layers, vocab_shard, fused_groups, split, native_step=None):
    from .runtime_v5 import generate_static_benchmark, StaticGraphDecoder
    from .optimize._hybrid_base import HybridPackedLinear
    res = generate_static_benchmark(model, input_ids=ids, max_new_tokens=new_tokens, device=device,
                                    use_cuda_graph=use_cuda_graph, compile_layers=compile_layers, vocab_shard=vocab_shard,
                                    native_step=native_step)
    dec = res.pop("decoder")
    res.update(linear_weight_bytes(model))
    res["shape"], res["mixed"], res["world"] = shape, mixed, world
    res["fused_sibling_groups"] = fused_groups
    res["all_reduces_per_token"] = sum(isinstance(m, AllReduceLinear) for m in model.modules()) if world > 1 else 0
    res["packed_gemvs_per_token"] = sum(isinstance(m, HybridPackedLinear) for m in model.modules())
    res["lm_head_rows_per_rank"] = int(model.lm_head.out_features)
    if split and use_cuda_graph and torch.device(device).type == "cuda":
        ids_d = ids.to(device)
        full, _ = _timed_decode(dec, ids_d, new_tokens)
        parts = {}
        for key, holder, attr in (("all_reduce", AllReduceLinear, "skip_collective"), ("packed_gemv", HybridPackedLinear, "skip_gemv")):
            if (key == "all_reduce" and world <= 1) or (key == "packed_gemv" and not mixed):
                parts[key] = 0.0
                continue
            setattr(holder, attr, True)
            try:
                d2 = StaticGraphDecoder(model, batch, prompt_len + new_tokens + 8, device=device, vocab_shard=vocab_shard,
                                        native_step=False if compile_layers else native_step)
                d2.prefill(ids_d)
                d2.capture()
                without, _ = _timed_decode(d2, ids_d, new_tokens)
            finally:
                setattr(holder, attr, False)
            parts[key] = max(0.0, full - without)
            del d2
        parts["other"] = max(0.0, full - parts["all_reduce"] - parts["packed_gemv"])
        parts["total"] = full
        res["split_ms_per_token"] = parts
    del dec
    return res
