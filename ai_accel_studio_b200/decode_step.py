"""One decode step of a Llama / Qwen2 style decoder with this package's own kernels between the GEMVs.

The reference's decode loop is the Hugging Face model under ``torch.compile(mode='reduce-overhead')``
(``ai_accel_lab/runtime_v5.py:7-23``): the normalisations, rotary embedding, cache update, attention,
SwiGLU product and residual additions between its packed GEMVs are whatever the framework generates.
Run eagerly those are some fifty small kernels per layer, and on a B200 they cost about twice what the
packed GEMVs cost.  ``NativeDecodeStep`` walks the same modules (the Linear layers are called as they
are: packed modules, fp16 ``nn.Linear``, tensor-parallel shards with their all-reduce, fused siblings)
and replaces everything in between by four kernels of ``include/qdecode_b200.h``:

    rmsnorm (+ residual update) -> q, k, v -> rope + cache append -> attention -> o
    rmsnorm (+ residual update) -> gate / up (+ silu * mul, fused into the GEMV where possible) -> down

It reads and writes the ``StaticCache`` tensors of the Hugging Face model in place, so the prompt can
still be processed by the framework's own forward.  Values are rounded to the activation type
wherever the framework's operators would round them; sums run in fp32 in a different order, so logits
agree to rounding, not bitwise.
"""
from __future__ import annotations

import ctypes as C

import torch
from torch import nn

from . import _cabi

_DT = {torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16}


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def rmsnorm(h: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    """``h += delta`` in place (when ``delta`` is given), then the RMS normalisation of ``h`` times ``weight``.
    ``h``, ``delta``: ``[rows, hidden]`` fp16 / bf16 CUDA tensors with unit inner stride."""
    if not h.is_cuda or h.dtype not in _DT or h.ndim != 2 or h.stride(1) != 1:
        raise ValueError("h must be a [rows, hidden] fp16/bf16 CUDA tensor with unit inner stride")
    if delta is not None and (delta.shape != h.shape or delta.dtype != h.dtype or delta.stride(1) != 1):
        raise ValueError("delta must match h")
    if weight.dtype != h.dtype or weight.numel() != h.shape[1] or not weight.is_contiguous():
        raise ValueError("weight must be a contiguous [hidden] tensor of h's dtype")
    y = out if out is not None else torch.empty_like(h, memory_format=torch.contiguous_format)
    with torch.cuda.device(h.device):
        _cabi.check(_cabi.lib().qdec_rmsnorm(_ptr(h), h.stride(0), _ptr(delta), 0 if delta is None else delta.stride(0),
                                             _ptr(weight), _ptr(y), y.stride(0), h.shape[0], h.shape[1], float(eps),
                                             _DT[h.dtype], _stream()))
    return y


def rope_append(q, k, v, cos, sin, pos, kcache, vcache, head_dim: int, status=None) -> None:
    """Rotate ``q`` in place, write the rotated ``k`` and ``v`` into the caches at position ``pos[0]``
    (``pos``: int64 CUDA tensor).  ``q``: ``[B, Hq * D]``, ``k`` / ``v``: ``[B, Hkv * D]``; ``cos`` / ``sin``:
    ``[rows, D]``; caches ``[B, Hkv, max_len, D]`` contiguous."""
    b = q.shape[0]
    hq, hkv = q.shape[1] // head_dim, k.shape[1] // head_dim
    if tuple(kcache.shape) != (b, hkv, kcache.shape[2], head_dim) or kcache.shape != vcache.shape or \
            not kcache.is_contiguous() or not vcache.is_contiguous():
        raise ValueError("caches must be contiguous [B, Hkv, max_len, D]")
    if pos.dtype != torch.int64 or not pos.is_cuda:
        raise ValueError("pos must be an int64 CUDA tensor")
    if cos.shape != sin.shape or cos.shape[1] != head_dim or not cos.is_contiguous() or not sin.is_contiguous() or cos.dtype != q.dtype:
        raise ValueError("cos / sin must be contiguous [rows, D] tables of q's dtype")
    for t in (q, k, v):
        if t.stride(1) != 1 or t.dtype != q.dtype:
            raise ValueError("q, k, v need unit inner stride and one dtype")
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().qdec_rope_append(_ptr(q), q.stride(0), _ptr(k), k.stride(0), _ptr(v), v.stride(0), _ptr(cos), _ptr(sin),
                                                 cos.shape[0], _ptr(pos), _ptr(kcache), _ptr(vcache), b, hq, hkv, head_dim,
                                                 kcache.shape[2], _ptr(status), _DT[q.dtype], _stream()))


def attention_workspace(batch: int, q_heads: int, kv_heads: int, head_dim: int, max_len: int, device) -> torch.Tensor:
    n = int(_cabi.lib().qdec_attention_workspace_bytes(batch, q_heads, kv_heads, head_dim, max_len))
    if n == 0:
        raise ValueError("bad attention sizes")
    return torch.zeros(n + 256, dtype=torch.uint8, device=device)


def attention(q, kcache, vcache, pos, scale: float, workspace: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Softmax attention of one query token per sequence over cache positions ``0 .. pos[0]``;
    returns ``[B, Hq * D]``."""
    b, hkv, max_len, d = kcache.shape
    hq = q.shape[1] // d
    o = out if out is not None else torch.empty((b, hq * d), dtype=q.dtype, device=q.device)
    off = (-workspace.data_ptr()) % 256
    with torch.cuda.device(q.device):
        _cabi.check(_cabi.lib().qdec_attention(_ptr(q), q.stride(0), _ptr(kcache), _ptr(vcache), _ptr(pos), _ptr(o), o.stride(0),
                                               b, hq, hkv, d, max_len, float(scale), C.c_void_p(workspace.data_ptr() + off),
                                               workspace.numel() - off, _DT[q.dtype], _stream()))
    return o


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if gate.shape != up.shape or gate.dtype != up.dtype or gate.ndim != 2 or gate.stride(1) != 1 or up.stride(1) != 1:
        raise ValueError("gate and up must be [rows, width] tensors of one dtype with unit inner stride")
    y = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    with torch.cuda.device(gate.device):
        _cabi.check(_cabi.lib().qdec_silu_mul(_ptr(gate), gate.stride(0), _ptr(up), up.stride(0), _ptr(y), y.stride(0),
                                              gate.shape[0], gate.shape[1], _DT[gate.dtype], _stream()))
    return y


def _is_silu(fn) -> bool:
    return isinstance(fn, nn.SiLU) or fn is torch.nn.functional.silu or type(fn).__name__ in ("SiLUActivation", "SiLU")


def unsupported_reason(model) -> str | None:
    """None if ``NativeDecodeStep`` can run this model, else why not (the caller then keeps the
    framework's own forward for the decode step)."""
    inner = getattr(model, "model", None)
    if inner is None or not hasattr(inner, "layers") or not hasattr(inner, "embed_tokens") or not hasattr(inner, "norm") \
            or not hasattr(inner, "rotary_emb") or not hasattr(model, "lm_head"):
        return "not a decoder with model.layers / embed_tokens / norm / rotary_emb / lm_head"
    cfg = model.config
    if getattr(cfg, "sliding_window", None) and getattr(cfg, "use_sliding_window", False):
        return "sliding-window attention"
    for layer in inner.layers:
        attn, mlp = getattr(layer, "self_attn", None), getattr(layer, "mlp", None)
        if attn is None or mlp is None or not hasattr(layer, "input_layernorm") or not hasattr(layer, "post_attention_layernorm"):
            return "a layer lacks self_attn / mlp / the two layer norms"
        if any(hasattr(attn, n) for n in ("q_norm", "k_norm")):
            return "per-head q / k normalisation"
        if not all(hasattr(attn, n) for n in ("q_proj", "k_proj", "v_proj", "o_proj")):
            return "attention without separate q / k / v / o projections"
        for norm in (layer.input_layernorm, layer.post_attention_layernorm):
            if not hasattr(norm, "weight") or not hasattr(norm, "variance_epsilon") or getattr(norm, "bias", None) is not None:
                return "a layer norm that is not a plain RMS norm"
        gated = type(mlp).__name__ == "GatedFeedForward"
        if not gated and (not all(hasattr(mlp, n) for n in ("gate_proj", "up_proj", "down_proj")) or not _is_silu(getattr(mlp, "act_fn", None))):
            return "a feed-forward block that is not SwiGLU"
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    if head_dim not in (64, 128):
        return f"head_dim {head_dim} (64 and 128 are built)"
    return None


_SIDE = {}


def _side_streams(device):
    """Two side streams per device, shared by every decode step on it, each with its own GEMV scratch buffer
    (taken from the pool now, i.e. before any graph capture)."""
    from . import ops
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _SIDE:
        _SIDE[key] = [torch.cuda.Stream(device=device) for _ in range(2)]
        for s in _SIDE[key]:
            ops.ensure_workspace(device, s)
    return _SIDE[key]


class NativeDecodeStep:
    """``step(tok, pos)``: logits ``[B, vocab]`` of the next token, given the current token ids ``[B, 1]``
    and their position (int64 CUDA tensor of one element, the same for every sequence), with the
    model's ``StaticCache`` updated in place.  Build it after the cache has been filled once (its
    tensors are allocated lazily by the first forward)."""

    def __init__(self, model, cache, batch: int, max_len: int):
        why = unsupported_reason(model)
        if why is not None:
            raise NotImplementedError(f"native decode step: {why}")
        self.model, self.inner = model, model.model
        cfg = model.config
        self.batch, self.max_len = int(batch), int(max_len)
        w = self.inner.embed_tokens.weight
        self.device, self.dtype = w.device, w.dtype
        if self.dtype not in _DT:
            raise NotImplementedError("native decode step: fp16 / bf16 models only")
        self.head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.layers = list(self.inner.layers)
        self.kv = []
        for i, _ in enumerate(self.layers):
            lay = cache.layers[i]
            k, v = getattr(lay, "keys", None), getattr(lay, "values", None)
            if k is None or v is None or k.ndim != 4 or not k.is_contiguous() or k.shape[2] != self.max_len or k.shape[0] != self.batch:
                raise RuntimeError("the static cache is not initialised for this batch / length: run a prefill first")
            self.kv.append((k, v))
        with torch.no_grad():
            ids = torch.arange(self.max_len, device=self.device)[None]
            cos, sin = self.inner.rotary_emb(torch.zeros(1, dtype=self.dtype, device=self.device), ids)
        self.cos = cos[0].to(self.dtype).contiguous()
        self.sin = sin[0].to(self.dtype).contiguous()
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        hq = max(int(getattr(l.self_attn.q_proj, "out_features")) // self.head_dim for l in self.layers)
        hkv = min(k.shape[1] for k, _ in self.kv)
        self.att_ws = attention_workspace(self.batch, hq, hkv, self.head_dim, self.max_len, self.device)
        self.side = _side_streams(self.device) if NativeDecodeStep.parallel_kv else None

    # Launch the k and v projections on side streams beside q when the three are separate modules: their grids are
    # small (one CTA per 16-row tile), so they run next to each other instead of one after the other
    # (Llama-3-8B shape, one GPU: 333 -> 362 tok/s).
    parallel_kv = True

    def _qkv(self, attn, x):
        from .optimize._hybrid_base import HybridPackedLinear
        mods = (attn.q_proj, attn.k_proj, attn.v_proj)
        if self.side is None or not all(isinstance(m, (HybridPackedLinear, nn.Linear)) for m in mods):
            return attn.q_proj(x), attn.k_proj(x), attn.v_proj(x)
        main = torch.cuda.current_stream(self.device)
        outs = [None, None]
        for i, (s, m) in enumerate(zip(self.side, (attn.k_proj, attn.v_proj))):
            s.wait_stream(main)                                  # x is ready
            with torch.cuda.stream(s):
                outs[i] = m(x)
        q = attn.q_proj(x)
        for s, o in zip(self.side, outs):
            main.wait_stream(s)
            o.record_stream(main)                                # consumed on the main stream: not to be recycled before that
        x.record_stream(self.side[0])
        x.record_stream(self.side[1])
        return q, outs[0], outs[1]

    # Fuse the all-reduce of the K-split projections into the normalisation that consumes their result
    # (comm.OneShotAllReduce.allreduce_rmsnorm) when tensor parallelism runs on the one-shot buffers.  Off by
    # default: one CTA per row does the push, the wait, the sum and the norm in sequence, and that measured slower
    # than the two kernels it replaces (Llama-3-70B shape on 2 GPUs: 85.7 against 88.0 tok/s).
    fuse_reduce = False

    @staticmethod
    def _project(linear, x):
        """A K-split projection that would all-reduce its result hands back its partial sum when the group's one-shot
        buffers can take it: the reduction is then fused into the normalisation that consumes it."""
        from .tp import AllReduceLinear
        if isinstance(linear, AllReduceLinear) and not AllReduceLinear.skip_collective:
            comm = AllReduceLinear.one_shot
            if NativeDecodeStep.fuse_reduce and comm is not None and comm.world > 1:
                y = linear.inner(x)
                if comm.fits_rows(y):
                    return y, comm
                if comm.fits(y):
                    return comm(y), None
                torch.distributed.all_reduce(y, group=linear.group)
                return y, None
        return linear(x), None

    @staticmethod
    def _norm(h, delta, comm, norm):
        if comm is not None:
            return comm.allreduce_rmsnorm(delta, h, norm.weight, norm.variance_epsilon)
        return rmsnorm(h, delta, norm.weight, norm.variance_epsilon)

    @torch.no_grad()
    def step(self, tok: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        inner, d = self.inner, self.head_dim
        h = inner.embed_tokens(tok).reshape(self.batch, -1).contiguous()
        delta = comm = None
        for i, layer in enumerate(self.layers):
            attn, mlp = layer.self_attn, layer.mlp
            x = self._norm(h, delta, comm, layer.input_layernorm)
            q, k, v = self._qkv(attn, x)
            kc, vc = self.kv[i]
            rope_append(q, k, v, self.cos, self.sin, pos, kc, vc, d, self.status)
            a = attention(q, kc, vc, pos, float(getattr(attn, "scaling", d ** -0.5)), self.att_ws)
            delta, comm = self._project(attn.o_proj, a)
            x = self._norm(h, delta, comm, layer.post_attention_layernorm)
            if type(mlp).__name__ == "GatedFeedForward":
                delta, comm = self._project(mlp.down_proj, mlp.gate_up(x))
            else:
                delta, comm = self._project(mlp.down_proj, silu_mul(mlp.gate_proj(x), mlp.up_proj(x)))
        x = self._norm(h, delta, comm, inner.norm)
        return self.model.lm_head(x)

    def check_status(self) -> int:
        """0, or 1 if a step was asked to write past the cache or the rotary table (synchronises)."""
        v = int(self.status.item())
        self.status.zero_()
        return v
