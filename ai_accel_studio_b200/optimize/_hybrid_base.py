"""Shared construction and forward logic of the hybrid packed Linear modules."""
from __future__ import annotations

import torch
from torch import nn
import torch.nn.functional as F

OUTLIER_COUNTS = (4, 8, 16, 32, 64)


def snap_outlier_count(requested: int, k: int) -> int:
    """Clamp to [0, K], then snap to the nearest of 4/8/16/32/64 (ties go to the smaller
    count), as both reference constructors do (ai_accel_lab/optimize/hybrid_int2.py:34-38,
    hybrid_int4.py:14-15).  The kernels accept any count; the snapping is kept so that modules
    built here hold exactly the columns the reference would pick."""
    oc = max(0, min(int(requested), k))
    if oc and oc not in OUTLIER_COUNTS:
        oc = min(OUTLIER_COUNTS, key=lambda v: abs(v - oc))
        oc = min(oc, k)
    return oc


def select_outliers(module: nn.Module, w: torch.Tensor, activation_rms, outlier_columns: int) -> torch.Tensor:
    """Register ``outlier_idx`` / ``outlier_weight`` and return the weight with those columns zeroed.

    Score = column RMS of W (times the activation RMS when given); the top columns are kept
    exactly in fp16 and removed from the quantised base so the two terms never double count."""
    n, k = w.shape
    oc = snap_outlier_count(outlier_columns, k)
    if not oc:
        module.register_buffer("outlier_idx", torch.empty(0, device=w.device, dtype=torch.int32))
        module.register_buffer("outlier_weight", torch.empty((n, 0), device=w.device, dtype=torch.float16))
        return w
    score = w.float().square().mean(0).sqrt()
    if activation_rms is not None:
        score = score * activation_rms.detach().float().to(w.device)[:k]
    idx = torch.topk(score, k=oc, largest=True, sorted=True).indices
    module.register_buffer("outlier_idx", idx.to(torch.int32))
    module.register_buffer("outlier_weight", w[:, idx].to(torch.float16).contiguous())
    base = w.clone()
    base[:, idx] = 0
    return base


class HybridPackedLinear(nn.Module):
    """Common forward: M <= 4 -> one fused GEMV launch; up to ``chunked_max_rows`` rows -> one fused launch per
    four rows; larger M -> CUDA dequantisation into the activation dtype + library GEMMs for the base, outlier
    and residual terms."""

    bits: int = 0
    residual_rank: int = 0
    # Measurement aid: when set, the decode path (every row count served by fused GEMVs) launches nothing and returns a zero buffer
    # of the right shape, so that replaying a decode step with and without the packed GEMVs tells how
    # much of the step they are.  Never set in production.
    skip_gemv: bool = False
    # Optional hint for the decode path: a static tensor (normally the packed codes of the module that
    # runs next) announced to L2 while this module's GEMV runs; see model_tools.chain_weight_prefetch.
    prefetch_next = None
    # Largest row count served by repeated fused GEMVs (groups of four rows) instead of the dequantise + GEMM route.
    chunked_max_rows: int = 16
    # Set by siblings.merge_gate_up: the rows are (8 gate, 8 up) blocks of a feed-forward block's two
    # input projections and forward returns silu(gate(x)) * up(x), of width out_features = rows / 2.
    gated_pairs: bool = False

    def _finish_init(self, pw, k: int, n: int, source_bias):
        self.register_buffer("packed", pw.packed)
        self.register_buffer("scales", pw.scales)
        self.original_k = pw.original_k
        self.padded_k = pw.padded_k
        self.group_size = pw.group_size
        self.in_features = k
        self.out_features = n
        self.graph_safe = False      # toggled by runtime_v5.prepare_static_compile; this build is always graph safe
        self.kernel = "auto"         # "auto" | "simt" | "mma": kernel family for the fused path
        if source_bias is None:
            self.bias = None
        else:
            self.register_buffer("bias", source_bias.detach().to(torch.float16))

    @classmethod
    def from_buffers(cls, packed, scales, original_k: int, group_size: int, outlier_idx=None,
                     outlier_weight=None, bias=None, res_u=None, res_v=None):
        """Build a module directly from packed buffers (no source ``nn.Linear``): what a loader
        that already holds a bundle's tensors, or a tensor-parallel sharder, needs.  ``cls`` must be
        one of the concrete classes (it fixes the bit width)."""
        if cls.bits not in (2, 4):
            raise TypeError("call from_buffers on HybridInt2Linear or HybridInt4Linear")
        self = cls.__new__(cls)
        nn.Module.__init__(self)
        n = int(packed.shape[0])
        dev = packed.device
        if outlier_idx is None or outlier_idx.numel() == 0:
            outlier_idx = torch.empty(0, device=dev, dtype=torch.int32)
            outlier_weight = torch.empty((n, 0), device=dev, dtype=torch.float16)
        self.register_buffer("outlier_idx", outlier_idx.to(torch.int32))
        self.register_buffer("outlier_weight", outlier_weight.to(torch.float16).contiguous())
        self.register_buffer("packed", packed.contiguous())
        self.register_buffer("scales", scales.to(torch.float16).contiguous())
        self.original_k = int(original_k)
        self.padded_k = int(packed.shape[1]) * (8 // cls.bits)
        self.group_size = int(group_size)
        self.in_features = int(original_k)
        self.out_features = n
        self.graph_safe = False
        self.kernel = "auto"
        self.backend = "auto"
        if bias is None:
            self.bias = None
        else:
            self.register_buffer("bias", bias.to(torch.float16))
        self.residual_rank = 0
        self.res_u = None
        self.res_v = None
        if res_u is not None and res_u.numel():
            self.set_residual(res_u, res_v)
        if packed.is_cuda:
            from .. import ops
            ops.ensure_workspace(packed.device)
        return self

    def effective_weight(self) -> torch.Tensor:
        """The float32 matrix this module multiplies by: dequantised base + outlier columns + U.V.
        Plain torch ops on whatever device the buffers live on -- for construction-time error
        analysis and the planner's quality measure, never for the forward pass."""
        p = self.packed
        if self.bits == 2:
            codes = torch.stack([(p >> s) & 3 for s in (0, 2, 4, 6)], dim=-1).reshape(p.shape[0], -1).long()
            from ..kernels.groupwise_int2 import INT2_LEVELS
            vals = torch.tensor(INT2_LEVELS, device=p.device, dtype=torch.float32)[codes]
        else:
            vals = (torch.stack([p & 15, p >> 4], dim=-1).reshape(p.shape[0], -1).to(torch.int16) - 8).float()
        w = (vals * self.scales.float().repeat_interleave(self.group_size, dim=1))[:, :self.original_k]
        if self.outlier_idx.numel():
            w.index_add_(1, self.outlier_idx.long(), self.outlier_weight.float())     # repeated columns add up
        if getattr(self, "residual_rank", 0):
            w = w + self.res_u.float() @ self.res_v.float()
        return w

    def set_residual(self, res_u: torch.Tensor, res_v: torch.Tensor) -> None:
        """Attach given low-rank factors ``res_u [N,r]``, ``res_v [r,K]`` (replacing any present)."""
        if res_u.shape[0] != self.packed.shape[0] or res_v.shape[1] != self.in_features or res_u.shape[1] != res_v.shape[0]:
            raise ValueError("res_u must be [N,r] and res_v [r,K]")
        dev = self.packed.device
        for name in ("res_u", "res_v"):
            if name in self.__dict__:
                del self.__dict__[name]     # plain None placeholders make way for buffers
            if name in self._buffers:
                del self._buffers[name]
        self.__dict__.pop("_call", None)
        self.register_buffer("res_u", res_u.detach().to(dev, torch.float16).contiguous())
        self.register_buffer("res_v", res_v.detach().to(dev, torch.float16).contiguous())
        self.residual_rank = int(res_u.shape[1])

    _LAUNCH_OPERANDS = frozenset(("packed", "scales", "bias", "outlier_idx", "outlier_weight", "res_u", "res_v", "residual_rank"))

    def __setattr__(self, name, value):
        if name in HybridPackedLinear._LAUNCH_OPERANDS:
            self.__dict__.pop("_call", None)          # the prepared launch holds the old tensor's address
        super().__setattr__(name, value)

    def _apply(self, fn, *args, **kwargs):
        self.__dict__.pop("_call", None)
        out = super()._apply(fn, *args, **kwargs)
        if self.packed.is_cuda:
            from .. import ops
            ops.ensure_workspace(self.packed.device)   # outside any graph capture, pointer-stable afterwards
        return out

    def _fused(self, xp: torch.Tensor) -> torch.Tensor:
        from .. import _cabi, ops
        if not torch.compiler.is_compiling():
            # eager: the prepared launch of this module for activations of this shape.  It is dropped whenever a
            # buffer is replaced (__setattr__, _apply, set_residual) and rebuilt when a setting has changed.
            d = self.__dict__
            pre = self.prefetch_next
            sig = (xp.shape[0], xp.dtype, xp.stride(0), xp.device, self.kernel, d.get("debug", 0), self.gated_pairs, id(pre))
            call = d.get("_call")
            if call is None or call.key != sig or call.keep[0] is not d["_buffers"]["packed"]:
                has_o = self.outlier_idx.numel() > 0
                call = ops.prepare_call(xp, self.packed, self.scales, self.bias, self.outlier_idx if has_o else None,
                                        self.outlier_weight if has_o else None,
                                        self.res_u if self.residual_rank else None, self.res_v if self.residual_rank else None,
                                        self.bits, self.group_size, self.original_k, 3 if self.gated_pairs else 0,
                                        self._kernel_code(), pre, sig)
                call.keep = (self.packed, self.scales, self.bias, self.outlier_idx, self.outlier_weight, self.res_u, self.res_v, pre)
                d["_call"] = call
            return call.run(xp)
        return ops.gemv(xp, self.packed, self.scales, self.bias, self.outlier_idx if self.outlier_idx.numel() else None,
                        self.outlier_weight if self.outlier_idx.numel() else None,
                        self.res_u if self.residual_rank else None, self.res_v if self.residual_rank else None,
                        self.bits, self.group_size, self.original_k, 3 if self.gated_pairs else 0, self._kernel_code(), self.prefetch_next)

    def _kernel_code(self) -> int:
        from .. import _cabi
        return _cabi.KERNEL[self.kernel] | (int(getattr(self, "debug", 0)) << 8)

    def forward_into(self, x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """Decode-path forward (at most 4 rows) written into ``out`` [M, out_features]: a CUDA tensor,
        or a pinned host tensor that the kernel then writes directly (no device-to-host copy)."""
        from .. import _cabi, ops
        if not x.is_cuda:
            raise RuntimeError(f"{type(self).__name__} computes on CUDA only (no CPU fallback); got a {x.device} tensor")
        xflat = x.reshape(-1, x.shape[-1])
        if xflat.shape[0] > 4:
            raise ValueError("forward_into is the decode path: at most 4 rows")
        xp = xflat if self.padded_k == self.original_k else F.pad(xflat, (0, self.padded_k - self.original_k))
        if xp.stride(1) != 1:
            xp = xp.contiguous()
        has_o = self.outlier_idx.numel() > 0
        return ops.gemv_into(xp, self.packed, self.scales, self.bias, self.outlier_idx if has_o else None,
                             self.outlier_weight if has_o else None,
                             self.res_u if self.residual_rank else None, self.res_v if self.residual_rank else None,
                             self.bits, self.group_size, self.original_k, 3 if self.gated_pairs else 0, self._kernel_code(), out, self.prefetch_next)

    def _dense(self, xflat: torch.Tensor) -> torch.Tensor:
        from .. import ops
        name = str(xflat.dtype).split(".")[-1]
        w = ops.dequant(self.packed, self.scales, self.bits, self.group_size, self.original_k, name)
        y = F.linear(xflat, w, None if self.bias is None else self.bias.to(xflat.dtype))
        if self.outlier_idx.numel():
            y = y + F.linear(xflat[:, self.outlier_idx.long()], self.outlier_weight.to(xflat.dtype))
        if self.residual_rank:
            y = y + F.linear(F.linear(xflat.to(self.res_v.dtype), self.res_v), self.res_u).to(y.dtype)
        if self.gated_pairs:
            pairs = y.view(y.shape[0], -1, 2, 8)
            y = (F.silu(pairs[:, :, 0, :]) * pairs[:, :, 1, :]).reshape(y.shape[0], -1)
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError(f"{type(self).__name__} computes on CUDA only (no CPU fallback); got a {x.device} tensor")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("fp16/bf16 activations required")
        shape = x.shape
        xflat = x.reshape(-1, shape[-1])
        if xflat.shape[0] <= self.chunked_max_rows and HybridPackedLinear.skip_gemv:
            key = (xflat.shape[0], x.dtype)
            cache = self.__dict__.setdefault("_skip_out", {})
            if key not in cache:
                cache[key] = torch.zeros((xflat.shape[0], self.out_features), dtype=x.dtype, device=x.device)
            y = cache[key]
        elif xflat.shape[0] <= 4:
            xp = xflat if self.padded_k == self.original_k else F.pad(xflat, (0, self.padded_k - self.original_k))
            if xp.stride(1) != 1:
                xp = xp.contiguous()
            y = self._fused(xp)
        elif xflat.shape[0] <= self.chunked_max_rows:
            y = self._fused_chunks(xflat)
        else:
            y = self._dense(xflat)
        return y.reshape(*shape[:-1], self.out_features)

    def _fused_chunks(self, xflat: torch.Tensor) -> torch.Tensor:
        """5 .. ``chunked_max_rows`` rows (a decode batch beyond the kernel's four): the fused GEMV over groups of
        four rows, written into one result.  The packed weights of one Linear stay in L2 between the launches,
        where dequantising the whole matrix for every token (the M > 4 route of the reference,
        ``ai_accel_lab/optimize/hybrid_int4.py:36-37``) would write and re-read 2 bytes per weight."""
        from .. import ops
        xp = xflat if self.padded_k == self.original_k else F.pad(xflat, (0, self.padded_k - self.original_k))
        if xp.stride(1) != 1:
            xp = xp.contiguous()
        has_o = self.outlier_idx.numel() > 0
        act = 3 if self.gated_pairs else 0
        y = torch.empty((xp.shape[0], self.out_features), dtype=xp.dtype, device=xp.device)
        for lo in range(0, xp.shape[0], 4):
            ops.gemv_into(xp[lo:lo + 4], self.packed, self.scales, self.bias, self.outlier_idx if has_o else None,
                          self.outlier_weight if has_o else None,
                          self.res_u if self.residual_rank else None, self.res_v if self.residual_rank else None,
                          self.bits, self.group_size, self.original_k, act, self._kernel_code(), y[lo:lo + 4], self.prefetch_next)
        return y
