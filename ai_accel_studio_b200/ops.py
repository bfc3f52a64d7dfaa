"""torch custom ops over the C ABI (namespace ``b200q``).

The ops are registered with ``torch.library`` together with fake (meta) implementations, so
``torch.compile`` traces through them without graph breaks and CUDA-graph capture records the
launches.  Each call passes raw device pointers and ``torch.cuda.current_stream()`` to the
shared library; nothing is synchronised and the only allocation is the output tensor.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi

_DT = {torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16, torch.float32: _cabi.F32}
_DT_NAME = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}

# Scratch buffers.  A workspace must not be shared by GEMVs that can overlap on the device (it holds
# the arrival counters and the launch tag of the residual projections), and calls on different
# streams can overlap.  So every (device, stream) pair gets a workspace of its own.  Device memory may
# not be allocated while a stream is being captured into a CUDA graph, therefore each device keeps a
# small pool allocated ahead of time (by ``ensure_workspace``: module construction, ``.to(device)``
# and the first eager call all run it) from which a stream that shows up during a capture is served.
_POOL_SIZE = 4
_POOL: dict[int, list] = {}                       # device index -> workspaces not yet bound to a stream
_WORKSPACE: dict[tuple, torch.Tensor] = {}       # (device index, stream handle) -> its workspace


def _device_index(dev: torch.device) -> int:
    return dev.index if dev.index is not None else torch.cuda.current_device()


def _new_workspace(idx: int) -> torch.Tensor:
    nbytes = _cabi.workspace_bytes(4, _cabi.MAX_M, 1, 256, 128, 64)   # shape independent
    return torch.zeros(nbytes, dtype=torch.uint8, device=torch.device("cuda", idx))


def ensure_workspace(device, stream=None) -> torch.Tensor:
    """The scratch buffer of ``stream`` (default: the current stream) on ``device``; zero-filled once.

    The first call for a device, which allocates that device's pool, must come before any CUDA-graph
    capture starts.  Calls outside a capture keep ``_POOL_SIZE`` spare buffers ready, so up to that many
    streams may issue their first GEMV inside one capture without any allocation.  Calls issued on one stream are ordered, so
    they share a workspace; calls on different streams get different ones and may overlap freely."""
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("qgemv workspace lives in CUDA memory")
    idx = _device_index(device)
    handle = (stream if stream is not None else torch.cuda.current_stream(idx)).cuda_stream
    ws = _WORKSPACE.get((idx, handle))
    if ws is not None:
        return ws
    capturing = torch.cuda.is_current_stream_capturing()
    pool = _POOL.get(idx)
    if pool is None:
        if capturing:
            raise RuntimeError("the qgemv scratch buffers must be created before CUDA-graph capture starts: "
                               "call ai_accel_studio_b200.ops.ensure_workspace(device) first")
        pool = _POOL[idx] = [_new_workspace(idx) for _ in range(_POOL_SIZE)]
    if not pool:
        if capturing:
            raise RuntimeError(f"more than {_POOL_SIZE} streams of one device issued packed GEMVs and the next one appeared "
                               "during a CUDA-graph capture: call ensure_workspace(device, stream) for it before capturing")
        pool.append(_new_workspace(idx))
    ws = _WORKSPACE[(idx, handle)] = pool.pop()
    if not capturing:
        while len(pool) < _POOL_SIZE:          # keep spares for streams that first appear inside a capture
            pool.append(_new_workspace(idx))
    return ws


def workspace_status(device, stream=None) -> int:
    """Read and clear the sticky status word of a stream's workspace (synchronises that stream).
    0: every GEMV since the last query completed normally; 1: a bounded wait inside a kernel ran out
    (its result is not to be trusted; the workspace and the context stay usable)."""
    import ctypes
    device = torch.device(device)
    idx = _device_index(device)
    st = stream if stream is not None else torch.cuda.current_stream(idx)
    ws = ensure_workspace(device, st)
    out = ctypes.c_int32(-1)
    with torch.cuda.device(idx):
        _cabi.check(_cabi.lib().qgemv_workspace_status(ws.data_ptr(), st.cuda_stream, ctypes.byref(out)))
        st.synchronize()
    return int(out.value)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor: this build has no CPU path")


ACT_SILU_MUL = 3      # qgemv_act: rows are (8 gate, 8 up) blocks, the output is silu(gate) * up of width N / 2


def _out_width(packed: torch.Tensor, act: int) -> int:
    n = int(packed.shape[0])
    if act == ACT_SILU_MUL:
        if n % 16:
            raise ValueError("the gated-pair activation needs an even number of 8-row blocks (N % 16 == 0)")
        return n // 2
    return n


def _problem(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, y, ws,
             bits, group, k_original, act, kernel, prefetch=None) -> _cabi.Problem:
    m, kpad = x.shape
    p = _cabi.Problem()
    p.bits, p.m, p.n, p.k_padded, p.k_original, p.group = bits, m, packed.shape[0], kpad, k_original, group
    p.act, p.x_dtype = act, _DT[x.dtype]
    p.kernel, p.debug = kernel & 0xff, kernel >> 8       # bits 8+ carry qgemv_problem.debug (tests, benchmarks)
    p.x, p.ldx = x.data_ptr(), x.stride(0)
    p.packed, p.ldp = packed.data_ptr(), packed.stride(0)
    p.scales, p.lds = scales.data_ptr(), scales.stride(0)
    p.bias = bias.data_ptr() if bias is not None else None
    oc = 0 if outlier_idx is None else int(outlier_idx.numel())
    p.outliers = oc
    if oc:
        p.outlier_idx, p.outlier_w, p.ldow = outlier_idx.data_ptr(), outlier_weight.data_ptr(), outlier_weight.stride(0)
    rank = 0 if res_u is None else int(res_u.shape[1])
    p.rank = rank
    if rank:
        p.res_u, p.ldu, p.res_v, p.ldv = res_u.data_ptr(), res_u.stride(0), res_v.data_ptr(), res_v.stride(0)
    p.y, p.ldy = y.data_ptr(), y.stride(0)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    if prefetch is not None and prefetch.is_cuda and prefetch.device == x.device:
        p.prefetch, p.prefetch_bytes = prefetch.data_ptr(), prefetch.numel() * prefetch.element_size()
    return p


def _check_gemv_inputs(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits):
    _require_cuda(x, "x")
    if x.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("the packed decode path requires fp16/bf16 activations")
    if x.ndim != 2 or x.shape[0] > _cabi.MAX_M or x.shape[0] < 1:
        raise ValueError("decode-specialized path is for [M,K] with 1 <= M <= 4")
    if x.stride(1) != 1:
        raise ValueError("x must have unit stride along K")
    if packed.dtype != torch.uint8 or scales.dtype != torch.float16:
        raise RuntimeError("packed must be uint8 and scales float16")
    if packed.shape[1] * (8 // bits) != x.shape[1]:
        raise ValueError("input must already be padded to packed K")
    for name, t, dt in (("bias", bias, torch.float16), ("outlier_weight", outlier_weight, torch.float16),
                        ("res_u", res_u, torch.float16), ("res_v", res_v, torch.float16),
                        ("outlier_idx", outlier_idx, torch.int32)):
        if t is not None:
            _require_cuda(t, name)
            if t.dtype != dt:
                raise RuntimeError(f"{name} must be {dt}")
            if t.ndim >= 1 and t.numel() and t.stride(-1) != 1:
                raise ValueError(f"{name} must have unit inner stride")


def gemv_eager(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
               outlier_idx: Optional[torch.Tensor], outlier_weight: Optional[torch.Tensor],
               res_u: Optional[torch.Tensor], res_v: Optional[torch.Tensor],
               bits: int, group: int, k_original: int, act: int, kernel: int,
               prefetch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[M,N] = act(x . dequant(W)^T + outlier term + low-rank residual + bias), M <= 4
    (``act`` 0 none, 1 ReLU, 2 SiLU; 3 = gated pairs, see ``ACT_SILU_MUL``: y is then [M, N/2]).

    ``prefetch``: an optional (contiguous, static) tensor -- normally the packed codes of the GEMV that
    follows -- which the kernel announces to L2 while it runs.

    Issued on the current stream with that stream's own scratch buffer (see ``ensure_workspace``), so
    GEMVs on different streams may overlap.  ``kernel``: ``_cabi.KERNEL[...]``, optionally OR-ed with
    ``debug_bits << 8``."""
    _check_gemv_inputs(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits)
    if outlier_idx is not None and outlier_idx.numel() == 0:
        outlier_idx = outlier_weight = None
    if res_u is not None and res_u.numel() == 0:
        res_u = res_v = None
    ws = ensure_workspace(x.device)
    y = torch.empty((x.shape[0], _out_width(packed, act)), dtype=x.dtype, device=x.device)
    prob = _problem(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, y, ws,
                    bits, group, k_original, act, kernel, prefetch)
    with torch.cuda.device(x.device):
        _cabi.run(prob, torch.cuda.current_stream().cuda_stream)
    return y


# The registered operator (traceable by Dynamo through its fake kernel) is the same function behind the
# dispatcher.  Eager callers that do not need tracing call ``gemv_eager`` and save the dispatcher's
# tens of microseconds per call, which is several times the kernel's own duration.
gemv = torch.library.custom_op("b200q::gemv", gemv_eager, mutates_args=())


class CachedCall:
    """A module's decode launch with everything that does not change between calls prepared once: the
    problem struct with the weight pointers filled in, keyed by the shapes and addresses it was built
    from.  ``run(x)`` then costs an output allocation, three pointer stores and the launch."""

    __slots__ = ("key", "problem", "out_width", "device_index", "keep")

    def __init__(self, key, problem, out_width, device_index):
        self.key, self.problem, self.out_width, self.device_index = key, problem, out_width, device_index
        self.keep = None                      # tensors the struct points at, when the caller does not hold them itself

    def run(self, x: torch.Tensor) -> torch.Tensor:
        import ctypes
        idx = self.device_index
        y = torch.empty((x.shape[0], self.out_width), dtype=x.dtype, device=x.device)
        stream = torch.cuda.current_stream(idx)
        handle = stream.cuda_stream
        ws = _WORKSPACE.get((idx, handle))
        if ws is None:
            ws = ensure_workspace(x.device, stream)
        p = self.problem
        p.x, p.y, p.workspace = x.data_ptr(), y.data_ptr(), ws.data_ptr()
        if torch.cuda.current_device() == idx:
            rc = _cabi.lib().qgemv_run(ctypes.byref(p), handle)
        else:
            with torch.cuda.device(idx):
                rc = _cabi.lib().qgemv_run(ctypes.byref(p), handle)
        if rc != 0:
            _cabi.check(rc)
        return y


def prepare_call(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits, group, k_original, act, kernel,
                 prefetch=None, key=None) -> CachedCall:
    """Validate once and build a ``CachedCall`` for activations shaped and strided like ``x``."""
    _check_gemv_inputs(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits)
    if outlier_idx is not None and outlier_idx.numel() == 0:
        outlier_idx = outlier_weight = None
    if res_u is not None and res_u.numel() == 0:
        res_u = res_v = None
    ws = ensure_workspace(x.device)
    width = _out_width(packed, act)
    y = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    prob = _problem(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, y, ws, bits, group, k_original, act,
                    kernel, prefetch)
    return CachedCall(key, prob, width, _device_index(x.device))


@gemv.register_fake
def _(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits, group, k_original, act, kernel, prefetch=None):
    return x.new_empty((x.shape[0], _out_width(packed, act)))


def gemv_into(x: torch.Tensor, packed: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor],
              outlier_idx: Optional[torch.Tensor], outlier_weight: Optional[torch.Tensor],
              res_u: Optional[torch.Tensor], res_v: Optional[torch.Tensor],
              bits: int, group: int, k_original: int, act: int, kernel: int, out: torch.Tensor,
              prefetch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Same computation as ``gemv`` written into ``out`` ([M, N], x.dtype, unit inner stride).

    ``out`` is a CUDA tensor on x's device or a *pinned* host tensor: pinned memory is addressable by
    the device, so the kernel's stores then go straight to host memory and no separate device-to-host
    copy is needed (worth it for results this small; the host must still wait for the stream before it
    reads them).  A plain function, not a registered op: it mutates its argument and is meant for
    serving loops, eager or captured in a CUDA graph."""
    _check_gemv_inputs(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, bits)
    if out.dtype != x.dtype or out.ndim != 2 or tuple(out.shape) != (x.shape[0], _out_width(packed, act)) or out.stride(1) != 1:
        raise ValueError("out must be [M, N] ([M, N/2] for the gated-pair activation) of x.dtype with unit inner stride")
    if out.is_cuda:
        if out.device != x.device:
            raise RuntimeError("out must be on x's device")
    elif not out.is_pinned():
        raise RuntimeError("a host result buffer must be pinned (page-locked) memory")
    if outlier_idx is not None and outlier_idx.numel() == 0:
        outlier_idx = outlier_weight = None
    if res_u is not None and res_u.numel() == 0:
        res_u = res_v = None
    ws = ensure_workspace(x.device)
    prob = _problem(x, packed, scales, bias, outlier_idx, outlier_weight, res_u, res_v, out, ws,
                    bits, group, k_original, act, kernel, prefetch)
    with torch.cuda.device(x.device):
        _cabi.run(prob, torch.cuda.current_stream().cuda_stream)
    return out


@torch.library.custom_op("b200q::dequant", mutates_args=())
def dequant(packed: torch.Tensor, scales: torch.Tensor, bits: int, group: int, k_original: int,
            dtype_name: str) -> torch.Tensor:
    """Dense [N, k_original] matrix, bit-identical to the torch expression of the reference."""
    _require_cuda(packed, "packed")
    _require_cuda(scales, "scales")
    dtype = _DT_NAME[dtype_name]
    if packed.dtype != torch.uint8 or scales.dtype != torch.float16 or packed.stride(1) != 1 or scales.stride(1) != 1:
        raise RuntimeError("packed must be uint8, scales float16, both with unit inner stride")
    n, kpad = packed.shape[0], packed.shape[1] * (8 // bits)
    out = torch.empty((n, k_original), dtype=dtype, device=packed.device)
    with torch.cuda.device(packed.device):
        _cabi.check(_cabi.lib().qdequant(bits, packed.data_ptr(), packed.stride(0), scales.data_ptr(), scales.stride(0),
                                         n, kpad, k_original, group, out.data_ptr(), out.stride(0), _DT[dtype],
                                         torch.cuda.current_stream().cuda_stream))
    return out


@dequant.register_fake
def _(packed, scales, bits, group, k_original, dtype_name):
    return packed.new_empty((packed.shape[0], k_original), dtype=_DT_NAME[dtype_name])


@torch.library.custom_op("b200q::unpack_codes", mutates_args=())
def unpack_codes(packed: torch.Tensor, bits: int) -> torch.Tensor:
    """One uint8 code per weight, [N, Kpad]."""
    _require_cuda(packed, "packed")
    if packed.dtype != torch.uint8 or packed.stride(1) != 1:
        raise RuntimeError("packed must be uint8 with unit inner stride")
    n, kpad = packed.shape[0], packed.shape[1] * (8 // bits)
    out = torch.empty((n, kpad), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        _cabi.check(_cabi.lib().qunpack_codes(bits, packed.data_ptr(), packed.stride(0), n, kpad,
                                              out.data_ptr(), out.stride(0), torch.cuda.current_stream().cuda_stream))
    return out


@unpack_codes.register_fake
def _(packed, bits):
    return packed.new_empty((packed.shape[0], packed.shape[1] * (8 // bits)))


def plan_name(x, packed, scales, bits, group, k_original, outliers=0, rank=0, kernel="auto"):
    """Name of the kernel variant a call of this shape would launch (no launch happens)."""
    ws = ensure_workspace(x.device)
    y = torch.empty((x.shape[0], packed.shape[0]), dtype=x.dtype, device=x.device)
    p = _problem(x, packed, scales, None, None, None, None, None, y, ws, bits, group, k_original, 0,
                 _cabi.KERNEL[kernel])
    return _cabi.plan_name(p)


def plan_launches(x, packed, scales, bits, group, k_original, outlier_idx=None, outlier_weight=None,
                  res_u=None, res_v=None, kernel="auto") -> int:
    """Number of kernel launches one call with these operands issues (no launch happens)."""
    ws = ensure_workspace(x.device)
    y = torch.empty((x.shape[0], packed.shape[0]), dtype=x.dtype, device=x.device)
    p = _problem(x, packed, scales, None, outlier_idx, outlier_weight, res_u, res_v, y, ws, bits, group,
                 k_original, 0, _cabi.KERNEL[kernel])
    return _cabi.plan_launches(p)


def plan_describe(x, packed, scales, bits, group, k_original, outlier_idx=None, outlier_weight=None,
                  res_u=None, res_v=None, kernel=0) -> dict:
    """What one call with these operands would launch (``qgemv_plan_describe``), as a dict; ``kernel`` is
    the integer selector ``gemv`` takes."""
    ws = ensure_workspace(x.device)
    y = torch.empty((x.shape[0], packed.shape[0]), dtype=x.dtype, device=x.device)
    p = _problem(x, packed, scales, None, outlier_idx, outlier_weight, res_u, res_v, y, ws, bits, group,
                 k_original, 0, kernel)
    info = _cabi.plan_describe(p)
    d = {name: int(getattr(info, name)) for name, _ in _cabi.PlanInfo._fields_}
    d["name"] = _cabi.plan_name(p)
    return d
