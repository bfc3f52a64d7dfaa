"""One-shot all-reduce of small fp16 / bf16 tensors over NVLink peer memory (``include/qcomm_b200.h``).

Used by tensor-parallel decode for the ``[M, hidden]`` partial results of the K-split projections:
one kernel per rank writes the rank's vector into every rank's receive buffer, raises flags, waits
(bounded) for the other ranks' flags and sums the slots in rank order.  The buffers are allocated
once per group with ``cudaMalloc`` inside the library and shared between the processes of the node
through CUDA inter-process handles that travel over ``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _cabi

_DT = {torch.float16: _cabi.F16, torch.bfloat16: _cabi.BF16}


class OneShotAllReduce:
    """``comm(t)`` sums ``t`` over the ranks of ``group`` in place (fp16 / bf16, contiguous, 16-byte
    aligned, a multiple of 8 and at most ``max_elems`` elements); every rank must make the same calls.
    ``peers`` may be given instead of a process group: a list of ``(slots_ptr, flags_ptr)`` device
    addresses per rank, for hosts that map the buffers themselves (and for single-process tests)."""

    def __init__(self, group=None, max_elems: int = 4 * 8192, device=None, wait_limit: int = 0, rank=None, world=None,
                 peers=None):
        lib = _cabi.lib()
        self.lib = lib
        self.group = group
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        if peers is None:
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = int(rank), int(world)
        if not 1 <= self.world <= _cabi.COMM_MAX_RANKS:
            raise ValueError(f"one-shot all-reduce handles 1..{_cabi.COMM_MAX_RANKS} ranks, not {self.world}")
        if max_elems % 8 or max_elems > _cabi.COMM_MAX_BLOCKS * 4096:
            raise ValueError("max_elems must be a multiple of 8 and at most 262144")
        self.max_elems = int(max_elems)
        self._owned, self._opened = [], []
        g = _cabi.CommGroup()
        g.rank, g.world, g.max_elems, g.wait_limit = self.rank, self.world, self.max_elems, int(wait_limit)
        with torch.cuda.device(self.device):
            g.state = self._alloc(lib.qcomm_state_bytes())
            if peers is not None:
                for r, (sp, fp) in enumerate(peers):
                    g.slots[r], g.flags[r] = sp, fp
            else:
                slots = self._alloc(lib.qcomm_slot_bytes(self.world, self.max_elems))
                flags = self._alloc(lib.qcomm_flag_bytes(self.world))
                mine = (self._export(slots), self._export(flags))
                every = [None] * self.world
                dist.all_gather_object(every, mine, group=group)
                for r, (hs, hf) in enumerate(every):
                    if r == self.rank:
                        g.slots[r], g.flags[r] = slots, flags
                    else:
                        g.slots[r], g.flags[r] = self._open(hs), self._open(hf)
                dist.barrier(group=group)            # every rank has mapped every buffer before anybody writes
        self.g = g

    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        _cabi.check(self.lib.qcomm_alloc(int(nbytes), C.byref(p)))
        self._owned.append(p.value)
        return p.value

    def _export(self, ptr: int) -> bytes:
        buf = C.create_string_buffer(_cabi.COMM_IPC_HANDLE_BYTES)
        _cabi.check(self.lib.qcomm_ipc_export(C.c_void_p(ptr), buf))
        return buf.raw

    def _open(self, handle: bytes) -> int:
        p = C.c_void_p()
        _cabi.check(self.lib.qcomm_ipc_open(C.create_string_buffer(handle, len(handle)), C.byref(p)))
        self._opened.append(p.value)
        return p.value

    def fits(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype in _DT and t.is_contiguous() and t.numel() % 8 == 0 and 0 < t.numel() <= self.max_elems
                and t.data_ptr() % 16 == 0)

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        if not self.fits(t):
            raise ValueError("tensor does not fit the one-shot all-reduce (fp16/bf16, contiguous, 16-byte aligned, "
                             f"a multiple of 8 and at most {self.max_elems} elements)")
        with torch.cuda.device(t.device):
            _cabi.check(self.lib.qcomm_allreduce(C.byref(self.g), C.c_void_p(t.data_ptr()), t.numel(), _DT[t.dtype],
                                                 C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return t

    def fits_rows(self, partial: torch.Tensor) -> bool:
        return (partial.is_cuda and partial.dtype in _DT and partial.ndim == 2 and partial.stride(1) == 1
                and partial.shape[1] % 8 == 0 and partial.shape[1] <= 16384 and partial.shape[0] <= _cabi.COMM_MAX_BLOCKS
                and partial.numel() <= self.max_elems and partial.data_ptr() % 16 == 0 and partial.stride(0) % 8 == 0)

    def allreduce_rmsnorm(self, partial: torch.Tensor, h: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        """One kernel for "all-reduce the K-split projection's partial result, add it to the residual stream,
        RMS-normalise": ``h += sum over ranks of partial`` in place, returns ``rmsnorm(h) * weight``.  ``partial`` and
        ``h``: ``[rows, hidden]``; counts as one call of the group's sequence, so every rank must make it."""
        if not self.fits_rows(partial):
            raise ValueError("partial does not fit the fused all-reduce (fp16/bf16 [rows, hidden], unit inner stride, 16-byte "
                             f"aligned rows, hidden a multiple of 8, at most {self.max_elems} elements)")
        if h.shape != partial.shape or h.dtype != partial.dtype or h.stride(1) != 1 or weight.dtype != h.dtype or \
                weight.numel() != h.shape[1] or not weight.is_contiguous():
            raise ValueError("h must match partial and weight must be a contiguous [hidden] tensor of the same dtype")
        y = torch.empty(h.shape, dtype=h.dtype, device=h.device)
        with torch.cuda.device(h.device):
            _cabi.check(self.lib.qcomm_allreduce_rmsnorm(C.byref(self.g), C.c_void_p(partial.data_ptr()), partial.stride(0),
                                                         C.c_void_p(h.data_ptr()), h.stride(0), C.c_void_p(weight.data_ptr()),
                                                         C.c_void_p(y.data_ptr()), y.stride(0), h.shape[0], h.shape[1], float(eps),
                                                         _DT[h.dtype], C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return y

    def status(self) -> int:
        """Read and clear the status word (synchronises the current stream): 0, or 1 if a wait for a peer ran out."""
        out = C.c_int32(-1)
        with torch.cuda.device(self.device):
            st = torch.cuda.current_stream()
            _cabi.check(self.lib.qcomm_status(C.byref(self.g), C.c_void_p(st.cuda_stream), C.byref(out)))
            st.synchronize()
        return int(out.value)

    def close(self):
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened:
                self.lib.qcomm_ipc_close(C.c_void_p(p))
            for p in self._owned:
                self.lib.qcomm_free(C.c_void_p(p))
        self._opened, self._owned = [], []
