"""ctypes binding of the C ABI declared in ``include/qgemv_b200.h``.

Nothing here touches torch: callers pass raw device addresses, sizes and a stream handle.
A missing or unloadable library is a hard error -- there is no fallback implementation.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libqgemv_b200.so"

OK = 0
ACT = {"none": 0, "relu": 1, "silu": 2, "swish": 2}
F16, BF16, F32 = 0, 1, 2
KERNEL = {"auto": 0, "simt": 1, "mma": 2, "mma_pipe": 3}
DEBUG_DROP_PROJECTIONS, DEBUG_NO_L2_HINT = 1, 2
MAX_M = 4
ABI_VERSION = 4

EXPORTS = ("qgemv_run", "qgemv_run_static", "qgemv_plan_launches", "qgemv_plan_describe", "qgemv_workspace_status", "qgemv_workspace_bytes", "qgemv_plan_name", "qdequant", "qunpack_codes",
           "qgemv_error_string", "qgemv_abi_version", "qgemv_sizeof_problem",
           "qcomm_slot_bytes", "qcomm_flag_bytes", "qcomm_state_bytes", "qcomm_allreduce", "qcomm_allreduce_rmsnorm", "qcomm_status", "qcomm_alloc", "qcomm_free",
           "qcomm_ipc_export", "qcomm_ipc_open", "qcomm_ipc_close",
           "qdec_rmsnorm", "qdec_rope_append", "qdec_attention_workspace_bytes", "qdec_attention", "qdec_silu_mul")
COMM_MAX_RANKS, COMM_MAX_BLOCKS, COMM_IPC_HANDLE_BYTES = 8, 64, 64


class Problem(C.Structure):
    """``struct qgemv_problem`` (field order and types must match the header)."""
    _fields_ = [
        ("bits", C.c_int32), ("m", C.c_int32), ("n", C.c_int32), ("k_padded", C.c_int32),
        ("k_original", C.c_int32), ("group", C.c_int32), ("act", C.c_int32), ("x_dtype", C.c_int32),
        ("outliers", C.c_int32), ("rank", C.c_int32), ("kernel", C.c_int32), ("debug", C.c_int32),
        ("x", C.c_void_p), ("ldx", C.c_int64),
        ("packed", C.c_void_p), ("ldp", C.c_int64),
        ("scales", C.c_void_p), ("lds", C.c_int64),
        ("bias", C.c_void_p),
        ("outlier_idx", C.c_void_p),
        ("outlier_w", C.c_void_p), ("ldow", C.c_int64),
        ("res_u", C.c_void_p), ("ldu", C.c_int64),
        ("res_v", C.c_void_p), ("ldv", C.c_int64),
        ("y", C.c_void_p), ("ldy", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("prefetch", C.c_void_p), ("prefetch_bytes", C.c_size_t),
    ]


class PlanInfo(C.Structure):
    """``struct qgemv_plan_info``."""
    _fields_ = [("family", C.c_int32), ("variant", C.c_int32), ("launches", C.c_int32), ("grid", C.c_int32),
                ("warps", C.c_int32), ("smem_bytes", C.c_int32), ("tile_aligned", C.c_int32),
                ("inline_projections", C.c_int32), ("ctas_per_sm", C.c_int32), ("stages", C.c_int32),
                ("run_chunks", C.c_int32), ("runs_per_tile", C.c_int32), ("epilogue_tiles", C.c_int32),
                ("l2_chunks", C.c_int32), ("projection_parts", C.c_int32), ("chunk_bytes", C.c_int32)]


class CommGroup(C.Structure):
    """``struct qcomm_group`` (include/qcomm_b200.h)."""
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("max_elems", C.c_int32), ("wait_limit", C.c_int32),
                ("slots", C.c_void_p * COMM_MAX_RANKS), ("flags", C.c_void_p * COMM_MAX_RANKS), ("state", C.c_void_p)]


class QgemvError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"qgemv error {code}: {message}")
        self.code = code


_lib = None


def lib():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m ai_accel_studio_b200.build` "
            "(needs nvcc with sm_100a support). There is no fallback implementation.")
    l = C.CDLL(str(LIB_PATH))
    l.qgemv_run.argtypes = [C.POINTER(Problem), C.c_void_p]
    l.qgemv_run.restype = C.c_int
    l.qgemv_run_static.argtypes = [C.POINTER(Problem), C.c_void_p]
    l.qgemv_run_static.restype = C.c_int
    l.qgemv_workspace_bytes.argtypes = [C.c_int] * 6
    l.qgemv_workspace_bytes.restype = C.c_size_t
    l.qgemv_plan_name.argtypes = [C.POINTER(Problem)]
    l.qgemv_plan_name.restype = C.c_char_p
    l.qgemv_plan_launches.argtypes = [C.POINTER(Problem)]
    l.qgemv_plan_launches.restype = C.c_int
    l.qgemv_plan_describe.argtypes = [C.POINTER(Problem), C.POINTER(PlanInfo)]
    l.qgemv_plan_describe.restype = C.c_int
    l.qgemv_workspace_status.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32)]
    l.qgemv_workspace_status.restype = C.c_int
    l.qcomm_slot_bytes.argtypes = [C.c_int, C.c_int]
    l.qcomm_slot_bytes.restype = C.c_size_t
    l.qcomm_flag_bytes.argtypes = [C.c_int]
    l.qcomm_flag_bytes.restype = C.c_size_t
    l.qcomm_state_bytes.argtypes = []
    l.qcomm_state_bytes.restype = C.c_size_t
    l.qcomm_allreduce.argtypes = [C.POINTER(CommGroup), C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    l.qcomm_allreduce.restype = C.c_int
    l.qcomm_allreduce_rmsnorm.argtypes = [C.POINTER(CommGroup), C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p,
                                          C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_float, C.c_int, C.c_void_p]
    l.qcomm_allreduce_rmsnorm.restype = C.c_int
    l.qcomm_status.argtypes = [C.POINTER(CommGroup), C.c_void_p, C.POINTER(C.c_int32)]
    l.qcomm_status.restype = C.c_int
    l.qcomm_alloc.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    l.qcomm_alloc.restype = C.c_int
    l.qcomm_free.argtypes = [C.c_void_p]
    l.qcomm_free.restype = C.c_int
    l.qcomm_ipc_export.argtypes = [C.c_void_p, C.c_void_p]
    l.qcomm_ipc_export.restype = C.c_int
    l.qcomm_ipc_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    l.qcomm_ipc_open.restype = C.c_int
    l.qcomm_ipc_close.argtypes = [C.c_void_p]
    l.qcomm_ipc_close.restype = C.c_int
    i64, vp, ci = C.c_int64, C.c_void_p, C.c_int
    l.qdec_rmsnorm.argtypes = [vp, i64, vp, i64, vp, vp, i64, ci, ci, C.c_float, ci, vp]
    l.qdec_rmsnorm.restype = ci
    l.qdec_rope_append.argtypes = [vp, i64, vp, i64, vp, i64, vp, vp, ci, vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, vp]
    l.qdec_rope_append.restype = ci
    l.qdec_attention_workspace_bytes.argtypes = [ci] * 5
    l.qdec_attention_workspace_bytes.restype = C.c_size_t
    l.qdec_attention.argtypes = [vp, i64, vp, vp, vp, vp, i64, ci, ci, ci, ci, ci, C.c_float, vp, C.c_size_t, ci, vp]
    l.qdec_attention.restype = ci
    l.qdec_silu_mul.argtypes = [vp, i64, vp, i64, vp, i64, ci, ci, ci, vp]
    l.qdec_silu_mul.restype = ci
    l.qdequant.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_int,
                           C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    l.qdequant.restype = C.c_int
    l.qunpack_codes.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
    l.qunpack_codes.restype = C.c_int
    l.qgemv_error_string.argtypes = []
    l.qgemv_error_string.restype = C.c_char_p
    l.qgemv_abi_version.argtypes = []
    l.qgemv_abi_version.restype = C.c_int
    l.qgemv_sizeof_problem.argtypes = []
    l.qgemv_sizeof_problem.restype = C.c_size_t
    if l.qgemv_sizeof_problem() != C.sizeof(Problem):
        raise RuntimeError("struct qgemv_problem layout mismatch between the binding and the library; rebuild it")
    if l.qgemv_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{LIB_PATH} has ABI version {l.qgemv_abi_version()}, expected {ABI_VERSION}; rebuild it")
    _lib = l
    return l


def last_error() -> str:
    return lib().qgemv_error_string().decode()


def check(code: int) -> None:
    if code != OK:
        raise QgemvError(code, last_error())


def workspace_bytes(bits: int, m: int, n: int, k_padded: int, group: int, rank: int) -> int:
    return int(lib().qgemv_workspace_bytes(bits, m, n, k_padded, group, rank))


def run(problem: Problem, stream: int) -> None:
    check(lib().qgemv_run(C.byref(problem), C.c_void_p(stream)))


def plan_launches(problem: Problem) -> int:
    r = int(lib().qgemv_plan_launches(C.byref(problem)))
    if r < 0:
        raise QgemvError(r, last_error())
    return r


def plan_describe(problem: Problem) -> PlanInfo:
    info = PlanInfo()
    check(lib().qgemv_plan_describe(C.byref(problem), C.byref(info)))
    return info


def run_static(problem: Problem, stream: int) -> None:
    """``qgemv_run_static``: the library's built-in scratch instead of a caller workspace."""
    check(lib().qgemv_run_static(C.byref(problem), C.c_void_p(stream)))


def plan_name(problem: Problem):
    r = lib().qgemv_plan_name(C.byref(problem))
    return None if r is None else r.decode()
