import ctypes
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"

# Output tolerance of the fused GEMV against the fp32-accumulate oracle (the bar the path is
# held to): |y - ref| <= ABS_TOL + REL_TOL * |ref| for every element, and
# ||y - ref||_2 <= REL_TOL * ||ref||_2 over the whole output.
ABS_TOL = 1e-2
REL_TOL = 1e-3


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def small_cases():
    z = np.load(GOLDEN / "small_cases.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    return z, meta


@pytest.fixture(scope="session")
def full_size():
    z = np.load(GOLDEN / "full_size.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    return z, meta


@pytest.fixture(scope="session")
def coracle():
    """The C restatement (oracle/qgemv_ref.c), built on demand with the committed Makefile."""
    lib = ROOT / "oracle" / "libqgemv_oracle.so"
    src = ROOT / "oracle" / "qgemv_ref.c"
    if not lib.exists() or lib.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle")], check=True, capture_output=True)
    l = ctypes.CDLL(str(lib))
    vp, i64, ci = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    l.qref_forward.argtypes = [vp, i64, ci, ci, vp, vp, i64, i64, i64, ci, ci, vp, vp, vp, ci, vp, vp, ci, ci, vp, vp]
    l.qref_forward.restype = None
    l.qref_dequant_f32.argtypes = [vp, vp, i64, i64, i64, ci, ci, vp]
    l.qref_unpack_codes.argtypes = [vp, i64, i64, ci, vp]
    l.qref_num_threads.restype = ci
    return l


def c_forward(lib, x16, bits, packed, scales, k, group, bias=None, oidx=None, ow=None, ru=None, rv=None,
              act=0, x_is_bf16=False):
    """Call qref_forward on numpy arrays; returns float32 [M, N]."""
    x16 = np.ascontiguousarray(x16)
    m, kpad = x16.shape
    n = packed.shape[0]

    def ptr(a):
        return None if a is None else np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p)
    keep = [np.ascontiguousarray(a) if a is not None else None for a in (packed, scales, bias, oidx, ow, ru, rv)]
    wbuf = np.empty((n, k), dtype=np.float32)
    y = np.empty((m, n), dtype=np.float32)
    oc = 0 if oidx is None else int(np.size(oidx))
    rank = 0 if ru is None else int(ru.shape[1])
    lib.qref_forward(x16.view(np.uint16).ctypes.data_as(ctypes.c_void_p), kpad, int(x_is_bf16), m,
                     ptr(keep[0]), ptr(keep[1]), n, kpad, k, group, bits, ptr(keep[2]),
                     ptr(keep[3]), ptr(keep[4]), oc, ptr(keep[5]), ptr(keep[6]), rank, act,
                     wbuf.ctypes.data_as(ctypes.c_void_p), y.ctypes.data_as(ctypes.c_void_p))
    return y


def assert_within_tolerance(y, ref, what=""):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert y.shape == ref.shape, (y.shape, ref.shape)
    diff = np.abs(y - ref)
    bound = ABS_TOL + REL_TOL * np.abs(ref)
    worst = float((diff - bound).max())
    assert worst <= 0, f"{what}: element error exceeds {ABS_TOL} + {REL_TOL}*|ref| by {worst:.3e} (max abs diff {diff.max():.3e})"
    nrm = float(np.linalg.norm(ref))
    if nrm > 0:
        rel = float(np.linalg.norm(y - ref)) / nrm
        assert rel <= REL_TOL, f"{what}: relative L2 error {rel:.3e} > {REL_TOL}"
