"""Build ``libqgemv_b200.so`` in-tree with nvcc for sm_100a.

    python -m ai_accel_studio_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libqgemv_b200.so"
# (source, extra defines, object name).  The two tensor-core-assisted kernels are compiled once per bit
# width so that the objects build in parallel.
UNITS = [
    ("qgemv_api.cu", [], "qgemv_api.o"),
    ("qgemv_simt.cu", [], "qgemv_simt.o"),
    ("qdequant.cu", [], "qdequant.o"),
    ("qcomm.cu", [], "qcomm.o"),
    ("qdecode.cu", [], "qdecode.o"),
    ("qgemv_mma.cu", ["-DQGEMV_INST_BITS=2"], "qgemv_mma_int2.o"),
    ("qgemv_mma.cu", ["-DQGEMV_INST_BITS=4"], "qgemv_mma_int4.o"),
    ("qgemv_pipe.cu", ["-DQGEMV_INST_BITS=2"], "qgemv_pipe_int2.o"),
    ("qgemv_pipe.cu", ["-DQGEMV_INST_BITS=4"], "qgemv_pipe_int4.o"),
]
OBJDIR = CSRC / "build"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
# No --use_fast_math: the dequantisation kernels must round exactly like IEEE arithmetic.


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit (12.8 or newer for sm_100a)")


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list((PKG.parent / "include").glob("*.h"))
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags: tuple = (), lib: Path = LIB) -> Path:
    """Compile the library if it is missing or older than its sources; return its path.

    ``extra_flags`` (e.g. ``("-DQGEMV_TRACE",)``) and ``lib`` let a measurement build sit beside the
    product build; objects of such a build go to their own directory."""
    if not force and not extra_flags and lib == LIB and not _stale():
        return lib
    nvcc = _nvcc()
    objdir = OBJDIR if not extra_flags else OBJDIR.with_name("build_" + "".join(c for c in "".join(extra_flags) if c.isalnum()))
    objdir.mkdir(parents=True, exist_ok=True)
    procs = []
    for src, defs, obj in UNITS:
        cmd = [nvcc, *NVCC_FLAGS, *defs, *extra_flags, "-c", str(CSRC / src), "-o", str(objdir / obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
    failed = []
    for cmd, pr in procs:
        out, err = pr.communicate()
        if pr.returncode != 0:
            failed.append(f"{' '.join(cmd)}\n{out}\n{err}")
        elif verbose:
            print(err)
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(failed))
    link = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-o", str(lib),
            *[str(objdir / obj) for _, _, obj in UNITS]]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed ({res.returncode}):\n{res.stdout}\n{res.stderr}")
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], help="extra -D flag for a measurement build, e.g. QGEMV_TRACE")
    ap.add_argument("--output", default=None, help="library path of a measurement build (default: the product library)")
    a = ap.parse_args()
    print(build(a.force, a.verbose, tuple("-D" + d for d in a.define), Path(a.output) if a.output else LIB))
    sys.exit(0)
