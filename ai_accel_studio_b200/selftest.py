"""Hot-path probes of the reference's self test on this package's kernels.

Mirrors the three probes of ``ai_accel_lab/selftest.py`` that touch the packed decode path
(``decode-int2-v4`` :99-111, ``decode-int4-v5`` :113-119, the CUDA-graph probe :121-134) with the
reference's inputs (x [1, 256] fp16, W [128, 256] / 16, group 64), comparison (against
``x @ unpack(fp16)^T``) and acceptance thresholds (max-abs error below 0.5 / 0.35, cosine above 0.999).
The rest of the reference's self test (Triton, Gluon, TorchAO, extension builds) probes components
this package does not have.

    python -m ai_accel_studio_b200.selftest
"""
from __future__ import annotations

import json

import torch
import torch.nn.functional as F

from .kernels.decode_int2 import decode_int2_linear
from .kernels.groupwise_int2 import pack_groupwise_int2, unpack_groupwise_int2
from .kernels.groupwise_int4 import decode_int4_linear, pack_groupwise_int4, unpack_groupwise_int4


def _probe(name, fn):
    try:
        out = fn()
        return dict(name=name, **out)
    except Exception as e:                      # the reference's report format: a failed probe carries its error
        return dict(name=name, ok=False, error=repr(e))


def _decode_probe(pack, unpack, decode, limit):
    x = torch.randn(1, 256, device="cuda", dtype=torch.float16)
    w = torch.randn(128, 256, device="cuda", dtype=torch.float16) / 16
    pw = pack(w, group_size=64)
    y = decode(x, pw)
    ref = x @ unpack(pw, dtype=torch.float16).t()
    torch.cuda.synchronize()
    max_err = float((y.float() - ref.float()).abs().max().item())
    cos = float(F.cosine_similarity(y.float(), ref.float(), dim=-1).mean().item())
    return dict(ok=max_err < limit and cos > 0.999, max_abs_error=max_err, cosine=cos)


def _graph_probe():
    """The packed GEMV captured in a CUDA graph and replayed (the reference captures a dense matmul)."""
    x = torch.randn(1, 256, device="cuda", dtype=torch.float16)
    pw = pack_groupwise_int2(torch.randn(128, 256, device="cuda", dtype=torch.float16) / 16, group_size=64)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            y = decode_int2_linear(x, pw)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = decode_int2_linear(x, pw)
    want = decode_int2_linear(x, pw)
    g.replay()
    torch.cuda.synchronize()
    return dict(ok=bool(torch.equal(y, want)))


def run_selftest() -> dict:
    report = dict(cuda=torch.cuda.is_available(), probes=[])
    if not report["cuda"]:
        report["probes"].append(dict(name="cuda", ok=False, error="no CUDA device: the packed decode path has no CPU implementation"))
        report["ok"] = False
        return report
    report["device"] = torch.cuda.get_device_name()
    report["probes"].append(_probe("decode-int2-v4", lambda: _decode_probe(pack_groupwise_int2, unpack_groupwise_int2, decode_int2_linear, 0.5)))
    report["probes"].append(_probe("decode-int4-v5", lambda: _decode_probe(pack_groupwise_int4, unpack_groupwise_int4, decode_int4_linear, 0.35)))
    report["probes"].append(_probe("cuda-graph", _graph_probe))
    report["ok"] = all(p["ok"] for p in report["probes"])
    return report


if __name__ == "__main__":
    print(json.dumps(run_selftest(), indent=1))
