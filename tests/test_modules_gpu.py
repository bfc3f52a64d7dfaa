"""The drop-in Linear wrappers on the GPU: fixtures made by the reference modules, the M > 4
path, state-dict round trips, CUDA-graph capture and torch.compile."""
import numpy as np
import pytest
import torch
from torch import nn

from oracle import qgemv_oracle as O
from conftest import assert_within_tolerance
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear

pytestmark = pytest.mark.gpu


def _build(c, z):
    nm = c["name"]
    lin = nn.Linear(c["k"], c["n"], bias=c["bias"])
    with torch.no_grad():
        lin.weight.copy_(torch.from_numpy(z[nm + ".w"]))
        if c["bias"]:
            lin.bias.copy_(torch.from_numpy(z[nm + ".srcbias"]))
    arms = torch.from_numpy(z[nm + ".arms"]) if c["aware"] else None
    if c["bits"] == 2:
        return HybridInt2Linear(lin, c["group"], arms, c["requested"], c["rank"])
    return HybridInt4Linear(lin, c["group"], arms, c["requested"])


def test_modules_reproduce_reference_outputs(small_cases):
    z, meta = small_cases
    for c in meta["hybrid_cases"]:
        nm = c["name"]
        mod = _build(c, z).to("cuda")
        host = O.PackedWeight(c["bits"], z[nm + ".packed"], z[nm + ".scales"], c["k"], c["padded_k"], c["group"])
        kw = dict(bias=z[nm + ".bias"] if c["bias"] else None, outlier_idx=z[nm + ".outlier_idx"],
                  outlier_weight=z[nm + ".outlier_weight"],
                  res_u=z[nm + ".res_u"] if c["rank"] else None, res_v=z[nm + ".res_v"] if c["rank"] else None)
        for m in (1, 2, 3, 4, 6):       # 6 rows: two fused launches (four rows + two rows)
            x = torch.from_numpy(z[f"{nm}.x{m}"])
            y = mod(x.cuda())
            assert y.dtype == torch.float16 and tuple(y.shape) == (m, c["n"])
            ref = O.gemv_f32(x.numpy(), host, **kw)
            assert_within_tolerance(y.float().cpu().numpy(), ref, f"{nm} m={m}")
            if m == 6:                  # the dequantise + GEMM route (what more than 16 rows take), forced
                mod.chunked_max_rows = 4
                yd = mod(x.cuda())
                del mod.chunked_max_rows
                assert np.abs(yd.float().cpu().numpy() - z[f"{nm}.y{m}"].astype(np.float32)).max() < 8e-3, (nm, m)
            # against what the reference module returned on the CPU (fp16 arithmetic on both sides)
            assert np.abs(y.float().cpu().numpy() - z[f"{nm}.y{m}"].astype(np.float32)).max() < 8e-3, (nm, m)
        x3 = torch.from_numpy(z[nm + ".x3d"])
        y3 = mod(x3.cuda())
        assert tuple(y3.shape) == (2, 2, c["n"])
        assert np.abs(y3.float().cpu().numpy() - z[nm + ".y3d"].astype(np.float32)).max() < 8e-3


def test_state_dict_round_trip_on_device(small_cases):
    z, meta = small_cases
    c = meta["hybrid_cases"][1]
    src = _build(c, z)
    dst = HybridInt2Linear(nn.Linear(c["k"], c["n"], bias=True), c["group"], None, c["requested"], c["rank"]).to("cuda")
    dst.load_state_dict(src.state_dict(), strict=False)
    x = torch.from_numpy(z[c["name"] + ".x2"]).cuda()
    assert torch.equal(dst(x), src.to("cuda")(x))


def test_int4_residual_extension():
    torch.manual_seed(0)
    lin = nn.Linear(512, 96, bias=False)
    plain = HybridInt4Linear(lin, 128, None, 8).cuda()
    u, v = torch.randn(96, 8) * 0.05, torch.randn(8, 512) * 0.05
    withres = HybridInt4Linear(lin, 128, None, 8, residual_factors=(u, v)).cuda()
    assert {"res_u", "res_v"} <= set(withres.state_dict())
    x = torch.randn(3, 512).half().cuda()
    want = plain(x).float() + (x.float() @ v.half().float().cuda().t()) @ u.half().float().cuda().t()
    assert (withres(x).float() - want).abs().max() < 5e-3
    svd = HybridInt4Linear(lin, 128, None, 8, residual_rank=4).cuda()
    w = lin.weight.detach().cuda()
    e_plain = (plain(x).float() - x.float() @ w.t()).norm()
    e_svd = (svd(x).float() - x.float() @ w.t()).norm()
    assert e_svd < e_plain


def test_forward_into_device_and_pinned_host_buffers():
    """forward_into writes the same bits as forward: into a device buffer, and straight into pinned
    host memory (fast and general kernels, fp16 and bf16)."""
    torch.manual_seed(3)
    mods = [HybridInt2Linear(nn.Linear(1024, 1000), 128, None, 8, 8).cuda(),
            HybridInt4Linear(nn.Linear(512, 96, bias=True), 128, None, 16).cuda(),
            HybridInt4Linear(nn.Linear(1000, 333), 40, None, 5).cuda()]       # general kernel (odd group, ragged N)
    for mod in mods:
        for dt in (torch.float16, torch.bfloat16):
            for m in (1, 4):
                x = torch.randn(m, mod.in_features).to(dt).cuda()
                want = mod(x)
                dev_out = torch.full((m, mod.out_features), float("nan"), dtype=dt, device="cuda")
                assert mod.forward_into(x, dev_out) is dev_out
                assert torch.equal(dev_out, want)
                host_out = torch.full((m, mod.out_features), float("nan"), dtype=dt).pin_memory()
                mod.forward_into(x, host_out)
                torch.cuda.synchronize()
                assert torch.equal(host_out, want.cpu())
    x = torch.randn(1, 512).half().cuda()
    with pytest.raises(RuntimeError):
        mods[1].forward_into(x, torch.empty((1, 96), dtype=torch.float16))            # pageable host memory
    with pytest.raises(ValueError):
        mods[1].forward_into(x, torch.empty((1, 97), dtype=torch.float16, device="cuda"))
    with pytest.raises(ValueError):
        mods[1].forward_into(torch.randn(5, 512).half().cuda(), torch.empty((5, 96), dtype=torch.float16, device="cuda"))


def test_fused_siblings_match_separate_modules():
    """q/k/v merged into one launch: the quantised term is the same arithmetic per row, the outlier
    and residual terms are summed over the merged column lists -> equal within the kernel tolerance,
    and equal to the oracle."""
    from ai_accel_studio_b200.optimize.siblings import merge_packed
    torch.manual_seed(5)
    k = 1024
    mods = []
    for n, oc in ((512, 16), (128, 8), (128, 8)):
        lin = nn.Linear(k, n, bias=False)
        with torch.no_grad():
            lin.weight[:, torch.randperm(k)[:8]] *= 6
        m = HybridInt4Linear(lin, 128, None, oc)
        m.set_residual(torch.randn(n, 8) * 0.03, torch.randn(8, k) * 0.03)
        mods.append(m.cuda())
    fused, sizes = merge_packed(mods)
    for m_rows in (1, 4):
        x = torch.randn(m_rows, k).half().cuda()
        parts = fused(x).split(sizes, dim=-1)
        for part, mod in zip(parts, mods):
            pw = O.PackedWeight(4, mod.packed.cpu().numpy(), mod.scales.cpu().numpy(), k, k, 128)
            ref = O.gemv_f32(x.cpu().numpy(), pw, None, mod.outlier_idx.cpu().numpy(), mod.outlier_weight.cpu().numpy(),
                             mod.res_u.cpu().numpy(), mod.res_v.cpu().numpy())
            assert_within_tolerance(part.float().cpu().numpy(), ref, "fused sibling slice vs oracle")
            assert (part.float() - mod(x).float()).abs().max() < 2e-3


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_shards_on_one_device(world, coracle):
    """Every row shard and every column shard of a packed module, run through the CUDA kernels on one
    device: row shards concatenate to, and column shards (re-based outlier indices, zero-weight padding
    columns, bias on rank 0 only, K/T-wide res_v) sum to, the unsharded module's oracle result."""
    from conftest import c_forward
    from ai_accel_studio_b200 import tp
    torch.manual_seed(40 + world)
    n, k = 1024, 4096
    for cls in (HybridInt2Linear, HybridInt4Linear):
        lin = nn.Linear(k, n, bias=True)
        with torch.no_grad():
            lin.weight.normal_(0, 0.02)
            lin.weight[:, torch.randperm(k)[:40]] *= 5          # clear outlier columns, unevenly spread over K
        full = cls(lin, 128, None, 32)
        full.set_residual(torch.randn(n, 8) * 0.02, torch.randn(8, k) * 0.02)
        np_ = lambda t_: t_.detach().cpu().numpy()
        for m in (1, 4):
            x = torch.randn(m, k).half()
            ref = c_forward(coracle, x.numpy(), full.bits, np_(full.packed), np_(full.scales), k, 128, np_(full.bias),
                            np_(full.outlier_idx), np_(full.outlier_weight), np_(full.res_u), np_(full.res_v))
            rows = [tp.shard_rows(full, r, world).cuda()(x.cuda()) for r in range(world)]
            assert_within_tolerance(torch.cat(rows, 1).float().cpu().numpy(), ref, f"{cls.__name__} row shards T={world} m={m}")
            ks = k // world
            cols = [tp.shard_cols(full, r, world) for r in range(world)]
            assert len({c.outlier_idx.numel() for c in cols}) == 1           # common padded outlier count
            assert all(c.bias is None for c in cols[1:]) and cols[0].bias is not None
            parts = [c.cuda()(x[:, r * ks:(r + 1) * ks].cuda()).float() for r, c in enumerate(cols)]
            total = torch.stack(parts).sum(0)                                  # what the all-reduce computes (fp32 here)
            # every rank rounds its partial result to fp16 before the sum: allow that on top of the tolerance
            assert np.abs(total.cpu().numpy() - ref).max() <= 1e-2 + 1e-3 * np.abs(ref).max() + world * 2.0 ** -11 * np.abs(ref).max()
            assert np.linalg.norm(total.cpu().numpy() - ref) <= 2e-3 * np.linalg.norm(ref)


def test_cuda_graph_capture_and_replay():
    torch.manual_seed(1)
    mods = [HybridInt2Linear(nn.Linear(1024, 1024), 128, None, 8, 4).cuda(),
            HybridInt4Linear(nn.Linear(1024, 1024), 128, None, 8).cuda()]
    x = torch.randn(1, 1024).half().cuda()
    eager = mods[1](mods[0](x))
    static_x = x.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            mods[1](mods[0](static_x))
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = mods[1](mods[0](static_x))
    g.replay()
    assert torch.equal(out, eager)
    x2 = torch.randn(1, 1024).half().cuda()
    static_x.copy_(x2)
    g.replay()
    assert torch.equal(out, mods[1](mods[0](x2)))


def test_torch_compile_traces_without_graph_break():
    torch.manual_seed(2)
    mod = HybridInt2Linear(nn.Linear(512, 256), 128, None, 4, 2).cuda()
    mod.graph_safe = True
    x = torch.randn(2, 512).half().cuda()
    fn = torch.compile(lambda t: torch.relu(mod(t)) * 2, fullgraph=True)
    assert torch.equal(fn(x), torch.relu(mod(x)) * 2)


def test_kernel_suite_rows_and_speed_gate():
    from ai_accel_studio_b200.kernel_suite import run_kernel_suite
    from ai_accel_studio_b200.optimize.planner_v5 import runtime_speedups
    rows = run_kernel_suite(m=1, n=512, k=1024, group_size=64, repeats=5)
    assert [r["method"] for r in rows] == ["torch-fp16", "decode-int2-v4", "decode-int4-v5"]
    assert rows[0]["nmse_vs_dense"] < 1e-6
    assert rows[2]["cosine_vs_dense"] > 0.99 and rows[1]["cosine_vs_dense"] > 0.85
    assert all(r["latency_ms"] > 0 and r["speedup"] > 0 for r in rows)
    lin = nn.Linear(1024, 512).cuda().half()
    cand = HybridInt4Linear(lin, 128, None, 8).cuda()
    d, p_, proj = runtime_speedups(lin, cand, torch.randn(32, 1024, device="cuda", dtype=torch.float16))
    assert d > 0 and p_ > 0 and proj > 0


def _r16(t, dtype):
    return t.to(dtype).float()


@pytest.mark.parametrize("bits,dtype", [(4, torch.float16), (2, torch.float16), (4, torch.bfloat16)])
def test_gated_pair_epilogue(bits, dtype):
    """gate / up merged with their rows interleaved in blocks of 8: one launch returns
    silu(gate(x)) * up(x), rounded where separate 16-bit operators round; compared with the oracle's
    float32 projections pushed through those roundings, with the unfused modules, and on the M > 4 path."""
    from ai_accel_studio_b200 import _cabi, ops
    from ai_accel_studio_b200.optimize.siblings import merge_gate_up
    torch.manual_seed(20 + bits)
    k, n = 1024, 2048 + 64
    cls = HybridInt2Linear if bits == 2 else HybridInt4Linear
    gate = cls(nn.Linear(k, n, bias=True), 128, None, 16)
    up = cls(nn.Linear(k, n, bias=False), 128, None, 8)
    up.set_residual(torch.randn(n, 8) * 0.02, torch.randn(8, k) * 0.02)
    fused = merge_gate_up(gate, up).cuda()
    gate, up = gate.cuda(), up.cuda()

    def np_(t):
        return t.cpu().numpy()
    for m_rows in (1, 3, 4):
        x = (torch.randn(m_rows, k) * 1.5).to(dtype).cuda()
        y = fused(x)
        assert y.shape == (m_rows, n) and y.dtype == dtype
        xs = x.float().cpu().numpy().astype(np.float32)
        refs = []
        for mod in (gate, up):
            pw = O.PackedWeight(bits, np_(mod.packed), np_(mod.scales), k, k, 128)
            refs.append(torch.from_numpy(O.gemv_f32(
                xs if dtype == torch.bfloat16 else np_(x), pw, None if mod.bias is None else np_(mod.bias), np_(mod.outlier_idx),
                np_(mod.outlier_weight), np_(mod.res_u) if mod.residual_rank else None,
                np_(mod.res_v) if mod.residual_rank else None)).float())
        g16, u16 = _r16(refs[0], dtype), _r16(refs[1], dtype)
        want = _r16(_r16(torch.nn.functional.silu(g16), dtype) * u16, dtype)
        tol = 1.6e-2 if dtype == torch.bfloat16 else 2e-3        # two units in the last place: a rounding may flip per stage
        err = (y.float().cpu() - want).abs()
        assert float((err / (tol * want.abs() + 1e-2)).max()) <= 1.0, float(err.max())
        sep = torch.nn.functional.silu(gate(x)) * up(x)
        assert float((y.float() - sep.float()).abs().max()) <= 2e-2 * float(sep.float().abs().max()) + 1e-3
    for rows in (9, 20):                    # 9 rows: three fused launches; 20 rows: dequantise + GEMM, then the same pairing
        x8 = torch.randn(rows, k).to(dtype).cuda()
        y8, sep8 = fused(x8), torch.nn.functional.silu(gate(x8)) * up(x8)
        assert y8.shape == (rows, n)
        assert float((y8.float() - sep8.float()).abs().max()) <= 2e-2 * float(sep8.float().abs().max()) + 1e-3
    with pytest.raises(_cabi.QgemvError) as e:                                      # no gated epilogue in the CUDA-core kernel
        ops.gemv(x8[:1].contiguous(), fused.packed, fused.scales, fused.bias, fused.outlier_idx, fused.outlier_weight, fused.res_u,
                 fused.res_v, bits, 128, k, ops.ACT_SILU_MUL, _cabi.KERNEL["simt"])
    assert e.value.code == -2
    assert ops.workspace_status("cuda") == 0


def test_prepared_launch_follows_the_module():
    """The eager decode path keeps a prepared launch per module; replacing a buffer, attaching a residual,
    changing the kernel or the activation shape must all be seen by the next call."""
    torch.manual_seed(31)
    k, n = 1024, 512
    a = HybridInt4Linear(nn.Linear(k, n, bias=True), 128, None, 8).cuda()
    b = HybridInt4Linear(nn.Linear(k, n, bias=True), 128, None, 8).cuda()
    x = torch.randn(1, k).half().cuda()
    ya, yb = a(x), b(x)
    assert not torch.equal(ya, yb) and torch.equal(a(x), ya)               # second call: the prepared launch
    a.packed = b.packed.clone()                                             # every operand swapped for b's, one at a time
    a.scales = b.scales.clone()
    a.bias = b.bias.clone()
    a.outlier_idx = b.outlier_idx.clone()
    a.outlier_weight = b.outlier_weight.clone()
    assert torch.equal(a(x), yb)
    a.set_residual(torch.randn(n, 4) * 0.05, torch.randn(4, k) * 0.05)
    y_res = a(x)
    assert not torch.equal(y_res, yb)
    x4 = torch.randn(4, k).half().cuda()
    assert a(x4).shape == (4, n)
    assert torch.equal(a(x), y_res)                                          # back to one row
    a.kernel = "simt"
    assert (a(x).float() - y_res.float()).abs().max() < 2e-3                 # another kernel, same answer to rounding
    moved = a.cpu().cuda()
    assert (moved(x).float() - y_res.float()).abs().max() < 2e-3
