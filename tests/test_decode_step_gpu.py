"""The decode-step kernels between the packed GEMVs (include/qdecode_b200.h) against the framework's
own operators: each kernel alone against the torch expression it replaces, then the whole step
(NativeDecodeStep) against the Hugging Face forward over the same static cache, token by token."""
import pytest
import torch
from torch import nn

from ai_accel_studio_b200 import _cabi, decode_step as ds, model_tools as mt
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.runtime_v5 import StaticGraphDecoder

pytestmark = pytest.mark.gpu

DTYPES = [torch.float16, torch.bfloat16]


def _ulp_close(got, want, dtype, ulps=1, frac_exact=0.98):
    """Equal up to `ulps` units in the last place of the 16-bit type, and bit-equal almost everywhere."""
    eps = 2.0 ** (-10 if dtype == torch.float16 else -7)
    g, w = got.float(), want.float()
    tol = ulps * eps * w.abs().clamp_min(2.0 ** -14)
    assert bool(((g - w).abs() <= tol).all()), float(((g - w).abs() / tol).max())
    assert float((got == want).float().mean()) >= frac_exact


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(1, 896), (4, 4096), (3, 8192), (2, 16384)])
def test_rmsnorm_with_residual_update(dtype, rows, hidden):
    torch.manual_seed(hidden + rows)
    h = (torch.randn(rows, hidden) * 2).to(dtype).cuda()
    delta = torch.randn(rows, hidden).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(hidden)).to(dtype).cuda()
    eps = 1e-5

    def ref(hh):
        f = hh.float()
        return w * (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)
    h1 = h.clone()
    y = ds.rmsnorm(h1, None, w, eps)
    assert torch.equal(h1, h)                                    # no delta: h is left alone
    _ulp_close(y, ref(h), dtype)
    h2 = h.clone()
    y2 = ds.rmsnorm(h2, delta, w, eps)
    assert torch.equal(h2, h + delta)                            # the residual stream is updated in place, rounded once
    _ulp_close(y2, ref(h + delta), dtype)
    wide = torch.zeros(rows, hidden + 64, dtype=dtype, device="cuda")      # strided rows
    wide[:, :hidden] = h
    y3 = ds.rmsnorm(wide[:, :hidden], None, w, eps)
    assert torch.equal(y3, y)
    with pytest.raises(_cabi.QgemvError):
        ds.rmsnorm(torch.zeros(1, 20, dtype=dtype, device="cuda"), None, torch.ones(20, dtype=dtype, device="cuda"), eps)


def _rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("batch,hq,hkv,d", [(1, 32, 8, 128), (2, 14, 2, 64), (4, 8, 1, 128)])
def test_rope_and_cache_append(dtype, batch, hq, hkv, d):
    torch.manual_seed(hq + d)
    max_len, p = 96, 37
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2).float() / d))
    ang = torch.arange(max_len).float()[:, None] * inv[None]
    emb = torch.cat([ang, ang], -1)
    cos, sin = emb.cos().to(dtype).cuda(), emb.sin().to(dtype).cuda()
    fused = torch.randn(batch, (hq + 2 * hkv) * d).to(dtype).cuda()             # q | k | v as one fused projection's output
    q, k, v = fused.split([hq * d, hkv * d, hkv * d], dim=-1)
    q0 = q.clone()
    kc = torch.randn(batch, hkv, max_len, d).to(dtype).cuda()
    vc = torch.randn(batch, hkv, max_len, d).to(dtype).cuda()
    kc0, vc0 = kc.clone(), vc.clone()
    pos = torch.tensor([p], dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ds.rope_append(q, k, v, cos, sin, pos, kc, vc, d, status)

    def rot(x, heads):                                                           # the framework's expression, in `dtype`
        xh = x.reshape(batch, heads, d)
        return (xh * cos[p]) + (_rotate_half(xh) * sin[p])
    assert torch.equal(q.reshape(batch, hq, d), rot(q0, hq))
    assert torch.equal(kc[:, :, p], rot(k, hkv)) and torch.equal(vc[:, :, p], v.reshape(batch, hkv, d))
    keep = torch.ones(max_len, dtype=torch.bool)
    keep[p] = False
    assert torch.equal(kc[:, :, keep], kc0[:, :, keep]) and torch.equal(vc[:, :, keep], vc0[:, :, keep])
    assert int(status.item()) == 0
    pos.fill_(max_len)                                                           # past the cache: nothing written, status raised
    before = (q.clone(), kc.clone())
    ds.rope_append(q, k, v, cos, sin, pos, kc, vc, d, status)
    assert int(status.item()) == 1 and torch.equal(q, before[0]) and torch.equal(kc, before[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("batch,hq,hkv,d,max_len,p", [(1, 32, 8, 128, 648, 600), (2, 14, 2, 64, 96, 17), (4, 8, 1, 128, 1160, 1159),
                                                       (1, 4, 2, 64, 64, 0), (3, 24, 8, 128, 40, 39), (1, 5, 1, 64, 300, 150)])
def test_attention_over_the_cache(dtype, batch, hq, hkv, d, max_len, p):
    torch.manual_seed(hq * d + p)
    q = torch.randn(batch, hq * d).to(dtype).cuda()
    kc = torch.randn(batch, hkv, max_len, d).to(dtype).cuda()
    vc = torch.randn(batch, hkv, max_len, d).to(dtype).cuda()
    kc[:, :, p + 1:] = 50.0                                                      # beyond the current position: must not be read
    vc[:, :, p + 1:] = float("nan")
    pos = torch.tensor([p], dtype=torch.int64, device="cuda")
    ws = ds.attention_workspace(batch, hq, hkv, d, max_len, "cuda")
    scale = d ** -0.5
    for _ in range(2):                                                           # twice: the arrival counters are left ready
        out = ds.attention(q, kc, vc, pos, scale, ws)
    g = hq // hkv
    kf = kc[:, :, :p + 1].float().repeat_interleave(g, dim=1)
    vf = vc[:, :, :p + 1].float().repeat_interleave(g, dim=1)
    att = torch.softmax(torch.einsum("bhd,bhjd->bhj", q.float().reshape(batch, hq, d), kf) * scale, -1)
    ref = torch.einsum("bhj,bhjd->bhd", att, vf).reshape(batch, hq * d)
    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3
    assert torch.isfinite(out.float()).all()
    assert float((out.float() - ref).abs().max()) <= tol * float(ref.abs().max()), float((out.float() - ref).abs().max())
    with pytest.raises(_cabi.QgemvError):
        ds.attention(q, kc, vc, pos, scale, ws[:64])                             # workspace too small


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    torch.manual_seed(1)
    for rows, width in ((1, 14336), (4, 4864), (3, 50)):
        g = (torch.randn(rows, width) * 3).to(dtype).cuda()
        u = torch.randn(rows, width).to(dtype).cuda()
        _ulp_close(ds.silu_mul(g, u), nn.functional.silu(g) * u, dtype, ulps=2)   # a flip of the rounded silu moves the product too
    wide = torch.randn(2, 4096 * 2).to(dtype).cuda()                            # two halves of one fused projection's output
    g, u = wide.split(4096, dim=-1)
    _ulp_close(ds.silu_mul(g, u), nn.functional.silu(g) * u, dtype, ulps=2)   # a flip of the rounded silu moves the product too


SHAPES = {
    "llama-like": dict(family="llama", layers=3, hidden=512, inter=1024, heads=8, kv_heads=2, head_dim=64, vocab=640, qkv_bias=False),
    "qwen-like": dict(family="qwen2", layers=2, hidden=896, inter=4864, heads=14, kv_heads=2, head_dim=64, vocab=1024, qkv_bias=True),
    "wide-heads": dict(family="llama", layers=2, hidden=1024, inter=2048, heads=8, kv_heads=2, head_dim=128, vocab=512, qkv_bias=False),
}


@pytest.mark.parametrize("side_streams", [True, False])
@pytest.mark.parametrize("shape,batch,fuse", [("llama-like", 1, False), ("llama-like", 2, True), ("qwen-like", 1, False),
                                              ("wide-heads", 3, True)])
def test_native_step_tracks_the_framework_forward(monkeypatch, shape, batch, fuse, side_streams):
    """Same model, same prompt, two static caches: at every step both paths get the same token and
    position; logits, and the keys / values appended to the caches, must agree to rounding."""
    monkeypatch.setitem(mt.SHAPES, shape, SHAPES[shape])
    monkeypatch.setattr(ds.NativeDecodeStep, "parallel_kv", side_streams)      # k / v beside q on side streams, or one after the other
    dev = torch.device("cuda")
    model = mt.build_fp16_model(shape, dev)
    probs = (0.0, 1.0, 0.0) if fuse else (0.5, 0.4, 0.1)                         # one bit width: every sibling set can merge
    mt.apply_plan(model, mt.seeded_plan(model, probs, seed=5))
    assert any(isinstance(m, (HybridInt2Linear, HybridInt4Linear)) for m in model.modules())
    vocab = SHAPES[shape]["vocab"]
    ids = torch.randint(0, vocab, (batch, 24), generator=torch.Generator().manual_seed(6)).to(dev)
    fw = StaticGraphDecoder(model, batch, 64, device=dev, native_step=False)
    fw.prefill(ids)
    if fuse:                                                                     # fused siblings and gated feed-forward blocks
        from ai_accel_studio_b200.optimize.siblings import fuse_decoder_siblings
        twin = mt.build_fp16_model(shape, dev)
        mt.apply_plan(twin, mt.seeded_plan(twin, probs, seed=5))
        assert fuse_decoder_siblings(twin) > 0
        assert any(type(m).__name__ == "GatedFeedForward" for m in twin.modules())
        native_model = twin
    else:
        native_model = model
    nv = StaticGraphDecoder(native_model, batch, 64, device=dev, native_step=True)
    nv.prefill(ids)
    assert nv.native is not None and fw.native is None
    tok, pos = fw.tok.clone(), fw.pos.clone()
    n0 = int(pos.item())
    with torch.no_grad():
        for _ in range(6):
            want = model(input_ids=tok, past_key_values=fw.cache, cache_position=pos, use_cache=True).logits[:, -1].float()
            got = nv.native.step(tok, pos).float()
            rel = float((got - want).norm() / want.norm())
            assert rel < 6e-3, rel
            tok = want.argmax(-1, keepdim=True)
            pos = pos + 1
    for lf, ln in zip(fw.cache.layers, nv.cache.layers):
        for a, b in ((lf.keys, ln.keys), (lf.values, ln.values)):
            a, b = a[:, :, n0:n0 + 6].float(), b[:, :, n0:n0 + 6].float()
            assert float((a - b).norm() / a.norm()) < 6e-3
    assert nv.native.check_status() == 0


def test_native_step_in_a_cuda_graph_equals_eager(monkeypatch):
    monkeypatch.setitem(mt.SHAPES, "llama-like", SHAPES["llama-like"])
    dev = torch.device("cuda")
    model = mt.build_fp16_model("llama-like", dev)
    mt.apply_plan(model, mt.seeded_plan(model, (0.6, 0.3, 0.1), seed=1))
    ids = torch.randint(0, 640, (2, 16), generator=torch.Generator().manual_seed(9)).to(dev)
    eager = StaticGraphDecoder(model, 2, 64, device=dev, native_step=True)
    first = eager.prefill(ids)
    tok_eager = torch.cat([first, eager.decode(20)], 1)
    graph = StaticGraphDecoder(model, 2, 64, device=dev, native_step=True)
    graph.prefill(ids)
    graph.capture()
    first = graph.prefill(ids)
    tok_graph = torch.cat([first, graph.decode(20)], 1)
    assert torch.equal(tok_eager, tok_graph)
    assert graph.native.check_status() == 0
    with pytest.raises(ValueError):
        graph.decode(64)                                                         # would run past the cache: refused on the host
