"""The torch expressions that the GPU tests of the decode-step kernels use as their oracle, pinned on the CPU to the
framework code they restate (transformers' Llama modules, imported here): RMS norm, rotary embedding with the
rotate-half convention, and one-token attention over a static cache through the model's own attention module."""
import pytest
import torch

transformers = pytest.importorskip("transformers")
from transformers import LlamaConfig                                                     # noqa: E402
from transformers.models.llama import modeling_llama as ml                                # noqa: E402


def test_rmsnorm_expression_is_the_frameworks():
    torch.manual_seed(0)
    norm = ml.LlamaRMSNorm(256, eps=1e-5)
    with torch.no_grad():
        norm.weight.copy_(1 + 0.1 * torch.randn(256))
    for dtype in (torch.float32, torch.bfloat16):
        x = torch.randn(3, 256).to(dtype)
        w = norm.weight.to(dtype)
        f = x.float()
        mine = w * (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-5)).to(dtype)      # tests/test_decode_step_gpu.py
        norm_t = ml.LlamaRMSNorm(256, eps=1e-5).to(dtype)
        with torch.no_grad():
            norm_t.weight.copy_(w)
        assert torch.equal(mine, norm_t(x))


def test_rope_expression_is_the_frameworks():
    torch.manual_seed(1)
    cfg = LlamaConfig(hidden_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=64, max_position_embeddings=128)
    rot = ml.LlamaRotaryEmbedding(cfg)
    pos = torch.tensor([[37]])
    q = torch.randn(1, 4, 1, 64)
    k = torch.randn(1, 2, 1, 64)
    cos, sin = rot(q, pos)                                                                   # [1, 1, 64] each
    q_ref, k_ref = ml.apply_rotary_pos_emb(q, k, cos, sin)

    def rotate_half(x):
        x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
        return torch.cat((-x2, x1), dim=-1)
    table_cos, table_sin = rot(q, torch.arange(128)[None])                                   # the decode step's tables: row = position
    c, s = table_cos[0, 37], table_sin[0, 37]
    assert torch.equal(q[0, :, 0] * c + rotate_half(q[0, :, 0]) * s, q_ref[0, :, 0])
    assert torch.equal(k[0, :, 0] * c + rotate_half(k[0, :, 0]) * s, k_ref[0, :, 0])


def test_attention_expression_is_the_frameworks():
    """softmax(q . K^T * scale) . V over positions 0..p with grouped-query heads, against the model's eager attention."""
    torch.manual_seed(2)
    b, hq, hkv, d, p = 2, 4, 2, 64, 9
    q = torch.randn(b, hq, 1, d)
    kc, vc = torch.randn(b, hkv, p + 1, d), torch.randn(b, hkv, p + 1, d)

    class Holder(torch.nn.Module):
        num_key_value_groups = hq // hkv
        training = False
    out, _ = ml.eager_attention_forward(Holder(), q, kc, vc, attention_mask=None, scaling=d ** -0.5)      # [b, 1, hq, d]
    g = hq // hkv
    att = torch.softmax(torch.einsum("bhd,bhjd->bhj", q[:, :, 0], kc.repeat_interleave(g, dim=1)) * d ** -0.5, -1)
    mine = torch.einsum("bhj,bhjd->bhd", att, vc.repeat_interleave(g, dim=1))
    assert torch.allclose(mine, out[:, 0], atol=1e-5)
