"""Whole-model decode on the GPU with swapped packed modules: the captured CUDA-graph decode
produces the same tokens as eager decoding, and the packed model tracks its own dequantised
(fp16 dense) twin."""
import pytest
import torch
from torch import nn

from ai_accel_studio_b200 import model_tools as mt
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.kernels.groupwise_int2 import unpack_groupwise_int2
from ai_accel_studio_b200.kernels.groupwise_int4 import unpack_groupwise_int4
from ai_accel_studio_b200.runtime_v5 import StaticGraphDecoder, generate_static_benchmark

pytestmark = pytest.mark.gpu


@pytest.fixture()
def tiny(monkeypatch):
    monkeypatch.setitem(mt.SHAPES, "tiny", dict(family="llama", layers=2, hidden=256, inter=512, heads=4, kv_heads=2,
                                                head_dim=64, vocab=320, qkv_bias=False))
    return "tiny"


def _dense_twin(mod):
    """nn.Linear holding exactly the weights the packed module represents (fp32 math, fp16 storage)."""
    w = (unpack_groupwise_int2 if mod.bits == 2 else unpack_groupwise_int4)(mod.packed_weight(), torch.float32)
    if mod.outlier_idx.numel():
        w[:, mod.outlier_idx.long()] += mod.outlier_weight.float()
    if mod.residual_rank:
        w += mod.res_u.float() @ mod.res_v.float()
    lin = nn.Linear(mod.in_features, mod.out_features, bias=mod.bias is not None, device=w.device, dtype=torch.float32)
    with torch.no_grad():
        lin.weight.copy_(w)
        if mod.bias is not None:
            lin.bias.copy_(mod.bias.float())
    return lin


def test_graph_decode_equals_eager_and_tracks_dense_twin(tiny):
    dev = torch.device("cuda")
    model = mt.build_fp16_model(tiny, dev)
    plan = mt.seeded_plan(model, (0.5, 0.4, 0.1), seed=3)
    mt.apply_plan(model, plan)
    assert any(isinstance(m, HybridInt2Linear) for m in model.modules())
    assert any(isinstance(m, HybridInt4Linear) for m in model.modules())
    ids = torch.randint(0, 320, (1, 16), generator=torch.Generator().manual_seed(2)).to(dev)

    eager = StaticGraphDecoder(model, 1, 64, device=dev)
    first = eager.prefill(ids)
    tok_eager = torch.cat([first, eager.decode(12)], 1)

    graph = StaticGraphDecoder(model, 1, 64, device=dev)
    graph.prefill(ids)
    graph.capture()
    first = graph.prefill(ids)
    tok_graph = torch.cat([first, graph.decode(12)], 1)
    assert torch.equal(tok_eager, tok_graph)

    # logits of one decode step vs the same model with dense fp32 twins of every packed layer
    with torch.no_grad():
        x = ids[:, :1]
        lg = model(input_ids=x).logits.float()
        twin = mt.build_fp16_model(tiny, dev)
        twin.load_state_dict({k: v for k, v in model.state_dict().items() if k in twin.state_dict()}, strict=False)
        mods = dict(model.named_modules())
        for name, m in mods.items():
            if isinstance(m, (HybridInt2Linear, HybridInt4Linear)):
                mt._set(twin, name, _dense_twin(m))
        twin = twin.float()
        ref = twin(input_ids=x).logits.float()
    rel = (lg - ref).norm() / ref.norm()
    assert rel < 2e-2, float(rel)          # fp16 model vs fp32 twin: activation rounding only

    res = generate_static_benchmark(model, input_ids=ids, max_new_tokens=8, device=dev, warmups=1)
    assert res["generated_tokens"] == 8 and res["decode_tokens_s"] > 0


@pytest.fixture()
def qwen_width(monkeypatch):
    """Qwen2.5-0.5B's layer shapes (hidden 896, intermediate 4864, 14 query / 2 key-value heads of 64,
    q/k/v bias) at reduced depth and vocabulary: K = 896 and 4864, N = 128 for the k/v projections."""
    monkeypatch.setitem(mt.SHAPES, "qwen-width", dict(family="qwen2", layers=3, hidden=896, inter=4864, heads=14, kv_heads=2,
                                                      head_dim=64, vocab=2048, qkv_bias=True))
    return "qwen-width"


def test_qwen_width_graph_decode_and_dense_twin(qwen_width):
    dev = torch.device("cuda")
    model = mt.build_fp16_model(qwen_width, dev)
    plan = mt.seeded_plan(model, (0.6, 0.3, 0.1), seed=0)
    mt.apply_plan(model, plan)
    packed = [m for m in model.modules() if isinstance(m, (HybridInt2Linear, HybridInt4Linear))]
    assert {m.in_features for m in packed} == {896, 4864} and 128 in {m.out_features for m in packed}
    assert any(m.bias is not None for m in packed)
    ids = torch.randint(0, 2048, (1, 24), generator=torch.Generator().manual_seed(4)).to(dev)

    eager = StaticGraphDecoder(model, 1, 96, device=dev)
    first = eager.prefill(ids)
    tok_eager = torch.cat([first, eager.decode(16)], 1)
    graph = StaticGraphDecoder(model, 1, 96, device=dev)
    graph.prefill(ids)
    graph.capture()
    first = graph.prefill(ids)
    tok_graph = torch.cat([first, graph.decode(16)], 1)
    assert torch.equal(tok_eager, tok_graph)

    with torch.no_grad():
        x = ids[:, :1]
        lg = model(input_ids=x).logits.float()
        twin = mt.build_fp16_model(qwen_width, dev)
        twin.load_state_dict({k: v for k, v in model.state_dict().items() if k in twin.state_dict()}, strict=False)
        for name, m in dict(model.named_modules()).items():
            if isinstance(m, (HybridInt2Linear, HybridInt4Linear)):
                mt._set(twin, name, _dense_twin(m))
        ref = twin.float()(input_ids=x).logits.float()
    rel = (lg - ref).norm() / ref.norm()
    assert rel < 2e-2, float(rel)
    from ai_accel_studio_b200 import ops
    assert ops.workspace_status(dev) == 0
