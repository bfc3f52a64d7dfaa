"""Model-level host logic on the CPU: local (sharded) configs, seeded plans, module swap, and the
static-cache greedy decoder against Hugging Face's own generate()."""
import pytest
import torch

from ai_accel_studio_b200 import model_tools as mt
from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
from ai_accel_studio_b200.runtime_v5 import StaticGraphDecoder, generate_static_benchmark
from ai_accel_studio_b200.tp import AllReduceLinear


@pytest.fixture()
def tiny(monkeypatch):
    monkeypatch.setitem(mt.SHAPES, "tiny", dict(family="llama", layers=2, hidden=256, inter=512, heads=4, kv_heads=2,
                                                head_dim=64, vocab=320, qkv_bias=False))
    return "tiny"


def test_local_config_shards_heads_and_mlp(tiny):
    c1, c2 = mt.local_config(tiny, 1), mt.local_config(tiny, 2)
    assert (c2.num_attention_heads, c2.num_key_value_heads, c2.intermediate_size) == (2, 1, 256)
    assert c2.hidden_size == c1.hidden_size == 256 and c2.head_dim == 64
    with pytest.raises(ValueError):
        mt.local_config(tiny, 4)                     # 2 kv heads cannot be split 4 ways
    cfg = mt.local_config("llama-3-70b", 8)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size) == (8, 1, 3584)


def test_seeded_plan_and_swap(tiny):
    model = mt.build_fp16_model(tiny, "cpu", world=2)
    assert sum(isinstance(m, AllReduceLinear) for m in model.modules()) == 4      # o_proj + down_proj, 2 layers
    plan = mt.seeded_plan(model, (0.6, 0.3, 0.1), seed=5, global_k={"o_proj": 256, "down_proj": 512})
    again = mt.seeded_plan(model, (0.6, 0.3, 0.1), seed=5, global_k={"o_proj": 256, "down_proj": 512})
    assert [(e.name, e.bits) for e in plan] == [(e.name, e.bits) for e in again]
    assert len(plan) == 14 and {e.bits for e in plan} <= {2, 4, 16}
    mt.apply_plan(model, plan)
    mods = dict(model.named_modules())
    for e in plan:
        m = mods[e.name]
        m = m.inner if isinstance(m, AllReduceLinear) else m
        if e.bits == 2:
            assert isinstance(m, HybridInt2Linear) and m.residual_rank == 8 and m.group_size == 128
        elif e.bits == 4:
            assert isinstance(m, HybridInt4Linear) and m.residual_rank == 8
        else:
            assert isinstance(m, torch.nn.Linear)
    b = mt.linear_weight_bytes(model)
    assert b["packed_bytes"] > 0 and b["fp16_bytes"] > 0


def test_static_decoder_matches_hf_generate(tiny):
    model = mt.build_fp16_model(tiny, "cpu").float()
    ids = torch.randint(0, 320, (2, 9), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ref = model.generate(ids, do_sample=False, max_new_tokens=6, min_new_tokens=6, cache_implementation="static",
                             pad_token_id=0)[:, 9:]
    dec = StaticGraphDecoder(model, 2, 32, device="cpu")
    first = dec.prefill(ids)
    rest = dec.decode(5)
    assert torch.equal(torch.cat([first, rest], 1), ref)
    res = generate_static_benchmark(model, input_ids=ids, max_new_tokens=6, device="cpu", warmups=1)
    assert torch.equal(res["tokens"], ref) and res["generated_tokens"] == 6 and res["decode_tokens_s"] > 0


def test_streaming_builder_follows_the_seeded_plan(tiny):
    """The model built layer by layer from a meta-device skeleton has exactly the planned modules,
    leaves nothing on the meta device, and under tensor parallelism wraps o_proj / down_proj."""
    for world in (1, 2):
        model, plan = mt.build_mixed_model_streaming(tiny, "cpu", world=world, seed=5)
        ref_plan = mt.seeded_plan(mt.build_fp16_model(tiny, "cpu", world=world), (0.6, 0.3, 0.1), seed=5,
                                  global_k={"o_proj": 256, "down_proj": 512})
        assert [(e.name, e.bits, e.outlier_columns) for e in plan] == [(e.name, e.bits, e.outlier_columns) for e in ref_plan]
        mods = dict(model.named_modules())
        for e in plan:
            m = mods[e.name]
            m = m.inner if isinstance(m, AllReduceLinear) else m
            want = {2: HybridInt2Linear, 4: HybridInt4Linear, 16: torch.nn.Linear}[e.bits]
            assert isinstance(m, want), (e.name, type(m))
            if e.bits != 16:
                assert m.residual_rank == 8 and m.graph_safe
        assert not any(t.is_meta for t in list(model.parameters()) + list(model.buffers()))
        assert sum(isinstance(m, AllReduceLinear) for m in model.modules()) == (4 if world == 2 else 0)
        assert float(model.model.norm.weight.float().mean()) == 1.0
        assert float(model.model.rotary_emb.inv_freq[0]) == 1.0


def _vocab_shard_rank(rank, world, port, ret):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mt.SHAPES["tiny"] = dict(family="llama", layers=2, hidden=256, inter=512, heads=4, kv_heads=2, head_dim=64,
                                 vocab=320, qkv_bias=False)
        model = mt.build_fp16_model("tiny", "cpu", seed=3).float()      # the same replica on every rank
        ids = torch.randint(0, 320, (2, 9), generator=torch.Generator().manual_seed(1))
        full = StaticGraphDecoder(model, 2, 32, device="cpu")
        want = torch.cat([full.prefill(ids), full.decode(6)], 1)
        rows = 320 // world
        head = torch.nn.Linear(256, rows, bias=False)
        with torch.no_grad():
            head.weight.copy_(model.lm_head.weight[rank * rows:(rank + 1) * rows])
        model.lm_head = head
        dec = StaticGraphDecoder(model, 2, 32, device="cpu", vocab_shard=(rank, world))
        got = torch.cat([dec.prefill(ids), dec.decode(6)], 1)
        ret[rank] = bool(torch.equal(got, want))
    finally:
        dist.destroy_process_group()


def test_vocabulary_sharded_greedy_token_two_ranks():
    """lm_head split by vocabulary rows over two gloo ranks: the exchanged (best logit, index) pairs
    pick the same tokens as the whole output projection."""
    import os
    import torch.multiprocessing as mp
    port = 31500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_vocab_shard_rank, args=(2, port, ret), nprocs=2, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_native_decode_step_recognises_what_it_can_run(monkeypatch):
    """Host-side gatekeeping of the decode-step kernels: Llama / Qwen2 style decoders qualify, anything the
    kernels do not cover is named, and a CPU decoder keeps the framework's forward."""
    from ai_accel_studio_b200 import decode_step as ds
    from ai_accel_studio_b200.runtime_v5 import StaticGraphDecoder
    monkeypatch.setitem(mt.SHAPES, "tiny", dict(family="llama", layers=2, hidden=128, inter=256, heads=2, kv_heads=1,
                                                head_dim=64, vocab=96, qkv_bias=False))
    model = mt.build_fp16_model("tiny", "cpu")
    assert ds.unsupported_reason(model) is None
    dec = StaticGraphDecoder(model.float(), 1, 16, device="cpu")
    dec.prefill(torch.randint(0, 96, (1, 4)))
    assert dec.native is None and dec.native_reason == "not a CUDA device"
    with pytest.raises(NotImplementedError):
        forced = StaticGraphDecoder(model, 1, 16, device="cpu", native_step=True)
        forced.prefill(torch.randint(0, 96, (1, 4)))
    model.model.layers[0].self_attn.q_norm = torch.nn.Identity()
    assert "q / k normalisation" in ds.unsupported_reason(model)
    del model.model.layers[0].self_attn.q_norm
    model.model.layers[1].mlp.act_fn = torch.nn.GELU()
    assert "SwiGLU" in ds.unsupported_reason(model)
    monkeypatch.setitem(mt.SHAPES, "odd-heads", dict(family="llama", layers=1, hidden=96, inter=128, heads=2, kv_heads=1,
                                                     head_dim=48, vocab=64, qkv_bias=False))
    assert "head_dim 48" in ds.unsupported_reason(mt.build_fp16_model("odd-heads", "cpu"))
    assert "not a decoder" in ds.unsupported_reason(torch.nn.Linear(4, 4))
