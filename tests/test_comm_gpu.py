"""One-shot all-reduce over peer memory (include/qcomm_b200.h).

On one GPU (this file's single-process tests) two ranks cannot run side by side -- kernels that wait
for each other must never be separate launches on one device -- so the two-rank data path is
checked in turns: a rank that goes early finds partners missing and its bounded wait runs out (the
status word says so and nothing hangs), the rank that goes last finds everybody's vector in place
and must produce the exact sum.  The real thing (two processes, two GPUs, compared
with NCCL) is the last test and needs two devices.
"""
import os

import pytest
import torch

from ai_accel_studio_b200 import _cabi
from ai_accel_studio_b200.comm import OneShotAllReduce

pytestmark = pytest.mark.gpu


def _buffers(world, max_elems):
    lib = _cabi.lib()
    slots = torch.zeros(lib.qcomm_slot_bytes(world, max_elems), dtype=torch.uint8, device="cuda")
    flags = torch.zeros(lib.qcomm_flag_bytes(world), dtype=torch.uint8, device="cuda")
    return slots, flags


def test_single_rank_group_is_the_identity_and_graph_capturable():
    keep = _buffers(1, 8192)
    comm = OneShotAllReduce(rank=0, world=1, max_elems=8192, peers=[(keep[0].data_ptr(), keep[1].data_ptr())])
    for dt in (torch.float16, torch.bfloat16):
        for n in (8, 4096, 8192):
            x = torch.randn(n, device="cuda").to(dt)
            y = x.clone()
            for _ in range(3):                      # both buffer halves get used
                comm(y)
            assert torch.equal(y, x)
    x = torch.randn(2, 4096, device="cuda").half()
    static = x.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm(static)
    torch.cuda.current_stream().wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        comm(static)
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(static, x) and comm.status() == 0
    with pytest.raises(ValueError):
        comm(torch.zeros(16384, device="cuda").half())              # larger than a slot
    with pytest.raises(ValueError):
        comm(torch.zeros(12, device="cuda").half())                 # not a multiple of 8
    comm.close()


def test_fused_allreduce_rmsnorm_single_rank_equals_the_plain_kernels():
    """World 1: the fused kernel must do exactly what rmsnorm(h, delta) does, eagerly and from a graph, and
    count as one call of the group's sequence (a plain all-reduce after it still works)."""
    from ai_accel_studio_b200 import decode_step as ds
    keep = _buffers(1, 4 * 8192)
    comm = OneShotAllReduce(rank=0, world=1, max_elems=4 * 8192, peers=[(keep[0].data_ptr(), keep[1].data_ptr())])
    torch.manual_seed(4)
    for dt in (torch.float16, torch.bfloat16):
        for rows, hidden in ((1, 4096), (4, 8192), (2, 896)):
            h = (torch.randn(rows, hidden) * 2).to(dt).cuda()
            part = torch.randn(rows, hidden).to(dt).cuda()
            w = (1 + 0.1 * torch.randn(hidden)).to(dt).cuda()
            h_ref = h.clone()
            y_ref = ds.rmsnorm(h_ref, part, w, 1e-5)
            for _ in range(3):                                       # both buffer halves
                h_got = h.clone()
                y_got = comm.allreduce_rmsnorm(part, h_got, w, 1e-5)
                assert torch.equal(h_got, h_ref) and torch.equal(y_got, y_ref), (dt, rows, hidden)
    v = torch.randn(4096, device="cuda").half()
    v2 = v.clone()
    comm(v2)
    assert torch.equal(v, v2)
    h = torch.randn(1, 4096, device="cuda").half()
    part, w = torch.randn(1, 4096, device="cuda").half(), torch.ones(4096, device="cuda").half()
    static_h = h.clone()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.allreduce_rmsnorm(part, static_h, w, 1e-5)
    torch.cuda.current_stream().wait_stream(s)
    static_h.copy_(h)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = comm.allreduce_rmsnorm(part, static_h, w, 1e-5)
    g.replay()
    torch.cuda.synchronize()
    h_ref = h.clone()
    assert torch.equal(y, ds.rmsnorm(h_ref, part, w, 1e-5)) and torch.equal(static_h, h_ref) and comm.status() == 0
    with pytest.raises(ValueError):
        comm.allreduce_rmsnorm(torch.zeros(8, 8192, device="cuda").half(), torch.zeros(8, 8192, device="cuda").half(),
                               torch.ones(8192, device="cuda").half(), 1e-5)      # 8 x 8192 elements exceed a slot
    comm.close()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_in_turns_and_the_wait_that_runs_out(world):
    """All ranks of a group on one device, one after the other (2 ranks: tagged words; 4 ranks: data + flags).
    Whoever goes before the last finds partners missing: its bounded wait runs out, the status word says so,
    nothing hangs.  The rank that goes last finds everybody's vector in place and must produce the exact sum."""
    n = 8192
    bufs = [_buffers(world, n) for _ in range(world)]
    peers = [(b[0].data_ptr(), b[1].data_ptr()) for b in bufs]
    # a short wait limit: a rank without partners gives up after ~100 probes instead of a second
    ranks = [OneShotAllReduce(rank=r, world=world, max_elems=n, peers=peers, wait_limit=100) for r in range(world)]
    g = torch.Generator(device="cuda").manual_seed(3)
    for rnd in range(4):                            # alternates the buffer halves; the order of the ranks rotates
        xs = [torch.randn(n, generator=g, device="cuda").half() for _ in range(world)]
        acc = torch.zeros(n, device="cuda")
        for x in xs:                                # rank order, fp32: what the kernel computes
            acc = acc + x.float()
        want = acc.half()
        order = [(rnd + i) % world for i in range(world)]
        ys = [x.clone() for x in xs]
        for r in order[:-1]:
            ranks[r](ys[r])
            torch.cuda.synchronize()                # the launch ended by itself although partners never came
            assert ranks[r].status() == 1           # ... and reported the wait that ran out
            assert ranks[r].status() == 0           # reading clears the word
        last = order[-1]
        ranks[last](ys[last])
        torch.cuda.synchronize()
        assert ranks[last].status() == 0            # every partner's vector was already there
        assert torch.equal(ys[last], want), rnd
    # the device is as usable as before
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    for r in ranks:
        r.close()


def _two_gpu_rank(rank, world, port, ret):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        comm = OneShotAllReduce(max_elems=4 * 8192)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        ok = True
        for n in (8, 1024, 8192, 4 * 8192):
            for dt in (torch.float16, torch.bfloat16):
                for _ in range(20):
                    x = torch.randn(n, generator=g, device="cuda").to(dt)
                    every = [torch.empty_like(x) for _ in range(world)]
                    dist.all_gather(every, x)
                    want = sum(e.float() for e in every).to(dt)       # rank order, fp32: what the kernel computes
                    y = x.clone()
                    comm(y)
                    ok = ok and bool(torch.equal(y, want))
        # the all-reduce fused with the residual update and RMS norm against NCCL + the plain kernels
        from ai_accel_studio_b200 import decode_step as ds
        for rows, hidden in ((1, 8192), (4, 4096), (2, 896)):
            for dt in (torch.float16, torch.bfloat16):
                for _ in range(10):
                    part = torch.randn((rows, hidden), generator=g, device="cuda").to(dt)
                    h = torch.randn((rows, hidden), generator=torch.Generator(device="cuda").manual_seed(7), device="cuda").to(dt)
                    w = torch.ones(hidden, device="cuda").to(dt)
                    every = [torch.empty_like(part) for _ in range(world)]
                    dist.all_gather(every, part)
                    delta = sum(e.float() for e in every).to(dt)
                    h_ref = h.clone()
                    y_ref = ds.rmsnorm(h_ref, delta, w, 1e-6)
                    h_got = h.clone()
                    y_got = comm.allreduce_rmsnorm(part, h_got, w, 1e-6)
                    ok = ok and bool(torch.equal(h_got, h_ref)) and bool(torch.equal(y_got, y_ref))
        # captured in a graph together with a producer kernel
        static = torch.zeros(8192, device="cuda").half()
        src = torch.randn(8192, generator=g, device="cuda").half()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            static.copy_(src)
            comm(static)
        torch.cuda.current_stream().wait_stream(s)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            static.copy_(src)
            comm(static)
        every = [torch.empty_like(src) for _ in range(world)]
        dist.all_gather(every, src)
        want = sum(e.float() for e in every).half()
        for _ in range(30):
            graph.replay()
        torch.cuda.synchronize()
        ok = ok and bool(torch.equal(static, want)) and comm.status() == 0
        ret[rank] = ok
        dist.barrier()
        comm.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus_match_nccl():
    import torch.multiprocessing as mp
    world = min(4, torch.cuda.device_count())
    port = 32500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_two_gpu_rank, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}


def _tp_rank(rank, world, port, ret):
    """One packed q/o-style pair sharded over the ranks: row shards need no communication, column
    shards end in AllReduceLinear (NCCL, then the one-shot kernel), eagerly and inside a CUDA graph."""
    import numpy as np
    import torch.distributed as dist
    from torch import nn
    from ai_accel_studio_b200 import tp
    from ai_accel_studio_b200.optimize import HybridInt2Linear, HybridInt4Linear
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        ok = True
        torch.manual_seed(21)                                   # the same unsharded modules on every rank
        n, k = 512, 2048
        for cls in (HybridInt2Linear, HybridInt4Linear):
            lin = nn.Linear(k, n, bias=True)
            with torch.no_grad():
                lin.weight.normal_(0, 0.02)
                lin.weight[:, torch.randperm(k)[:24]] *= 5
            full = cls(lin, 128, None, 16)
            full.set_residual(torch.randn(n, 8) * 0.02, torch.randn(8, k) * 0.02)
            x = torch.randn(2, k).half()
            want = full.cuda()(x.cuda()).float()
            rows = tp.shard_rows(full, rank, world).cuda()(x.cuda())
            every = [torch.empty_like(rows) for _ in range(world)]
            dist.all_gather(every, rows)
            ok = ok and bool((torch.cat(every, 1).float() - want).abs().max() <= 2e-3)
            ks = k // world
            col = tp.AllReduceLinear(tp.shard_cols(full, rank, world).cuda())
            xs = x[:, rank * ks:(rank + 1) * ks].contiguous().cuda()
            tol = 1e-2 + 1e-3 * float(want.abs().max()) + world * 2.0 ** -11 * float(want.abs().max())
            for one_shot in (False, True):
                tp.AllReduceLinear.one_shot = OneShotAllReduce(max_elems=8192) if one_shot else None
                y = col(xs)
                ok = ok and bool((y.float() - want).abs().max() <= tol)
                s = torch.cuda.Stream()
                s.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(s):
                    col(xs)
                torch.cuda.current_stream().wait_stream(s)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    yg = col(xs)
                for _ in range(5):
                    g.replay()
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(yg, y))
                if one_shot:
                    ok = ok and tp.AllReduceLinear.one_shot.status() == 0
                    dist.barrier()
                    tp.AllReduceLinear.one_shot.close()
                    tp.AllReduceLinear.one_shot = None
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_linear_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    port = 33500 + (os.getpid() % 2000)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_tp_rank, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {r: True for r in range(world)}
