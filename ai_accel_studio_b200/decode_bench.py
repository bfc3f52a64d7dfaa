"""Whole-model greedy decode benchmark on random-init decoder shapes.

    python -m ai_accel_studio_b200.decode_bench --shape llama-3-8b --batch 1 --prompt 512 --new 128
    torchrun --nproc-per-node 8 -m ai_accel_studio_b200.decode_bench --shape llama-3-70b --probs 0.7 0.3 0.0 ...

Prints one JSON line per variant (mixed-bit packed modules, and the untouched fp16 model as the
cuBLAS comparator): decode tokens/s, TTFT, weight bytes per token and the bandwidth they imply.
Timing protocol: ai_accel_studio_b200.runtime_v5.generate_static_benchmark (StaticCache, explicit
CUDA graph of the decode step, CUDA events).  With more than one rank the model is tensor
parallel (one process per GPU, NCCL all-reduce inside the captured graph) and rank 0 prints.
"""
from __future__ import annotations

import argparse
import gc
import json
import os

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--new", type=int, default=128)
    ap.add_argument("--layers", type=int, default=None, help="truncate the model (for quick checks)")
    ap.add_argument("--probs", type=float, nargs=3, default=(0.6, 0.3, 0.1), help="P(INT2) P(INT4) P(FP16)")
    ap.add_argument("--variants", nargs="+", default=["mixed", "fp16"], choices=["mixed", "fp16"])
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--compile-layers", action="store_true",
                    help="fuse the non-GEMV work of each decoder layer with torch.compile (regional compilation)")
    ap.add_argument("--fuse-siblings", action="store_true",
                    help="merge q/k/v and gate/up projections that share bit width and group size into one launch each")
    ap.add_argument("--prefetch-hints", action="store_true",
                    help="announce the next Linear's weights to L2 while a packed GEMV runs (honoured by the mma_pipe kernel only)")
    ap.add_argument("--split", action="store_true",
                    help="also replay the decode step without the all-reduces / without the packed GEMVs and report their share")
    ap.add_argument("--replicated-lm-head", action="store_true",
                    help="tensor parallel: keep the whole output projection on every rank instead of vocab / world rows")
    ap.add_argument("--framework-step", action="store_true",
                    help="run the work between the GEMVs (norms, rotary embedding, attention, SwiGLU) with the framework's "
                         "operators instead of this package's decode-step kernels")
    ap.add_argument("--serial-kv", action="store_true",
                    help="do not launch the k and v projections on side streams beside q where the three are separate launches")
    ap.add_argument("--fused-reduce", action="store_true",
                    help="tensor parallel: fuse every all-reduce into the RMS normalisation that consumes its result")
    ap.add_argument("--nccl-all-reduce", action="store_true",
                    help="tensor parallel: all-reduce the K-split projections with NCCL instead of the one-shot peer-memory kernel")
    a = ap.parse_args()

    import torch.distributed as dist
    from ai_accel_studio_b200 import model_tools as mt

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if a.fused_reduce or a.serial_kv:
        from ai_accel_studio_b200.decode_step import NativeDecodeStep
        NativeDecodeStep.fuse_reduce = a.fused_reduce
        NativeDecodeStep.parallel_kv = not a.serial_kv
    for variant in a.variants:
        res = mt.decode_benchmark(a.shape, dev, a.batch, a.prompt, a.new, tuple(a.probs), variant == "mixed", world,
                                  a.layers, use_cuda_graph=not a.no_graph, compile_layers=a.compile_layers,
                                  fuse_siblings=a.fuse_siblings, split=a.split, shard_vocab=not a.replicated_lm_head,
                                  prefetch_hints=a.prefetch_hints, one_shot=not a.nccl_all_reduce, native_step=False if a.framework_step else None)
        if world > 1:
            t = torch.tensor([res["aggregate_decode_tokens_s"]], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)          # the slowest rank sets the pace
            res["aggregate_decode_tokens_s"] = float(t[0])
        if rank == 0:
            tps = res["aggregate_decode_tokens_s"]
            line = dict(shape=a.shape, variant=variant, world=world, batch=a.batch, prompt_tokens=a.prompt,
                        new_tokens=res["generated_tokens"], layers=a.layers, decode_tokens_s=tps,
                        ttft_ms=res["ttft_ms"], weight_bytes_per_rank=res["total"], packed_bytes=res["packed_bytes"],
                        fp16_bytes=res["fp16_bytes"],
                        weight_GBps_per_gpu=res["total"] * tps / a.batch / 1e9,
                        peak_vram_gb=res.get("peak_vram_gb"), cuda_graph=not a.no_graph,
                        compiled_layers=a.compile_layers, fused_sibling_groups=res.get("fused_sibling_groups", 0),
                        all_reduces_per_token=res.get("all_reduces_per_token"), packed_gemvs_per_token=res.get("packed_gemvs_per_token"),
                        lm_head_rows_per_rank=res.get("lm_head_rows_per_rank"), all_reduce_impl=res.get("all_reduce_impl"), decode_step=res.get("decode_step"),
                        one_shot_status=res.get("one_shot_status"), split_ms_per_token=res.get("split_ms_per_token"))
            print(json.dumps(line), flush=True)
        del res
        gc.collect()
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
