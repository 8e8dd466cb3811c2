"""Decode throughput of a Llama-3-70B-shaped tensor-parallel decoder (random weights), tokens/s.

    python -m torch.distributed.run --nproc-per-node 8 -m gpu_ipc_example_b200.bench_decoder

80 layers, hidden 8192, 64 query / 8 KV heads of 128, SwiGLU FFN 28672, vocabulary 128256, RMSNorm
eps 1e-5, RoPE theta 5e5, fp16 N(0, 0.02) weights; batch 32, one new token per sequence at a
2048-token context, uniform random token ids.  Two fused all-reduce + RMSNorm per layer.

Each arm (`--arms`) builds the same model with a different way of doing the two all-reduces per layer
(see models/llama.py: "gemm", "allreduce", "nccl") and replays one decode step from a CUDA graph, so
the host is out of the picture; time is device time by CUDA events, max over ranks.  One JSON line per
arm: tokens/s = batch / step time, plus the weight-streaming floor (per-rank weight and KV bytes at the
measured HBM rate).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from gpu_ipc_example_b200 import Communicator
from gpu_ipc_example_b200.models.llama import LlamaConfig, LlamaTP


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--arms", nargs="*", default=["nccl", "allreduce", "gemm"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--no-kernels", action="store_true", help="plain PyTorch ops for RoPE / cache append / attention / SiLU*up")
    ap.add_argument("--pack", action="store_true", help="gemm arm: row-parallel weights packed by Communicator.pack_weight")
    ap.add_argument("--own-projections", nargs="?", const="both", default=None, choices=["both", "qkv", "gate_up"],
                    help="QKV and / or gate/up through the library's weight-streaming kernel instead of the framework's matmul")
    ap.add_argument("--breakdown", action="store_true", help="also time the stages of one eager step with CUDA events")
    ap.add_argument("--per-rank-shapes-of", type=int, default=0,
                    help="single-GPU dry run: use the per-rank shapes of this tensor-parallel degree with a world of one")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    multi = world > 1
    if multi:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = LlamaConfig.llama3_70b()
    cfg.layers = args.layers
    if args.per_rank_shapes_of:
        tp = args.per_rank_shapes_of
        cfg.n_heads //= tp
        cfg.n_kv_heads //= tp
        cfg.ffn //= tp
        cfg.vocab //= tp
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            hbm = float(json.load(f)["hbm_gbs"]) * 1e9
        peaks = "measured"
    except (OSError, KeyError, ValueError):
        hbm, peaks = 6.65e12, "fallback"

    g = torch.Generator(device="cuda").manual_seed(99)
    tokens = torch.randint(0, cfg.vocab, (args.batch,), device="cuda", generator=g)
    for arm in args.arms:
        if arm == "nccl" and not multi:
            continue
        comm = None
        if multi:
            comm = Communicator.from_torch_distributed(local, staging_bytes=256 << 20, device_seq=True)
        elif arm in ("gemm", "allreduce"):
            comm = Communicator.virtual(1, local, staging_bytes=256 << 20, device_seq=True)
        model = LlamaTP(cfg, comm, batch=args.batch, max_ctx=args.ctx, fusion=arm, seed=3,
                        kernels=False if args.no_kernels else None, pack_weights=args.pack,
                        local_gemm=True if args.own_projections == "both" else args.own_projections)
        model.pos = args.ctx - 1  # attend over a full context (the cache holds zeros: timing only)
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up: allocations, workspaces, cuBLAS heuristics
                model.pos = args.ctx - 1
                out = model.decode(tokens)
            stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            model.pos = args.ctx - 1
            with torch.cuda.graph(graph, stream=stream):
                out = model.decode(tokens)
            graph.replay()
            stream.synchronize()
            if multi:
                dist.barrier()
                torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(args.steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps * 1e-3], device="cuda", dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if comm is not None:
            comm.check()
        step = float(t.item())
        stages = None
        if args.breakdown:
            model.pos = args.ctx - 1
            model.stage_events = []
            with torch.cuda.stream(stream):
                model.decode(tokens)
                stream.synchronize()
            acc = {}
            for name, a, b in model.stage_events:
                acc[name] = acc.get(name, 0.0) + a.elapsed_time(b)
            stages = {k: round(v, 3) for k, v in acc.items()}  # ms per step, eager launches (host gaps included)
            model.stage_events = None
        kv_bytes = 2 * args.batch * model.hkv * args.ctx * cfg.head_dim * 2 * cfg.layers
        floor = (model.weight_bytes_per_rank() + kv_bytes) / hbm
        if rank == 0:
            print(json.dumps({
                "arm": arm, "world": world, "layers": cfg.layers, "batch": args.batch, "ctx": args.ctx,
                "ms_per_step": round(step * 1e3, 4), "tokens_per_s": round(args.batch / step, 1),
                "weight_and_kv_stream_floor_ms": round(floor * 1e3, 4), "fraction_of_floor": round(floor / step, 3),
                "kernels": bool(model.kernels), "packed_weights": bool(args.pack and arm == "gemm"),
                "stage_ms_eager": stages, "peaks": peaks, "next_token_sample": int(out[0]),
            }), flush=True)
        del model, graph
        if comm is not None:
            comm.close()
        torch.cuda.empty_cache()
    if multi:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
