"""Multi-GPU leg of the benchmark: the expert-parallel MoE layer, one process per GPU.

Per rank: 65536 tokens (bf16 ~ N(0,1), hidden 7168), top-8 Zipf(1.2) routing over 256 experts
sharded 256/G per rank, MXFP8 weights ~ N(0, 0.02).  One step = the whole layer (dispatch
all-to-all, quantise, FC1 + SwiGLU, FC2 with gating, combine all-to-all).  Weak scaling: tokens
per GPU are fixed.  FLOPs = 2 * routed rows * (N1 K1 + N2 K2) summed over ranks, true rows only.
"""

from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

EXPERTS, HIDDEN, INTER, TOPK = 256, 7168, 2048, 8


def run(args, tokens_per_gpu: int = 65536):
    from . import synthetic
    from .ep_layer import ExpertParallelMoE

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    e_local = EXPERTS // world
    w1, sfw1 = synthetic.make_weights(e_local, 2 * INTER, HIDDEN, 100 + rank, dev)
    w2, sfw2 = synthetic.make_weights(e_local, HIDDEN, INTER, 200 + rank, dev)
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, EXPERTS, group)

    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn(tokens_per_gpu, HIDDEN, generator=g, device=dev).to(torch.bfloat16)
    rank_w = torch.arange(1, EXPERTS + 1, device=dev, dtype=torch.float32).pow(-1.2)
    perm = torch.randperm(EXPERTS, generator=torch.Generator(device=dev).manual_seed(7), device=dev)  # same on every rank
    w = torch.empty(EXPERTS, device=dev)
    w[perm] = rank_w
    ids = torch.multinomial(w.expand(tokens_per_gpu, EXPERTS), TOPK, replacement=False, generator=g).to(torch.int32)
    prob = torch.softmax(torch.randn(tokens_per_gpu, TOPK, generator=g, device=dev), dim=-1)

    def barrier():
        if world > 1:
            dist.barrier()

    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        y = layer(x, ids, prob)
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(args.steps):
        y = layer(x, ids, prob)
    stop.record(stream)
    torch.cuda.synchronize()
    barrier()
    ms = torch.tensor([start.elapsed_time(stop) / args.steps], device=dev)
    rows_recv = torch.tensor([float(layer.last_plan.rows_received)], device=dev)
    rows_max = rows_recv.clone()
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
        dist.all_reduce(rows_recv, op=dist.ReduceOp.SUM)
    ms = ms.item()
    total_rows = tokens_per_gpu * TOPK * world
    flops = 2.0 * total_rows * (2 * INTER * HIDDEN + HIDDEN * INTER)
    value = flops / (ms * 1e-3) / 1e12
    finite = bool(torch.isfinite(y.float()).all().item())
    if rank == 0:
        line = {
            "metric": "MXFP8 grouped-GEMM+SwiGLU TFLOP/s",
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp8_e4m3 x ue8m0 block scales, f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": f"expert-parallel MoE layer: E=256 sharded {e_local}/GPU, hidden 7168, intermediate 2048, {tokens_per_gpu} tokens/GPU top-8 Zipf(1.2); dispatch all-to-all + quantise + FC1 + FC2 + combine all-to-all",
                "parallelism": f"ep{world}",
                "l2": "inputs larger than L2 (0.94 GB tokens, 11 GB local weights), no flush",
                "rows_received_max_over_mean": rows_max.item() / (rows_recv.item() / world),
                "pct_of_fp8_nominal_4500_per_gpu": 100.0 * value / world / 4500.0,
                "output_finite": finite,
            },
            "gpu_launches": args.steps * 9,
            "e2e": None,
            "roofline": None,
            "cpu_baseline": None,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
