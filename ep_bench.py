"""Multi-GPU leg of the benchmark: the expert-parallel MoE layer, one process per GPU.

Per rank: 65536 tokens (bf16 ~ N(0,1), hidden 7168), top-8 Zipf(1.2) routing over 256 experts
sharded 256/G per rank, MXFP8 weights ~ N(0, 0.02).  One step = the whole layer (quantise and
dispatch to the owning ranks, FC1 + SwiGLU, FC2 with gating, return of the result rows, top-k sum);
rows cross NVLink by peer stores from the kernels (default) or by NCCL all-to-all
(B200MOE_EP_PATH=nccl).  Experts are placed by load (default: an untimed observation of the routing
re-shards them once, weights move between ranks) or contiguously (B200MOE_EP_PLACEMENT=contiguous).  Weak scaling: tokens
per GPU are fixed.  FLOPs = 2 * routed rows * (N1 K1 + N2 K2) summed over ranks, true rows only.
"""

from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

EXPERTS, HIDDEN, INTER, TOPK = 256, 7168, 2048, 8


def _synthetic_tokens(tokens: int, dev, seed: int):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(tokens, HIDDEN, generator=g, device=dev).to(torch.bfloat16)
    rank_w = torch.arange(1, EXPERTS + 1, device=dev, dtype=torch.float32).pow(-1.2)
    perm = torch.randperm(EXPERTS, generator=torch.Generator(device=dev).manual_seed(7), device=dev)  # same on every rank
    w = torch.empty(EXPERTS, device=dev)
    w[perm] = rank_w
    ids = torch.multinomial(w.expand(tokens, EXPERTS), TOPK, replacement=False, generator=g).to(torch.int32)
    prob = torch.softmax(torch.randn(tokens, TOPK, generator=g, device=dev), dim=-1)
    return x, ids, prob


def layer_flops(tokens_total: int) -> float:
    return 2.0 * tokens_total * TOPK * (2 * INTER * HIDDEN + HIDDEN * INTER)


def single_gpu_layer(dev, steps: int = 5, warmup: int = 3, tokens: int = 65536) -> dict:
    """The same layer with all 256 experts on one GPU (no exchange): the like-for-like N = 1 point of
    the multi-GPU series."""
    from cudnn_frontend_b200 import synthetic
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    w1, sfw1 = synthetic.make_weights(EXPERTS, 2 * INTER, HIDDEN, 100, dev)
    w2, sfw2 = synthetic.make_weights(EXPERTS, HIDDEN, INTER, 200, dev)
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, EXPERTS, None)
    x, ids, prob = _synthetic_tokens(tokens, dev, 1000)
    for _ in range(warmup):
        layer.forward_fused(x, ids, prob)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        layer.forward_fused(x, ids, prob)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    layer.release_peer_buffers()
    return {"tflops": layer_flops(tokens) / (ms * 1e-3) / 1e12, "ms": ms, "tokens": tokens, "launches_per_step": 7}


def _step_roofline(tflops_per_gpu: float, peaks):
    """Whole step against the tensor roof: algorithmic FLOPs of FC1 + FC2 per GPU and step over the step
    time (the two GEMMs are about three quarters of a step), peak = twice the measured sustained bf16
    rate as for the single-GPU line."""
    if not peaks:
        return None
    peak = 2.0 * peaks["bf16_sustained"]
    return {"bound": "tensor", "achieved": tflops_per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": tflops_per_gpu / peak, "traffic": None,
            "kernel": "whole step per GPU (quantise+dispatch, FC1, FC2, combine)",
            "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS.json (dense fp8 proxy)"}  # fmt: skip


def _timed(step, steps, warmup, stream, barrier):
    """Warm-up, then `steps` calls between two events (barrier + synchronize on both sides), an event after
    every step too.  Returns (ms per step over the region, sorted single-step times)."""
    for _ in range(warmup):
        step()
    barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record(stream)
    for i in range(steps):
        step()
        ev[i + 1].record(stream)
    torch.cuda.synchronize()
    barrier()
    return ev[0].elapsed_time(ev[steps]) / steps, sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))


def run(args, tokens_per_gpu: int = 65536):
    from cudnn_frontend_b200 import synthetic
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

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

    x, ids, prob = _synthetic_tokens(tokens_per_gpu, dev, 1000 + rank)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(v):
        tns = torch.tensor([float(v)], device=dev)
        if world > 1:
            dist.all_reduce(tns, op=dist.ReduceOp.MAX)
        return tns.item()

    # data path: "peer" = rows cross NVLink by stores from the dispatch kernel and by device-to-device
    # copies of result rows, in expert chunks beside the GEMMs; "peer-direct" = one dispatch kernel, result
    # rows stored from the FC2 epilogue, nothing overlapped; "nccl" = all-to-all of rows
    path = os.environ.get("B200MOE_EP_PATH", "peer")
    micro = int(os.environ.get("B200MOE_EP_MICRO_BATCHES", "1"))

    def run_layer(xx, ii, pp, which=None):
        which = which or path
        if which == "peer":
            return layer.forward_fused(xx, ii, pp)
        if which == "peer-direct":
            return layer.forward_fused(xx, ii, pp, chunks=0)
        if which == "peer-chunked":
            return layer.forward_fused(xx, ii, pp, chunks=5)
        return layer.forward_pipelined(xx, ii, pp, micro) if micro > 1 else layer(xx, ii, pp)

    stream = torch.cuda.current_stream()
    steps, warmup = args.steps, max(args.warmup, 3)
    sampler = getattr(args, "clock_sampler", None)
    import contextlib

    def measure(which=None, with_clocks=False):
        with (sampler(local) if with_clocks and sampler is not None and rank == 0 else contextlib.nullcontext()) as clk:
            ms, per = _timed(lambda: run_layer(x, ids, prob, which), steps, warmup, stream, barrier)
        rows_recv = torch.tensor([float(layer.last_rows_received)], device=dev)
        rows_max = rows_recv.clone()
        if world > 1:
            dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
            dist.all_reduce(rows_recv, op=dist.ReduceOp.SUM)
        return dict(ms=max_over_ranks(ms), median_ms=max_over_ranks(per[len(per) // 2]), min_ms=max_over_ranks(per[0]),
                    rows_ratio=rows_max.item() / (rows_recv.item() / world), clk=None if clk is None else clk.summary())  # fmt: skip

    flops = layer_flops(tokens_per_gpu * world)
    placement = os.environ.get("B200MOE_EP_PLACEMENT", "balanced")
    side = {}
    if world > 1 and placement == "balanced" and not getattr(args, "no_extras", False):
        # the plain sharding (expert e on rank e // (E / G)) first, as a side measurement
        r = measure()
        side["contiguous_placement"] = {"ms_per_step": r["ms"], "tflops": flops / (r["ms"] * 1e-3) / 1e12,
                                        "rows_received_max_over_mean": r["rows_ratio"]}  # fmt: skip
    if world > 1 and placement == "balanced":
        # Load-aware placement, as production systems do it: the routing histogram of an EARLIER batch
        # (another seed than the batch that is timed), summed over ranks, re-shards the experts so that
        # every rank gets about the same number of rows; the weights move between the ranks once.
        _, ids_prev, _ = _synthetic_tokens(tokens_per_gpu, dev, 5000 + rank)
        hist = torch.bincount(ids_prev.reshape(-1).long(), minlength=EXPERTS).float()
        dist.all_reduce(hist)
        layer.rebalance(hist)
        del ids_prev

    # one untimed step through both data paths on the same inputs: the NCCL all-to-all path is the check
    y = run_layer(x, ids, prob)
    finite = bool(torch.isfinite(y.float()).all().item())
    matches = None
    if world > 1:
        y_nccl = layer(x, ids, prob)
        matches = bool(max_over_ranks(0.0 if torch.equal(y, y_nccl) else 1.0) == 0.0)
        del y_nccl

    chunks_used = layer.default_chunks() if path == "peer" else 0
    head = measure(with_clocks=True)
    ms = head["ms"]
    breakdown_path = os.environ.get("B200MOE_EP_BREAKDOWN")
    if breakdown_path and world > 1 and path == "peer":
        # one extra step with a timing event at every phase boundary of the chunked peer path (caller's stream):
        # every rank writes its own list, "<path>.rank<r>"
        form = None if chunks_used > 0 else "peer-chunked"  # the events sit in the chunked form
        run_layer(x, ids, prob, form)  # untimed: side streams and operators of this form exist afterwards
        layer.step_events = []
        dist.barrier()
        torch.cuda.synchronize()
        run_layer(x, ids, prob, form)
        torch.cuda.synchronize()
        evs = layer.step_events
        layer.step_events = None
        rows = [{"phase": evs[i][0], "ms": evs[i - 1][1].elapsed_time(evs[i][1])} for i in range(1, len(evs))]
        total = evs[0][1].elapsed_time(evs[-1][1])
        with open(f"{breakdown_path}.rank{rank}", "w") as f:
            json.dump({"rank": rank, "world": world, "rows_received": int(layer.last_rows_received), "total_ms": total, "phases": rows}, f, indent=1)
    value = flops / (ms * 1e-3) / 1e12
    if world > 1 and path == "peer" and not getattr(args, "no_extras", False):
        # the other form of the peer path beside the default one
        if chunks_used > 0:
            r = measure("peer-direct")
            side["peer_direct_path"] = {"ms_per_step": r["ms"], "tflops": flops / (r["ms"] * 1e-3) / 1e12,
                                        "what": "one dispatch kernel, result rows stored over NVLink from the FC2 epilogue, no overlap"}  # fmt: skip
        else:
            r = measure("peer-chunked")
            side["peer_chunked_path"] = {"ms_per_step": r["ms"], "tflops": flops / (r["ms"] * 1e-3) / 1e12,
                                         "what": "5 expert chunks, result copies beside the GEMMs"}  # fmt: skip

    # end to end: tokens, expert ids and gate probabilities start in pinned host memory every step and the
    # layer's output goes back to pinned host memory; the transfers overlap the neighbouring steps (a copy
    # stream per direction, two buffers each, events both ways)
    x_h, ids_h, prob_h = x.cpu().pin_memory(), ids.cpu().pin_memory(), prob.cpu().pin_memory()
    in_bufs = [(torch.empty_like(x), torch.empty_like(ids), torch.empty_like(prob)) for _ in range(2)]
    out_bufs = [torch.empty((tokens_per_gpu, HIDDEN), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    out_h = [torch.empty((tokens_per_gpu, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    computed = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]
    step_no = [0]

    def start_copy(i):
        x_d, ids_d, prob_d = in_bufs[i % 2]
        with torch.cuda.stream(h2d_stream):
            if i >= 2:
                h2d_stream.wait_event(consumed[i % 2])
            x_d.copy_(x_h, non_blocking=True)
            ids_d.copy_(ids_h, non_blocking=True)
            prob_d.copy_(prob_h, non_blocking=True)
            copied[i % 2].record(h2d_stream)

    def e2e_step():
        i = step_no[0]
        if i == 0:
            start_copy(0)
        start_copy(i + 1)
        x_d, ids_d, prob_d = in_bufs[i % 2]
        stream.wait_event(copied[i % 2])
        out = run_layer(x_d, ids_d, prob_d)
        consumed[i % 2].record(stream)
        if i >= 2:
            stream.wait_event(drained[i % 2])
        out_bufs[i % 2].copy_(out)
        computed[i % 2].record(stream)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(computed[i % 2])
            out_h[i % 2].copy_(out_bufs[i % 2], non_blocking=True)
            drained[i % 2].record(d2h_stream)
        step_no[0] = i + 1

    e2e_steps = max(steps // 4, 3)
    for _ in range(2):
        e2e_step()
    barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    stream.wait_stream(d2h_stream)  # the last outputs have reached the host
    stop.record(stream)
    torch.cuda.synchronize()
    barrier()
    ms_e2e = max_over_ranks(start.elapsed_time(stop) / e2e_steps)
    e2e_same = bool(max_over_ranks(0.0 if torch.equal(out_h[(step_no[0] - 1) % 2], y.cpu()) else 1.0) == 0.0)
    h2d = x_h.numel() * 2 + ids_h.numel() * 4 + prob_h.numel() * 4
    d2h = out_h[0].numel() * 2
    if rank == 0:
        line = {
            "metric": "MXFP8 grouped-GEMM+SwiGLU TFLOP/s",
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": ms,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp8_e4m3 x ue8m0 block scales, f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": f"expert-parallel MoE layer: E=256 sharded {e_local}/GPU, hidden 7168, intermediate 2048, {tokens_per_gpu} tokens/GPU top-8 Zipf(1.2); one step = quantise + dispatch to the owning ranks, FC1 + SwiGLU, FC2 with gating, return + top-k sum",
                "parallelism": f"ep{world}",
                "data_path": {"peer": (f"peer stores over NVLink from the quantise+dispatch kernel, result rows returned by device-to-device copies beside the GEMMs of {chunks_used} expert chunks"
                                       if chunks_used > 0 else "peer stores over NVLink from the quantise+dispatch kernel and from the FC2 epilogue (the default on two ranks)"),
                              "peer-direct": "peer stores over NVLink from the quantise+dispatch kernel and from the FC2 epilogue; nothing overlapped",
                              "nccl": f"NCCL all-to-all, {micro} micro-batch(es)"}[path],
                "l2": "inputs larger than L2 (0.94 GB tokens, 11 GB local weights), no flush",
                "expert_placement": (placement + " (histogram of an earlier batch, another seed than the timed one)" if placement == "balanced" else placement) if world > 1 else "single rank",
                "rows_received_max_over_mean": head["rows_ratio"],
                "pct_of_fp8_nominal_4500_per_gpu": 100.0 * value / world / 4500.0,
                "output_finite": finite,
                "output_matches_nccl_path": matches,
            },
            "timing": {"median_ms": head["median_ms"], "min_ms": head["min_ms"], "steps": steps},
            "gpu_launches": steps * ((6 + 3 * chunks_used if chunks_used > 0 else 7) if path != "nccl" else 5 * micro),
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e, "steps": e2e_steps, "output_on_host_matches": e2e_same,
                    "note": "bytes are one rank's, the value is the aggregate over ranks; inputs of step i + 1 and the output of step i - 1 travel while step i computes; the region ends when the last output is on the host"},
            "roofline": _step_roofline(value / world, getattr(args, "peaks", None)),
            "clocks": head["clk"],
            "cpu_baseline": None,
            "extras": side,
        }  # fmt: skip
        print(json.dumps(line))
    layer.release_peer_buffers()
    if world > 1:
        dist.destroy_process_group()
