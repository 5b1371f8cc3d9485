"""Benchmark of the MXFP8 MoE grouped-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 (default): one step = one FC1 call (MXFP8 grouped GEMM + SwiGLU, bf16 D + per-expert amax)
on the Mixtral-shape configuration (E=8, K=4096, N=2x14336, 16384 tokens top-2 -> 32768 routed
rows, groups padded to 128), inputs resident in HBM.  FLOPs = 2 * routed rows * N * K (no
padding counted).  N > 1 (under torchrun): one step = the expert-parallel MoE layer (all-to-all
dispatch, quantise, FC1, FC2, all-to-all combine) with 65536 tokens per GPU.

`--impl reference` times the CPU restatement of the reference's PyTorch implementation of the
same path (oracle/) on the host cores on a bounded sample of the same workload.

Prints one JSON line (rank 0).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "MXFP8 grouped-GEMM+SwiGLU TFLOP/s"
# reduced Mixtral-shape case for profiler captures: same K, a quarter of N, a quarter of the rows;
# operands (A 33 MB + B 235 MB) still exceed the 126 MB L2
SMALL_CASE = dict(experts=8, k=4096, n=7168, tokens=4096, topk=2, routing="uniform")
UNIT = "TFLOP/s"
FP8_NOMINAL_TFLOPS = 4500.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    BAD = {
        0x8: "hw_slowdown",
        0x40: "hw_thermal_slowdown",
        0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap",
    }

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None

    def __enter__(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = None
            try:
                import torch

                uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid)
                h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)

            def loop():
                while not self._stop.is_set():
                    try:
                        self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        mask = pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)
                        for bit, name in self.BAD.items():
                            if mask & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(self.period)

            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
        except Exception:
            self._thread = None
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def time_steps(fn, steps, warmup, stream, barrier=None):
    """W untimed calls, then K calls bracketed by (barrier +) synchronize on both sides; CUDA
    events on the launching stream.  Returns milliseconds per step."""
    import torch

    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return start.elapsed_time(stop) / steps


# ---------------------------------------------------------------------------------------------
# CPU baseline (the oracle port of the reference's PyTorch implementation)
# ---------------------------------------------------------------------------------------------
def cpu_baseline_fc1(sample_experts=2, rows_per_expert=512, n=28672, k=4096, seed=0, repeats=1):
    import numpy as np
    import torch

    from oracle import mxfp8_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rng = np.random.default_rng(seed)
    m = sample_experts * rows_per_expert
    a = rng.integers(0, 256, (m, k), dtype=np.uint8)
    a[(a & 0x7F) == 0x7F] = 0  # no NaN encodings
    b = rng.integers(0, 256, (sample_experts, n, k), dtype=np.uint8)
    b[(b & 0x7F) == 0x7F] = 0
    sfa = rng.integers(118, 122, (m, k // 32), dtype=np.uint8)
    sfb = rng.integers(118, 122, (sample_experts, n, k // 32), dtype=np.uint8)
    offs = (np.arange(1, sample_experts + 1) * rows_per_expert).astype(np.int32)
    alpha = np.ones(sample_experts, dtype=np.float32)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.fc1_reference(a, sfa, b, sfb, offs, alpha, None)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    flops = 2.0 * m * n * k
    return {
        "value": flops / best / 1e12,
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": f"{sample_experts} experts x {rows_per_expert} rows of the Mixtral-shape FC1 (N={n}, K={k}), {best:.2f} s",
    }


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    vals = []
    base = None
    for _ in range(max(args.warmup, 0) + max(args.steps, 1)):
        base = cpu_baseline_fc1(sample_experts=1, rows_per_expert=256)
        vals.append(base["value"])
    vals = vals[max(args.warmup, 0) :]
    value = sum(vals) / len(vals)
    base["value"] = value
    flops_sample = 2.0 * 256 * 28672 * 4096
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": flops_sample / (value * 1e12) * 1e3,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "Mixtral-shape FC1 (E=8,K=4096,N=28672), CPU port of the reference's PyTorch implementation, sample of 1 expert x 256 rows per step"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# N = 1: Mixtral-shape FC1
# ---------------------------------------------------------------------------------------------
def bench_single(args):
    import torch

    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import moe, ops, synthetic

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream()
    peaks = load_peaks()
    cfg = synthetic.CONFIGS["c2"] if args.workload == "c2" else SMALL_CASE
    prob_ = synthetic.make_problem(cfg, dev, seed=0, m_aligned=128)
    e, n, k = cfg["experts"], cfg["n"], cfg["k"]
    m = prob_["m_rows"]
    flops = prob_["flops"]

    def make_full_op():
        """The output set of the reference's wrapper for fp8 inputs: C (bf16), D and D_col (E4M3), row
        and column scale factors."""
        d8 = torch.empty((m, n // 2, 1), dtype=torch.float8_e4m3fn, device=dev)
        dc8 = torch.empty((m, n // 2, 1), dtype=torch.float8_e4m3fn, device=dev)
        c = torch.empty((m, n, 1), dtype=torch.bfloat16, device=dev)
        sr, sc = ops.empty_sf(m, n // 2, 1, device=dev), ops.empty_sf(n // 2, m, 1, device=dev)
        norm = torch.ones(1, device=dev)
        op = cf.GroupedGemmSwigluSm100(prob_["a"], prob_["b"], c, d8, prob_["sfa"], prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                                       dc8, sample_sfd_row=sr, sample_sfd_col=sc, sample_norm_const=norm, sample_prob=prob_["prob"],
                                       sf_vec_size=32, m_aligned=128)  # fmt: skip
        assert op.check_support()
        op.compile()

        def step():
            op.execute(prob_["a"], prob_["b"], c, d8, prob_["sfa"], prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                       d_col_tensor=dc8, sfd_row_tensor=sr, sfd_col_tensor=sc, norm_const_tensor=norm, prob_tensor=prob_["prob"])  # fmt: skip

        return step, (c, d8, dc8, sr, sc)

    def make_op(write_c):
        d = torch.empty((m, n // 2, 1), dtype=torch.bfloat16, device=dev)
        c = torch.empty((m, n, 1), dtype=torch.bfloat16, device=dev) if write_c else None
        amax = torch.full((e, 1), float("-inf"), dtype=torch.float32, device=dev)
        op = cf.GroupedGemmSwigluSm100(prob_["a"], prob_["b"], c, d, prob_["sfa"], prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                                       None, sample_amax=amax, sample_prob=prob_["prob"], sf_vec_size=32, m_aligned=128)  # fmt: skip
        assert op.check_support()
        op.compile()

        def step():
            op.execute(prob_["a"], prob_["b"], c, d, prob_["sfa"], prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                       amax_tensor=amax, prob_tensor=prob_["prob"])  # fmt: skip

        return step, (c, d, amax)

    step, outs = make_full_op() if args.outputs == "full" else make_op(write_c=False)
    with ClockSampler(0) as clk:
        ms = time_steps(step, args.steps, args.warmup, stream)
    value = flops / (ms * 1e-3) / 1e12
    assert ops.device_status(clear=True) == 0, "a bounded wait inside the kernel gave up"
    if args.kernel_only:
        print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms, "steps": args.steps, "warmup": args.warmup,
                          "config": {"workload": f"kernel only, {args.workload}: {cfg}"}, "clocks": clk.summary()}))  # fmt: skip
        return

    # the same call with the bf16 pre-activation C also written, and with the full output set of the
    # reference's wrapper (C, E4M3 D and D_col, row and column scale factors)
    step_c, outs_c = make_op(write_c=True)
    ms_c = time_steps(step_c, max(args.steps // 2, 3), 3, stream)
    del outs_c, step_c
    step_f, outs_f = make_full_op()
    ms_full = time_steps(step_f, max(args.steps // 2, 3), 3, stream)
    del outs_f, step_f

    # ---- end to end through the public API from pinned host memory -------------------------
    # Every step copies its own inputs from pinned host memory and reads its result (per-expert amax)
    # back.  As in a serving loop, the copy of step i + 1 runs on a copy stream while step i computes:
    # two sets of device input buffers, events in both directions.
    routing = prob_["routing"]
    t, topk = routing.topk_ids.shape
    x_host = prob_["x"].cpu().pin_memory()
    ids_host = routing.topk_ids.cpu().pin_memory()
    p_host = routing.topk_prob.cpu().pin_memory()
    m_max = ((t * topk + e * 127 + 127) // 128) * 128
    in_bufs = [(torch.empty_like(prob_["x"]), torch.empty_like(routing.topk_ids), torch.empty_like(routing.topk_prob)) for _ in range(2)]
    xg = torch.empty((m_max, k), dtype=torch.bfloat16, device=dev)
    pg = torch.empty((m_max,), dtype=torch.float32, device=dev)
    aq = torch.empty((m_max, k), dtype=torch.float8_e4m3fn, device=dev)
    sfa = ops.empty_sf(m_max, k, 1, device=dev)
    d2 = torch.empty((m_max, n // 2, 1), dtype=torch.bfloat16, device=dev)
    amax2 = torch.full((e, 1), float("-inf"), dtype=torch.float32, device=dev)
    amax_host = torch.empty((e, 1), dtype=torch.float32).pin_memory()
    op2 = cf.GroupedGemmSwigluSm100(aq.view(m_max, k, 1), prob_["b"], None, d2, sfa, prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                                    None, sample_amax=amax2, sample_prob=pg.view(m_max, 1, 1), sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op2.check_support()
    op2.compile()
    copy_stream = torch.cuda.Stream()
    copied = [torch.cuda.Event() for _ in range(2)]  # inputs of the buffer have landed
    consumed = [torch.cuda.Event() for _ in range(2)]  # the step that read the buffer is done with it
    step_no = [0]

    def start_copy(i):
        x_dev, ids_dev, p_dev = in_bufs[i % 2]
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[i % 2])
            x_dev.copy_(x_host, non_blocking=True)
            ids_dev.copy_(ids_host, non_blocking=True)
            p_dev.copy_(p_host, non_blocking=True)
            copied[i % 2].record(copy_stream)

    def e2e_step():
        i = step_no[0]
        if i == 0:
            start_copy(0)
        start_copy(i + 1)  # the next step's inputs travel while this step computes
        x_dev, ids_dev, p_dev = in_bufs[i % 2]
        stream.wait_event(copied[i % 2])
        counts, offs, dst = moe.route(ids_dev, e, 128)
        moe.scatter_rows(x_dev, dst, xg, rows_per_src=topk, in_prob=p_dev.view(-1), out_prob=pg)
        moe.zero_pad_rows(xg, counts, offs, pg)
        ops.quantize_mxfp8_out(xg, aq, sfa)
        consumed[i % 2].record(stream)
        op2.execute(aq.view(m_max, k, 1), prob_["b"], None, d2, sfa, prob_["sfb"], offs, prob_["alpha"], amax_tensor=amax2,
                    prob_tensor=pg.view(m_max, 1, 1))  # fmt: skip
        amax_host.copy_(amax2, non_blocking=True)
        step_no[0] = i + 1

    ms_e2e = time_steps(e2e_step, max(args.steps // 2, 3), 3, stream)
    torch.cuda.synchronize()
    h2d = x_host.numel() * 2 + ids_host.numel() * 4 + p_host.numel() * 4
    e2e = {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": e * 4,
           "ms_per_step": ms_e2e, "launches_per_step": 7,
           "note": "host-to-device copy of step i + 1 overlaps the kernels of step i (copy stream, two input buffers)"}  # fmt: skip
    e2e_amax_ok = bool(torch.allclose(amax_host.view(-1), outs[2].cpu().view(-1), rtol=1e-5))

    # ---- quantiser bandwidth (the other new kernel of the path) -----------------------------
    xq = torch.randn(32768, 4096, device=dev).to(torch.bfloat16)
    q_out = torch.empty((32768, 4096), dtype=torch.float8_e4m3fn, device=dev)
    sf_out = ops.empty_sf(32768, 4096, 1, device=dev)
    ms_q = time_steps(lambda: ops.quantize_mxfp8_out(xq, q_out, sf_out), 20, 3, stream)
    q_bytes = 32768 * 4096 * (2 + 1 + 1 / 32)
    quant = {"gbs": q_bytes / (ms_q * 1e-3) / 1e9, "frac_of_measured_hbm": q_bytes / (ms_q * 1e-3) / 1e9 / peaks["hbm_gbs"], "shape": [32768, 4096]}
    del xq, q_out, sf_out

    extras = {"fc1_with_c_store_tflops": flops / (ms_c * 1e-3) / 1e12, "fc1_full_output_set_tflops": flops / (ms_full * 1e-3) / 1e12, "quantiser": quant, "e2e_amax_matches_resident_run": e2e_amax_ok}
    if not args.no_extras:
        del prob_, outs, op2, xg, aq, d2, in_bufs
        torch.cuda.empty_cache()
        extras.update(bench_other_configs(dev, stream))
        torch.cuda.empty_cache()
        import ep_bench

        # the workload of the multi-GPU runs (--gpus 2/4/8) with all experts on this GPU
        extras["ep_layer_1gpu"] = ep_bench.single_gpu_layer(dev)

    cpu = cpu_baseline_fc1()
    peak = 2.0 * peaks["bf16_sustained"]
    routed = t * topk
    prob_bytes = routed * k * (1 + 1 / 32) + e * n * k * (1 + 1 / 32) + routed * (n // 2) * 2
    line = {
        "metric": METRIC,
        "value": value,
        "unit": UNIT,
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp8_e4m3 x ue8m0 block scales, f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": "Mixtral-shape FC1: E=8, K=4096, N=2x14336, 16384 tokens top-2 uniform (32768 routed rows), groups padded to 128, bf16 D + per-expert amax",
            "l2": "inputs larger than L2 (A 134 MB + B 940 MB per step), no flush",
            "pct_of_fp8_nominal_4500": 100.0 * value / FP8_NOMINAL_TFLOPS,
        },
        "roofline": {
            "bound": "tensor",
            "achieved": value,
            "peak": peak,
            "unit": UNIT,
            "frac": value / peak,
            # HBM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum) from the one-pass ncu
            # launch list of this same workload (profiles/bench_c2_launch_list.md); algorithmic bytes beside it
            "traffic": 1.60e9 + 0.93e9 if args.workload == "c2" else None,
            "traffic_unit": "bytes per launch (ncu, this workload)",
            "algorithmic_bytes": prob_bytes,
            "peak_source": f"2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS.json (dense fp8 proxy)",
            "kernel": "grouped_gemm_kernel<FC1, dense>",
        },
        "cpu_baseline": cpu,
        "e2e": e2e,
        "gpu_launches": args.steps,
        "clocks": clk.summary(),
        "extras": extras,
    }
    print(json.dumps(line))


def bench_other_configs(dev, stream):
    """DeepSeek-shape FC1 (dense and discrete weights) and FC2; reported beside the headline."""
    import torch

    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops, synthetic

    out = {}
    p3 = synthetic.make_problem("c3", dev, seed=1, m_aligned=128)
    cfg = p3["cfg"]
    e, n, k, m = cfg["experts"], cfg["n"], cfg["k"], p3["m_rows"]
    d8 = torch.empty((m, n // 2, 1), dtype=torch.float8_e4m3fn, device=dev)
    sfd_row = ops.empty_sf(m, n // 2, 1, device=dev)
    norm = torch.ones(1, device=dev)
    dbf = torch.empty((m, n // 2, 1), dtype=torch.bfloat16, device=dev)
    amax = torch.full((e, 1), float("-inf"), dtype=torch.float32, device=dev)
    op = cf.GroupedGemmSwigluSm100(p3["a"], p3["b"], None, dbf, p3["sfa"], p3["sfb"], p3["padded_offsets"], p3["alpha"], None,
                                   sample_amax=amax, sample_prob=None, sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op.check_support()
    op.compile()
    ms = time_steps(lambda: op.execute(p3["a"], p3["b"], None, dbf, p3["sfa"], p3["sfb"], p3["padded_offsets"], p3["alpha"], amax_tensor=amax), 10, 3, stream)
    active = int((p3["routing"].counts > 0).sum().item())
    bytes3 = p3["routing"].routed_rows * k * (1 + 1 / 32) + active * n * k * (1 + 1 / 32) + p3["routing"].routed_rows * (n // 2) * 2
    out["deepseek_fc1_dense"] = {"tflops": p3["flops"] / (ms * 1e-3) / 1e12, "ms": ms, "gbs": bytes3 / (ms * 1e-3) / 1e9, "padded_rows": m, "active_experts": active}

    # discrete weights: one allocation per expert
    b_store = p3["b"].permute(2, 0, 1)  # [E, n, k]
    sf_flat = torch.as_strided(p3["sfb"].view(torch.uint8), (p3["sfb"].numel(),), (1,))
    per = sf_flat.numel() // e
    b_list = [b_store[i].clone() for i in range(e)]
    sf_list = [sf_flat[i * per : (i + 1) * per].clone() for i in range(e)]
    b_ptrs = torch.tensor([x.data_ptr() for x in b_list], dtype=torch.int64, device=dev)
    sfb_ptrs = torch.tensor([x.data_ptr() for x in sf_list], dtype=torch.int64, device=dev)
    opd = cf.DiscreteGroupedGemmSwigluSm100(p3["a"], e, (n, k), torch.float8_e4m3fn, None, dbf, p3["sfa"], p3["padded_offsets"], p3["alpha"], None,
                                            sample_amax=amax, sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert opd.check_support()
    opd.compile()
    ms_d = time_steps(lambda: opd.execute(p3["a"], b_ptrs, None, dbf, p3["sfa"], sfb_ptrs, p3["padded_offsets"], p3["alpha"], amax_tensor=amax), 10, 3, stream)
    out["deepseek_fc1_discrete"] = {"tflops": p3["flops"] / (ms_d * 1e-3) / 1e12, "ms": ms_d}
    del b_list, sf_list, opd

    # FC1 with MXFP8 output feeds FC2
    d_col = None
    op8 = cf.GroupedGemmSwigluSm100(p3["a"], p3["b"], None, d8, p3["sfa"], p3["sfb"], p3["padded_offsets"], p3["alpha"], d8,
                                    sample_sfd_row=sfd_row, sample_sfd_col=ops.empty_sf(n // 2, m, 1, device=dev), sample_norm_const=norm,
                                    sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op8.check_support()
    op8.compile()
    op8.execute(p3["a"], p3["b"], None, d8, p3["sfa"], p3["sfb"], p3["padded_offsets"], p3["alpha"], sfd_row_tensor=sfd_row, norm_const_tensor=norm)
    del p3["b"], p3["sfb"], b_store, sf_flat
    torch.cuda.empty_cache()
    cfg4 = synthetic.CONFIGS["c4"]
    n4, k4 = cfg4["n"], cfg4["k"]
    w2, sfw2 = synthetic.make_weights(e, n4, k4, 7, dev)
    d4 = torch.empty((m, n4, 1), dtype=torch.float8_e4m3fn, device=dev)
    sfd4 = ops.empty_sf(m, n4, 1, device=dev)
    op4 = cf.GroupedGemmQuantSm100(d8, sfd_row, p3["padded_offsets"], p3["alpha"], d4, sample_d_col=d4, sample_b=w2, sample_sfb=sfw2,
                                   sample_sfd_row=sfd4, sample_sfd_col=ops.empty_sf(n4, m, 1, device=dev), sample_norm_const=norm,
                                   sample_prob=p3["prob"], sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op4.check_support()
    op4.compile()
    ms4 = time_steps(lambda: op4.execute(d8, sfd_row, p3["padded_offsets"], p3["alpha"], d4, b_tensor=w2, sfb_tensor=sfw2, sfd_row_tensor=sfd4,
                                         norm_const_tensor=norm, prob_tensor=p3["prob"]), 10, 3, stream)  # fmt: skip
    flops4 = 2.0 * p3["routing"].routed_rows * n4 * k4
    bytes4 = p3["routing"].routed_rows * k4 * (1 + 1 / 32) + active * n4 * k4 * (1 + 1 / 32) + p3["routing"].routed_rows * n4 * (1 + 1 / 32)
    out["deepseek_fc2_quant"] = {"tflops": flops4 / (ms4 * 1e-3) / 1e12, "ms": ms4, "gbs": bytes4 / (ms4 * 1e-3) / 1e9}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the DeepSeek-shape side measurements")
    ap.add_argument("--workload", default="c2", choices=["c2", "small"], help="c2 = Mixtral-shape FC1 (the benchmark); small = reduced case for profiler captures")
    ap.add_argument("--outputs", default="d", choices=["d", "full"], help="with --kernel-only: d = bf16 D + amax (the benchmark); full = C + E4M3 D + D_col + scale factors")
    ap.add_argument("--kernel-only", action="store_true", help="time the FC1 kernel only (no end-to-end, CPU baseline or side measurements)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "own" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        import ep_bench

        args.peaks = load_peaks()
        args.clock_sampler = ClockSampler
        ep_bench.run(args)
    else:
        bench_single(args)


if __name__ == "__main__":
    main()
