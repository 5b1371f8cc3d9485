"""Benchmark of the MXFP8 MoE grouped-GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1 (default): one step = one FC1 call (MXFP8 grouped GEMM + SwiGLU, bf16 D + per-expert amax)
on the Mixtral-shape configuration (E=8, K=4096, N=2x14336, 16384 tokens top-2 -> 32768 routed
rows, groups padded to 128), inputs resident in HBM.  FLOPs = 2 * routed rows * N * K (no
padding counted).  N > 1 (under torchrun): one step = the expert-parallel MoE layer (quantise +
dispatch, FC1, FC2, return, top-k sum) with 65536 tokens per GPU.

The K timed steps run back to back between two events; an event after every step also gives the
median and the minimum step.  A second region of at least two seconds gives the sustained figure
with the SM clock sampled over it.  Every side measurement follows the reference's protocol
(test/python/sdpa/helpers.py:399-441): 3 warm-ups, 10 trials with an L2 flush between them,
median and best.

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
# reduced DeepSeek-shape case for profiler captures: Zipf rows over 64 experts of the full K and N
# (weights 64 x 29 MB = 1.9 GB: far larger than L2)
DEEPSEEK_SMALL_CASE = dict(experts=64, k=7168, n=4096, tokens=2048, topk=8, routing="zipf")
UNIT = "TFLOP/s"
FP8_NOMINAL_TFLOPS = 4500.0
WORKLOAD = ("Mixtral-shape FC1: E=8, K=4096, N=2x14336, 16384 tokens top-2 uniform (32768 routed rows), groups padded to 128, "
            "bf16 D + per-expert amax")  # fmt: skip
SUSTAINED_SECONDS = 2.0


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def load_traffic(key):
    """HBM bytes per launch of a kernel on a workload, as recorded beside its profile summary
    (profiles/traffic.json: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture)."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            entry = json.load(f).get(key)
        return None if entry is None else float(entry["dram_bytes_read"]) + float(entry["dram_bytes_write"])
    except (OSError, ValueError, KeyError, TypeError):
        return None


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
    """W untimed calls, then K calls bracketed by (barrier +) synchronize on both sides; CUDA events
    on the launching stream, one after every step as well.  Returns (milliseconds per step over the
    whole region, statistics of the single steps)."""
    import torch

    for _ in range(warmup):
        fn()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    ev[0].record(stream)
    for i in range(steps):
        fn()
        ev[i + 1].record(stream)
    torch.cuda.synchronize()
    if barrier:
        barrier()
    per = sorted(ev[i].elapsed_time(ev[i + 1]) for i in range(steps))
    return ev[0].elapsed_time(ev[steps]) / steps, {"median_ms": per[len(per) // 2], "min_ms": per[0], "max_ms": per[-1], "steps": steps}


_FLUSH = {}


def time_trials(fn, stream, trials=10, warmup=3, repeat=1):
    """The reference's timing protocol: `warmup` untimed calls, then `trials` timed ones with a 256 MiB
    write between them so that nothing of the previous trial stays in L2; `repeat` calls per trial for
    kernels too short to time alone.  Returns {"median_ms", "min_ms", "trials"} per call."""
    import torch

    dev = torch.cuda.current_device()
    if dev not in _FLUSH:
        _FLUSH[dev] = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(trials):
        _FLUSH[dev].zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        for _ in range(repeat):
            fn()
        e.record(stream)
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e) / repeat)
    times.sort()
    return {"median_ms": times[len(times) // 2], "min_ms": times[0], "trials": trials}


def time_sustained(fn, stream, ms_per_step, seconds, device_index):
    """Back-to-back calls for at least `seconds`, with the SM clock sampled over the region."""
    import torch

    steps = max(int(seconds * 1e3 / max(ms_per_step, 1e-3)) + 1, 10)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(device_index) as clk:
        s.record(stream)
        for _ in range(steps):
            fn()
        e.record(stream)
        torch.cuda.synchronize()
    return s.elapsed_time(e) / steps, steps, clk.summary()


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


def cpu_baseline_c1(repeats=3):
    """Configuration c1 (E=4, K=256, N=1024, 512 tokens top-1, groups padded to 256) at full size through
    the oracle port, unit scale factors as in the reference's bf16 path; best of `repeats`."""
    import numpy as np
    import torch

    from oracle import mxfp8_oracle as orc

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    rng = np.random.default_rng(1)
    e, k, n, t = 4, 256, 1024, 512
    ids = rng.integers(0, e, t)
    counts, offs, dst = orc.route_rows(ids, e, 256)
    m = int(offs[-1])
    a = np.zeros((m, k), dtype=np.uint8)
    a[dst] = rng.integers(0, 120, (t, k), dtype=np.uint8)
    b = rng.integers(0, 120, (e, n, k), dtype=np.uint8)
    sfa = np.full((m, k // 32), 127, dtype=np.uint8)  # scale factors of one
    sfb = np.full((e, n, k // 32), 127, dtype=np.uint8)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.fc1_reference(a, sfa, b, sfb, offs, np.ones(e, dtype=np.float32), None)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": 2.0 * t * n * k / best / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "seconds": best,
            "sample": "configuration c1 at full size (512 routed rows, padded to 256 per expert), best of 3"}  # fmt: skip


def reference_gpu_kernel():
    """The reference's own FC1 GPU kernel (its CuTe-DSL grouped_gemm_swiglu_wrapper_sm100, JIT-compiled from the
    overlay under baseline/_ref) on the benchmark's configuration, timed with the reference's protocol: 3 warm-ups,
    10 trials with an L2 flush, median and best.  Inputs are made with plain torch (nothing of this package runs):
    E4M3 operands of N(0, 1) values scaled to the E4M3 range, unit scale factors, 16384 tokens top-2 uniform, groups
    padded to 256 (the only alignment the reference accepts), full output set (C, E4M3 D and D_col, scales).
    Returns None where the overlay, a GPU or the CuTe DSL is missing; only ever run in a 1-GPU process."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "cudnn")) or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return None
    try:
        import torch

        if not torch.cuda.is_available():
            return None
        sys.path.insert(0, ref_dir)
        try:
            import cuda.bindings.driver as cuda
            import cudnn as ref
        finally:
            sys.path.remove(ref_dir)
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        e, k, n, tokens, topk = 8, 4096, 28672, 16384, 2
        g = torch.Generator(device=dev).manual_seed(0)
        ids = torch.multinomial(torch.ones(tokens, e, device=dev), topk, replacement=False, generator=g)
        counts = torch.bincount(ids.reshape(-1), minlength=e)
        padded = (counts + 255) // 256 * 256
        offsets = torch.cumsum(padded, 0).to(torch.int32)
        m = int(offsets[-1].item())
        a = (torch.randn(m, k, generator=g, device=dev) * 100.0).clamp_(-448, 448)
        starts = offsets.long() - padded
        rows = torch.arange(m, device=dev)
        owner = torch.searchsorted(offsets.long(), rows, right=True).clamp(max=e - 1)
        a[(rows - starts[owner]) >= counts[owner]] = 0  # padding rows of every group are zero
        a = torch.as_strided(a.to(torch.float8_e4m3fn), (m, k, 1), (k, 1, m * k))
        b = torch.empty((e, n, k), dtype=torch.float8_e4m3fn, device=dev)
        for i in range(e):
            b[i] = (torch.randn(n, k, generator=g, device=dev) * 100.0).clamp_(-448, 448).to(torch.float8_e4m3fn)
        b = b.permute(1, 2, 0)

        def unit_sf(mn, l):  # 128x4 layout, every scale 2^-7
            rm, rk = (mn + 127) // 128, (k // 32 + 3) // 4
            flat = torch.full((l * rm * rk * 512,), 120, dtype=torch.uint8, device=dev)
            return torch.as_strided(flat.view(torch.float8_e8m0fnu), (32, 4, rm, 4, rk, l), (16, 4, rk * 512, 1, 512, rm * rk * 512))

        sfa, sfb = unit_sf(m, 1), unit_sf(n, e)
        alpha, norm = torch.ones(e, device=dev), torch.ones(1, device=dev)
        prob = torch.rand(m, 1, 1, generator=g, device=dev)
        stream = torch.cuda.current_stream()
        cu_stream = cuda.CUstream(stream.cuda_stream)

        def step():
            ref.grouped_gemm_swiglu_wrapper_sm100(a, b, sfa, sfb, offsets, alpha, norm_const_tensor=norm, prob_tensor=prob, d_dtype=torch.float8_e4m3fn,
                                                  sf_vec_size=32, m_aligned=256, mma_tiler_mn=(256, 256), current_stream=cu_stream)  # fmt: skip

        t0 = time.perf_counter()
        step()
        torch.cuda.synchronize()
        jit_s = time.perf_counter() - t0
        t = time_trials(step, stream)
        ms_b2b, _ = time_steps(step, 20, 3, stream)
        flops = 2.0 * tokens * topk * n * k
        return {"kernel": "the reference's BlockScaledContiguousGroupedGemmKernel through grouped_gemm_swiglu_wrapper_sm100 (CuTe DSL, JIT)",
                "workload": "c2 FC1: E=8, K=4096, N=28672, 32768 routed rows, groups padded to 256; C + E4M3 D + D_col + row and column scales",
                "tflops": flops / (t["median_ms"] * 1e-3) / 1e12, "timing": t, "ms_back_to_back": ms_b2b,
                "tflops_back_to_back": flops / (ms_b2b * 1e-3) / 1e12, "first_call_s": jit_s,
                "compare_with": "extras.vs_reference_kernel of the own arm (both kernels on the same tensors in one process)"}  # fmt: skip
    except Exception as exc:  # a JIT or import failure on this box is a result, not an error of the arm
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:300]}


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
    base["sample"] = "every step = 1 expert x 256 rows of the workload's FC1 (N=28672, K=4096) through the CPU port of the reference's PyTorch implementation"
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
        "config": {"workload": WORKLOAD},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    gpu_kernel = reference_gpu_kernel() if args.gpus == 1 else None
    if gpu_kernel is not None:
        # beside the CPU figure this arm is defined by: what the reference's own sm_100 kernel does on this GPU
        line["extras"] = {"reference_gpu_kernel": gpu_kernel}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# head to head with the reference's own GPU kernel (only where its overlay is present: 1-GPU calls)
# ---------------------------------------------------------------------------------------------
def vs_reference_kernel(prob256, stream):
    """Interleaved A B A B timing of the reference's grouped_gemm_swiglu_wrapper_sm100 (its CuTe-DSL
    kernel, JIT-compiled from the overlay under baseline/_ref) and this package's wrapper on the same c2
    tensors: groups padded to 256, mma_tiler (256, 256), full output set (C, E4M3 D and D_col, row and
    column scales).  Returns None when the overlay is absent."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "cudnn")):
        return None
    import torch

    sys.path.insert(0, ref_dir)
    try:
        import cuda.bindings.driver as cuda
        import cudnn as ref

        ref_fn = ref.grouped_gemm_swiglu_wrapper_sm100
    except Exception as exc:  # the overlay exists but cannot be imported on this box
        return {"unavailable": f"{type(exc).__name__}: {exc}"[:200]}
    finally:
        sys.path.remove(ref_dir)
    import cudnn_frontend_b200 as ours

    p = prob256
    norm = torch.ones(1, device="cuda")
    cu_stream = cuda.CUstream(stream.cuda_stream)
    common = dict(norm_const_tensor=norm, prob_tensor=p["prob"], d_dtype=torch.float8_e4m3fn, sf_vec_size=32, m_aligned=256)

    def run_ref():
        return ref_fn(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], mma_tiler_mn=(256, 256), current_stream=cu_stream, **common)

    def run_own():
        return ours.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], **common)

    try:
        t0 = time.perf_counter()
        r_ref = run_ref()
        torch.cuda.synchronize()
        jit_s = time.perf_counter() - t0
    except Exception as exc:
        return {"unavailable": f"reference kernel failed: {type(exc).__name__}: {exc}"[:200]}
    r_own = run_own()
    torch.cuda.synchronize()
    same = {key: bool(torch.equal(r_ref[key].view(torch.uint8), r_own[key].view(torch.uint8))) for key in ("d_tensor", "d_col_tensor")}
    same["c_tensor"] = bool(torch.equal(r_ref["c_tensor"], r_own["c_tensor"]))
    del r_ref, r_own
    rounds = 12
    for _ in range(3):
        run_ref()
        run_own()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * rounds + 1)]
    ev[0].record(stream)
    for i in range(rounds):
        run_ref()
        ev[2 * i + 1].record(stream)
        run_own()
        ev[2 * i + 2].record(stream)
    torch.cuda.synchronize()
    t_ref = sorted(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(rounds))
    t_own = sorted(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(rounds))
    # isolated launches (L2 flushed, GPU idle before each), the two kernels taking turns so that both see
    # the same power and clock state of the GPU
    dev = torch.cuda.current_device()
    if dev not in _FLUSH:
        _FLUSH[dev] = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    iso = {"ref": [], "own": []}
    for _ in range(10):
        for name, fn in (("ref", run_ref), ("own", run_own)):
            _FLUSH[dev].zero_()
            s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_.record(stream)
            fn()
            e_.record(stream)
            torch.cuda.synchronize()
            iso[name].append(s_.elapsed_time(e_))
    iso_ref = {"median_ms": sorted(iso["ref"])[5], "min_ms": min(iso["ref"])}
    iso_own = {"median_ms": sorted(iso["own"])[5], "min_ms": min(iso["own"])}
    return {
        "workload": "c2 FC1 through both wrappers: groups padded to 256, C + E4M3 D + D_col + row and column scales",
        "protocol": "interleaved A B A B in one queue (medians of 12 rounds); isolated = 10 trials each with an L2 flush and an idle GPU before "
                    "every launch, the two kernels taking turns",
        "reference_ms": t_ref[rounds // 2], "own_ms": t_own[rounds // 2], "own_over_reference": t_ref[rounds // 2] / t_own[rounds // 2],
        "reference_isolated_ms": iso_ref["median_ms"], "own_isolated_ms": iso_own["median_ms"],
        "own_over_reference_isolated": iso_ref["median_ms"] / iso_own["median_ms"],
        "outputs_bit_identical": same, "reference_first_call_s": jit_s,
        "timed_through": "both wrappers (output allocation included on both sides)",
    }  # fmt: skip


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
    cfg = {"c2": synthetic.CONFIGS["c2"], "small": SMALL_CASE, "deepseek-small": DEEPSEEK_SMALL_CASE}[args.workload]
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
        ms, step_stats = time_steps(step, args.steps, args.warmup, stream)
    value = flops / (ms * 1e-3) / 1e12
    assert ops.device_status(clear=True) == 0, "a bounded wait inside the kernel gave up"
    if args.kernel_only:
        print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms, "steps": args.steps, "warmup": args.warmup,
                          "config": {"workload": f"kernel only, {args.workload}: {cfg}"}, "timing": step_stats, "clocks": clk.summary()}))  # fmt: skip
        return

    # the same launch for at least two seconds: what the GPU sustains under its power cap, with the clock it ran at
    ms_sus, steps_sus, clk_sus = time_sustained(step, stream, ms, SUSTAINED_SECONDS, 0)
    value_sus = flops / (ms_sus * 1e-3) / 1e12
    sustained = {"value": value_sus, "unit": UNIT, "ms_per_step": ms_sus, "steps": steps_sus, "seconds": ms_sus * steps_sus * 1e-3,
                 "sm_mhz_median": clk_sus["sm_mhz"], "reasons": clk_sus["reasons"],
                 "mcycles_per_step": None if not clk_sus["sm_mhz"] else ms_sus * 1e-3 * clk_sus["sm_mhz"],
                 "pct_of_fp8_nominal_4500": 100.0 * value_sus / FP8_NOMINAL_TFLOPS}  # fmt: skip

    # the same call with the bf16 pre-activation C also written, and with the full output set of the
    # reference's wrapper (C, E4M3 D and D_col, row and column scale factors)
    step_c, outs_c = make_op(write_c=True)
    t_c = time_trials(step_c, stream)
    del outs_c, step_c
    step_f, outs_f = make_full_op()
    t_full = time_trials(step_f, stream)
    del outs_f, step_f

    # ---- end to end through the public API from pinned host memory -------------------------
    # Every step copies its own inputs from pinned host memory and copies its result (the bf16 D and the
    # per-expert amax) back to pinned host memory.  As in a serving loop the transfers overlap the
    # kernels: inputs of step i + 1 travel while step i computes, the result of step i travels while step
    # i + 1 computes (a copy stream per direction, two buffers each, events both ways).
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
    d_bufs = [torch.empty((m_max, n // 2, 1), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    amax_bufs = [torch.full((e, 1), float("-inf"), dtype=torch.float32, device=dev) for _ in range(2)]
    d_host = [torch.empty((m, n // 2), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    amax_host = [torch.empty((e, 1), dtype=torch.float32).pin_memory() for _ in range(2)]
    op2 = cf.GroupedGemmSwigluSm100(aq.view(m_max, k, 1), prob_["b"], None, d_bufs[0], sfa, prob_["sfb"], prob_["padded_offsets"], prob_["alpha"],
                                    None, sample_amax=amax_bufs[0], sample_prob=pg.view(m_max, 1, 1), sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op2.check_support()
    op2.compile()
    h2d_stream, d2h_stream = torch.cuda.Stream(), torch.cuda.Stream()
    copied = [torch.cuda.Event() for _ in range(2)]  # inputs of the buffer have landed
    consumed = [torch.cuda.Event() for _ in range(2)]  # the step that read the input buffer is done with it
    computed = [torch.cuda.Event() for _ in range(2)]  # the step's result is complete
    drained = [torch.cuda.Event() for _ in range(2)]  # the result buffer has been copied out
    step_no = [0]

    def start_copy(i):
        x_dev, ids_dev, p_dev = in_bufs[i % 2]
        with torch.cuda.stream(h2d_stream):
            if i >= 2:
                h2d_stream.wait_event(consumed[i % 2])
            x_dev.copy_(x_host, non_blocking=True)
            ids_dev.copy_(ids_host, non_blocking=True)
            p_dev.copy_(p_host, non_blocking=True)
            copied[i % 2].record(h2d_stream)

    def e2e_step():
        i = step_no[0]
        if i == 0:
            start_copy(0)
        start_copy(i + 1)  # the next step's inputs travel while this step computes
        x_dev, ids_dev, p_dev = in_bufs[i % 2]
        d_dev, amax_dev = d_bufs[i % 2], amax_bufs[i % 2]
        stream.wait_event(copied[i % 2])
        if i >= 2:
            stream.wait_event(drained[i % 2])  # the result of step i - 2 has left this buffer
        counts, offs, dst = moe.route(ids_dev, e, 128)
        moe.scatter_rows(x_dev, dst, xg, rows_per_src=topk, in_prob=p_dev.view(-1), out_prob=pg)
        moe.zero_pad_rows(xg, counts, offs, pg)
        ops.quantize_mxfp8_out(xg, aq, sfa)
        consumed[i % 2].record(stream)
        amax_dev.fill_(float("-inf"))
        op2.execute(aq.view(m_max, k, 1), prob_["b"], None, d_dev, sfa, prob_["sfb"], offs, prob_["alpha"], amax_tensor=amax_dev,
                    prob_tensor=pg.view(m_max, 1, 1))  # fmt: skip
        computed[i % 2].record(stream)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(computed[i % 2])
            d_host[i % 2].copy_(d_dev[:m, :, 0], non_blocking=True)
            amax_host[i % 2].copy_(amax_dev, non_blocking=True)
            drained[i % 2].record(d2h_stream)
        step_no[0] = i + 1

    def e2e_region(steps):
        torch.cuda.synchronize()
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record(stream)
        for _ in range(steps):
            e2e_step()
        stream.wait_stream(d2h_stream)  # the last results have reached the host
        e_.record(stream)
        torch.cuda.synchronize()
        return s_.elapsed_time(e_) / steps

    e2e_region(3)
    e2e_steps = max(args.steps // 2, 10)
    ms_e2e = e2e_region(e2e_steps)
    last = (step_no[0] - 1) % 2
    h2d = x_host.numel() * 2 + ids_host.numel() * 4 + p_host.numel() * 4
    d2h = d_host[0].numel() * 2 + e * 4
    e2e = {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": ms_e2e, "steps": e2e_steps, "launches_per_step": 8,
           "d2h_gbs": d2h / (ms_e2e * 1e-3) / 1e9,
           "note": "per step: tokens, expert ids and gate probabilities from pinned host memory, the bf16 D and amax back to pinned host "
                   "memory; transfers overlap the kernels of the neighbouring steps; the region ends when the last result is on the host; "
                   "the result copy (0.94 GB over PCIe) is the longest leg of a step"}  # fmt: skip
    e2e_ok = bool(torch.allclose(amax_host[last].view(-1), outs[2].cpu().view(-1), rtol=1e-5)) and bool(
        torch.equal(d_host[last], outs[1][:m, :, 0].cpu()))

    # ---- quantiser bandwidth (the other new kernel of the path) -----------------------------
    xq = torch.randn(32768, 4096, device=dev).to(torch.bfloat16)
    q_out = torch.empty((32768, 4096), dtype=torch.float8_e4m3fn, device=dev)
    sf_out = ops.empty_sf(32768, 4096, 1, device=dev)
    q_bytes = 32768 * 4096 * (2 + 1 + 1 / 32)
    t_q = time_trials(lambda: ops.quantize_mxfp8_out(xq, q_out, sf_out), stream)
    # and back to back for at least half a second (the input is larger than L2, so nothing is reused between calls)
    reps = max(int(0.6e3 / t_q["median_ms"]) + 1, 100)  # at least half a second even when back-to-back calls run faster than the flushed median
    ms_q_long, _ = time_steps(lambda: ops.quantize_mxfp8_out(xq, q_out, sf_out), reps, 3, stream)
    quant = {"gbs": q_bytes / (t_q["median_ms"] * 1e-3) / 1e9, "gbs_best": q_bytes / (t_q["min_ms"] * 1e-3) / 1e9,
             "gbs_sustained": q_bytes / (ms_q_long * 1e-3) / 1e9, "sustained_calls": reps, "sustained_seconds": ms_q_long * reps * 1e-3,
             "frac_of_measured_hbm": q_bytes / (ms_q_long * 1e-3) / 1e9 / peaks["hbm_gbs"], "shape": [32768, 4096], "timing": t_q}  # fmt: skip
    del xq, q_out, sf_out

    extras = {"fc1_with_c_store": {"tflops": flops / (t_c["median_ms"] * 1e-3) / 1e12, "timing": t_c},
              "fc1_full_output_set": {"tflops": flops / (t_full["median_ms"] * 1e-3) / 1e12, "timing": t_full},
              "quantiser": quant, "e2e_result_on_host_matches_resident_run": e2e_ok}  # fmt: skip
    routed = t * topk
    prob_bytes = routed * k * (1 + 1 / 32) + e * n * k * (1 + 1 / 32) + routed * (n // 2) * 2
    if not args.no_extras:
        del prob_, outs, op2, xg, aq, d_bufs, in_bufs, d_host, step
        torch.cuda.empty_cache()
        if args.workload == "c2":
            p256 = synthetic.make_problem("c2", dev, seed=0, m_aligned=256)
            h2h = vs_reference_kernel(p256, stream)
            if h2h is not None:
                extras["vs_reference_kernel"] = h2h
            del p256
            torch.cuda.empty_cache()
        extras.update(bench_other_configs(dev, stream, peaks))
        torch.cuda.empty_cache()
        extras.update(bench_fp4(dev, stream))
        torch.cuda.empty_cache()
        extras.update(bench_backward(dev, stream))
        torch.cuda.empty_cache()
        import ep_bench

        # the workload of the multi-GPU runs (--gpus 2/4/8) with all experts on this GPU
        extras["ep_layer_1gpu"] = ep_bench.single_gpu_layer(dev)

    cpu = cpu_baseline_fc1()
    cpu["c1_full_size"] = cpu_baseline_c1()
    peak_burst, peak_sus = 2.0 * peaks["bf16"], 2.0 * peaks["bf16_sustained"]
    region_s = ms * args.steps * 1e-3
    burst_region = region_s < 1.0  # a region this short runs at the clock of a cold, un-capped GPU
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
            "workload": WORKLOAD,
            "l2": "inputs larger than L2 (A 134 MB + B 940 MB per step), no flush",
            "pct_of_fp8_nominal_4500": 100.0 * value / FP8_NOMINAL_TFLOPS,
        },
        "timing": step_stats,
        "value_sustained": sustained,
        "roofline": {
            "bound": "tensor",
            "achieved": value,
            "peak": peak_burst if burst_region else peak_sus,
            "unit": UNIT,
            "frac": value / (peak_burst if burst_region else peak_sus),
            "frac_burst": value / peak_burst,
            "frac_sustained": value_sus / peak_sus,
            "peak_burst": peak_burst,
            "peak_sustained": peak_sus,
            "timed_region_s": region_s,
            # HBM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum), recorded beside the
            # profile summary of this workload; the algorithmic bytes beside it
            "traffic": load_traffic("grouped_gemm_fc1_c2") if args.workload == "c2" else None,
            "traffic_unit": "bytes per launch (ncu, this workload)",
            "algorithmic_bytes": prob_bytes,
            "peak_source": f"2 x bf16_tflops (burst) / 2 x bf16_tflops_sustained of {peaks['source']} MEASURED_PEAKS.json: no fp8 peak is measured, "
                           "twice the bf16 cuBLAS rate stands in for it; frac uses the burst figure for a timed region under one second, frac_sustained "
                           "compares the two-second region with the sustained figure",
            "kernel": "grouped_gemm_kernel<FC1, dense>",
        },
        "cpu_baseline": cpu,
        "e2e": e2e,
        "gpu_launches": args.steps,
        "clocks": clk.summary(),
        "extras": extras,
    }  # fmt: skip
    print(json.dumps(line))


def bench_other_configs(dev, stream, peaks):
    """DeepSeek-shape FC1 (dense and discrete weights, static and dynamic scheduler) and FC2; reported
    beside the headline.  These are the HBM-bound configurations: GB/s of algorithmic bytes against the
    measured copy rate."""
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
    active = int((p3["routing"].counts > 0).sum().item())
    rows = p3["routing"].routed_rows
    bytes3 = rows * k * (1 + 1 / 32) + active * n * k * (1 + 1 / 32) + rows * (n // 2) * 2

    def report(t, flops, nbytes, **more):
        gbs = nbytes / (t["median_ms"] * 1e-3) / 1e9
        return {"tflops": flops / (t["median_ms"] * 1e-3) / 1e12, "ms": t["median_ms"], "ms_best": t["min_ms"], "gbs": gbs,
                "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], **more}  # fmt: skip

    for dyn in (False, True):
        op = cf.GroupedGemmGluSm100(p3["a"], None, dbf, p3["sfa"], p3["padded_offsets"], p3["alpha"], None, sample_b=p3["b"], sample_sfb=p3["sfb"],
                                    sample_amax=amax, sf_vec_size=32, m_aligned=128, use_dynamic_sched=dyn)  # fmt: skip
        assert op.check_support()
        op.compile()
        t3 = time_trials(lambda: op.execute(p3["a"], None, dbf, p3["sfa"], p3["padded_offsets"], p3["alpha"], b_tensor=p3["b"], sfb_tensor=p3["sfb"],
                                            amax_tensor=amax), stream)  # fmt: skip
        out["deepseek_fc1_dense" + ("_dynamic_sched" if dyn else "")] = report(t3, p3["flops"], bytes3, padded_rows=m, active_experts=active)

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
    t_d = time_trials(lambda: opd.execute(p3["a"], b_ptrs, None, dbf, p3["sfa"], sfb_ptrs, p3["padded_offsets"], p3["alpha"], amax_tensor=amax), stream)
    out["deepseek_fc1_discrete"] = report(t_d, p3["flops"], bytes3)
    del b_list, sf_list, opd

    # FC1 with MXFP8 output feeds FC2
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
    flops4 = 2.0 * rows * n4 * k4
    bytes4 = rows * k4 * (1 + 1 / 32) + active * n4 * k4 * (1 + 1 / 32) + rows * n4 * (1 + 1 / 32)
    for dyn in (False, True):
        op4 = cf.GroupedGemmQuantSm100(d8, sfd_row, p3["padded_offsets"], p3["alpha"], d4, sample_d_col=d4, sample_b=w2, sample_sfb=sfw2,
                                       sample_sfd_row=sfd4, sample_sfd_col=ops.empty_sf(n4, m, 1, device=dev), sample_norm_const=norm,
                                       sample_prob=p3["prob"], sf_vec_size=32, m_aligned=128, use_dynamic_sched=dyn)  # fmt: skip
        assert op4.check_support()
        op4.compile()
        t4 = time_trials(lambda: op4.execute(d8, sfd_row, p3["padded_offsets"], p3["alpha"], d4, b_tensor=w2, sfb_tensor=sfw2, sfd_row_tensor=sfd4,
                                             norm_const_tensor=norm, prob_tensor=p3["prob"]), stream)  # fmt: skip
        out["deepseek_fc2_quant" + ("_dynamic_sched" if dyn else "")] = report(t4, flops4, bytes4)
    out["protocol"] = "3 warm-ups, 10 trials with a 256 MiB L2 flush between them, median (ms) and best (ms_best)"
    return out


def bench_fp4(dev, stream):
    """The Mixtral-shape FC1 with FP4 operands (random E2M1 bytes; E4M3 scales per 16 = NVFP4, E8M0 per 32 =
    MXFP4), bf16 D + amax, same rows and offsets as the headline: reported beside it."""
    import torch

    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops, synthetic

    cfg = synthetic.CONFIGS["c2"]
    e, n, k = cfg["experts"], cfg["n"], cfg["k"]
    r = synthetic.make_routing(cfg["tokens"], e, cfg["topk"], cfg["routing"], 0, dev, 128)
    m = r.m_rows
    g = torch.Generator(device=dev).manual_seed(5)
    a8 = torch.randint(0, 256, (m, k // 2), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
    b8 = torch.randint(0, 256, (e, n, k // 2), generator=g, device=dev, dtype=torch.int32).to(torch.uint8)
    a = torch.as_strided(a8.view(torch.float4_e2m1fn_x2), (m, k // 2, 1), (k // 2, 1, m * k // 2))
    b = b8.view(torch.float4_e2m1fn_x2).permute(1, 2, 0)
    d = torch.empty((m, n // 2, 1), dtype=torch.bfloat16, device=dev)
    amax = torch.full((e, 1), float("-inf"), dtype=torch.float32, device=dev)
    alpha = torch.ones(e, device=dev)
    flops = 2.0 * r.routed_rows * n * k
    out = {}
    for name, sf_vec, sf_dtype, lo, hi in (("nvfp4", 16, torch.float8_e4m3fn, 0x30, 0x46), ("mxfp4", 32, torch.float8_e8m0fnu, 124, 131)):
        def rand_sf(mn, l):
            t = ops.empty_sf(mn, k, l, device=dev, dtype=sf_dtype, sf_vec=sf_vec)
            flat = torch.as_strided(t.view(torch.uint8), (t.numel(),), (1,))
            flat.copy_(torch.randint(lo, hi, (t.numel(),), generator=g, device=dev, dtype=torch.int32).to(torch.uint8))
            return t

        sfa, sfb = rand_sf(m, 1), rand_sf(n, e)
        op = cf.GroupedGemmSwigluSm100(a, b, None, d, sfa, sfb, r.padded_offsets, alpha, None, sample_amax=amax, sf_vec_size=sf_vec, m_aligned=128)
        assert op.check_support()
        op.compile()
        t = time_trials(lambda: op.execute(a, b, None, d, sfa, sfb, r.padded_offsets, alpha, amax_tensor=amax), stream)
        out["fc1_" + name] = {"tflops": flops / (t["median_ms"] * 1e-3) / 1e12, "timing": t, "pct_of_fp4_nominal_9000": 100.0 * flops / (t["median_ms"] * 1e-3) / 9e15,
                              "operands": f"E2M1 with {'E4M3' if sf_vec == 16 else 'E8M0'} scales per {sf_vec} elements"}  # fmt: skip
    return out


def bench_backward(dev, stream, small=False):
    """The backward pair on the Mixtral shape (E=8, hidden 4096, intermediate 14336, 32768 routed rows): dSwiGLU
    (gradient GEMM with K = hidden, N = intermediate, fused activation backward, E4M3 D_row / D_col with scales) and
    the weight gradient of FC1 (m = hidden, n = 2 x intermediate, the experts split the 32768 tokens), bf16 output.
    small: a quarter of the intermediate size and of the rows, for profiler captures."""
    import torch

    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops, synthetic

    out = {}
    cfg = dict(experts=8, k=4096, n=3584 if small else 14336, tokens=4096 if small else 16384, topk=2, routing="uniform")
    p = synthetic.make_problem(cfg, dev, seed=4, m_aligned=128)
    e, n, k, m = cfg["experts"], cfg["n"], cfg["k"], p["m_rows"]
    g = torch.Generator(device=dev).manual_seed(8)
    c_fwd = torch.empty((m, 2 * n), device=dev).uniform_(-3, 3, generator=g).to(torch.bfloat16).view(m, 2 * n, 1)
    d_row = torch.empty((m, 2 * n, 1), dtype=torch.float8_e4m3fn, device=dev)
    d_col = torch.empty_like(d_row)
    dprob = torch.zeros((m, 1, 1), device=dev)
    sfd_row, sfd_col = ops.empty_sf(m, 2 * n, 1, device=dev), ops.empty_sf(2 * n, m, 1, device=dev)
    beta, norm = torch.ones(e, device=dev), torch.ones(1, device=dev)
    op = cf.GroupedGemmDswigluSm100(p["a"], p["b"], c_fwd, d_row, d_col, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], beta, p["prob"], dprob,
                                    sample_sfd_row=sfd_row, sample_sfd_col=sfd_col, sample_norm_const=norm, sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op.check_support()
    op.compile()
    t = time_trials(lambda: op.execute(p["a"], p["b"], c_fwd, d_row, d_col, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], beta, p["prob"], dprob,
                                       sfd_row_tensor=sfd_row, sfd_col_tensor=sfd_col, norm_const_tensor=norm), stream)  # fmt: skip
    out["dswiglu_mixtral"] = {"tflops": p["flops"] / (t["median_ms"] * 1e-3) / 1e12, "timing": t,
                              "outputs": f"E4M3 D_row and D_col [{m}, {2 * n}] with row and column scales, dprob"}  # fmt: skip
    del p, c_fwd, d_row, d_col, sfd_row, sfd_col, op
    torch.cuda.empty_cache()

    m_w, n_w, tokens = 4096, (7168 if small else 28672), 32768
    a = torch.empty((m_w, tokens), device=dev).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn)
    b = torch.empty((n_w, tokens), device=dev).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn).t()
    cols = tokens // 32
    sfa = torch.randint(124, 131, (m_w, cols), generator=g, device=dev, dtype=torch.int32).to(torch.uint8).view(torch.float8_e8m0fnu)
    sfb = torch.randint(124, 131, (n_w, cols), generator=g, device=dev, dtype=torch.int32).to(torch.uint8).view(torch.float8_e8m0fnu)
    offs = torch.arange(1, e + 1, device=dev, dtype=torch.int32) * (tokens // e)
    w = torch.empty((e, m_w, n_w), dtype=torch.bfloat16, device=dev)
    opw = cf.GroupedGemmWgradSm100(a, b, sfa, sfb, offs, sample_wgrad=w, sf_vec_size=32)
    assert opw.check_support()
    opw.compile()
    tw = time_trials(lambda: opw.execute(a, b, sfa, sfb, offs, wgrad_tensor=w), stream)
    flops_w = 2.0 * tokens * m_w * n_w
    out["wgrad_mixtral_fc1"] = {"tflops": flops_w / (tw["median_ms"] * 1e-3) / 1e12, "timing": tw, "outputs": f"bf16 [8, {m_w}, {n_w}]"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the DeepSeek-shape side measurements")
    ap.add_argument("--workload", default="c2", choices=["c2", "small", "deepseek-small"],
                    help="c2 = Mixtral-shape FC1 (the benchmark); small / deepseek-small = reduced cases for profiler captures")  # fmt: skip
    ap.add_argument("--outputs", default="d", choices=["d", "full"], help="with --kernel-only: d = bf16 D + amax (the benchmark); full = C + E4M3 D + D_col + scale factors")
    ap.add_argument("--kernel-only", action="store_true", help="time the FC1 kernel only (no end-to-end, CPU baseline or side measurements)")
    ap.add_argument("--backward-only", action="store_true", help="time the dSwiGLU and weight-gradient kernels only (--workload small: reduced sizes for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "own" else args.warmup
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.backward_only:
        import torch

        torch.cuda.set_device(0)
        print(json.dumps(bench_backward(torch.device("cuda", 0), torch.cuda.current_stream(), small=args.workload == "small")))
        return
    if world > 1 or args.gpus > 1:
        import ep_bench

        args.peaks = load_peaks()
        args.clock_sampler = ClockSampler
        ep_bench.run(args)
    else:
        bench_single(args)


if __name__ == "__main__":
    main()
