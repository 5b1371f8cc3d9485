"""Run the reference's own CuTe-DSL grouped-GEMM kernels next to this repository's on one GPU.

Needs the overlay made by baseline/make_ref_overlay.py (baseline/_ref/cudnn) and the CuTe DSL
(nvidia-cutlass-dsl) of the image.  For each case the same device tensors go through

    reference:  cudnn.grouped_gemm_swiglu_wrapper_sm100 / grouped_gemm_quant_wrapper_sm100
    here:       cudnn_frontend_b200.<same names>

with the reference's constraints (groups padded to 256, mma_tiler (256, 256)), then outputs are
compared (C bf16, E8M0 scale bytes, E4M3 ULP distance) and both are timed with CUDA events
(3 warm-ups, 10 trials, 256 MiB L2 flush between trials, median and best; back to back; and
interleaved A B A B in one queue, which is the comparison that is independent of the GPU's power state).  Results go to
<out dir>/reference_kernels_<cases>.json; the tiny cases' inputs and reference-kernel outputs are saved
to <out dir>/reference_kernel_*golden.npz so they can be committed as golden vectors (tests/golden/).  The
output directory is --out (or the environment variable B200MOE_OUT_DIR); one of the two is required.

    python baseline/run_reference_kernels.py --cases tiny      # one case per process: the reference's
    python baseline/run_reference_kernels.py --cases c2        # wrapper cache does not key on the expert count
    python baseline/run_reference_kernels.py --cases c4        # FC2 (grouped_gemm_quant): fc2_tiny, fc2_mixtral, c4
"""

import argparse
import json
import os
import sys
import time
import traceback

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

OUT_DIR = os.environ.get("B200MOE_OUT_DIR")  # main() replaces it with --out when given


def timed(fn, trials=10, warmup=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(trials):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    ordered = sorted(times)
    return ordered[len(ordered) // 2], ordered[0], times


def timed_back_to_back(fn, steps=20, warmup=3):
    """Sustained protocol: `steps` launches in a row between two events (what bench.py does)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps


def timed_interleaved(fn_a, fn_b, rounds=30, warmup=3):
    """A B A B ... in one queue, every call bracketed by events: both kernels see the same clocks,
    temperature and power state.  Returns the median ms of each."""
    for _ in range(warmup):
        fn_a()
        fn_b()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * rounds + 1)]
    ev[0].record()
    for i in range(rounds):
        fn_a()
        ev[2 * i + 1].record()
        fn_b()
        ev[2 * i + 2].record()
    torch.cuda.synchronize()
    ta = sorted(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(rounds))
    tb = sorted(ev[2 * i + 1].elapsed_time(ev[2 * i + 2]) for i in range(rounds))
    return ta[rounds // 2], tb[rounds // 2]


def ulp(a, b):
    def order(v):
        v = v.to(torch.int32)
        mag = v & 0x7F
        return torch.where((v & 0x80) != 0, -mag, mag)

    return (order(a) - order(b)).abs()


def run_case(name, cfg, out):
    import cuda.bindings.driver as cuda
    import cudnn as ref  # the overlay

    import cudnn_frontend_b200 as ours
    from cudnn_frontend_b200 import synthetic

    p = synthetic.make_problem(cfg, "cuda", seed=3, m_aligned=256)
    n, k = cfg["n"], cfg["k"]
    if cfg.get("ab") == "e5m2":
        # same shapes and scale factors, operands drawn directly in E5M2 (reinterpreting E4M3 bytes would hit its Inf / NaN codes)
        g5 = torch.Generator(device="cuda").manual_seed(11)
        m_all = p["a"].shape[0]
        a5 = torch.randn(m_all, k, generator=g5, device="cuda").to(torch.float8_e5m2)
        p["a"] = torch.as_strided(a5, (m_all, k, 1), (k, 1, m_all * k))
        p["b"] = (torch.randn(cfg["experts"], n, k, generator=g5, device="cuda") * 0.5).to(torch.float8_e5m2).permute(1, 2, 0)
    norm = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    d_dtype = {"e5m2": torch.float8_e5m2, "bf16": torch.bfloat16}.get(cfg.get("d"), torch.float8_e4m3fn)
    d16 = d_dtype == torch.bfloat16  # scale factors generated, D and D_col hold the scaled values in bf16
    common = dict(norm_const_tensor=norm, prob_tensor=p["prob"], d_dtype=d_dtype, sf_vec_size=32, m_aligned=256)
    res = {"case": name, "cfg": cfg, "m_rows": p["m_rows"], "flops": p["flops"]}

    t0 = time.time()
    r_ref = ref.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"],
                                                  mma_tiler_mn=(256, 256), current_stream=stream, **common)  # fmt: skip
    torch.cuda.synchronize()
    res["ref_first_call_s"] = time.time() - t0
    r_own = ours.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], **common)
    torch.cuda.synchronize()

    if PROFILE_ONLY:  # two launches of each kernel for a profiler capture, nothing else
        ref.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"],
                                              mma_tiler_mn=(256, 256), current_stream=stream, **common)  # fmt: skip
        ours.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], **common)
        torch.cuda.synchronize()
        return
    m = p["m_rows"]
    c_ref, c_own = r_ref["c_tensor"][:m].float(), r_own["c_tensor"][:m].float()
    res["c_rel_fro"] = float((c_ref - c_own).norm() / c_ref.norm())
    res["c_equal_frac"] = float((r_ref["c_tensor"][:m] == r_own["c_tensor"][:m]).float().mean())

    def flat(t):
        t = t.view(torch.uint8)
        return torch.as_strided(t, (t.numel(),), (1,))

    sf_r, sf_o = flat(r_ref["sfd_row_tensor"]), flat(r_own["sfd_row_tensor"])
    res["sfd_row_bytes_equal_frac"] = float((sf_r == sf_o).float().mean())
    def raw(t):  # [m, n_out] bytes (FP8) or 16-bit patterns (bf16)
        t2 = t[:m, :, 0]
        return t2.view(torch.uint8) if t.element_size() == 1 else t2.contiguous().view(torch.int16)

    d_r, d_o = raw(r_ref["d_tensor"]), raw(r_own["d_tensor"])
    dc_r, dc_o = raw(r_ref["d_col_tensor"]), raw(r_own["d_col_tensor"])
    if d16:
        res["d_bf16_equal_frac"] = float((d_r == d_o).float().mean())
        res["d_col_bf16_equal_frac"] = float((dc_r == dc_o).float().mean())
        res["amax_equal"] = bool(torch.equal(r_ref["amax_tensor"], r_own["amax_tensor"]))
    else:
        u = ulp(d_r, d_o)
        res["d_e4m3_within_1ulp_frac"] = float((u <= 1).float().mean())
        res["d_e4m3_equal_frac"] = float((u == 0).float().mean())
        uc = ulp(dc_r, dc_o)
        res["d_col_within_1ulp_frac"] = float((uc <= 1).float().mean())
    sc_r, sc_o = flat(r_ref["sfd_col_tensor"]), flat(r_own["sfd_col_tensor"])
    res["sfd_col_bytes_equal_frac"] = float((sc_r == sc_o).float().mean())

    def run_ref():
        return ref.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"],
                                                     mma_tiler_mn=(256, 256), current_stream=stream, **common)  # fmt: skip

    def run_own():
        return ours.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], **common)

    # alternate the two kernels so that both see the same thermal / power state of the GPU
    order = [("own", run_own), ("ref", run_ref)] if OWN_FIRST else [("ref", run_ref), ("own", run_own)]
    iso, b2b = {}, {"ref": [], "own": []}
    for name_, fn in order:
        iso[name_] = timed(fn)
    for _ in range(3):
        for name_, fn in order:
            b2b[name_].append(timed_back_to_back(fn))
    ms_ref, ms_own = iso["ref"], iso["own"]
    il_ref, il_own = timed_interleaved(run_ref, run_own)
    res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
    res["own_over_ref_interleaved"] = il_ref / il_own
    res["order"] = [n for n, _ in order]
    res["ref_ms_median_best"] = ms_ref[:2]
    res["own_ms_median_best"] = ms_own[:2]
    res["ref_ms_trials"] = ms_ref[2]
    res["own_ms_trials"] = ms_own[2]
    res["ref_ms_back_to_back_rounds"] = b2b["ref"]
    res["own_ms_back_to_back_rounds"] = b2b["own"]
    res["ref_ms_back_to_back"] = sorted(b2b["ref"])[1]
    res["own_ms_back_to_back"] = sorted(b2b["own"])[1]
    res["own_over_ref_back_to_back"] = res["ref_ms_back_to_back"] / res["own_ms_back_to_back"]
    res["ref_tflops"] = p["flops"] / (ms_ref[0] * 1e-3) / 1e12
    res["own_tflops"] = p["flops"] / (ms_own[0] * 1e-3) / 1e12
    res["own_over_ref"] = ms_ref[0] / ms_own[0]
    out.append(res)
    print(json.dumps(res), flush=True)

    if name in ("tiny", "tiny_e5m2", "tiny_d_e5m2", "tiny_deepk", "tiny_d_bf16"):
        np.savez_compressed(
            os.path.join(OUT_DIR, {"tiny": "reference_kernel_golden.npz", "tiny_e5m2": "reference_kernel_e5m2_golden.npz",
                                   "tiny_d_e5m2": "reference_kernel_d_e5m2_golden.npz",
                                   "tiny_deepk": "reference_kernel_deepk_golden.npz",
                                   "tiny_d_bf16": "reference_kernel_d_bf16_golden.npz"}[name]),
            a=p["a"][:, :, 0].view(torch.uint8).cpu().numpy(),
            b=p["b"].permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(),
            sfa=flat(p["sfa"]).cpu().numpy(),
            sfb=flat(p["sfb"]).cpu().numpy(),
            offsets=p["padded_offsets"].cpu().numpy(),
            prob=p["prob"].view(-1).cpu().numpy(),
            c=r_ref["c_tensor"][:, :, 0].view(torch.int16).cpu().numpy(),
            d=d_r.cpu().numpy(),
            d_col=dc_r.cpu().numpy(),
            amax=(r_ref["amax_tensor"].cpu().numpy() if d16 else np.zeros(0, dtype=np.float32)),
            sfd_row=sf_r.cpu().numpy(),
            sfd_col=sc_r.cpu().numpy(),
        )


def run_case_fc2(name, cfg, out):
    """FC2: grouped GEMM + gating + MXFP8 re-quantisation (grouped_gemm_quant), full output set."""
    import cuda.bindings.driver as cuda
    from cudnn.grouped_gemm.grouped_gemm_quant.api import grouped_gemm_quant_wrapper_sm100 as ref_quant  # the overlay

    import cudnn_frontend_b200 as ours
    from cudnn_frontend_b200 import synthetic

    p = synthetic.make_problem(cfg, "cuda", seed=5, m_aligned=256)
    norm = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    kw = dict(b_tensor=p["b"], sfb_tensor=p["sfb"], norm_const_tensor=norm, prob_tensor=p["prob"], d_dtype=torch.float8_e4m3fn,
              sf_vec_size=32, m_aligned=256)  # fmt: skip
    res = {"case": name, "op": "fc2", "cfg": cfg, "m_rows": p["m_rows"], "flops": p["flops"]}

    def run_ref():
        return ref_quant(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], mma_tiler_mn=(256, 256), current_stream=stream, **kw)

    def run_own():
        return ours.grouped_gemm_quant_wrapper_sm100(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], **kw)

    t0 = time.time()
    r_ref = run_ref()
    torch.cuda.synchronize()
    res["ref_first_call_s"] = time.time() - t0
    r_own = run_own()
    torch.cuda.synchronize()
    if PROFILE_ONLY:
        run_ref()
        run_own()
        torch.cuda.synchronize()
        return
    m = p["m_rows"]

    def flat(t):
        t = t.view(torch.uint8)
        return torch.as_strided(t, (t.numel(),), (1,))

    u = ulp(r_ref["d_tensor"][:m].view(torch.uint8), r_own["d_tensor"][:m].view(torch.uint8))
    res["d_e4m3_equal_frac"] = float((u == 0).float().mean())
    res["d_e4m3_within_1ulp_frac"] = float((u <= 1).float().mean())
    uc = ulp(r_ref["d_col_tensor"][:m].view(torch.uint8), r_own["d_col_tensor"][:m].view(torch.uint8))
    res["d_col_equal_frac"] = float((uc == 0).float().mean())
    res["sfd_row_bytes_equal_frac"] = float((flat(r_ref["sfd_row_tensor"]) == flat(r_own["sfd_row_tensor"])).float().mean())
    res["sfd_col_bytes_equal_frac"] = float((flat(r_ref["sfd_col_tensor"]) == flat(r_own["sfd_col_tensor"])).float().mean())

    iso_ref, iso_own = timed(run_ref), timed(run_own)
    res["ref_ms_median_best"], res["own_ms_median_best"] = iso_ref[:2], iso_own[:2]
    res["ref_ms_back_to_back"] = sorted(timed_back_to_back(run_ref) for _ in range(3))[1]
    res["own_ms_back_to_back"] = sorted(timed_back_to_back(run_own) for _ in range(3))[1]
    il_ref, il_own = timed_interleaved(run_ref, run_own)
    res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
    res["own_over_ref_interleaved"] = il_ref / il_own
    res["own_over_ref_back_to_back"] = res["ref_ms_back_to_back"] / res["own_ms_back_to_back"]
    res["own_over_ref"] = iso_ref[0] / iso_own[0]
    res["ref_tflops_interleaved"] = p["flops"] / (il_ref * 1e-3) / 1e12
    res["own_tflops_interleaved"] = p["flops"] / (il_own * 1e-3) / 1e12
    out.append(res)
    print(json.dumps(res), flush=True)

    if name == "fc2_tiny":
        np.savez_compressed(
            os.path.join(OUT_DIR, "reference_kernel_fc2_golden.npz"),
            a=p["a"][:, :, 0].view(torch.uint8).cpu().numpy(),
            b=p["b"].permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(),
            sfa=flat(p["sfa"]).cpu().numpy(),
            sfb=flat(p["sfb"]).cpu().numpy(),
            offsets=p["padded_offsets"].cpu().numpy(),
            prob=p["prob"].view(-1).cpu().numpy(),
            d=r_ref["d_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(),
            d_col=r_ref["d_col_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(),
            sfd_row=flat(r_ref["sfd_row_tensor"]).cpu().numpy(),
            sfd_col=flat(r_ref["sfd_col_tensor"]).cpu().numpy(),
        )


def run_case_glu(name, cfg, out):
    """Unified FC1 (grouped_gemm_glu): GeGLU + fused bf16 bias, dense weights, full output set."""
    import cuda.bindings.driver as cuda
    from cudnn.grouped_gemm.grouped_gemm_glu.api import grouped_gemm_glu_wrapper_sm100 as ref_glu  # the overlay

    import cudnn_frontend_b200 as ours
    from cudnn_frontend_b200 import synthetic

    p = synthetic.make_problem(cfg, "cuda", seed=9, m_aligned=256)
    n, e = cfg["n"], cfg["experts"]
    norm = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(4)
    bias = torch.empty((e, n), dtype=torch.float32, device="cuda").uniform_(-2.0, 2.0, generator=g).to(torch.bfloat16).t()
    res = {"case": name, "op": "glu", "cfg": cfg, "m_rows": p["m_rows"], "flops": p["flops"]}
    m = p["m_rows"]

    def flat(t):
        t = t.view(torch.uint8)
        return torch.as_strided(t, (t.numel(),), (1,))

    saved = {}
    for act in ("geglu", "swiglu"):
        kw = dict(b_tensor=p["b"], sfb_tensor=p["sfb"], bias_tensor=bias, norm_const_tensor=norm, prob_tensor=p["prob"],
                  d_dtype=torch.float8_e4m3fn, sf_vec_size=32, m_aligned=256, act_func=act)  # fmt: skip
        r_ref = ref_glu(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], mma_tiler_mn=(256, 256), current_stream=stream, **kw)
        torch.cuda.synchronize()
        r_own = ours.grouped_gemm_glu_wrapper_sm100(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], **kw)
        torch.cuda.synchronize()
        res[f"{act}_c_equal_frac"] = float((r_ref["c_tensor"][:m] == r_own["c_tensor"][:m]).float().mean())
        u = ulp(r_ref["d_tensor"][:m].view(torch.uint8), r_own["d_tensor"][:m].view(torch.uint8))
        res[f"{act}_d_equal_frac"] = float((u == 0).float().mean())
        uc = ulp(r_ref["d_col_tensor"][:m].view(torch.uint8), r_own["d_col_tensor"][:m].view(torch.uint8))
        res[f"{act}_d_col_equal_frac"] = float((uc == 0).float().mean())
        res[f"{act}_sfd_row_bytes_equal_frac"] = float((flat(r_ref["sfd_row_tensor"]) == flat(r_own["sfd_row_tensor"])).float().mean())
        res[f"{act}_sfd_col_bytes_equal_frac"] = float((flat(r_ref["sfd_col_tensor"]) == flat(r_own["sfd_col_tensor"])).float().mean())
        if act == "geglu":
            saved = dict(
                c=r_ref["c_tensor"][:, :, 0].view(torch.int16).cpu().numpy(),
                d=r_ref["d_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(),
                d_col=r_ref["d_col_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(),
                sfd_row=flat(r_ref["sfd_row_tensor"]).cpu().numpy(),
                sfd_col=flat(r_ref["sfd_col_tensor"]).cpu().numpy(),
            )
            if not PROFILE_ONLY and name != "glu_tiny":
                il_ref, il_own = timed_interleaved(
                    lambda: ref_glu(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], mma_tiler_mn=(256, 256), current_stream=stream, **kw),
                    lambda: ours.grouped_gemm_glu_wrapper_sm100(p["a"], p["sfa"], p["padded_offsets"], p["alpha"], **kw))
                res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
                res["own_over_ref_interleaved"] = il_ref / il_own
    out.append(res)
    print(json.dumps(res), flush=True)
    if name == "glu_tiny":
        np.savez_compressed(
            os.path.join(OUT_DIR, "reference_kernel_glu_golden.npz"),
            a=p["a"][:, :, 0].view(torch.uint8).cpu().numpy(),
            b=p["b"].permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(),
            sfa=flat(p["sfa"]).cpu().numpy(),
            sfb=flat(p["sfb"]).cpu().numpy(),
            offsets=p["padded_offsets"].cpu().numpy(),
            prob=p["prob"].view(-1).cpu().numpy(),
            bias=bias.t().contiguous().view(torch.int16).cpu().numpy(),  # [E, N] bf16 bits
            **saved,
        )


def run_case_fp4(name, cfg, out):
    """FC1 with FP4 operands (float4_e2m1fn_x2): bf16 C and bf16 D, no scale-factor generation.
    cfg["sf"] = (sf_vec_size, "e8m0" | "e4m3")."""
    import cuda.bindings.driver as cuda
    import cudnn as ref  # the overlay

    import cudnn_frontend_b200 as ours
    from cudnn_frontend_b200 import ops, synthetic

    e, n, k = cfg["experts"], cfg["n"], cfg["k"]
    sf_vec, sf_kind = cfg["sf"]
    sf_dtype = torch.float8_e4m3fn if sf_kind == "e4m3" else torch.float8_e8m0fnu
    r = synthetic.make_routing(cfg["tokens"], e, cfg["topk"], cfg["routing"], 3, "cuda", 256)
    m = r.m_rows
    g = torch.Generator(device="cuda").manual_seed(17)
    a8 = torch.randint(0, 256, (m, k // 2), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    # padding rows of every group are zero (amax covers them)
    ends = r.padded_offsets.long()
    starts = torch.cat([ends.new_zeros(1), ends[:-1]])
    rows = torch.arange(m, device="cuda")
    owner = torch.searchsorted(ends, rows, right=True).clamp(max=e - 1)
    a8[(rows - starts[owner]) >= r.counts.long()[owner]] = 0
    b8 = torch.randint(0, 256, (e, n, k // 2), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8)
    a = torch.as_strided(a8.view(torch.float4_e2m1fn_x2), (m, k // 2, 1), (k // 2, 1, m * k // 2))
    b = b8.view(torch.float4_e2m1fn_x2).permute(1, 2, 0)
    lo, hi = (0x30, 0x46) if sf_kind == "e4m3" else (124, 131)

    def rand_sf(mn, l):
        t = ops.empty_sf(mn, k, l, device="cuda", dtype=sf_dtype, sf_vec=sf_vec)
        flat_ = torch.as_strided(t.view(torch.uint8), (t.numel(),), (1,))
        flat_.copy_(torch.randint(lo, hi, (t.numel(),), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8))
        return t

    sfa, sfb = rand_sf(m, 1), rand_sf(n, e)
    alpha = torch.ones(e, device="cuda")
    prob = torch.zeros(m, device="cuda")
    prob[r.dst_row.long()] = r.topk_prob.reshape(-1)
    prob = prob.view(m, 1, 1)
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    res = {"case": name, "op": "fc1_fp4", "cfg": {k_: v for k_, v in cfg.items()}, "m_rows": m, "flops": 2.0 * r.routed_rows * n * k}

    # Through the operator classes with no amax tensor: the reference's amax code (its atomic_max_float32) does not
    # compile with the CuTe DSL release of this image, and its wrapper always allocates amax for a bf16 D.
    def outputs():
        return dict(c_tensor=torch.empty_strided((m, n, 1), (n, 1, m * n), dtype=torch.bfloat16, device="cuda"),
                    d_tensor=torch.empty_strided((m, n // 2, 1), (n // 2, 1, m * n // 2), dtype=torch.bfloat16, device="cuda"))  # fmt: skip

    r_ref, r_own = outputs(), outputs()
    d_col_dummy = torch.empty_like(r_ref["d_tensor"])
    mk = dict(sample_prob=prob, mma_tiler_mn=(256, 256), sf_vec_size=sf_vec, m_aligned=256)
    op_ref = ref.GroupedGemmSwigluSm100(a, b, r_ref["c_tensor"], r_ref["d_tensor"], sfa, sfb, r.padded_offsets, alpha, d_col_dummy, **mk)
    op_own = ours.GroupedGemmSwigluSm100(a, b, r_own["c_tensor"], r_own["d_tensor"], sfa, sfb, r.padded_offsets, alpha, None, **mk)
    t0 = time.time()
    assert op_ref.check_support()
    op_ref.compile()
    assert op_own.check_support()
    op_own.compile()

    def run_ref():
        op_ref.execute(a, b, r_ref["c_tensor"], r_ref["d_tensor"], sfa, sfb, r.padded_offsets, alpha, d_col_tensor=d_col_dummy, prob_tensor=prob,
                       current_stream=stream)  # fmt: skip

    def run_own():
        op_own.execute(a, b, r_own["c_tensor"], r_own["d_tensor"], sfa, sfb, r.padded_offsets, alpha, prob_tensor=prob)

    run_ref()
    torch.cuda.synchronize()
    res["ref_first_call_s"] = time.time() - t0
    run_own()
    torch.cuda.synchronize()
    if PROFILE_ONLY:
        run_ref()
        run_own()
        torch.cuda.synchronize()
        return
    bits = lambda t: t[:m, :, 0].contiguous().view(torch.int16)  # noqa: E731
    res["c_equal_frac"] = float((bits(r_ref["c_tensor"]) == bits(r_own["c_tensor"])).float().mean())
    res["d_equal_frac"] = float((bits(r_ref["d_tensor"]) == bits(r_own["d_tensor"])).float().mean())
    if not name.startswith("fp4_tiny"):
        il_ref, il_own = timed_interleaved(run_ref, run_own, rounds=12)
        res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
        res["own_over_ref_interleaved"] = il_ref / il_own
        res["ref_tflops_interleaved"] = res["flops"] / (il_ref * 1e-3) / 1e12
        res["own_tflops_interleaved"] = res["flops"] / (il_own * 1e-3) / 1e12
    out.append(res)
    print(json.dumps(res), flush=True)
    if name.startswith("fp4_tiny"):
        def flat(t):
            t = t.view(torch.uint8)
            return torch.as_strided(t, (t.numel(),), (1,))

        np.savez_compressed(
            os.path.join(OUT_DIR, f"reference_kernel_{name}_golden.npz"),
            a=a8.cpu().numpy(), b=b8.cpu().numpy(), sfa=flat(sfa).cpu().numpy(), sfb=flat(sfb).cpu().numpy(),
            offsets=r.padded_offsets.cpu().numpy(), prob=prob.view(-1).cpu().numpy(),
            c=bits(r_ref["c_tensor"]).cpu().numpy(), d=bits(r_ref["d_tensor"]).cpu().numpy(),
            sf_vec=np.int32(sf_vec), sf_is_e4m3=np.int32(sf_kind == "e4m3"),
        )  # fmt: skip


def run_case_dswiglu(name, cfg, out):
    """dSwiGLU backward (grouped_gemm_dswiglu): fp8 operands, bf16 forward C, E4M3 D_row / D_col with row and column
    scales, dprob."""
    import cuda.bindings.driver as cuda
    from cudnn.grouped_gemm.grouped_gemm_dswiglu.api import grouped_gemm_dswiglu_wrapper_sm100 as ref_dswiglu  # the overlay

    import cudnn_frontend_b200 as ours
    from cudnn_frontend_b200 import synthetic

    p = synthetic.make_problem(cfg, "cuda", seed=13, m_aligned=256)
    e, n, k = cfg["experts"], cfg["n"], cfg["k"]
    m = p["m_rows"]
    g = torch.Generator(device="cuda").manual_seed(6)
    c_fwd = torch.empty((m, 2 * n), device="cuda").uniform_(-3, 3, generator=g).to(torch.bfloat16)
    c_fwd = torch.as_strided(c_fwd, (m, 2 * n, 1), (2 * n, 1, m * 2 * n))  # the reference checks the stride of the unit dimension too
    beta = torch.tensor([1.0, 0.5] * (e // 2) + [2.0] * (e % 2), device="cuda")
    norm = torch.tensor([1.0], dtype=torch.float32, device="cuda")
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    kw = dict(norm_const_tensor=norm, d_dtype=torch.float8_e4m3fn, sf_vec_size=32, m_aligned=256)
    res = {"case": name, "op": "dswiglu", "cfg": cfg, "m_rows": m, "flops": 2.0 * p["routing"].routed_rows * n * k}

    def run_ref():
        return ref_dswiglu(p["a"], p["b"], c_fwd, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], beta, p["prob"], mma_tiler_mn=(256, 256),
                           current_stream=stream, **kw)  # fmt: skip

    def run_own():
        return ours.grouped_gemm_dswiglu_wrapper_sm100(p["a"], p["b"], c_fwd, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], beta, p["prob"], **kw)

    t0 = time.time()
    r_ref = run_ref()
    torch.cuda.synchronize()
    res["ref_first_call_s"] = time.time() - t0
    r_own = run_own()
    torch.cuda.synchronize()
    if PROFILE_ONLY:
        run_ref()
        run_own()
        torch.cuda.synchronize()
        return

    def flat(t):
        t = t.view(torch.uint8)
        return torch.as_strided(t, (t.numel(),), (1,))

    for key in ("d_row_tensor", "d_col_tensor"):
        u = ulp(r_ref[key][:m].view(torch.uint8), r_own[key][:m].view(torch.uint8))
        res[key + "_equal_frac"] = float((u == 0).float().mean())
        res[key + "_within_1ulp_frac"] = float((u <= 1).float().mean())
    res["sfd_row_bytes_equal_frac"] = float((flat(r_ref["sfd_row_tensor"]) == flat(r_own["sfd_row_tensor"])).float().mean())
    res["sfd_col_bytes_equal_frac"] = float((flat(r_ref["sfd_col_tensor"]) == flat(r_own["sfd_col_tensor"])).float().mean())
    dp_r, dp_o = r_ref["dprob_tensor"].view(-1), r_own["dprob_tensor"].view(-1)
    res["dprob_rel_fro"] = float((dp_r - dp_o).norm() / dp_r.norm())
    if not name.endswith("tiny"):
        il_ref, il_own = timed_interleaved(run_ref, run_own, rounds=12)
        res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
        res["own_over_ref_interleaved"] = il_ref / il_own
    out.append(res)
    print(json.dumps(res), flush=True)
    if name.endswith("tiny"):
        np.savez_compressed(
            os.path.join(OUT_DIR, "reference_kernel_dswiglu_golden.npz"),
            a=p["a"][:, :, 0].view(torch.uint8).cpu().numpy(), b=p["b"].permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(),
            sfa=flat(p["sfa"]).cpu().numpy(), sfb=flat(p["sfb"]).cpu().numpy(), offsets=p["padded_offsets"].cpu().numpy(),
            prob=p["prob"].view(-1).cpu().numpy(), beta=beta.cpu().numpy(), c_fwd=c_fwd[:, :, 0].view(torch.int16).cpu().numpy(),
            d_row=r_ref["d_row_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(), d_col=r_ref["d_col_tensor"][:m, :, 0].view(torch.uint8).cpu().numpy(),
            sfd_row=flat(r_ref["sfd_row_tensor"]).cpu().numpy(), sfd_col=flat(r_ref["sfd_col_tensor"]).cpu().numpy(),
            dprob=r_ref["dprob_tensor"].view(-1).cpu().numpy(),
        )  # fmt: skip


def run_case_wgrad(name, cfg, out):
    """Weight gradient (grouped_gemm_wgrad): fp8 operands with E8M0 scales per 32 tokens, bf16 output, dense mode."""
    import cuda.bindings.driver as cuda
    from cudnn.grouped_gemm.grouped_gemm_wgrad.api import grouped_gemm_wgrad_wrapper_sm100 as ref_wgrad  # the overlay

    import cudnn_frontend_b200 as ours

    m, n, groups = cfg["m"], cfg["n"], cfg["groups"]
    tokens, e = sum(groups), len(groups)
    g = torch.Generator(device="cuda").manual_seed(23)
    a = torch.empty((m, tokens), device="cuda").uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn)
    b_store = torch.empty((n, tokens), device="cuda").uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn)
    b = b_store.t()  # (tokens, n), contiguous along the tokens
    cols = (tokens // 32 + 3) // 4 * 4

    def rand_sf(rows):
        rows_p = (rows + 127) // 128 * 128
        return torch.randint(124, 131, (rows_p, cols), generator=g, device="cuda", dtype=torch.int32).to(torch.uint8).view(torch.float8_e8m0fnu)

    sfa, sfb = rand_sf(m), rand_sf(n)
    offs = torch.tensor(np.cumsum(groups), dtype=torch.int32, device="cuda")
    stream = cuda.CUstream(torch.cuda.current_stream().cuda_stream)
    res = {"case": name, "op": "wgrad", "cfg": cfg, "flops": 2.0 * tokens * m * n}

    def run_ref():
        return ref_wgrad(a, b, sfa, sfb, offs, sf_vec_size=32, mma_tiler_mn=(256, 256), current_stream=stream)["wgrad_tensor"]

    def run_own():
        return ours.grouped_gemm_wgrad_wrapper_sm100(a, b, sfa, sfb, offs, sf_vec_size=32)["wgrad_tensor"]

    t0 = time.time()
    w_ref = run_ref()
    torch.cuda.synchronize()
    res["ref_first_call_s"] = time.time() - t0
    w_own = run_own()
    torch.cuda.synchronize()
    if PROFILE_ONLY:
        run_ref()
        run_own()
        torch.cuda.synchronize()
        return
    res["wgrad_equal_frac"] = float((w_ref.view(torch.int16) == w_own.view(torch.int16)).float().mean())
    res["wgrad_rel_fro"] = float((w_ref.float() - w_own.float()).norm() / w_ref.float().norm())
    if not name.endswith("tiny"):
        il_ref, il_own = timed_interleaved(run_ref, run_own, rounds=12)
        res["ref_ms_interleaved"], res["own_ms_interleaved"] = il_ref, il_own
        res["own_over_ref_interleaved"] = il_ref / il_own
        res["ref_tflops_interleaved"] = res["flops"] / (il_ref * 1e-3) / 1e12
        res["own_tflops_interleaved"] = res["flops"] / (il_own * 1e-3) / 1e12
    out.append(res)
    print(json.dumps(res), flush=True)
    if name.endswith("tiny"):
        np.savez_compressed(
            os.path.join(OUT_DIR, "reference_kernel_wgrad_golden.npz"),
            a=a.view(torch.uint8).cpu().numpy(), b=b_store.view(torch.uint8).cpu().numpy(), sfa=sfa.view(torch.uint8).cpu().numpy().reshape(-1),
            sfb=sfb.view(torch.uint8).cpu().numpy().reshape(-1), offsets=offs.cpu().numpy(), wgrad=w_ref.view(torch.int16).cpu().numpy(),
        )  # fmt: skip


PROFILE_ONLY = False
OWN_FIRST = False

CASES = {
    # reduced Mixtral shape for profiler captures (operands still exceed L2)
    "mid": dict(experts=8, k=4096, n=7168, tokens=4096, topk=2, routing="uniform"),
    # small enough to commit its inputs and the reference kernel's outputs as a fixture
    "tiny": dict(experts=2, k=128, n=128, tokens=128, topk=2, routing="uniform"),
    "tiny_e5m2": dict(experts=2, k=128, n=128, tokens=128, topk=2, routing="uniform", ab="e5m2"),
    "tiny_d_e5m2": dict(experts=2, k=128, n=128, tokens=128, topk=2, routing="uniform", d="e5m2"),
    # eight k-tiles deep (the accumulation across k-tiles and the wrap of the shared-memory ring), still small enough to commit
    "tiny_deepk": dict(experts=2, k=1024, n=128, tokens=64, topk=2, routing="uniform"),
    # scale factors generated with a bf16 D: D and D_col hold the scaled values (block maximum mapped to 1), amax too
    "tiny_d_bf16": dict(experts=2, k=128, n=128, tokens=128, topk=2, routing="uniform", d="bf16"),
    "small": dict(experts=4, k=512, n=512, tokens=512, topk=2, routing="uniform"),
    "c2": dict(experts=8, k=4096, n=28672, tokens=16384, topk=2, routing="uniform"),
    "c3": dict(experts=256, k=7168, n=4096, tokens=8192, topk=8, routing="zipf"),
    # FC2 (grouped_gemm_quant) cases: K = intermediate size, N = hidden size
    "fc2_tiny": dict(experts=2, k=128, n=256, tokens=128, topk=2, routing="uniform"),
    "fc2_mixtral": dict(experts=8, k=14336, n=4096, tokens=16384, topk=2, routing="uniform"),
    "c4": dict(experts=256, k=2048, n=7168, tokens=8192, topk=8, routing="zipf"),
    # reduced Mixtral-shape FC2 for profiler captures
    "fc2_mid": dict(experts=8, k=3584, n=4096, tokens=4096, topk=2, routing="uniform"),
}
FC2_CASES = ("fc2_tiny", "fc2_mixtral", "c4", "fc2_mid")
# unified GLU API (GeGLU + fused bias): glu_tiny records a fixture, glu_mid compares speed
CASES["glu_tiny"] = dict(experts=2, k=128, n=128, tokens=128, topk=2, routing="uniform")
CASES["glu_mid"] = dict(experts=8, k=4096, n=7168, tokens=4096, topk=2, routing="uniform")
GLU_CASES = ("glu_tiny", "glu_mid")
# FP4 operands: NVFP4 (E4M3 scales per 16), MXFP4 (E8M0 per 32) and E8M0 per 16; the tiny ones record fixtures
# (two k-tiles of 256 elements deep), the others compare speed
# backward pair: dSwiGLU (K = hidden, N = intermediate; D is 2 N wide) and the weight gradient (experts split the tokens)
CASES["dswiglu_tiny"] = dict(experts=2, k=256, n=128, tokens=128, topk=2, routing="uniform")
CASES["dswiglu_mid"] = dict(experts=8, k=4096, n=3584, tokens=4096, topk=2, routing="uniform")
CASES["wgrad_tiny"] = dict(m=384, n=640, groups=[256, 384])
CASES["wgrad_mid"] = dict(m=4096, n=7168, groups=[4096] * 8)
CASES["fp4_tiny_nvfp4"] = dict(experts=2, k=512, n=128, tokens=128, topk=2, routing="uniform", sf=(16, "e4m3"))
CASES["fp4_tiny_mxfp4"] = dict(experts=2, k=512, n=128, tokens=128, topk=2, routing="uniform", sf=(32, "e8m0"))
CASES["fp4_tiny_e8m0x16"] = dict(experts=2, k=512, n=128, tokens=128, topk=2, routing="uniform", sf=(16, "e8m0"))
CASES["fp4_mid_nvfp4"] = dict(experts=8, k=4096, n=7168, tokens=4096, topk=2, routing="uniform", sf=(16, "e4m3"))
CASES["fp4_c2_nvfp4"] = dict(experts=8, k=4096, n=28672, tokens=16384, topk=2, routing="uniform", sf=(16, "e4m3"))
CASES["fp4_c2_mxfp4"] = dict(experts=8, k=4096, n=28672, tokens=16384, topk=2, routing="uniform", sf=(32, "e8m0"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--cases", default="tiny")
    ap.add_argument("--own-first", action="store_true", help="time this repository's kernel before the reference's")
    ap.add_argument("--profile", action="store_true", help="launch each kernel twice and exit (for ncu)")
    ap.add_argument("--out", default=None, help="output directory (else the environment variable B200MOE_OUT_DIR)")
    args = ap.parse_args()
    global PROFILE_ONLY, OWN_FIRST, OUT_DIR
    OUT_DIR = args.out or OUT_DIR
    if not OUT_DIR:
        ap.error("give the output directory with --out or B200MOE_OUT_DIR")
    PROFILE_ONLY = args.profile
    OWN_FIRST = args.own_first
    os.makedirs(OUT_DIR, exist_ok=True)
    out = []
    for name in args.cases.split(","):
        try:
            (run_case_dswiglu if name.startswith("dswiglu") else run_case_wgrad if name.startswith("wgrad") else run_case_fp4 if name.startswith("fp4_") else run_case_glu if name in GLU_CASES else run_case_fc2 if name in FC2_CASES else run_case)(
                name, CASES[name], out)
        except Exception as exc:  # keep going: a JIT failure of one case is a result too
            out.append({"case": name, "error": f"{type(exc).__name__}: {exc}"})
            traceback.print_exc()
        with open(os.path.join(OUT_DIR, f"reference_kernels_{args.cases.replace(',', '_')}.json"), "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
