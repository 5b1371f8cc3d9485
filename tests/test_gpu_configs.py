"""Parity at the sizes the benchmark configurations use.

The small cases of test_gpu_parity.py never leave one raster group, one or two k-tiles and a
handful of experts.  Here the CUDA path runs

  * one expert of more than 9000 rows (three raster groups of the tile schedule),
  * 256 experts with Zipf-distributed rows, empty experts included, at K = 7168 (56 k-tiles: the
    shared-memory ring wraps 9 to 14 times per tile), checked in full against the oracle,
  * the benchmark's configurations c2, c3 (dense and discrete weights) and c4 at full size, with
    the oracle evaluated on whole row tiles of three experts (the one with most rows, the one
    with fewest, the last non-empty one) over all of N,
  * configuration c1 (the reference's CPU-runnable bf16 case) after MXFP8 quantisation.

Gates as everywhere: E8M0 bytes bit-exact up to the documented power-of-two ties, bf16 relative
Frobenius error <= 2e-2, E4M3 within 1 ULP on >= 99.9 %.
"""

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H
from tests import test_gpu_parity as P

pytestmark = pytest.mark.gpu

BF16_GATE = 2e-2


@pytest.fixture(params=["single", "pair"])
def tile_mode(request, monkeypatch):
    monkeypatch.setenv("B200MOE_TILE_MODE", request.param)
    return request.param


def _fp8_bytes(rng, shape, max_exp_field=8):
    """Random E4M3 bytes with a bounded exponent field (|value| <= 3.75 for the default): no NaN codes,
    and sums over thousands of products stay far from float32 overflow."""
    sign = rng.integers(0, 2, shape, dtype=np.uint8) << 7
    exp = rng.integers(0, max_exp_field + 1, shape, dtype=np.uint8) << 3
    return sign | exp | rng.integers(0, 8, shape, dtype=np.uint8)


# ---------------------------------------------------------------------------------------------
# (a) more than one raster group
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["fc1", "fc2"])
def test_expert_with_three_raster_groups(kind, tile_mode):
    """9100 rows of one expert = 72 row tiles of 128 (36 of 256): raster groups hold 4096 rows, so the
    schedule walks three groups, the last one partial; the second expert (130 rows) is a light one."""
    fp8 = kind == "fc1"
    out, ref, info = P._run(kind, 51, [9100, 130], 512, 256, d_fp8=fp8)
    P._check(kind, out, ref, info, d_fp8=fp8)


# ---------------------------------------------------------------------------------------------
# (b) 256 experts, Zipf rows, empty experts, deep K
# ---------------------------------------------------------------------------------------------
def _zipf_groups(experts, slots, empty, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.arange(1, experts + 1, dtype=torch.float32).pow(-1.2)[torch.randperm(experts, generator=g)]
    w[list(empty)] = 0
    ids = torch.multinomial(w, slots, replacement=True, generator=g)
    return torch.bincount(ids, minlength=experts).tolist()


@pytest.mark.parametrize("kind,n,k", [("fc1", 512, 7168), ("fc2", 512, 2048)])
def test_256_experts_zipf_rows_deep_k(kind, n, k, tile_mode):
    e = 256
    groups = _zipf_groups(e, 8192, empty=(0, 5, 100, 254, 255), seed=7)
    assert groups[0] == 0 and groups[-1] == 0 and max(groups) > 600 and sum(1 for g_ in groups if g_ == 0) >= 5
    rng = np.random.default_rng(77)
    m_rows = orc.padded_end_offsets(groups, 128)[0]
    a = _fp8_bytes(rng, (m_rows, k))
    b = _fp8_bytes(rng, (e, n, k), max_exp_field=6)
    sfa = rng.integers(125, 130, (m_rows, k // 32), dtype=np.uint8)
    sfb = rng.integers(125, 130, (e, n, k // 32), dtype=np.uint8)
    out, ref, info = P._run(kind, 52, groups, n, k, d_fp8=True, operands=(a, b, sfa, sfb), write_c=False)
    P._check(kind, out, ref, info, d_fp8=True)


# ---------------------------------------------------------------------------------------------
# (c) the benchmark's configurations at full size, oracle on sampled row tiles
# ---------------------------------------------------------------------------------------------
def _flat_bytes(sf6d):
    t = sf6d.view(torch.uint8)
    return torch.as_strided(t, (t.numel(),), (1,))


def _sample_experts(counts):
    """(expert, first row inside the expert, rows) of the tiles to check: the first and the last row tile
    of the expert with most rows, the whole expert with fewest (non-zero) rows, the last tile of the last
    non-empty expert."""
    counts = np.asarray(counts)
    nz = np.nonzero(counts)[0]
    heavy = int(nz[np.argmax(counts[nz])])
    light = int(nz[np.argmin(counts[nz])])
    last = int(nz[-1])
    picks = [(heavy, 0, 128), (heavy, (int(counts[heavy]) - 1) // 128 * 128, None), (light, 0, None), (last, (int(counts[last]) - 1) // 128 * 128, None)]
    out = []
    for ex, first, rows in picks:
        rows = int(min(128, counts[ex] - first)) if rows is None else int(min(rows, counts[ex]))
        if (ex, first) not in [(o[0], o[1]) for o in out]:
            out.append((ex, first, rows))
    return out


def _host_rows(t2d, r0, r1):
    return t2d[r0:r1].contiguous().view(torch.uint8).cpu().numpy()


def _check_sampled_tiles(kind, prob_, b_store, sfb6, e, n, k, outs, d_fp8, prob_rows, counts):
    """Oracle on the sampled tiles.  ``outs``: dict with d (and sfd_row, d_col, sfd_col, amax) tensors."""
    offs = prob_["padded_offsets"].cpu().numpy()
    m_rows = int(offs[-1])
    starts = np.concatenate([[0], offs[:-1]])
    a2d = prob_["a"][:, :, 0]
    sfa_flat = _flat_bytes(prob_["sfa"]).cpu().numpy()
    sfb_flat = _flat_bytes(sfb6)
    rest_k = (k // 32 + 3) // 4
    per_expert_sf = ((n + 127) // 128) * rest_k * 512
    n_out = n // 2 if kind == "fc1" else n
    d_all = outs["d"][:, :, 0]
    for ex, first, rows in _sample_experts(counts):
        r0 = int(starts[ex]) + first
        a = _host_rows(a2d, r0, r0 + rows)
        kb = np.arange(k // 32)
        sfa = sfa_flat[orc.sf_offset(np.arange(r0, r0 + rows)[:, None], kb[None, :], rest_k)]
        b = b_store[ex].contiguous().view(torch.uint8).cpu().numpy()[None]
        sfb = orc.sf_unpack(sfb_flat[ex * per_expert_sf : (ex + 1) * per_expert_sf].cpu().numpy(), n, k // 32, 1)
        pr = None if prob_rows is None else prob_rows[r0 : r0 + rows].float().cpu().numpy()
        local_offs = np.asarray([rows], dtype=np.int32)
        one = np.ones(1, dtype=np.float32)
        fn = orc.fc1_reference if kind == "fc1" else orc.fc2_reference
        ref = fn(a, sfa, b, sfb, local_offs, one, pr, norm_const=1.0 if d_fp8 else None)
        if not d_fp8:
            got = d_all[r0 : r0 + rows].float().cpu().numpy()
            assert H.rel_fro(got, ref["d"][:rows]) <= BF16_GATE, (ex, first)
            if rows == counts[ex]:  # the sample covers the whole expert: its amax is fully determined
                np.testing.assert_allclose(outs["amax"].view(-1)[ex].item(), ref["amax"][0], rtol=1e-2)
        else:
            got = _host_rows(d_all, r0, r0 + rows)
            sf_all = _flat_bytes(outs["sfd_row"]).cpu().numpy()
            nb = (n_out + 31) // 32
            sfr = sf_all[orc.sf_offset(np.arange(r0, r0 + rows)[:, None], np.arange(nb)[None, :], (nb + 3) // 4)]
            mism = sfr != ref["sfd_row"]
            assert mism.mean() <= 1e-3, f"expert {ex}: {mism.sum()} of {mism.size} row scales differ"
            same = np.repeat(~mism, 32, axis=1)[:, :n_out]
            H.assert_e4m3_within_one_ulp(got[same], ref["d_q"][same])
            if outs.get("d_col") is not None and first == 0 and rows % 32 == 0:
                # complete 32-row blocks from the expert's first row: column scales are determined by the sample
                gotc = _host_rows(outs["d_col"][:, :, 0], r0, r0 + rows)
                sfc_all = _flat_bytes(outs["sfd_col"]).cpu().numpy()
                rb = np.arange(r0 // 32, (r0 + rows) // 32)
                sfc = sfc_all[orc.sf_offset(np.arange(n_out)[:, None], rb[None, :], ((m_rows + 31) // 32 + 3) // 4)]
                mism = sfc != ref["sfd_col"]
                assert mism.mean() <= 1e-3, f"expert {ex}: {mism.sum()} of {mism.size} column scales differ"
                same = np.repeat(~mism.T, 32, axis=0)[:rows]
                H.assert_e4m3_within_one_ulp(gotc[same], ref["d_col_q"][same])


def test_config_c2_full_size_sampled():
    """Mixtral-shape FC1 exactly as the benchmark runs it (bf16 D + per-expert amax, groups padded to
    128, the library's own tile-mode choice), then with the reference wrapper's output set."""
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops, synthetic

    p = synthetic.make_problem("c2", "cuda", seed=0, m_aligned=128)
    cfg = p["cfg"]
    e, n, k, m = cfg["experts"], cfg["n"], cfg["k"], p["m_rows"]
    counts = p["routing"].counts.cpu().numpy()
    b_store = p["b"].permute(2, 0, 1)
    d = torch.empty((m, n // 2, 1), dtype=torch.bfloat16, device="cuda")
    amax = torch.full((e, 1), float("-inf"), device="cuda")
    op = cf.GroupedGemmSwigluSm100(p["a"], p["b"], None, d, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], None,
                                   sample_amax=amax, sample_prob=p["prob"], sf_vec_size=32, m_aligned=128)  # fmt: skip
    assert op.check_support()
    op.compile()
    op.execute(p["a"], p["b"], None, d, p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], amax_tensor=amax, prob_tensor=p["prob"])
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    _check_sampled_tiles("fc1", p, b_store, p["sfb"], e, n, k, dict(d=d, amax=amax), False, p["prob"].view(-1), counts)
    # amax of every expert against max |D| over its rows (padding rows are zero rows): a checksum over all
    # tiles.  amax is taken before the bf16 rounding of D; rounding is monotonic, so the rounded amax is the
    # maximum of the rounded values.
    offs = p["padded_offsets"].cpu().tolist()
    start = 0
    for ex, end in enumerate(offs):
        assert amax[ex].to(torch.bfloat16).item() == d[start:end].abs().max().item(), ex
        start = end
    del d
    # the reference wrapper's output set: C, E4M3 D and D_col, row and column scales
    res = cf.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"],
                                               norm_const_tensor=torch.ones(1, device="cuda"), prob_tensor=p["prob"],
                                               d_dtype=torch.float8_e4m3fn, sf_vec_size=32, m_aligned=128)  # fmt: skip
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    _check_sampled_tiles("fc1", p, b_store, p["sfb"], e, n, k,
                         dict(d=res["d_tensor"], sfd_row=res["sfd_row_tensor"], d_col=res["d_col_tensor"], sfd_col=res["sfd_col_tensor"]),
                         True, p["prob"].view(-1), counts)  # fmt: skip


def test_configs_c3_and_c4_full_size_sampled():
    """DeepSeek-shape FC1 with dense and with discrete weights (E = 256, K = 7168, Zipf rows), its MXFP8
    output fed to the DeepSeek-shape FC2 (K = 2048, N = 7168) as configuration c4 does; static and
    dynamic tile scheduler."""
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops, synthetic

    dev = "cuda"
    p = synthetic.make_problem("c3", dev, seed=1, m_aligned=128)
    cfg = p["cfg"]
    e, n, k, m = cfg["experts"], cfg["n"], cfg["k"], p["m_rows"]
    counts = p["routing"].counts.cpu().numpy()
    norm = torch.ones(1, device=dev)

    def fc1_outputs():
        return dict(d=torch.zeros((m, n // 2, 1), dtype=torch.float8_e4m3fn, device=dev), d_col=torch.zeros((m, n // 2, 1), dtype=torch.float8_e4m3fn, device=dev),
                    sfd_row=ops.empty_sf(m, n // 2, 1, device=dev, zero=True), sfd_col=ops.empty_sf(n // 2, m, 1, device=dev, zero=True))  # fmt: skip

    o = fc1_outputs()
    op = cf.GroupedGemmSwigluSm100(p["a"], p["b"], None, o["d"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], o["d_col"],
                                   sample_sfd_row=o["sfd_row"], sample_sfd_col=o["sfd_col"], sample_norm_const=norm, sf_vec_size=32,
                                   m_aligned=128)  # fmt: skip
    assert op.check_support()
    op.compile()
    op.execute(p["a"], p["b"], None, o["d"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], d_col_tensor=o["d_col"],
               sfd_row_tensor=o["sfd_row"], sfd_col_tensor=o["sfd_col"], norm_const_tensor=norm)  # fmt: skip
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    b_store = p["b"].permute(2, 0, 1)
    _check_sampled_tiles("fc1", p, b_store, p["sfb"], e, n, k, o, True, None, counts)

    # discrete weights (one allocation per expert) and the dynamic scheduler: bitwise the same result
    sf_flat = _flat_bytes(p["sfb"])
    per = sf_flat.numel() // e
    b_list = [b_store[i].clone() for i in range(e)]
    sf_list = [sf_flat[i * per : (i + 1) * per].clone() for i in range(e)]
    b_ptrs = torch.tensor([x.data_ptr() for x in b_list], dtype=torch.int64, device=dev)
    sfb_ptrs = torch.tensor([x.data_ptr() for x in sf_list], dtype=torch.int64, device=dev)
    for dynamic in (False, True):
        o2 = fc1_outputs()
        opd = cf.DiscreteGroupedGemmSwigluSm100(p["a"], e, (n, k), torch.float8_e4m3fn, None, o2["d"], p["sfa"], p["padded_offsets"], p["alpha"],
                                                o2["d_col"], sample_sfd_row=o2["sfd_row"], sample_sfd_col=o2["sfd_col"], sample_norm_const=norm,
                                                sf_vec_size=32, m_aligned=128, use_dynamic_sched=dynamic)  # fmt: skip
        assert opd.check_support()
        opd.compile()
        opd.execute(p["a"], b_ptrs, None, o2["d"], p["sfa"], sfb_ptrs, p["padded_offsets"], p["alpha"], d_col_tensor=o2["d_col"],
                    sfd_row_tensor=o2["sfd_row"], sfd_col_tensor=o2["sfd_col"], norm_const_tensor=norm)  # fmt: skip
        torch.cuda.synchronize()
        assert ops.device_status(clear=True) == 0
        for key in ("d", "d_col"):
            assert torch.equal(o[key].view(torch.uint8), o2[key].view(torch.uint8)), (key, dynamic)
        for key in ("sfd_row", "sfd_col"):
            assert torch.equal(_flat_bytes(o[key]), _flat_bytes(o2[key])), (key, dynamic)
        del o2, opd
    del b_list, sf_list, b_store
    del p["b"], p["sfb"]
    torch.cuda.empty_cache()

    # c4: FC2 on FC1's quantised output
    cfg4 = synthetic.CONFIGS["c4"]
    n4, k4 = cfg4["n"], cfg4["k"]
    assert k4 == n // 2
    w2, sfw2 = synthetic.make_weights(e, n4, k4, 7, dev)
    p4 = dict(a=o["d"], sfa=o["sfd_row"], padded_offsets=p["padded_offsets"])
    res = {}
    for dynamic in (False, True):
        r = cf.grouped_gemm_quant_wrapper_sm100(o["d"], o["sfd_row"], p["padded_offsets"], p["alpha"], b_tensor=w2, sfb_tensor=sfw2,
                                                norm_const_tensor=norm, prob_tensor=p["prob"], d_dtype=torch.float8_e4m3fn, sf_vec_size=32,
                                                m_aligned=128, use_dynamic_sched=dynamic)  # fmt: skip
        torch.cuda.synchronize()
        assert ops.device_status(clear=True) == 0
        res[dynamic] = r
    for key in ("d_tensor", "d_col_tensor"):
        assert torch.equal(res[False][key].view(torch.uint8), res[True][key].view(torch.uint8)), key
    for key in ("sfd_row_tensor", "sfd_col_tensor"):
        assert torch.equal(_flat_bytes(res[False][key]), _flat_bytes(res[True][key])), key
    r = res[False]
    _check_sampled_tiles("fc2", p4, w2.permute(2, 0, 1), sfw2, e, n4, k4,
                         dict(d=r["d_tensor"], sfd_row=r["sfd_row_tensor"], d_col=r["d_col_tensor"], sfd_col=r["sfd_col_tensor"]),
                         True, p["prob"].view(-1), counts)  # fmt: skip


# ---------------------------------------------------------------------------------------------
# (d) configuration c1: the reference's CPU-runnable bf16 case
# ---------------------------------------------------------------------------------------------
def test_config_c1_against_the_bf16_reference_path():
    """c1 (E=4, K=256, N=1024, 512 tokens top-1): the reference has no bf16 grouped kernel; its PyTorch
    path computes this case with unit scale factors on bf16 operands.  The CUDA path quantises both
    operands to MXFP8 first.  Two checks: (1) against the oracle on the same quantised operands, at the
    2e-2 gate; (2) against the bf16, unit-scale result: E4M3 keeps three mantissa bits, which alone puts
    the quantised path 3.8 % (C) and 5.4 % (D) away from the bf16 result in relative Frobenius norm (the
    CPU oracle measures the same distance), so that comparison is bounded by 8e-2, not 2e-2."""
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import synthetic

    p = synthetic.make_problem("c1", "cuda", seed=0, m_aligned=256)
    cfg = p["cfg"]
    e, n, k, m = cfg["experts"], cfg["n"], cfg["k"], p["m_rows"]
    res = cf.grouped_gemm_swiglu_wrapper_sm100(p["a"], p["b"], p["sfa"], p["sfb"], p["padded_offsets"], p["alpha"], sf_vec_size=32, m_aligned=256)
    torch.cuda.synchronize()
    c = res["c_tensor"][:, :, 0].float().cpu().numpy()
    d = res["d_tensor"][:, :, 0].float().cpu().numpy()
    offs = p["padded_offsets"].cpu().numpy()
    a = p["a"][:, :, 0].view(torch.uint8).cpu().numpy()
    b = p["b"].permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy()
    sfa = H.sf_to_numpy(p["sfa"], m, k // 32)[0]
    sfb = H.sf_to_numpy(p["sfb"], n, k // 32, e)
    ref = orc.fc1_reference(a, sfa, b, sfb, offs, np.ones(e, dtype=np.float32), None)
    assert H.rel_fro(c, ref["c"]) <= BF16_GATE and H.rel_fro(d, ref["d"]) <= BF16_GATE
    np.testing.assert_allclose(res["amax_tensor"].cpu().numpy().reshape(-1), ref["amax"], rtol=1e-2)
    # the bf16 unit-scale reference of the same tokens and weights: dequantise nothing, use the originals
    x = p["x"].float().cpu().numpy()
    dst = p["routing"].dst_row.cpu().numpy()
    xg = np.zeros((m, k), dtype=np.float32)
    xg[dst] = x
    g = torch.Generator(device="cuda").manual_seed(2)
    w = (torch.randn(e * n, k, generator=g, device="cuda") * 0.02).to(torch.bfloat16).float().cpu().numpy().reshape(e, n, k)
    c_bf = np.zeros((m, n), dtype=np.float32)
    start = 0
    for ex, end in enumerate(offs.tolist()):
        c_bf[start:end] = xg[start:end] @ w[ex].T
        start = end
    d_bf = orc.swiglu_interleaved(c_bf, None)
    assert H.rel_fro(c[dst], c_bf[dst]) <= 8e-2
    assert H.rel_fro(d[dst], d_bf[dst]) <= 8e-2


# ---------------------------------------------------------------------------------------------
# failure paths, in the forms that cannot fault a GPU
# ---------------------------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_the_next_launch_is_correct(tile_mode):
    """A launch whose B-side producer issues no load (test hook) on a one-CTA (one-pair) grid with a
    20 ms wait limit: the MMA warp's wait for the stage (or the epilogue's for the accumulator) runs out,
    the kernel takes its abort path (abort flag, fall-through, TMEM freed) and returns; the status word
    names the wait.  The next ordinary launch on the same context must be correct."""
    import time

    from cudnn_frontend_b200 import ops

    groups, n, k = [256, 128], 512, 256
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands(81, valid, n, k, len(groups))
    H.zero_padding_rows(a, groups, aligned)
    ta, tb = H.dev_fp8(a).view(valid, k, 1), H.dev_fp8(b).permute(1, 2, 0)
    tsfa, tsfb = H.dev_sf(sfa, valid, k), H.dev_sf(sfb, n, k, len(groups))
    toffs = torch.from_numpy(offs).cuda()
    alpha = torch.ones(len(groups), device="cuda")
    prob = torch.rand(valid, device="cuda") + 0.1
    d = torch.zeros((valid, n, 1), dtype=torch.bfloat16, device="cuda")
    amax = torch.full((len(groups), 1), float("-inf"), device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    common = dict(a=ta, sfa=tsfa, b=tb, sfb=tsfb, padded_offsets=toffs, alpha=alpha, prob=prob, d=d, amax=amax, m_rows=valid, n=n, k=k,
                  num_experts=len(groups))  # fmt: skip
    assert ops.device_status(clear=True) == 0
    t0 = time.perf_counter()
    ops.launch_grouped_gemm("fc2", **common, sm_margin=sms - 2, wait_limit_ms=20, test_skip_b_loads=True)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    status = ops.device_status(clear=True)
    assert status in (101, 102, 104), status
    assert elapsed < 2.0, f"the starved launch took {elapsed:.2f} s"
    # the context is intact: an ordinary launch computes the right answer
    d.zero_()
    amax.fill_(float("-inf"))
    ops.launch_grouped_gemm("fc2", **common)
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    ref = orc.fc2_reference(a, sfa, b, sfb, offs, np.ones(len(groups), dtype=np.float32), prob.cpu().numpy())
    assert H.rel_fro(d[:, :, 0].float().cpu().numpy(), ref["d"]) <= BF16_GATE


def test_dispatch_row_outside_the_peer_buffer_is_skipped_and_reported():
    """b200moe_dispatch_quantize_peer with a destination row beyond row_capacity: the store is skipped,
    nothing outside the buffers is written, and the status word reads 301."""
    from cudnn_frontend_b200 import moe, ops
    from cudnn_frontend_b200.peer_memory import PeerBuffer

    t, k, h, e = 64, 2, 256, 4
    g = torch.Generator().manual_seed(5)
    x = torch.randn(t, h, generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32).cuda()
    prob = torch.rand(t * k, generator=g).cuda()
    counts, _, local_row = moe.route(ids.view(-1), e, 1)
    cap = 256
    pitch = moe.dispatch_record_pitch(h)
    q = PeerBuffer(cap * h)
    rec = PeerBuffer(cap * pitch)
    q.local.fill_(0xAB)
    rec.local.fill_(0xFF)
    guard_q = q.local.clone()
    assert ops.device_status(clear=True) == 0
    # every row of expert 3 is sent beyond the capacity; the others land inside
    delta = torch.zeros(e, dtype=torch.int32, device="cuda")
    delta[3] = cap + 1000
    moe.dispatch_quantize_peer(x, ids, local_row, delta, prob, e, 1, 0, t * k, cap, q.ptrs_dev, rec.ptrs_dev)
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 301
    rows_in = int(counts[:3].sum().item())
    assert rows_in > 0 and int(counts[3].item()) > 0
    changed = (q.local.view(cap, h) != guard_q.view(cap, h)).any(dim=1)
    assert int(changed.sum().item()) <= rows_in and not bool(changed[rows_in:].any())
    q.close()
    rec.close()
