"""dSwiGLU (backward of FC1's activation) through the operator class and the wrapper against the CPU oracle and
the fixture made by the reference's own PyTorch function.

Cases follow the reference's matrix (test/python/fe_api/test_grouped_gemm_dswiglu_utils.py:24-130): fp8 operands with
an E4M3 D_row / D_col and row and column scales, C in bf16 or E4M3, B K- or N-major, discrete_col_sfd on and off;
FP4 operands with a bf16 or float32 D_row and amax.  Gates: E8M0 bytes equal but for block maxima that land on a
power of two (at most 1e-3 of them), E4M3 within 1 ULP on 99.9 % where the scales agree, bf16 / float32 outputs and
dprob within 2e-2 relative Frobenius error.
"""

import os

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["single", "pair"])
def tile_mode(request, monkeypatch):
    monkeypatch.setenv("B200MOE_TILE_MODE", request.param)
    return request.param


def _bf16_np(x):
    return torch.from_numpy(x).to(torch.bfloat16).float().numpy()


def _case(seed, groups, n, k, *, c_dtype=torch.bfloat16, n_major=False, discrete_col_sfd=False, m_aligned=128, wrapper=False, norm=1.0):
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops

    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, m_aligned)
    a, b, sfa, sfb = H.gen_operands(seed, valid, n, k, e)
    H.zero_padding_rows(a, groups, aligned)
    rng = np.random.default_rng(seed)
    alpha = rng.integers(1, 3, e).astype(np.float32)
    beta = rng.choice([0.5, 1.0, 2.0], e).astype(np.float32)
    prob = rng.uniform(0.1, 1.0, valid).astype(np.float32)
    c_t = torch.from_numpy(rng.uniform(-3, 3, (valid, 2 * n)).astype(np.float32)).to(c_dtype)
    c_f32 = c_t.float().numpy()
    ref = orc.dswiglu_reference(a, sfa, b, sfb, c_f32, offs, alpha, beta, prob, norm_const=norm)

    ta = H.dev_fp8(a).view(valid, k, 1)
    tb_store = H.dev_fp8(b)
    tb = tb_store.transpose(1, 2).contiguous().permute(2, 1, 0) if n_major else tb_store.permute(1, 2, 0)
    tsfa, tsfb = H.dev_sf(sfa, valid, k), H.dev_sf(sfb, n, k, e)
    tc = c_t.cuda().view(valid, 2 * n, 1)
    toffs, talpha, tbeta = torch.from_numpy(offs).cuda(), torch.from_numpy(alpha).cuda(), torch.from_numpy(beta).cuda()
    tprob = torch.from_numpy(prob).cuda().view(valid, 1, 1)
    tnorm = torch.tensor([norm], device="cuda")
    if wrapper:
        out = cf.grouped_gemm_dswiglu_wrapper_sm100(ta, tb, tc, tsfa, tsfb, toffs, talpha, tbeta, tprob, norm_const_tensor=tnorm, d_dtype=torch.float8_e4m3fn,
                                                    sf_vec_size=32, m_aligned=m_aligned, discrete_col_sfd=discrete_col_sfd)  # fmt: skip
    else:
        d_row = torch.zeros((valid, 2 * n, 1), dtype=torch.float8_e4m3fn, device="cuda")
        d_col = torch.zeros_like(d_row)
        dprob = torch.zeros((valid, 1, 1), device="cuda")
        sfd_row, sfd_col = ops.empty_sf(valid, 2 * n, 1, zero=True), ops.empty_sf(2 * n, valid, 1, zero=True)
        op = cf.GroupedGemmDswigluSm100(ta, tb, tc, d_row, d_col, tsfa, tsfb, toffs, talpha, tbeta, tprob, dprob, sample_sfd_row=sfd_row,
                                        sample_sfd_col=sfd_col, sample_norm_const=tnorm, sf_vec_size=32, m_aligned=m_aligned,
                                        discrete_col_sfd=discrete_col_sfd)  # fmt: skip
        assert op.check_support()
        op.compile()
        op.execute(ta, tb, tc, d_row, d_col, tsfa, tsfb, toffs, talpha, tbeta, tprob, dprob, sfd_row_tensor=sfd_row, sfd_col_tensor=sfd_col,
                   norm_const_tensor=tnorm)  # fmt: skip
        out = dict(d_row_tensor=d_row, d_col_tensor=d_col, dprob_tensor=dprob, sfd_row_tensor=sfd_row, sfd_col_tensor=sfd_col)
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    return ref, out, valid, offs, groups, aligned


def _check_fp8_outputs(ref, out, valid, n2, offs, groups, aligned, discrete_col_sfd=False):
    sfr = H.sf_to_numpy(out["sfd_row_tensor"], valid, n2 // 32)[0]
    assert (sfr != ref["sfd_row"]).mean() <= 1e-3
    dq = out["d_row_tensor"][:, :, 0].view(torch.uint8).cpu().numpy()
    same = np.repeat(sfr == ref["sfd_row"], 32, axis=1)
    H.assert_e4m3_within_one_ulp(dq[same], ref["d_q"][same])
    # dequantised D against the float32 gradient
    deq = orc.dequantize_rows(dq, sfr)
    assert H.rel_fro(deq, ref["d"]) <= 6e-2  # E4M3 carries 3 mantissa bits
    np.testing.assert_allclose(out["dprob_tensor"].view(-1).cpu().numpy(), ref["dprob"], rtol=2e-2, atol=2e-2 * np.abs(ref["dprob"]).max())
    if not discrete_col_sfd:
        sfc = H.sf_to_numpy(out["sfd_col_tensor"], n2, valid // 32)[0]
        assert (sfc != ref["sfd_col"]).mean() <= 1e-3
        dcq = out["d_col_tensor"][:, :, 0].view(torch.uint8).cpu().numpy()
        same_c = np.repeat((sfc == ref["sfd_col"]).T, 32, axis=0)
        H.assert_e4m3_within_one_ulp(dcq[same_c], ref["d_col_q"][same_c])
    else:
        # every expert has its own block of column scales, rows counted from the expert's first row
        flat = torch.as_strided(out["sfd_col_tensor"].view(torch.uint8), (out["sfd_col_tensor"].numel(),), (1,)).cpu().numpy()
        start = 0
        for g_, al in zip(groups, aligned):
            if al:
                rows = al
                blk = flat[(start // 128) * ((n2 + 127) // 128) * 512 :]
                got = orc.sf_unpack(blk, n2, rows // 32)[0]
                _, want = orc.quantize_cols(ref["d"][start : start + rows], 1.0)
                assert (got != want).mean() <= 2e-3
            start += al


@pytest.mark.parametrize("c_dtype", [torch.bfloat16, torch.float8_e4m3fn])
@pytest.mark.parametrize("n_major", [False, True])
def test_dswiglu_fp8_matches_oracle(tile_mode, c_dtype, n_major):
    groups, n, k = [200, 0, 128, 300], 256, 384
    ref, out, valid, offs, groups, aligned = _case(5, groups, n, k, c_dtype=c_dtype, n_major=n_major)
    _check_fp8_outputs(ref, out, valid, 2 * n, offs, groups, aligned)


def test_dswiglu_wrapper_ragged_n_and_discrete_col_sfd(tile_mode):
    # n = 160: five 32-column blocks, the tile's last three blocks lie beyond N; per-expert column scale blocks
    ref, out, valid, offs, groups, aligned = _case(9, [256, 128, 384], 160, 256, wrapper=True, discrete_col_sfd=True)
    _check_fp8_outputs(ref, out, valid, 320, offs, groups, aligned, discrete_col_sfd=True)
    ref, out, valid, offs, groups, aligned = _case(10, [256, 128, 384], 160, 256, wrapper=True, m_aligned=256)
    _check_fp8_outputs(ref, out, valid, 320, offs, groups, aligned)


def test_dswiglu_matches_the_reference_pytorch_fixture(golden_dir, tile_mode):
    """Inputs and float32 outputs of the reference's run_grouped_gemm_dswiglu_ref (tests/golden/dswiglu.npz, made by
    tests/golden/make_golden.py): the kernel with FP4-style outputs disabled is compared through its E4M3 D_row."""
    import cudnn_frontend_b200 as cf

    g = np.load(os.path.join(golden_dir, "dswiglu.npz"))
    m, k = g["a"].shape
    e, n, _ = g["b"].shape
    c_bits = torch.from_numpy(g["c_fwd"].astype(np.int16)).view(torch.bfloat16)
    out = cf.grouped_gemm_dswiglu_wrapper_sm100(
        H.dev_fp8(g["a"]).view(m, k, 1), H.dev_fp8(g["b"]).permute(1, 2, 0), c_bits.cuda().view(m, 2 * n, 1), H.dev_sf(g["sfa"], m, k),
        H.dev_sf(g["sfb"], n, k, e), torch.from_numpy(g["offsets"]).cuda(), torch.from_numpy(g["alpha"]).cuda(), torch.from_numpy(g["beta"]).cuda(),
        torch.from_numpy(g["prob"]).cuda().view(m, 1, 1), norm_const_tensor=torch.ones(1, device="cuda"), d_dtype=torch.float8_e4m3fn, sf_vec_size=32,
        m_aligned=256)  # fmt: skip
    torch.cuda.synchronize()
    sfr = H.sf_to_numpy(out["sfd_row_tensor"], m, 2 * n // 32)[0]
    deq = orc.dequantize_rows(out["d_row_tensor"][:, :, 0].view(torch.uint8).cpu().numpy(), sfr)
    assert H.rel_fro(deq, g["d_ref"]) <= 6e-2
    np.testing.assert_allclose(out["dprob_tensor"].view(-1).cpu().numpy(), g["dprob_ref"], rtol=2e-2, atol=2e-2 * np.abs(g["dprob_ref"]).max())


@pytest.mark.parametrize("sf_vec,sf_dtype,d_dtype", [(16, "e4m3", torch.bfloat16), (32, "e8m0", torch.float32), (16, "e8m0", torch.bfloat16)])
def test_dswiglu_fp4_matches_oracle(tile_mode, sf_vec, sf_dtype, d_dtype):
    import cudnn_frontend_b200 as cf

    groups, n, k = [130, 256, 0, 64], 128, 512
    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands_fp4(3, valid, n, k, e, sf_vec, sf_dtype)
    H.zero_padding_rows(a, groups, aligned)
    rng = np.random.default_rng(4)
    alpha = np.ones(e, np.float32)
    beta = rng.choice([0.5, 1.0], e).astype(np.float32)
    prob = rng.uniform(0.1, 1.0, valid).astype(np.float32)
    c_t = torch.from_numpy(rng.uniform(-3, 3, (valid, 2 * n)).astype(np.float32)).to(torch.bfloat16)
    ref = orc.dswiglu_reference(a, sfa, b, sfb, c_t.float().numpy(), offs, alpha, beta, prob, ab_dtype="e2m1", sf_vec=sf_vec, sf_dtype=sf_dtype)
    sft = torch.float8_e4m3fn if sf_dtype == "e4m3" else torch.float8_e8m0fnu
    fp4 = lambda x, shape: torch.from_numpy(np.ascontiguousarray(x)).cuda().view(torch.float4_e2m1fn_x2).view(*shape)  # noqa: E731
    out = cf.grouped_gemm_dswiglu_wrapper_sm100(
        fp4(a, (valid, k // 2, 1)), fp4(b, (e, n, k // 2)).permute(1, 2, 0), c_t.cuda().view(valid, 2 * n, 1),
        H.dev_sf(sfa, valid, k, 1, sf_vec=sf_vec, dtype=sft), H.dev_sf(sfb, n, k, e, sf_vec=sf_vec, dtype=sft), torch.from_numpy(offs).cuda(),
        torch.from_numpy(alpha).cuda(), torch.from_numpy(beta).cuda(), torch.from_numpy(prob).cuda().view(valid, 1, 1), d_dtype=d_dtype,
        sf_vec_size=sf_vec, m_aligned=128)  # fmt: skip
    torch.cuda.synchronize()
    d = out["d_row_tensor"][:, :, 0].float().cpu().numpy()
    assert H.rel_fro(d, ref["d"]) <= 2e-2
    np.testing.assert_allclose(out["dprob_tensor"].view(-1).cpu().numpy(), ref["dprob"], rtol=2e-2, atol=2e-2 * np.abs(ref["dprob"]).max())
    if d_dtype == torch.float32:
        assert out["amax_tensor"] is None
    else:
        amax = out["amax_tensor"].view(e, 2).cpu().numpy()
        live = np.isfinite(ref["amax"][:, 0])
        np.testing.assert_allclose(amax[live], ref["amax"][live], rtol=2e-2)
        assert np.all(np.isneginf(amax[~live]))


@pytest.mark.parametrize("b_major,dynamic", [("k", False), ("n", False), ("k", True)])
def test_discrete_dswiglu_equals_dense_bitwise(tile_mode, b_major, dynamic):
    """One weight allocation per expert behind b_ptrs / sfb_ptrs (K- or N-major, static or dynamic scheduler) gives
    the same bytes as the dense operator (the reference checks its discrete kernels the same way,
    test/python/fe_api/test_discrete_grouped_gemm_swiglu.py:448-688)."""
    import cudnn_frontend_b200 as cf

    groups, n, k = [256, 0, 130, 384], 192, 256
    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands(17, valid, n, k, e)
    H.zero_padding_rows(a, groups, aligned)
    rng = np.random.default_rng(17)
    ta = H.dev_fp8(a).view(valid, k, 1)
    tb_store = H.dev_fp8(b)
    tsfa, tsfb = H.dev_sf(sfa, valid, k), H.dev_sf(sfb, n, k, e)
    tc = torch.from_numpy(rng.uniform(-3, 3, (valid, 2 * n)).astype(np.float32)).to(torch.bfloat16).cuda().view(valid, 2 * n, 1)
    toffs = torch.from_numpy(offs).cuda()
    talpha, tbeta = torch.ones(e, device="cuda"), torch.full((e,), 0.5, device="cuda")
    tprob = torch.from_numpy(rng.uniform(0.1, 1.0, valid).astype(np.float32)).cuda().view(valid, 1, 1)
    norm = torch.ones(1, device="cuda")
    kw = dict(norm_const_tensor=norm, d_dtype=torch.float8_e4m3fn, sf_vec_size=32, m_aligned=128)
    dense = cf.grouped_gemm_dswiglu_wrapper_sm100(ta, tb_store.permute(1, 2, 0), tc, tsfa, tsfb, toffs, talpha, tbeta, tprob, **kw)
    bl = [(tb_store[i].t().contiguous() if b_major == "n" else tb_store[i].clone()) for i in range(e)]
    sl = [H.dev_sf(sfb[i], n, k) for i in range(e)]
    b_ptrs = torch.tensor([x.data_ptr() for x in bl], dtype=torch.int64, device="cuda")
    sfb_ptrs = torch.tensor([x.data_ptr() for x in sl], dtype=torch.int64, device="cuda")
    dprob = torch.zeros((valid, 1, 1), device="cuda")
    disc = cf.discrete_grouped_gemm_dswiglu_wrapper_sm100(ta, b_ptrs, tc, tsfa, sfb_ptrs, toffs, talpha, tbeta, tprob, dprob, n, torch.float8_e4m3fn,
                                                          b_major=b_major, use_dynamic_sched=dynamic, **kw)  # fmt: skip
    torch.cuda.synchronize()
    for key in ("d_row_tensor", "d_col_tensor"):
        assert torch.equal(dense[key].view(torch.uint8), disc[key].view(torch.uint8)), key
    sfr_a = H.sf_to_numpy(dense["sfd_row_tensor"], valid, 2 * n // 32)
    sfr_b = H.sf_to_numpy(disc["sfd_row_tensor"], valid, 2 * n // 32)
    np.testing.assert_array_equal(sfr_a, sfr_b)
    # dprob is accumulated with atomic adds from two tile halves per row: equal up to the order of two additions
    torch.testing.assert_close(dense["dprob_tensor"], disc["dprob_tensor"], rtol=1e-5, atol=1e-5)
