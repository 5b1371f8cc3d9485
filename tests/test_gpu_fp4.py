"""FP4 operands (E2M1, two per byte) through the operator classes against the CPU oracle: MXFP4 (E8M0
scales per 32 elements), E8M0 per 16 and NVFP4 (E4M3 scales per 16), FC1 and FC2, both tile modes.

The cases follow the reference's FP4 matrix (test/python/fe_api/test_grouped_gemm_swiglu_utils.py:59-110):
bf16 C, bf16 or float32 D, no scale-factor generation.  Gates: bf16 outputs within 2e-2 relative Frobenius
error of the float32 reference; the float32 D within 1e-5 (the products are exact in float32, only the
summation order differs).
"""

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

BF16_GATE = 2e-2
F32_GATE = 1e-5
FORMATS = [(32, "e8m0"), (16, "e8m0"), (16, "e4m3")]


@pytest.fixture(params=["single", "pair"])
def tile_mode(request, monkeypatch):
    monkeypatch.setenv("B200MOE_TILE_MODE", request.param)
    return request.param


def _sf_torch(sf_dtype):
    return torch.float8_e4m3fn if sf_dtype == "e4m3" else torch.float8_e8m0fnu


def _fp4(x_bytes, shape):
    return torch.from_numpy(np.ascontiguousarray(x_bytes)).cuda().view(torch.float4_e2m1fn_x2).view(*shape)


def _run_fc1(seed, groups, n, k, sf_vec, sf_dtype, d_dtype=torch.bfloat16, wrapper=False, m_aligned=128):
    import cudnn_frontend_b200 as cf

    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, m_aligned)
    a, b, sfa, sfb = H.gen_operands_fp4(seed, valid, n, k, e, sf_vec, sf_dtype)
    H.zero_padding_rows(a, groups, aligned)
    rng = np.random.default_rng(seed)
    alpha = rng.integers(1, 3, e).astype(np.float32)
    prob = rng.uniform(0.1, 1.0, valid).astype(np.float32)
    ref = orc.fc1_reference(a, sfa, b, sfb, offs, alpha, prob, ab_dtype="e2m1", sf_vec=sf_vec, sf_dtype=sf_dtype)
    ta = _fp4(a, (valid, k // 2, 1))
    tb = _fp4(b, (e, n, k // 2)).permute(1, 2, 0)
    tsfa = H.dev_sf(sfa, valid, k, 1, sf_vec=sf_vec, dtype=_sf_torch(sf_dtype))
    tsfb = H.dev_sf(sfb, n, k, e, sf_vec=sf_vec, dtype=_sf_torch(sf_dtype))
    toffs, talpha = torch.from_numpy(offs).cuda(), torch.from_numpy(alpha).cuda()
    tprob = torch.from_numpy(prob).cuda().view(valid, 1, 1)
    if wrapper:
        out = cf.grouped_gemm_swiglu_wrapper_sm100(ta, tb, tsfa, tsfb, toffs, talpha, prob_tensor=tprob, d_dtype=d_dtype, sf_vec_size=sf_vec,
                                                   m_aligned=m_aligned)  # fmt: skip
        c, d, amax = out["c_tensor"], out["d_tensor"], out["amax_tensor"]
        assert out["sfd_row_tensor"] is None and out["sfd_col_tensor"] is None
    else:
        c = torch.empty((valid, n, 1), dtype=torch.bfloat16, device="cuda")
        d = torch.empty((valid, n // 2, 1), dtype=d_dtype, device="cuda")
        amax = torch.full((e, 1), float("-inf"), device="cuda") if d_dtype != torch.float32 else None
        op = cf.GroupedGemmSwigluSm100(ta, tb, c, d, tsfa, tsfb, toffs, talpha, None, sample_amax=amax, sample_prob=tprob, sf_vec_size=sf_vec,
                                       m_aligned=m_aligned)  # fmt: skip
        assert op.check_support()
        op.compile()
        op.execute(ta, tb, c, d, tsfa, tsfb, toffs, talpha, amax_tensor=amax, prob_tensor=tprob)
    torch.cuda.synchronize()
    from cudnn_frontend_b200 import ops

    assert ops.device_status(clear=True) == 0
    return ref, c[:, :, 0].float().cpu().numpy(), d[:, :, 0].float().cpu().numpy(), None if amax is None else amax.cpu().numpy().reshape(-1)


@pytest.mark.parametrize("sf_vec,sf_dtype", FORMATS)
def test_fc1_fp4_matches_oracle(tile_mode, sf_vec, sf_dtype):
    # 512 = two full k-tiles of 256 elements; 384 leaves half a k-tile and, per 16, an incomplete run of scale chunks
    for k in (512, 384):
        ref, c, d, amax = _run_fc1(11 + k, [130, 0, 256, 77], 256, k, sf_vec, sf_dtype)
        assert H.rel_fro(c, ref["c"]) <= BF16_GATE
        assert H.rel_fro(d, ref["d"]) <= BF16_GATE
        live = np.isfinite(ref["amax"])
        np.testing.assert_allclose(amax[live], ref["amax"][live], rtol=2e-2)
        assert np.all(np.isneginf(amax[~live]))


def test_fc1_fp4_float32_d_is_nearly_exact(tile_mode):
    ref, c, d, amax = _run_fc1(5, [256, 128], 512, 1024, 32, "e8m0", d_dtype=torch.float32)
    assert amax is None
    assert H.rel_fro(d, ref["d"]) <= 5e-3  # SwiGLU uses the approximate exponential and reciprocal
    # the pre-activation C is stored in bf16: compare D against the oracle evaluated on exactly that input instead
    assert H.rel_fro(c, ref["c"]) <= 4e-3


def test_fc1_fp4_deep_k_wrapper(tile_mode):
    # 14 k-tiles: the ring (4 to 6 stages) wraps several times and the single scale-factor buffer in TMEM is rewritten 13 times
    ref, c, d, amax = _run_fc1(9, [300, 128, 0, 512], 512, 3584, 16, "e4m3", wrapper=True)
    assert H.rel_fro(c, ref["c"]) <= BF16_GATE
    assert H.rel_fro(d, ref["d"]) <= BF16_GATE


@pytest.mark.parametrize("sf_vec,sf_dtype", FORMATS)
def test_fc2_fp4_matches_oracle(tile_mode, sf_vec, sf_dtype):
    import cudnn_frontend_b200 as cf

    groups, n, k = [200, 128, 0, 384], 384, 768
    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands_fp4(21, valid, n, k, e, sf_vec, sf_dtype)
    H.zero_padding_rows(a, groups, aligned)
    rng = np.random.default_rng(3)
    alpha = rng.integers(1, 3, e).astype(np.float32)
    prob = rng.uniform(0.1, 1.0, valid).astype(np.float32)
    ref = orc.fc2_reference(a, sfa, b, sfb, offs, alpha, prob, ab_dtype="e2m1", sf_vec=sf_vec, sf_dtype=sf_dtype)
    for d_dtype in (torch.bfloat16,) + ((torch.float32,) if sf_vec == 32 else ()):
        out = cf.grouped_gemm_quant_wrapper_sm100(
            _fp4(a, (valid, k // 2, 1)), H.dev_sf(sfa, valid, k, 1, sf_vec=sf_vec, dtype=_sf_torch(sf_dtype)), torch.from_numpy(offs).cuda(),
            torch.from_numpy(alpha).cuda(), b_tensor=_fp4(b, (e, n, k // 2)).permute(1, 2, 0),
            sfb_tensor=H.dev_sf(sfb, n, k, e, sf_vec=sf_vec, dtype=_sf_torch(sf_dtype)), prob_tensor=torch.from_numpy(prob).cuda().view(valid, 1, 1),
            d_dtype=d_dtype, sf_vec_size=sf_vec, m_aligned=128)  # fmt: skip
        torch.cuda.synchronize()
        d = out["d_tensor"][:, :, 0].float().cpu().numpy()
        assert H.rel_fro(d, ref["d"]) <= (F32_GATE if d_dtype == torch.float32 else BF16_GATE)
        assert out["sfd_row_tensor"] is None


def test_fp4_rejections():
    import cudnn_frontend_b200 as cf

    valid, n, k, e = 128, 128, 256, 1
    a, b, sfa, sfb = H.gen_operands_fp4(1, valid, n, k, e, 16, "e4m3")
    args = (_fp4(a, (valid, k // 2, 1)), _fp4(b, (e, n, k // 2)).permute(1, 2, 0), H.dev_sf(sfa, valid, k, 1, sf_vec=16, dtype=torch.float8_e4m3fn),
            H.dev_sf(sfb, n, k, e, sf_vec=16, dtype=torch.float8_e4m3fn), torch.tensor([128], dtype=torch.int32, device="cuda"), torch.ones(1, device="cuda"))  # fmt: skip
    with pytest.raises(NotImplementedError):  # the reference disables fp4 + sf_vec 16 + float32 D
        cf.grouped_gemm_swiglu_wrapper_sm100(*args, d_dtype=torch.float32, sf_vec_size=16, m_aligned=128)
    with pytest.raises(ValueError):  # an FP8 D is not a valid output type for FP4 operands
        cf.grouped_gemm_swiglu_wrapper_sm100(*args, d_dtype=torch.float8_e4m3fn, sf_vec_size=16, m_aligned=128)
    with pytest.raises(ValueError):  # E4M3 scale factors go with sf_vec_size 16 only
        cf.grouped_gemm_swiglu_wrapper_sm100(*args, d_dtype=torch.bfloat16, sf_vec_size=32, m_aligned=128)


def test_uint8_operands_are_raw_packed_fp4(tile_mode):
    """The reference reads uint8 A / B as raw packed FP4 (python/cudnn/api_base.py:602-609): the same bytes as uint8
    tensors give the same C and D as float4_e2m1fn_x2 tensors, through the wrapper and through the class."""
    import cudnn_frontend_b200 as cf

    valid, n, k, e = 256, 256, 512, 2
    a, b, sfa, sfb = H.gen_operands_fp4(5, valid, n, k, e, 16, "e4m3")
    ta, tb = _fp4(a, (valid, k // 2, 1)), _fp4(b, (e, n, k // 2)).permute(1, 2, 0)
    rest = (H.dev_sf(sfa, valid, k, 1, sf_vec=16, dtype=torch.float8_e4m3fn), H.dev_sf(sfb, n, k, e, sf_vec=16, dtype=torch.float8_e4m3fn),
            torch.tensor([128, 256], dtype=torch.int32, device="cuda"), torch.ones(e, device="cuda"))  # fmt: skip
    kw = dict(d_dtype=torch.bfloat16, sf_vec_size=16, m_aligned=128)
    want = cf.grouped_gemm_swiglu_wrapper_sm100(ta, tb, *rest, **kw)
    got = cf.grouped_gemm_swiglu_wrapper_sm100(ta.view(torch.uint8), tb.view(torch.uint8), *rest, **kw)
    torch.cuda.synchronize()
    for key in ("c_tensor", "d_tensor", "amax_tensor"):
        assert torch.equal(want[key], got[key]), key
    c, d = torch.empty_like(want["c_tensor"]), torch.empty_like(want["d_tensor"])
    amax = torch.full((e, 1), float("-inf"), device="cuda")
    op = cf.GroupedGemmSwigluSm100(ta.view(torch.uint8), tb.view(torch.uint8), c, d, *rest, None, sample_amax=amax, sf_vec_size=16, m_aligned=128)
    assert op.check_support()
    op.compile()
    op.execute(ta.view(torch.uint8), tb.view(torch.uint8), c, d, *rest, amax_tensor=amax)
    torch.cuda.synchronize()
    assert torch.equal(c, want["c_tensor"]) and torch.equal(d, want["d_tensor"])


@pytest.mark.parametrize("fixture", ["reference_kernel_fc1_fp4_nvfp4.npz", "reference_kernel_fc1_fp4_mxfp4.npz", "reference_kernel_fc1_fp4_e8m0x16.npz"])
def test_fc1_fp4_is_bit_identical_to_the_reference_kernel_fixture(golden_dir, tile_mode, fixture):
    """Inputs and outputs of cudnn-frontend's GroupedGemmSwigluSm100 with float4_e2m1fn_x2 operands (bf16 C and
    D, groups padded to 256) recorded on a B200: C and D must match bit for bit in both tile modes."""
    import os

    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops

    g = np.load(os.path.join(golden_dir, fixture))
    m, kb = g["a"].shape
    e, n, _ = g["b"].shape
    k = 2 * kb
    sf_vec = int(g["sf_vec"])
    sf_t = torch.float8_e4m3fn if int(g["sf_is_e4m3"]) else torch.float8_e8m0fnu

    def sf(flat, mn, l):
        shape, stride = ops.sf_shape_stride(mn, k, l, sf_vec)
        return torch.as_strided(torch.from_numpy(flat).cuda().view(sf_t), shape, stride)

    out = cf.grouped_gemm_swiglu_wrapper_sm100(
        _fp4(g["a"], (m, kb, 1)), _fp4(g["b"], (e, n, kb)).permute(1, 2, 0), sf(g["sfa"], m, 1), sf(g["sfb"], n, e),
        torch.from_numpy(g["offsets"]).cuda(), torch.ones(e, device="cuda"), prob_tensor=torch.from_numpy(g["prob"]).cuda().view(m, 1, 1),
        d_dtype=torch.bfloat16, sf_vec_size=sf_vec, m_aligned=256)  # fmt: skip
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out["c_tensor"][:, :, 0].contiguous().view(torch.int16).cpu().numpy(), g["c"])
    np.testing.assert_array_equal(out["d_tensor"][:, :, 0].contiguous().view(torch.int16).cpu().numpy(), g["d"])


def test_discrete_and_glu_fp4_equal_dense_bitwise(tile_mode):
    """FP4 weights behind per-expert pointers (discrete FC1) and through the unified GLU front end (GeGLU and a
    fused bias) give the same bits as the dense FC1 on the same operands."""
    import cudnn_frontend_b200 as cf

    groups, n, k, sf_vec, sf_dtype = [128, 300, 0, 64], 256, 768, 16, "e4m3"
    e = len(groups)
    valid, aligned, offs = orc.padded_end_offsets(groups, 128)
    a, b, sfa, sfb = H.gen_operands_fp4(31, valid, n, k, e, sf_vec, sf_dtype)
    H.zero_padding_rows(a, groups, aligned)
    ta = _fp4(a, (valid, k // 2, 1))
    tb = _fp4(b, (e, n, k // 2))
    tsfa = H.dev_sf(sfa, valid, k, 1, sf_vec=sf_vec, dtype=torch.float8_e4m3fn)
    tsfb = H.dev_sf(sfb, n, k, e, sf_vec=sf_vec, dtype=torch.float8_e4m3fn)
    toffs, talpha = torch.from_numpy(offs).cuda(), torch.ones(e, device="cuda")
    # seeded: the dense wrapper keeps a running amax per cached configuration, so both tile modes must see the same rows
    prob = torch.from_numpy(np.random.default_rng(7).uniform(0.1, 1.0, valid).astype(np.float32)).cuda().view(valid, 1, 1)
    kw = dict(prob_tensor=prob, d_dtype=torch.bfloat16, sf_vec_size=sf_vec, m_aligned=128)
    dense = cf.grouped_gemm_swiglu_wrapper_sm100(ta, tb.permute(1, 2, 0), tsfa, tsfb, toffs, talpha, **kw)
    bl = [tb[i].clone() for i in range(e)]
    sl = [H.dev_sf(sfb[i], n, k, 1, sf_vec=sf_vec, dtype=torch.float8_e4m3fn) for i in range(e)]
    b_ptrs = torch.tensor([x.data_ptr() for x in bl], dtype=torch.int64, device="cuda")
    sfb_ptrs = torch.tensor([x.data_ptr() for x in sl], dtype=torch.int64, device="cuda")
    disc = cf.discrete_grouped_gemm_swiglu_wrapper_sm100(ta, b_ptrs, tsfa, sfb_ptrs, toffs, talpha, n, torch.float4_e2m1fn_x2, **kw)
    torch.cuda.synchronize()
    assert torch.equal(dense["c_tensor"], disc["c_tensor"]) and torch.equal(dense["d_tensor"], disc["d_tensor"])
    assert torch.equal(dense["amax_tensor"], disc["amax_tensor"])

    # GeGLU + bias through the unified front end, dense and discrete, against the oracle
    rng = np.random.default_rng(2)
    bias = rng.uniform(-2, 2, (e, n)).astype(np.float32)
    tbias = torch.from_numpy(bias).cuda().to(torch.bfloat16).t()  # (n, e), stride (1, n)
    ref = orc.fc1_reference(a, sfa, b, sfb, offs, np.ones(e, np.float32), prob.view(-1).cpu().numpy(), bias=orc.bf16_round(bias).T,
                            act_func="geglu", ab_dtype="e2m1", sf_vec=sf_vec, sf_dtype=sf_dtype)  # fmt: skip
    g1 = cf.grouped_gemm_glu_wrapper_sm100(ta, tsfa, toffs, talpha, b_tensor=tb.permute(1, 2, 0), sfb_tensor=tsfb, bias_tensor=tbias, act_func="geglu", **kw)
    g2 = cf.grouped_gemm_glu_wrapper_sm100(ta, tsfa, toffs, talpha, b_ptrs=b_ptrs, sfb_ptrs=sfb_ptrs, n=n, b_dtype=torch.float4_e2m1fn_x2,
                                           bias_tensor=tbias, act_func="geglu", **kw)  # fmt: skip
    torch.cuda.synchronize()
    assert torch.equal(g1["d_tensor"], g2["d_tensor"]) and torch.equal(g1["c_tensor"], g2["c_tensor"])
    assert H.rel_fro(g1["c_tensor"][:, :, 0].float().cpu().numpy(), ref["c"]) <= BF16_GATE
    assert H.rel_fro(g1["d_tensor"][:, :, 0].float().cpu().numpy(), ref["d"]) <= BF16_GATE
