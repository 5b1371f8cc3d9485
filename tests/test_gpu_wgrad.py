"""Weight gradient (the experts partition the token dimension) through the operator class and the wrapper against
the CPU oracle.  Cases follow the reference's test (test/python/fe_api/test_grouped_gemm_wgrad_utils.py:118-215:
m = 384, n = 640, token groups [256, 384], bf16 output, fp8 with E8M0 scales per 32, FP4 with E8M0 per 32 and with
E4M3 per 16 plus per-expert global scales), widened by an empty expert, accumulation and float32 / fp16 outputs.
Gate: relative Frobenius error <= 2e-2 of the float32 reference for bf16 / fp16 outputs, <= 1e-5 for float32.
"""

import os

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["single", "pair"], autouse=True)
def tile_mode(request, monkeypatch):
    """Every case runs with 128 x 256 single-CTA tiles and with 256 x 256 CTA-pair tiles."""
    monkeypatch.setenv("B200MOE_TILE_MODE", request.param)
    return request.param


def _operands(seed, m, n, groups, fmt):
    """fmt: ("e4m3", 32, "e8m0") | ("e2m1", 32, "e8m0") | ("e2m1", 16, "e4m3") ..."""
    ab, sf_vec, sf_dtype = fmt
    g = torch.Generator().manual_seed(seed)
    tokens = sum(groups)
    if ab == "e2m1":
        a = torch.randint(0, 256, (m, tokens // 2), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
        b = torch.randint(0, 256, (n, tokens // 2), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    else:
        a = torch.empty(m, tokens).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
        b = torch.empty(n, tokens).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    lo, hi = (0x30, 0x46) if sf_dtype == "e4m3" else (124, 131)
    sfa = [torch.randint(lo, hi, (m, t // sf_vec), generator=g, dtype=torch.int32).to(torch.uint8).numpy() for t in groups]
    sfb = [torch.randint(lo, hi, (n, t // sf_vec), generator=g, dtype=torch.int32).to(torch.uint8).numpy() for t in groups]
    return a, b, sfa, sfb


def _device(a, b, sfa, sfb, groups, fmt, m, n):
    ab, sf_vec, sf_dtype = fmt
    tokens = sum(groups)
    sft = torch.float8_e4m3fn if sf_dtype == "e4m3" else torch.float8_e8m0fnu
    if ab == "e2m1":
        ta = torch.from_numpy(a).cuda().view(torch.float4_e2m1fn_x2)  # (m, tokens / 2)
        tb = torch.from_numpy(b).cuda().view(torch.float4_e2m1fn_x2).t()  # (tokens / 2, n), packed along dim 0
    else:
        ta = torch.from_numpy(a).cuda().view(torch.float8_e4m3fn)
        tb = torch.from_numpy(b).cuda().view(torch.float8_e4m3fn).t()  # (tokens, n) with strides (1, tokens)
    cols = (tokens // sf_vec + 3) // 4 * 4

    def scales(groups_, rows):
        flat = orc.wgrad_pack_scales(groups_)
        rows_p = (rows + 127) // 128 * 128
        buf = np.full(rows_p * cols, 0xFF, dtype=np.uint8)  # nothing may depend on bytes past the last expert's block
        buf[: flat.size] = flat
        return torch.from_numpy(buf).cuda().view(sft).view(rows_p, cols)

    offs = torch.tensor(np.cumsum(groups), dtype=torch.int32, device="cuda")
    return ta, tb, scales(sfa, m), scales(sfb, n), offs


FORMATS = [("e4m3", 32, "e8m0"), ("e2m1", 32, "e8m0"), ("e2m1", 16, "e4m3"), ("e2m1", 16, "e8m0")]


@pytest.mark.parametrize("fmt", FORMATS)
def test_wgrad_matches_oracle(fmt):
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops

    m, n, groups = 384, 640, [256, 384]
    a, b, sfa, sfb = _operands(1, m, n, groups, fmt)
    ta, tb, tsfa, tsfb, offs = _device(a, b, sfa, sfb, groups, fmt, m, n)
    gs = None
    if fmt[2] == "e4m3":
        gs = (np.array([1.0, 2.0], np.float32), np.array([0.5, 1.5], np.float32))
    ref = orc.wgrad_reference(a, b, sfa, sfb, np.cumsum(groups), None if gs is None else gs[0], None if gs is None else gs[1], ab_dtype=fmt[0],
                              sf_vec=fmt[1], sf_dtype=fmt[2])  # fmt: skip
    kw = {} if gs is None else dict(global_scale_a=torch.from_numpy(gs[0]).cuda(), global_scale_b=torch.from_numpy(gs[1]).cuda())
    out = cf.grouped_gemm_wgrad_wrapper_sm100(ta, tb, tsfa, tsfb, offs, sf_vec_size=fmt[1], **kw)["wgrad_tensor"]
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    assert out.shape == (2, m, n) and out.dtype == torch.bfloat16
    assert H.rel_fro(out.float().cpu().numpy(), ref) <= 2e-2


def test_wgrad_ragged_groups_empty_expert_accumulate_and_float32():
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops

    # an empty expert, rows and columns that do not fill their last tile (m = 200, n = 288), nine k-tiles in the last
    # expert (the ring wraps twice).  Groups are multiples of 128 tokens: the reference's scale-tensor shape
    # (round_up(rows, 128), round_up(tokens / 32, 4)) holds the experts' blocks only then.
    m, n, groups = 200, 288, [128, 0, 256, 1152]
    fmt = ("e4m3", 32, "e8m0")
    a, b, sfa, sfb = _operands(2, m, n, groups, fmt)
    ta, tb, tsfa, tsfb, offs = _device(a, b, sfa, sfb, groups, fmt, m, n)
    ref = orc.wgrad_reference(a, b, sfa, sfb, np.cumsum(groups))
    e = len(groups)
    for dtype, gate in ((torch.float32, 1e-5), (torch.float16, 2e-2)):
        w = torch.full((e, m, n), 7.0, dtype=dtype, device="cuda")
        op = cf.GroupedGemmWgradSm100(ta, tb, tsfa, tsfb, offs, sample_wgrad=w, sf_vec_size=32)
        assert op.check_support()
        op.compile()
        op.execute(ta, tb, tsfa, tsfb, offs, wgrad_tensor=w)
        torch.cuda.synchronize()
        assert H.rel_fro(w.float().cpu().numpy(), ref) <= gate
        assert float(w[1].abs().max()) == 0.0  # the expert without tokens gets zeros, not what was there
        acc = cf.GroupedGemmWgradSm100(ta, tb, tsfa, tsfb, offs, sample_wgrad=w, sf_vec_size=32, accumulate_on_output=True)
        assert acc.check_support()
        acc.compile()
        acc.execute(ta, tb, tsfa, tsfb, offs, wgrad_tensor=w)
        torch.cuda.synchronize()
        assert H.rel_fro(w.float().cpu().numpy(), 2.0 * ref) <= max(gate, 1e-3 if dtype == torch.float16 else 0)
    assert ops.device_status(clear=True) == 0


def test_wgrad_unaligned_group_is_reported_not_computed():
    import cudnn_frontend_b200 as cf
    from cudnn_frontend_b200 import ops

    m, n, groups = 128, 256, [128, 128]
    fmt = ("e4m3", 32, "e8m0")
    a, b, sfa, sfb = _operands(3, m, n, groups, fmt)
    ta, tb, tsfa, tsfb, _ = _device(a, b, sfa, sfb, groups, fmt, m, n)
    offs = torch.tensor([100, 256], dtype=torch.int32, device="cuda")  # 100 tokens: not a whole number of scale blocks
    out = cf.grouped_gemm_wgrad_wrapper_sm100(ta, tb, tsfa, tsfb, offs, sf_vec_size=32)["wgrad_tensor"]
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 202
    assert float(out.float().abs().max()) == 0.0


def test_wgrad_is_bit_identical_to_the_reference_kernel_fixture(golden_dir):
    """Inputs and the bf16 output of cudnn-frontend's grouped_gemm_wgrad_wrapper_sm100 recorded on a B200: every bit
    of the [E, m, n] result must match."""
    import cudnn_frontend_b200 as cf

    g = np.load(os.path.join(golden_dir, "reference_kernel_wgrad.npz"))
    m, tokens = g["a"].shape
    n = g["b"].shape[0]
    cols = (tokens // 32 + 3) // 4 * 4
    ta = torch.from_numpy(g["a"]).cuda().view(torch.float8_e4m3fn)
    tb = torch.from_numpy(g["b"]).cuda().view(torch.float8_e4m3fn).t()
    sfa = torch.from_numpy(g["sfa"]).cuda().view(torch.float8_e8m0fnu).view(-1, cols)
    sfb = torch.from_numpy(g["sfb"]).cuda().view(torch.float8_e8m0fnu).view(-1, cols)
    out = cf.grouped_gemm_wgrad_wrapper_sm100(ta, tb, sfa, sfb, torch.from_numpy(g["offsets"]).cuda(), sf_vec_size=32)["wgrad_tensor"]
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.view(torch.int16).cpu().numpy(), g["wgrad"])


def test_wgrad_discrete_output_equals_dense():
    """One [m, n] allocation per expert behind wgrad_ptrs (the reference's discrete output mode) holds what the dense
    [E, m, n] tensor holds."""
    import cudnn_frontend_b200 as cf

    m, n, groups = 384, 640, [256, 0, 384]
    fmt = ("e4m3", 32, "e8m0")
    a, b, sfa, sfb = _operands(5, m, n, groups, fmt)
    ta, tb, tsfa, tsfb, offs = _device(a, b, sfa, sfb, groups, fmt, m, n)
    dense = cf.grouped_gemm_wgrad_wrapper_sm100(ta, tb, tsfa, tsfb, offs, sf_vec_size=32)["wgrad_tensor"]
    outs = [torch.full((m, n), 3.0, dtype=torch.bfloat16, device="cuda") for _ in groups]
    ptrs = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device="cuda")
    cf.grouped_gemm_wgrad_wrapper_sm100(ta, tb, tsfa, tsfb, offs, output_mode="discrete", wgrad_ptrs=ptrs, sf_vec_size=32)
    torch.cuda.synchronize()
    for e, o in enumerate(outs):
        assert torch.equal(o, dense[e])
