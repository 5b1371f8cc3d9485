"""Shared helpers of the GPU parity tests: seeded operands, device upload, comparisons."""

from __future__ import annotations

import numpy as np
import torch

from oracle import mxfp8_oracle as orc


def gen_operands(seed, m_rows, n, k, e, sf_lo=124, sf_hi=131, scale=2.0, dtype=torch.float8_e4m3fn):
    """Random E4M3 (or E5M2) bytes (uniform(-scale, scale) cast) and E8M0 bytes in [sf_lo, sf_hi)."""
    g = torch.Generator().manual_seed(seed)
    a = torch.empty(m_rows, k).uniform_(-scale, scale, generator=g).to(dtype).view(torch.uint8).numpy()
    b = torch.empty(e, n, k).uniform_(-scale, scale, generator=g).to(dtype).view(torch.uint8).numpy()
    kb = (k + 31) // 32
    sfa = torch.randint(sf_lo, sf_hi, (m_rows, kb), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    sfb = torch.randint(sf_lo, sf_hi, (e, n, kb), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    return a, b, sfa, sfb


def gen_operands_fp4(seed, m_rows, n, k, e, sf_vec=16, sf_dtype="e4m3"):
    """Random packed E2M1 bytes ([rows, k/2], every nibble pattern) and scale bytes per ``sf_vec`` elements:
    E8M0 in [124, 131) or positive E4M3 in [0.5, 3.5]."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randint(0, 256, (m_rows, k // 2), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    b = torch.randint(0, 256, (e, n, k // 2), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    kb = (k + sf_vec - 1) // sf_vec
    lo, hi = (0x30, 0x46) if sf_dtype == "e4m3" else (124, 131)
    sfa = torch.randint(lo, hi, (m_rows, kb), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    sfb = torch.randint(lo, hi, (e, n, kb), generator=g, dtype=torch.int32).to(torch.uint8).numpy()
    return a, b, sfa, sfb


def zero_padding_rows(a, groups, aligned):
    start = 0
    for g_, al in zip(groups, aligned):
        a[start + g_ : start + al] = 0
        start += al
    return a


def dev_fp8(x, device="cuda", dtype=torch.float8_e4m3fn):
    return torch.from_numpy(np.ascontiguousarray(x)).to(device).view(dtype)


def dev_sf(sf_bytes, mn, k, l=1, device="cuda", sf_vec=32, dtype=torch.float8_e8m0fnu):
    """[L, MN, KB] / [MN, KB] scale bytes -> 6-D tensor (E8M0, or E4M3 with ``dtype``) in the 128x4 layout.
    Unused bytes of the layout are set to 0xFF (NaN) on purpose: nothing may depend on them."""
    from cudnn_frontend_b200 import ops

    flat = torch.from_numpy(orc.sf_pack(sf_bytes, fill=0xFF)).to(device)
    shape, stride = ops.sf_shape_stride(mn, k, l, sf_vec)
    return torch.as_strided(flat.view(dtype), shape, stride)


def sf_to_numpy(sf6d, mn, kb, l=1):
    """6-D scale tensor (any 1-byte dtype) -> [L, MN, KB] uint8 on the host."""
    t = sf6d.view(torch.uint8)
    flat = torch.as_strided(t, (t.numel(),), (1,)).cpu().numpy()
    return orc.sf_unpack(flat, mn, kb, l)


def rel_fro(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-300))


def assert_close_like_reference(got, ref_f32, dtype=torch.bfloat16, atol=1e-1, rtol=1e-2):
    """The reference's own check: cast the float32 reference to the output dtype, then
    atol 0.1 / rtol 1e-2 (test/python/fe_api/test_grouped_gemm_swiglu_utils.py:725-726)."""
    ref = torch.from_numpy(np.asarray(ref_f32)).to(dtype).to(torch.float32)
    torch.testing.assert_close(torch.as_tensor(got, dtype=torch.float32), ref, atol=atol, rtol=rtol)


def assert_e4m3_within_one_ulp(got_bytes, ref_bytes, frac=0.999):
    ulp = orc.e4m3_ulp_distance(got_bytes, ref_bytes)
    ok = float((ulp <= 1).mean())
    assert ok >= frac, f"only {ok:.5f} of E4M3 outputs within 1 ULP (need {frac})"
    return float((ulp == 0).mean())
