"""Generate the golden fixtures of tests/golden/ from the reference's own PyTorch code.

Run where the reference checkout is available (the REFERENCE_ROOT environment variable, else a
directory ``reference`` next to this repository); no GPU is needed:

    python tests/golden/make_golden.py

It imports the reference's test utilities in place (nothing is copied), feeds them seeded
inputs, and stores inputs + outputs as small .npz files:

* sf_layout.npz        scale-factor 128x4 layout, produced by the reference's
                       create_sf_layout_tensor + cvt_sf_MKL_to_M32x4xrm_K4xrk_L
                       (test/python/fe_api/test_fe_api_utils.py:12-25,95-114)
* offsets.npz          create_mask (test/python/fe_api/test_grouped_gemm_swiglu_utils.py:270-312)
* fc1_swiglu.npz       run_grouped_gemm_swiglu_ref, float32 branch (same file, :472-573)
* fc2_quant.npz        run_grouped_gemm_quant_ref, float32 branch
                       (test/python/fe_api/test_grouped_gemm_quant_utils.py:270-345)
* dswiglu.npz          run_grouped_gemm_dswiglu_ref, float32 branch with amax
                       (test/python/fe_api/test_grouped_gemm_dswiglu_utils.py:334-491)

The re-quantisation branch of those functions (generate_sfd=True) needs a GPU and the CuTe
DSL, so it is not part of these fixtures.  The reference_kernel_*.npz files are different: they
hold inputs and outputs of the reference's own CuTe-DSL kernels recorded on a B200 by
baseline/run_reference_kernels.py (cases tiny, tiny_e5m2, fc2_tiny, glu_tiny; after
baseline/make_ref_overlay.py).
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))

# The reference's helpers call .cuda() and query the device capability at import time.
torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
torch.Tensor.cuda = lambda self, *a, **k: self
sys.path.insert(0, os.path.join(REF, "test", "python"))
sys.path.insert(0, os.path.join(REF, "test", "python", "fe_api"))

import test_fe_api_utils as fu  # noqa: E402
import test_grouped_gemm_dswiglu_utils as du  # noqa: E402
import test_grouped_gemm_quant_utils as qu  # noqa: E402
import test_grouped_gemm_swiglu_utils as su  # noqa: E402
from cutlass.cute.runtime import from_dlpack  # noqa: E402


def ref_sf_layout(sf_mkl: torch.Tensor, mn: int, k: int) -> np.ndarray:
    """[MN, KB, L] float32 -> flat buffer in the reference's 128x4 layout."""
    l = sf_mkl.shape[2]
    cute_t, sf_k = fu.create_sf_layout_tensor(l, mn, k, 32)
    assert sf_k == sf_mkl.shape[1]
    fu.cvt_sf_MKL_to_M32x4xrm_K4xrk_L(from_dlpack(sf_mkl), from_dlpack(cute_t))
    flat = torch.as_strided(cute_t, (cute_t.numel(),), (1,))
    return flat.numpy().copy(), tuple(cute_t.shape), tuple(cute_t.stride())


def gen_operands(g, m, n, k, e):
    a = torch.empty(m, k).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn)
    b = torch.empty(e, n, k).uniform_(-2, 2, generator=g).to(torch.float8_e4m3fn)
    sfa = torch.randint(125, 130, (m, k // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    sfb = torch.randint(125, 130, (e, n, k // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    return a, b, sfa, sfb


def expand_sf(sf_u8: torch.Tensor) -> torch.Tensor:
    """E8M0 bytes [..., KB] -> float32 [..., KB*32] (value repeated per element)."""
    return sf_u8.view(torch.float8_e8m0fnu).to(torch.float32).repeat_interleave(32, dim=-1)


def main():
    g = torch.Generator().manual_seed(20240)

    # ---- scale-factor layout --------------------------------------------------------
    l, mn, k = 2, 300, 288  # ragged on purpose: 3 row blocks, 9 K blocks -> 3 K groups
    kb = fu.ceil_div(k, 32)
    vals = torch.randint(1, 255, (l, mn, kb), generator=g, dtype=torch.int32).to(torch.float32)
    flat, shape, stride = ref_sf_layout(vals.permute(1, 2, 0), mn, k)
    np.savez_compressed(
        os.path.join(HERE, "sf_layout.npz"),
        values=vals.numpy().astype(np.uint8),
        flat=flat.astype(np.uint8),
        shape=np.asarray(shape),
        stride=np.asarray(stride),
        mn=mn,
        k=k,
    )

    # ---- offsets ----------------------------------------------------------------------
    groups = [64, 256, 0, 320, 1]
    valid_m, aligned, offs = su.create_mask(groups, 256)
    np.savez_compressed(
        os.path.join(HERE, "offsets.npz"),
        groups=np.asarray(groups),
        valid_m=valid_m,
        aligned=np.asarray(aligned),
        offsets=offs.numpy(),
    )

    # ---- FC1: grouped GEMM + SwiGLU ---------------------------------------------------
    e, n, k = 3, 64, 64
    groups = [200, 1, 256]
    valid_m, aligned, offs = su.create_mask(groups, 256)
    a, b, sfa, sfb = gen_operands(g, valid_m, n, k, e)
    alpha = torch.randint(-2, 2, (e,), generator=g).float()
    prob = torch.randint(-2, 2, (valid_m, 1, 1), generator=g).float()
    ref = su.run_grouped_gemm_swiglu_ref(
        a_ref=a.float().unsqueeze(-1),
        b_ref=b.float().permute(1, 2, 0),
        sfa_ref=expand_sf(sfa).unsqueeze(-1),
        sfb_ref=expand_sf(sfb).permute(1, 2, 0),
        alpha_tensor=alpha,
        prob_tensor=prob,
        aligned_group_m_list=aligned,
        valid_m=valid_m,
        generate_amax=True,
        generate_sfd=False,
    )
    np.savez_compressed(
        os.path.join(HERE, "fc1_swiglu.npz"),
        a=a.view(torch.uint8).numpy(),
        b=b.view(torch.uint8).numpy(),
        sfa=sfa.numpy(),
        sfb=sfb.numpy(),
        offsets=offs.numpy(),
        alpha=alpha.numpy(),
        prob=prob.numpy().reshape(-1),
        c_ref=ref["c_ref"][:, :, 0].numpy(),
        d_ref=ref["d_ref"][:, :, 0].numpy(),
        amax_ref=ref["amax_ref"].numpy(),
    )

    # ---- FC2: grouped GEMM + alpha + prob -------------------------------------------------
    e, n, k = 3, 96, 64
    groups = [256, 100, 0]
    valid_m, aligned, offs = su.create_mask(groups, 256)
    a, b, sfa, sfb = gen_operands(g, valid_m, n, k, e)
    alpha = torch.randint(-2, 2, (e,), generator=g).float()
    prob = torch.empty(valid_m, 1, 1).uniform_(0, 1, generator=g)
    ref = qu.run_grouped_gemm_quant_ref(
        a_ref=a.float().unsqueeze(-1),
        b_ref=b.float().permute(1, 2, 0),
        sfa_ref=expand_sf(sfa).unsqueeze(-1),
        sfb_ref=expand_sf(sfb).permute(1, 2, 0),
        alpha_tensor=alpha,
        prob_tensor=prob,
        aligned_group_m_list=aligned,
        valid_m=valid_m,
        generate_amax=False,  # the reference's amax helper rejects an empty group
        generate_sfd=False,
    )
    np.savez_compressed(
        os.path.join(HERE, "fc2_quant.npz"),
        a=a.view(torch.uint8).numpy(),
        b=b.view(torch.uint8).numpy(),
        sfa=sfa.numpy(),
        sfb=sfb.numpy(),
        offsets=offs.numpy(),
        alpha=alpha.numpy(),
        prob=prob.numpy().reshape(-1),
        d_ref=ref["d_ref"][:, :, 0].numpy(),
    )
    # ---- dSwiGLU: backward of FC1's activation ---------------------------------------------
    e, n, k = 3, 64, 96
    groups = [256, 40, 512]
    valid_m, aligned, offs = su.create_mask(groups, 256)
    a, b, sfa, sfb = gen_operands(g, valid_m, n, k, e)
    alpha = torch.randint(1, 3, (e,), generator=g).float()
    beta = torch.tensor([1.0, 0.5, 2.0])
    prob = torch.empty(valid_m, 1, 1).uniform_(0.1, 1, generator=g)
    c_fwd = torch.empty(valid_m, 2 * n, 1).uniform_(-3, 3, generator=g).to(torch.bfloat16)
    ref = du.run_grouped_gemm_dswiglu_ref(
        a_ref=a.float().unsqueeze(-1),
        b_ref=b.float().permute(1, 2, 0),
        c_ref=c_fwd.float(),
        sfa_ref=expand_sf(sfa).unsqueeze(-1),
        sfb_ref=expand_sf(sfb).permute(1, 2, 0),
        alpha_tensor=alpha,
        beta_tensor=beta,
        prob_tensor=prob,
        aligned_group_m_list=aligned,
        valid_m=valid_m,
        generate_amax=True,
        generate_sfd=False,
    )
    np.savez_compressed(
        os.path.join(HERE, "dswiglu.npz"),
        a=a.view(torch.uint8).numpy(),
        b=b.view(torch.uint8).numpy(),
        sfa=sfa.numpy(),
        sfb=sfb.numpy(),
        offsets=offs.numpy(),
        alpha=alpha.numpy(),
        beta=beta.numpy(),
        prob=prob.numpy().reshape(-1),
        c_fwd=c_fwd.view(torch.int16).numpy()[:, :, 0],
        d_ref=ref["d_ref"][:, :, 0].numpy(),
        dprob_ref=ref["dprob_ref"].numpy().reshape(-1),
        amax_ref=ref["amax_ref"].numpy().reshape(e, 2),
    )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
