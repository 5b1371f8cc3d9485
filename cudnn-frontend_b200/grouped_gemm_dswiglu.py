"""Backward of FC1's activation: contiguous block-scaled grouped GEMM with a fused dSwiGLU epilogue.

Same names, arguments and error behaviour as the reference's ``GroupedGemmDswigluSm100`` /
``grouped_gemm_dswiglu_wrapper_sm100`` (python/cudnn/grouped_gemm/grouped_gemm_dswiglu/api.py:52-695,
:697-923).  ``A (m, k, 1)`` is the gradient that arrives at FC2's input side, ``B (n, k, l)`` the FC2 weights seen
from that side (K- or N-major for fp8), ``C (m, 2n, 1)`` the pre-activation FC1 wrote in the forward pass.  The
kernel computes ``G = alpha_e^2 (A SFA)(B_e SFB_e)^T`` and, per 32-column block ``j`` of ``G``,

    D[:, 64j      : 64j + 32] = G_j * prob * up_j * sig_j * (1 + gate_j * (1 - sig_j))    (gradient of the gate)
    D[:, 64j + 32 : 64j + 64] = G_j * prob * gate_j * sig_j                              (gradient of the up half)
    dprob                   += row sums of G * gate * sig * up

with ``gate / up`` the even / odd 32-column blocks of ``beta_e * C`` and ``sig = sigmoid(gate)``; ``D_row`` and
``D_col`` come out row- and column-quantised (fp8 operands) or as a 16-bit / float32 ``D_row`` with an ``(l, 2, 1)``
amax (FP4 operands), as in the reference.

``DiscreteGroupedGemmDswigluSm100`` / ``discrete_grouped_gemm_dswiglu_wrapper_sm100``
(python/cudnn/discrete_grouped_gemm/discrete_grouped_gemm_dswiglu/api.py:70-768, :770-1000) are the same operator
with one weight allocation per expert behind ``b_ptrs`` / ``sfb_ptrs``, K- or N-major (``b_major``), optionally with the
dynamic tile scheduler.

Differences a caller can observe: groups may be padded to any multiple of 128 rows; ``act_func`` other than
``"dswiglu"``, a float32 ``C`` and the dbias output are not built (``NotImplementedError``).  ``epilogue_op``
(``"relu"``, ``"srelu"``) is validated and then has no effect, exactly as in the reference: its kernel takes the
lambda as a parameter and never applies it (grouped_gemm_dswiglu_quant.py:543, :1533).
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from . import ops
from .api_base import OperatorBase, TensorSpec, TupleDict, as_packed_fp4, ceil_div, check_tile_and_cluster, packed_fp4_dtype, pick_tile_mode

_SF_STRIDE_MSG = "scale-factor tensors must use the 128x4 layout (32, 4, rest_mn, 4, rest_k, l)"


class GroupedGemmDswigluSm100(OperatorBase):
    def __init__(
        self,
        sample_a: torch.Tensor,
        sample_b: torch.Tensor,
        sample_c: torch.Tensor,
        sample_d_row: torch.Tensor,
        sample_d_col: Optional[torch.Tensor],
        sample_sfa: torch.Tensor,
        sample_sfb: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_beta: torch.Tensor,
        sample_prob: torch.Tensor,
        sample_dprob: torch.Tensor,
        sample_sfd_row: Optional[torch.Tensor] = None,
        sample_sfd_col: Optional[torch.Tensor] = None,
        sample_amax: Optional[torch.Tensor] = None,
        sample_norm_const: Optional[torch.Tensor] = None,
        acc_dtype: torch.dtype = torch.float32,
        mma_tiler_mn: Tuple[int, int] = (256, 256),
        cluster_shape_mn: Optional[Tuple[int, int]] = None,
        sf_vec_size: int = 16,
        vector_f32: bool = False,
        m_aligned: int = 256,
        discrete_col_sfd: bool = False,
        epilogue_op: Optional[str] = None,
        _discrete: Optional[dict] = None,
    ):
        """``_discrete`` is how :class:`DiscreteGroupedGemmDswigluSm100` describes its weights (``num_experts``,
        ``b_shape``, ``b_dtype``, ``b_major``, ``use_dynamic_sched``); ``sample_b`` / ``sample_sfb`` are then ``None``."""
        super().__init__()
        self.discrete = _discrete is not None
        self._dw = _discrete or {}
        self.use_dynamic_sched = bool(self._dw.get("use_dynamic_sched", False))
        self._workspace = None
        self.a = TensorSpec.of(as_packed_fp4(sample_a), "sample_a")
        self.b = TensorSpec.of(as_packed_fp4(sample_b), "sample_b")
        self.c = TensorSpec.of(sample_c, "sample_c")
        self.d_row = TensorSpec.of(sample_d_row, "sample_d_row")
        self.d_col = TensorSpec.of(sample_d_col, "sample_d_col")
        self.sfa = TensorSpec.of(sample_sfa, "sample_sfa")
        self.sfb = TensorSpec.of(sample_sfb, "sample_sfb")
        self.padded_offsets = TensorSpec.of(sample_padded_offsets, "sample_padded_offsets")
        self.alpha = TensorSpec.of(sample_alpha, "sample_alpha")
        self.beta = TensorSpec.of(sample_beta, "sample_beta")
        self.prob = TensorSpec.of(sample_prob, "sample_prob")
        self.dprob = TensorSpec.of(sample_dprob, "sample_dprob")
        self.sfd_row = TensorSpec.of(sample_sfd_row, "sample_sfd_row")
        self.sfd_col = TensorSpec.of(sample_sfd_col, "sample_sfd_col")
        self.amax = TensorSpec.of(sample_amax, "sample_amax")
        self.norm_const = TensorSpec.of(sample_norm_const, "sample_norm_const")
        self.expert_cnt = self.padded_offsets.shape[0]
        self.acc_dtype = acc_dtype
        self.mma_tiler_mn = tuple(mma_tiler_mn)
        self.use_2cta_instrs = self.mma_tiler_mn[0] == 256
        self.cluster_shape_mn = tuple(cluster_shape_mn) if cluster_shape_mn is not None else ((2, 1) if self.use_2cta_instrs else (1, 1))
        self.sf_vec_size = sf_vec_size
        self.vector_f32 = vector_f32
        self.m_aligned = m_aligned
        self.discrete_col_sfd = discrete_col_sfd
        self._value_error_if(
            epilogue_op not in (None, "none", "identity", "relu", "srelu"),
            f"Invalid epilogue operation: {epilogue_op}. Valid values: None, 'none', 'identity', 'relu', 'srelu'",
        )
        self.epilogue_op = epilogue_op
        self.num_cluster_overlap_margin = int(os.getenv("CUDNNFE_CLUSTER_OVERLAP_MARGIN", "0"))

    def check_support(self) -> bool:
        sfd_parts = [self.sfd_row, self.sfd_col, self.norm_const]
        all_none = all(x is None for x in sfd_parts)
        none_none = all(x is not None for x in sfd_parts)
        self._value_error_if(not (all_none or none_none), "sfd_row, sfd_col, and norm_const must be all None or all not None")
        self.generate_sfd = none_none
        if self.discrete_col_sfd and not self.generate_sfd:
            self._logger.warning("discrete_col_sfd is True but generate_sfd is False, discrete_col_sfd will be ignored")
            self.discrete_col_sfd = False

        self._value_error_if(len(self.a.shape) != 3, "A must be (m, k, 1)")
        a_l = self.a.logical()  # FP4 operands: two elements per byte along K
        tensor_m, k, _ = a_l.shape
        if self.discrete:
            b_l = None
            self._value_error_if(len(self._dw["b_shape"]) < 2, "b_shape must be (n, k)")
            n, b_k = self._dw["b_shape"][0], self._dw["b_shape"][1]
            l = int(self._dw["num_experts"])
            self._value_error_if(b_k != k, f"B K dimension ({b_k}) must match A K dimension ({k})")
            self._value_error_if(self.padded_offsets.shape[0] != l, f"padded_offsets length ({self.padded_offsets.shape[0]}) must equal num_experts ({l})")
            self._value_error_if(self._dw["b_major"] not in ("k", "n"), f"b_major must be 'k' or 'n', got {self._dw['b_major']}")
        else:
            self._value_error_if(len(self.b.shape) != 3, "B must be (n, k, l)")
            b_l = self.b.logical()
            n, _, l = b_l.shape
        self._check_shape(a_l, (tensor_m, k, 1), "A")
        self._check_shape(b_l, (n, k, l), "B")
        self._check_shape(self.c, (tensor_m, n * 2, 1), "C")
        self._check_shape(self.d_row, (tensor_m, n * 2, 1), "D_row")
        self._check_shape(self.d_col, (tensor_m, n * 2, 1), "D_col")
        rest_k = ceil_div(ceil_div(k, self.sf_vec_size), 4)
        self._check_shape(self.sfa, (32, 4, ceil_div(tensor_m, 128), 4, rest_k, 1), "SFA")
        self._check_shape(self.sfb, (32, 4, ceil_div(n, 128), 4, rest_k, l), "SFB")
        rest_n2 = ceil_div(ceil_div(n * 2, self.sf_vec_size), 4)
        self._check_shape(self.sfd_row, (32, 4, ceil_div(tensor_m, 128), 4, rest_n2, 1), "SFD_row")
        rest_m = ceil_div(ceil_div(tensor_m, self.sf_vec_size), 4)
        self._check_shape(self.sfd_col, (32, 4, ceil_div(n * 2, 128), 4, rest_m, 1), "SFD_col")
        self._check_shape(self.padded_offsets, (l,), "padded_offsets")
        self._check_shape(self.alpha, (l,), "alpha")
        self._check_shape(self.beta, (l,), "beta")
        self._check_shape(self.prob, (tensor_m, 1, 1), "prob")
        self._check_shape(self.dprob, (tensor_m, 1, 1), "dprob")
        self._check_shape(self.amax, (l, 2, 1), "amax")
        self._check_shape(self.norm_const, (1,), "norm_const")

        self._check_stride(a_l, (k, 1, tensor_m * k), "A must have k-major layout")
        self.ab_dtype = self._check_dtype(self.a, [torch.float4_e2m1fn_x2, torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn], "A/B")
        self._check_dtype(self.b, self.ab_dtype, "B", "B must have the same dtype as A")
        fp4 = self._is_fp4x2(self.ab_dtype)
        self._b_nmajor = False
        if self.discrete:
            self._value_error_if(self._dw["b_dtype"] != self.ab_dtype, f"b_dtype ({self._dw['b_dtype']}) must match A dtype ({self.ab_dtype})")
            self._value_error_if(fp4 and self._dw["b_major"] != "k", "b_major must be 'k' when ab_dtype is fp4")
            self._b_nmajor = self._dw["b_major"] == "n"
        elif not fp4 and n > 1 and k > 1 and self.b.stride[0] == 1 and self.b.stride[1] == n:
            self._check_stride(self.b, (1, n, n * k), "For fp8 ab_dtype, B must have k- or n-major layout")
            self._b_nmajor = True
        else:
            self._check_stride(b_l, (k, 1, n * k), "For fp4 ab_dtype, B must have k-major layout" if fp4 else "For fp8 ab_dtype, B must have k- or n-major layout")
        self._check_stride(self.c, (n * 2, 1, tensor_m * n * 2), "C must have n-major layout")
        self._check_stride(self.d_row, (n * 2, 1, tensor_m * n * 2), "D_row must have n-major layout")
        self._check_stride(self.d_col, (n * 2, 1, tensor_m * n * 2), "D_col must have n-major layout")
        for spec, mn, kk, ll in ((self.sfa, tensor_m, k, 1), (self.sfb, n, k, l), (self.sfd_row, tensor_m, n * 2, 1), (self.sfd_col, n * 2, tensor_m, 1)):
            if spec is not None:
                self._check_stride(spec, ops.sf_shape_stride(mn, kk, ll, self.sf_vec_size)[1], _SF_STRIDE_MSG)

        self.sf_dtype = self._check_dtype(self.sfa, [torch.float8_e8m0fnu, torch.float8_e4m3fn], "SFA/SFB/SFD_row/SFD_col")
        for spec, label in ((self.sfb, "SFB"), (self.sfd_row, "SFD_row"), (self.sfd_col, "SFD_col")):
            self._check_dtype(spec, self.sf_dtype, label, f"{label} must have the same dtype as SFA")
        self._value_error_if(self.sf_vec_size not in (16, 32), f"sf_vec_size must be 16 or 32, got {self.sf_vec_size}")
        self._value_error_if(self.sf_dtype == torch.float8_e4m3fn and self.sf_vec_size == 32, f"sf_dtype {self.sf_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._value_error_if(self._is_fp8(self.ab_dtype) and self.sf_vec_size == 16, f"ab_dtype {self.ab_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._check_dtype(self.acc_dtype, torch.float32, "Accumulator", "Accumulator must be float32")
        self._check_dtype(self.prob, torch.float32, "Prob", "Prob must be float32")
        self._check_dtype(self.dprob, torch.float32, "Dprob", "Dprob must be float32")
        self.c_dtype = self._check_dtype(self.c, [torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2], "C")
        self._value_error_if(
            self._is_fp8(self.c_dtype) and self.vector_f32,
            "Invalid configuration: fp8 ab_dtype, c_dtype, and vector_f32 is not supported. Please use vector_f32=False or c_dtype=bfloat16 instead",
        )
        if fp4:
            self.d_dtype = self._check_dtype(self.d_row, [torch.float16, torch.bfloat16, torch.float32], "D_row", "D_row must be fp16, bf16, or float32 when ab_dtype is fp4")
        else:
            self.d_dtype = self._check_dtype(self.d_row, [torch.float8_e4m3fn, torch.float8_e5m2], "D_row", "D_row must be fp8 dtype when ab_dtype is fp8")
        self._check_dtype(self.d_col, self.d_dtype, "D_col", "D_col must have the same dtype as D_row")
        self._check_dtype(self.padded_offsets, torch.int32, "padded_offsets")
        self._check_dtype(self.alpha, torch.float32, "alpha")
        self._check_dtype(self.beta, torch.float32, "beta")
        self._check_dtype(self.amax, torch.float32, "amax")
        self._check_dtype(self.norm_const, torch.float32, "norm_const")

        check_tile_and_cluster(self, self.mma_tiler_mn, self.cluster_shape_mn, self.m_aligned, only_n256=False)
        self._value_error_if(k % (32 if fp4 else 16) != 0 or n % 16 != 0, "Invalid tensor alignment: tensors must be 16B aligned")
        if self.expert_cnt > 1024:
            raise ValueError(f"expert_cnt must be <= 1024, got {self.expert_cnt}")

        # what this build implements of the reference's surface
        self._not_implemented_error_if(self.c_dtype == torch.float32, "a float32 C is not built (bf16, fp16, E4M3 and E5M2 are)")
        self._not_implemented_error_if(fp4 and k % 64 != 0, f"FP4 operands need k to be a multiple of 64, got {k}")
        self._not_implemented_error_if(fp4 and self.generate_sfd, "scale-factor generation is built for fp8 operands only")
        self._not_implemented_error_if(not fp4 and not self.generate_sfd, "fp8 operands need sfd_row, sfd_col and norm_const (an FP8 D)")
        self._not_implemented_error_if(fp4 and self.sf_vec_size == 16 and self.d_dtype == torch.float32, "fp4 ab_dtype, sf_vec_size 16, d_dtype float32 is not supported")
        self._value_error_if(n % 32 != 0, f"n must be a multiple of 32 (32-column gate / up blocks), got {n}")
        self._value_error_if(self.generate_sfd and self.d_col is None, "sample_d_col is required when scale factors are generated")
        self._n = n
        self._require_sm100()
        self._is_supported = True
        return True

    def compile(self) -> None:
        if not self._is_supported:
            self.check_support()
        ops._lib.load()  # fails loudly when the CUDA library is missing
        nbytes = ops.workspace_bytes(self.expert_cnt, self.discrete, self.use_dynamic_sched)
        if nbytes and self._workspace is None:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.a.device)
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        b_tensor: torch.Tensor,
        c_tensor: torch.Tensor,
        d_row_tensor: torch.Tensor,
        d_col_tensor: Optional[torch.Tensor],
        sfa_tensor: torch.Tensor,
        sfb_tensor: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        beta_tensor: torch.Tensor,
        prob_tensor: torch.Tensor,
        dprob_tensor: torch.Tensor,
        sfd_row_tensor: Optional[torch.Tensor] = None,
        sfd_col_tensor: Optional[torch.Tensor] = None,
        amax_tensor: Optional[torch.Tensor] = None,
        norm_const_tensor: Optional[torch.Tensor] = None,
        current_stream=None,
    ) -> None:
        """Launch on ``current_stream``; allocates nothing.  ``dprob_tensor`` must be zero on entry (the kernel adds
        to it); ``amax_tensor`` ``(l, 2, 1)`` is only ever raised."""
        a_tensor = as_packed_fp4(a_tensor)
        b_tensor = as_packed_fp4(b_tensor)
        self._ensure_compiled()
        if a_tensor.shape[0] == 0:
            return
        gen = bool(self.generate_sfd) and sfd_row_tensor is not None and norm_const_tensor is not None
        # discrete weights: b_tensor / sfb_tensor carry the int64 pointer arrays
        ops.grouped_gemm_op(
            "dswiglu",
            a=a_tensor,
            sfa=sfa_tensor,
            b=None if self.discrete else b_tensor,
            sfb=None if self.discrete else sfb_tensor,
            b_ptrs=b_tensor if self.discrete else None,
            sfb_ptrs=sfb_tensor if self.discrete else None,
            workspace=self._workspace,
            dynamic_sched=self.use_dynamic_sched,
            padded_offsets=padded_offsets,
            alpha=alpha_tensor,
            beta=beta_tensor,
            prob=prob_tensor,
            dprob=dprob_tensor,
            norm_const=norm_const_tensor if gen else None,
            c=c_tensor,
            d=d_row_tensor,
            d_col=d_col_tensor if gen else None,
            amax=None if gen or d_row_tensor.dtype == torch.float32 else amax_tensor,
            sfd_row=sfd_row_tensor if gen else None,
            sfd_col=sfd_col_tensor if gen else None,
            n=self._n,
            discrete_col_sfd=self.discrete_col_sfd,
            sm_margin=self.num_cluster_overlap_margin,
            tile_mode=pick_tile_mode(self.mma_tiler_mn, self.m_aligned),
            stream=current_stream,
            b_nmajor=self._b_nmajor,
            sf_vec_size=self.sf_vec_size,
        )


_cache_of_GroupedGemmDswigluSm100Objects = {}


def _alloc_sfd(mn: int, k: int, sf_vec_size: int, dtype, device) -> torch.Tensor:
    shape = (1, ceil_div(mn, 128), ceil_div(ceil_div(k, sf_vec_size), 4), 32, 4, 4)
    return torch.empty(shape, dtype=dtype, device=device).permute(3, 4, 1, 5, 2, 0)


def grouped_gemm_dswiglu_wrapper_sm100(
    a_tensor: torch.Tensor,
    b_tensor: torch.Tensor,
    c_tensor: torch.Tensor,
    sfa_tensor: torch.Tensor,
    sfb_tensor: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha_tensor: torch.Tensor,
    beta_tensor: Optional[torch.Tensor],
    prob_tensor: torch.Tensor,
    norm_const_tensor: Optional[torch.Tensor] = None,
    acc_dtype: torch.dtype = torch.float32,
    d_dtype: torch.dtype = torch.bfloat16,
    cd_major: str = "n",
    mma_tiler_mn: Tuple[int, int] = (256, 256),
    cluster_shape_mn: Optional[Tuple[int, int]] = None,
    sf_vec_size: int = 16,
    vector_f32: bool = False,
    m_aligned: int = 256,
    discrete_col_sfd: bool = False,
    epilogue_op: Optional[str] = None,
    current_stream=None,
    dprob_tensor_buf: Optional[torch.Tensor] = None,
    amax_tensor_buf: Optional[torch.Tensor] = None,
) -> TupleDict:
    """One-shot dSwiGLU.  Returns ``TupleDict(d_row_tensor, d_col_tensor, dprob_tensor, amax_tensor, sfd_row_tensor,
    sfd_col_tensor)``; ``dprob`` is zeroed here before the launch, amax (16-bit ``d_dtype``) is allocated per cached
    configuration like the reference's (api.py:838-860) and starts at -inf."""
    a_tensor = as_packed_fp4(a_tensor)
    b_tensor = as_packed_fp4(b_tensor)
    valid_m = a_tensor.shape[0]
    n, _, l = b_tensor.shape
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    dev = a_tensor.device
    d_row_tensor = torch.empty_strided((valid_m, n * 2, 1), (n * 2, 1, valid_m * n * 2), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n * 2, 1), (n * 2, 1, valid_m * n * 2), dtype=d_dtype, device=dev)
    dprob_tensor = dprob_tensor_buf.zero_() if dprob_tensor_buf is not None else torch.zeros((valid_m, 1, 1), dtype=torch.float32, device=dev)
    if valid_m == 0:
        amax_tensor = torch.full((l, 2, 1), float("-inf"), dtype=torch.float32, device=dev) if d_dtype in (torch.bfloat16, torch.float16) else None
        return TupleDict(d_row_tensor=d_row_tensor, d_col_tensor=d_col_tensor, dprob_tensor=dprob_tensor, amax_tensor=amax_tensor, sfd_row_tensor=None, sfd_col_tensor=None)
    sfd_row_tensor = sfd_col_tensor = None
    if a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and sfa_tensor.dtype in (torch.float8_e8m0fnu, torch.float8_e4m3fn):
        sfd_row_tensor = _alloc_sfd(valid_m, n * 2, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n * 2, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    key = (
        a_tensor.dtype, b_tensor.dtype, c_tensor.dtype, sfa_tensor.dtype, tuple(a_tensor.shape[1:]), tuple(b_tensor.shape), tuple(b_tensor.stride()),
        norm_const_tensor is not None, acc_dtype, d_dtype, tuple(mma_tiler_mn), None if cluster_shape_mn is None else tuple(cluster_shape_mn),
        sf_vec_size, vector_f32, m_aligned, discrete_col_sfd, epilogue_op, str(dev),
    )  # fmt: skip
    hit = _cache_of_GroupedGemmDswigluSm100Objects.get(key)
    if hit is None:
        cached_beta = torch.ones(l, dtype=torch.float32, device=dev) if beta_tensor is None else None
        cached_amax = torch.full((l, 2, 1), float("-inf"), dtype=torch.float32, device=dev) if d_dtype in (torch.bfloat16, torch.float16) else None
        op = GroupedGemmDswigluSm100(
            sample_a=a_tensor, sample_b=b_tensor, sample_c=c_tensor, sample_d_row=d_row_tensor, sample_d_col=d_col_tensor, sample_sfa=sfa_tensor,
            sample_sfb=sfb_tensor, sample_padded_offsets=padded_offsets, sample_alpha=alpha_tensor,
            sample_beta=cached_beta if beta_tensor is None else beta_tensor, sample_prob=prob_tensor, sample_dprob=dprob_tensor,
            sample_amax=cached_amax, sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor,
            sample_norm_const=norm_const_tensor if sfd_row_tensor is not None else None, acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn,
            cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size, vector_f32=vector_f32, m_aligned=m_aligned,
            discrete_col_sfd=discrete_col_sfd, epilogue_op=epilogue_op,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_GroupedGemmDswigluSm100Objects[key] = (op, cached_amax, cached_beta)
    else:
        op, cached_amax, cached_beta = hit
    amax_tensor = amax_tensor_buf if amax_tensor_buf is not None else cached_amax
    if beta_tensor is not None:
        effective_beta = beta_tensor
    elif cached_beta is not None:
        effective_beta = cached_beta
    else:
        effective_beta = torch.ones(l, dtype=torch.float32, device=dev)
    op.execute(
        a_tensor=a_tensor, b_tensor=b_tensor, c_tensor=c_tensor, d_row_tensor=d_row_tensor, d_col_tensor=d_col_tensor, sfa_tensor=sfa_tensor,
        sfb_tensor=sfb_tensor, padded_offsets=padded_offsets, alpha_tensor=alpha_tensor, beta_tensor=effective_beta, prob_tensor=prob_tensor,
        dprob_tensor=dprob_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
        norm_const_tensor=norm_const_tensor if sfd_row_tensor is not None else None, current_stream=current_stream,
    )  # fmt: skip
    return TupleDict(d_row_tensor=d_row_tensor, d_col_tensor=d_col_tensor, dprob_tensor=dprob_tensor, amax_tensor=amax_tensor,
                     sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)  # fmt: skip


class DiscreteGroupedGemmDswigluSm100(GroupedGemmDswigluSm100):
    """dSwiGLU with one weight allocation per expert: ``b_ptrs`` / ``sfb_ptrs`` are int64 device arrays of the experts'
    ``[n, k]`` (``b_major="k"``) or ``[k, n]`` (``"n"``) weights and of their 128x4 scale tensors."""

    def __init__(
        self,
        sample_a: torch.Tensor,
        num_experts: int,
        b_shape: Tuple[int, ...],
        b_dtype: torch.dtype,
        sample_c: torch.Tensor,
        sample_d_row: torch.Tensor,
        sample_d_col: Optional[torch.Tensor],
        sample_sfa: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_beta: torch.Tensor,
        sample_prob: torch.Tensor,
        sample_dprob: torch.Tensor,
        sample_dbias: Optional[torch.Tensor] = None,
        sample_sfd_row: Optional[torch.Tensor] = None,
        sample_sfd_col: Optional[torch.Tensor] = None,
        sample_amax: Optional[torch.Tensor] = None,
        sample_norm_const: Optional[torch.Tensor] = None,
        acc_dtype: torch.dtype = torch.float32,
        mma_tiler_mn: Tuple[int, int] = (256, 256),
        cluster_shape_mn: Optional[Tuple[int, int]] = None,
        sf_vec_size: int = 16,
        vector_f32: bool = False,
        m_aligned: int = 256,
        discrete_col_sfd: bool = False,
        act_func: str = "dswiglu",
        b_major: str = "k",
        epilogue_op: Optional[str] = None,
        use_dynamic_sched: bool = False,
    ):
        super().__init__(
            sample_a, None, sample_c, sample_d_row, sample_d_col, sample_sfa, None, sample_padded_offsets, sample_alpha, sample_beta, sample_prob,
            sample_dprob, sample_sfd_row=sample_sfd_row, sample_sfd_col=sample_sfd_col, sample_amax=sample_amax, sample_norm_const=sample_norm_const,
            acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size, vector_f32=vector_f32,
            m_aligned=m_aligned, discrete_col_sfd=discrete_col_sfd, epilogue_op=epilogue_op,
            _discrete=dict(num_experts=num_experts, b_shape=tuple(b_shape), b_dtype=packed_fp4_dtype(b_dtype), b_major=b_major, use_dynamic_sched=use_dynamic_sched),
        )  # fmt: skip
        self._value_error_if(act_func not in ("dswiglu", "dgeglu"), f"act_func must be 'dswiglu' or 'dgeglu', got {act_func}")
        self.act_func = act_func
        self.dbias = TensorSpec.of(sample_dbias, "sample_dbias")

    def check_support(self) -> bool:
        self._not_implemented_error_if(self.act_func != "dswiglu", f"act_func {self.act_func!r} is not built ('dswiglu' is)")
        self._not_implemented_error_if(self.dbias is not None, "the dbias output is not built")
        return super().check_support()

    def execute(
        self,
        a_tensor: torch.Tensor,
        b_ptrs: torch.Tensor,
        c_tensor: torch.Tensor,
        d_row_tensor: torch.Tensor,
        d_col_tensor: Optional[torch.Tensor],
        sfa_tensor: torch.Tensor,
        sfb_ptrs: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        beta_tensor: torch.Tensor,
        prob_tensor: torch.Tensor,
        dprob_tensor: torch.Tensor,
        dbias_tensor: Optional[torch.Tensor] = None,
        sfd_row_tensor: Optional[torch.Tensor] = None,
        sfd_col_tensor: Optional[torch.Tensor] = None,
        amax_tensor: Optional[torch.Tensor] = None,
        norm_const_tensor: Optional[torch.Tensor] = None,
        current_stream=None,
    ) -> None:
        """Launch on ``current_stream``; allocates nothing and never reads the pointer values on the host."""
        a_tensor = as_packed_fp4(a_tensor)
        from .discrete_grouped_gemm_swiglu import _require_pointer_tensor

        if dbias_tensor is not None:
            raise NotImplementedError("the dbias output is not built")
        _require_pointer_tensor(b_ptrs, "b_ptrs", self.expert_cnt)
        _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", self.expert_cnt)
        super().execute(a_tensor, b_ptrs, c_tensor, d_row_tensor, d_col_tensor, sfa_tensor, sfb_ptrs, padded_offsets, alpha_tensor, beta_tensor,
                        prob_tensor, dprob_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
                        norm_const_tensor=norm_const_tensor, current_stream=current_stream)  # fmt: skip


_cache_of_DiscreteGroupedGemmDswigluSm100Objects = {}


def discrete_grouped_gemm_dswiglu_wrapper_sm100(
    a_tensor: torch.Tensor,
    b_ptrs: torch.Tensor,
    c_tensor: torch.Tensor,
    sfa_tensor: torch.Tensor,
    sfb_ptrs: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha_tensor: torch.Tensor,
    beta_tensor: torch.Tensor,
    prob_tensor: torch.Tensor,
    dprob_tensor: torch.Tensor,
    n: int,
    b_dtype: torch.dtype,
    generate_dbias: bool = False,
    norm_const_tensor: Optional[torch.Tensor] = None,
    acc_dtype: torch.dtype = torch.float32,
    d_dtype: torch.dtype = torch.bfloat16,
    cd_major: str = "n",
    mma_tiler_mn: Tuple[int, int] = (256, 256),
    cluster_shape_mn: Optional[Tuple[int, int]] = None,
    sf_vec_size: int = 16,
    vector_f32: bool = False,
    m_aligned: int = 256,
    discrete_col_sfd: bool = False,
    act_func: str = "dswiglu",
    b_major: str = "k",
    epilogue_op: Optional[str] = None,
    use_dynamic_sched: bool = False,
    current_stream=None,
) -> TupleDict:
    """One-shot discrete-weight dSwiGLU.  The caller owns ``dprob_tensor`` (zeroed by the caller, as in the reference).
    Returns ``TupleDict(d_row_tensor, d_col_tensor, dprob_tensor, dbias_tensor, amax_tensor, sfd_row_tensor,
    sfd_col_tensor)``."""
    a_tensor = as_packed_fp4(a_tensor)
    b_dtype = packed_fp4_dtype(b_dtype)
    from .discrete_grouped_gemm_swiglu import _require_pointer_tensor

    if generate_dbias:
        raise NotImplementedError("the dbias output is not built")
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    _require_pointer_tensor(b_ptrs, "b_ptrs")
    l = b_ptrs.shape[0]
    _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", l)
    valid_m, k, _ = a_tensor.shape
    if a_tensor.dtype == torch.float4_e2m1fn_x2:
        k *= 2
    dev = a_tensor.device
    d_row_tensor = torch.empty_strided((valid_m, n * 2, 1), (n * 2, 1, valid_m * n * 2), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n * 2, 1), (n * 2, 1, valid_m * n * 2), dtype=d_dtype, device=dev)
    sfd_row_tensor = sfd_col_tensor = amax_tensor = None
    if a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        sfd_row_tensor = _alloc_sfd(valid_m, n * 2, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n * 2, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    if d_dtype in (torch.bfloat16, torch.float16):
        amax_tensor = torch.full((l, 2, 1), float("-inf"), dtype=torch.float32, device=dev)
    out = TupleDict(d_row_tensor=d_row_tensor, d_col_tensor=d_col_tensor, dprob_tensor=dprob_tensor, dbias_tensor=None, amax_tensor=amax_tensor,
                    sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)  # fmt: skip
    if valid_m == 0:
        return out
    key = (a_tensor.dtype, c_tensor.dtype, sfa_tensor.dtype, b_dtype, tuple(a_tensor.shape[1:]), n, l, norm_const_tensor is not None, acc_dtype, d_dtype,
           tuple(mma_tiler_mn), None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, vector_f32, m_aligned, discrete_col_sfd,
           act_func, b_major, epilogue_op, use_dynamic_sched, str(dev))  # fmt: skip
    op = _cache_of_DiscreteGroupedGemmDswigluSm100Objects.get(key)
    if op is None:
        op = DiscreteGroupedGemmDswigluSm100(
            a_tensor, l, (n, k), b_dtype, c_tensor, d_row_tensor, d_col_tensor, sfa_tensor, padded_offsets, alpha_tensor, beta_tensor, prob_tensor,
            dprob_tensor, sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor, sample_amax=amax_tensor,
            sample_norm_const=norm_const_tensor if sfd_row_tensor is not None else None, acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn,
            cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size, vector_f32=vector_f32, m_aligned=m_aligned,
            discrete_col_sfd=discrete_col_sfd, act_func=act_func, b_major=b_major, epilogue_op=epilogue_op, use_dynamic_sched=use_dynamic_sched,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_DiscreteGroupedGemmDswigluSm100Objects[key] = op
    op.execute(a_tensor, b_ptrs, c_tensor, d_row_tensor, d_col_tensor, sfa_tensor, sfb_ptrs, padded_offsets, alpha_tensor, beta_tensor, prob_tensor,
               dprob_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
               norm_const_tensor=norm_const_tensor if sfd_row_tensor is not None else None, current_stream=current_stream)  # fmt: skip
    return out
