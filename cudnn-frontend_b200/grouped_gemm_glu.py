"""Unified FC1: grouped GEMM + GLU activation for dense and discrete weights.

Same names, arguments and error behaviour as the reference's ``GroupedGemmGluSm100`` /
``grouped_gemm_glu_wrapper_sm100`` (python/cudnn/grouped_gemm/grouped_gemm_glu/api.py:99-133,
1094-1117, 1212-1243), its successor to both FC1 classes: one signature for dense weights
(``sample_b`` / ``sample_sfb``) and discrete ones (``num_experts`` / ``b_shape`` / ``b_dtype``, pointer
tensors at execute time), ``act_func`` in {"swiglu", "geglu"} and an optional fused bias ``(n, l)``
with stride ``(1, n)``:

    C = alpha_e * acc + bias_e            (stored as bf16 when a C tensor is given)
    swiglu:  D = up * gate * sigmoid(gate) * prob
    geglu:   gate <= 7, -7 <= up <= 7 (after the C store);  D = (up + 1) * gate * sigmoid(1.702 gate) * prob

The class owns one of this package's two FC1 operators and forwards to it; both launch the same
kernel.  ``use_dynamic_sched=True`` hands tiles out through an atomic counter in either weight mode;
``b_major="n"`` (discrete mode) takes per-expert ``[k][n]`` weights.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .api_base import OperatorBase, TupleDict, as_packed_fp4, packed_fp4_dtype
from .discrete_grouped_gemm_swiglu import DiscreteGroupedGemmSwigluSm100
from .grouped_gemm_quant import _require_pointer_tensor
from .grouped_gemm_swiglu import GroupedGemmSwigluSm100, _alloc_sfd


class GroupedGemmGluSm100(OperatorBase):
    def __init__(
        self,
        sample_a: torch.Tensor,
        sample_c: Optional[torch.Tensor],
        sample_d: torch.Tensor,
        sample_sfa: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_d_col: Optional[torch.Tensor],
        # dense mode
        sample_b: Optional[torch.Tensor] = None,
        sample_sfb: Optional[torch.Tensor] = None,
        sample_bias: Optional[torch.Tensor] = None,
        # discrete mode
        num_experts: Optional[int] = None,
        b_shape: Optional[Tuple[int, ...]] = None,
        b_dtype: Optional[torch.dtype] = None,
        # optional quantisation outputs
        sample_sfd_row: Optional[torch.Tensor] = None,
        sample_sfd_col: Optional[torch.Tensor] = None,
        sample_amax: Optional[torch.Tensor] = None,
        sample_norm_const: Optional[torch.Tensor] = None,
        sample_prob: Optional[torch.Tensor] = None,
        # configuration
        acc_dtype: torch.dtype = torch.float32,
        mma_tiler_mn: Tuple[int, int] = (256, 256),
        cluster_shape_mn: Optional[Tuple[int, int]] = None,
        sf_vec_size: int = 16,
        vector_f32: bool = False,
        m_aligned: int = 256,
        discrete_col_sfd: bool = False,
        act_func: str = "swiglu",
        b_major: str = "k",
        use_dynamic_sched: bool = False,
    ):
        super().__init__()
        dense = sample_b is not None or sample_sfb is not None
        discrete = num_experts is not None or b_shape is not None
        self._value_error_if(dense and discrete, "Provide either (sample_b, sample_sfb) or (num_experts, b_shape, b_dtype), not both")
        self._value_error_if(not dense and not discrete, "Must provide either (sample_b, sample_sfb) or (num_experts, b_shape, b_dtype)")
        self.discrete = discrete
        self.act_func = act_func
        self.b_major = b_major
        self.use_dynamic_sched = use_dynamic_sched
        common = dict(sample_sfd_row=sample_sfd_row, sample_sfd_col=sample_sfd_col, sample_amax=sample_amax,
                      sample_norm_const=sample_norm_const, sample_prob=sample_prob, acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn,
                      cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size, vector_f32=vector_f32, m_aligned=m_aligned,
                      discrete_col_sfd=discrete_col_sfd, sample_bias=sample_bias, act_func=act_func)  # fmt: skip
        if discrete:
            self._value_error_if(num_experts is None or b_shape is None or b_dtype is None, "discrete mode needs num_experts, b_shape and b_dtype")
            self._op = DiscreteGroupedGemmSwigluSm100(sample_a, num_experts, b_shape, b_dtype, sample_c, sample_d, sample_sfa,
                                                      sample_padded_offsets, sample_alpha, sample_d_col, b_major=b_major,
                                                      use_dynamic_sched=use_dynamic_sched, **common)  # fmt: skip
        else:
            self._value_error_if(sample_b is None or sample_sfb is None, "dense mode needs sample_b and sample_sfb")
            self._op = GroupedGemmSwigluSm100(sample_a, sample_b, sample_c, sample_d, sample_sfa, sample_sfb, sample_padded_offsets,
                                              sample_alpha, sample_d_col, **common)  # fmt: skip
            self._op.use_dynamic_sched = bool(use_dynamic_sched)
        self.expert_cnt = self._op.expert_cnt

    def check_support(self) -> bool:
        self._value_error_if(self.b_major not in ("k", "n"), f"b_major must be 'k' or 'n', got {self.b_major}")
        # dense weights carry their layout in their strides (K-major only for FC1, as in the reference);
        # b_major describes the allocations behind the pointers of discrete mode
        self._is_supported = self._op.check_support()
        return self._is_supported

    def compile(self) -> None:
        if not self._is_supported:
            self.check_support()
        self._op.compile()
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        c_tensor: Optional[torch.Tensor],
        d_tensor: torch.Tensor,
        sfa_tensor: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        b_tensor: Optional[torch.Tensor] = None,
        sfb_tensor: Optional[torch.Tensor] = None,
        bias_tensor: Optional[torch.Tensor] = None,
        b_ptrs: Optional[torch.Tensor] = None,
        sfb_ptrs: Optional[torch.Tensor] = None,
        d_col_tensor: Optional[torch.Tensor] = None,
        sfd_row_tensor: Optional[torch.Tensor] = None,
        sfd_col_tensor: Optional[torch.Tensor] = None,
        amax_tensor: Optional[torch.Tensor] = None,
        norm_const_tensor: Optional[torch.Tensor] = None,
        prob_tensor: Optional[torch.Tensor] = None,
        current_stream=None,
    ) -> None:
        """Dense mode: supply ``b_tensor`` and ``sfb_tensor``; discrete mode: ``b_ptrs`` and ``sfb_ptrs``.
        Bias fusion is fixed at construction (``sample_bias``)."""
        self._ensure_compiled()
        tail = dict(d_col_tensor=d_col_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
                    norm_const_tensor=norm_const_tensor, prob_tensor=prob_tensor, current_stream=current_stream, bias_tensor=bias_tensor)  # fmt: skip
        if self.discrete:
            if b_ptrs is None or sfb_ptrs is None:
                raise ValueError("discrete mode needs b_ptrs and sfb_ptrs")
            self._op.execute(a_tensor, b_ptrs, c_tensor, d_tensor, sfa_tensor, sfb_ptrs, padded_offsets, alpha_tensor, **tail)
        else:
            if b_tensor is None or sfb_tensor is None:
                raise ValueError("dense mode needs b_tensor and sfb_tensor")
            self._op.execute(a_tensor, b_tensor, c_tensor, d_tensor, sfa_tensor, sfb_tensor, padded_offsets, alpha_tensor, **tail)


_cache_of_GroupedGemmGluSm100Objects = {}


def grouped_gemm_glu_wrapper_sm100(
    a_tensor: torch.Tensor,
    sfa_tensor: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha_tensor: torch.Tensor,
    b_tensor: Optional[torch.Tensor] = None,
    sfb_tensor: Optional[torch.Tensor] = None,
    bias_tensor: Optional[torch.Tensor] = None,
    b_ptrs: Optional[torch.Tensor] = None,
    sfb_ptrs: Optional[torch.Tensor] = None,
    n: Optional[int] = None,
    b_dtype: Optional[torch.dtype] = None,
    b_major: str = "k",
    norm_const_tensor: Optional[torch.Tensor] = None,
    prob_tensor: Optional[torch.Tensor] = None,
    acc_dtype: torch.dtype = torch.float32,
    c_dtype: torch.dtype = torch.bfloat16,
    d_dtype: torch.dtype = torch.bfloat16,
    cd_major: str = "n",
    mma_tiler_mn: Tuple[int, int] = (256, 256),
    cluster_shape_mn: Optional[Tuple[int, int]] = None,
    sf_vec_size: int = 16,
    vector_f32: bool = False,
    m_aligned: int = 256,
    discrete_col_sfd: bool = False,
    act_func: str = "swiglu",
    use_dynamic_sched: bool = False,
    current_stream=None,
) -> TupleDict:
    """One-shot unified FC1.  Dense mode: ``b_tensor`` + ``sfb_tensor``; discrete mode: ``b_ptrs``,
    ``sfb_ptrs``, ``n`` and ``b_dtype``.  Allocates the outputs, reuses a cached operator per
    configuration and returns ``TupleDict(c_tensor, d_tensor, d_col_tensor, amax_tensor,
    sfd_row_tensor, sfd_col_tensor)``."""
    a_tensor = as_packed_fp4(a_tensor)
    b_tensor = as_packed_fp4(b_tensor)
    b_dtype = packed_fp4_dtype(b_dtype)
    dense = b_tensor is not None
    discrete = b_ptrs is not None
    if dense and discrete:
        raise ValueError("Provide either (b_tensor, sfb_tensor) or (b_ptrs, sfb_ptrs), not both")
    if not dense and not discrete:
        raise ValueError("Must provide either (b_tensor, sfb_tensor) or (b_ptrs, sfb_ptrs)")
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    valid_m, k, _ = a_tensor.shape
    if a_tensor.dtype == torch.float4_e2m1fn_x2:
        k *= 2  # two elements per byte
    if dense:
        n_full, _, l = b_tensor.shape
    else:
        _require_pointer_tensor(b_ptrs, "b_ptrs")
        if n is None or b_dtype is None:
            raise ValueError("discrete mode needs n and b_dtype")
        n_full, l = n, b_ptrs.shape[0]
    n_out = n_full // 2
    dev = a_tensor.device
    c_tensor = torch.empty_strided((valid_m, n_full, 1), (n_full, 1, valid_m * n_full), dtype=c_dtype, device=dev)
    d_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    sfd_row_tensor = sfd_col_tensor = amax_tensor = None
    fp8_in = a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
    if fp8_in and (d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2) or norm_const_tensor is not None):
        sfd_row_tensor = _alloc_sfd(valid_m, n_out, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n_out, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    if d_dtype in (torch.bfloat16, torch.float16):
        amax_tensor = torch.full((l, 1), float("-inf"), dtype=torch.float32, device=dev)
    out = TupleDict(c_tensor=c_tensor, d_tensor=d_tensor, d_col_tensor=d_col_tensor, amax_tensor=amax_tensor,
                    sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)  # fmt: skip
    if valid_m == 0:
        return out
    key = (dense, a_tensor.dtype, sfa_tensor.dtype, c_dtype, d_dtype, acc_dtype, (valid_m, k), (n_full, l), tuple(mma_tiler_mn),
           None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, vector_f32, m_aligned, discrete_col_sfd,
           act_func, b_major, use_dynamic_sched, prob_tensor is not None, norm_const_tensor is not None,
           None if bias_tensor is None else bias_tensor.dtype, str(dev))  # fmt: skip
    op = _cache_of_GroupedGemmGluSm100Objects.get(key)
    if op is None:
        mode = dict(sample_b=b_tensor, sample_sfb=sfb_tensor) if dense else dict(num_experts=l, b_shape=(n_full, k), b_dtype=b_dtype)
        op = GroupedGemmGluSm100(
            a_tensor, c_tensor, d_tensor, sfa_tensor, padded_offsets, alpha_tensor, d_col_tensor, sample_bias=bias_tensor,
            sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor, sample_amax=amax_tensor,
            sample_norm_const=norm_const_tensor if sfd_row_tensor is not None else None, sample_prob=prob_tensor,
            acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size,
            vector_f32=vector_f32, m_aligned=m_aligned, discrete_col_sfd=discrete_col_sfd, act_func=act_func, b_major=b_major,
            use_dynamic_sched=use_dynamic_sched, **mode,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_GroupedGemmGluSm100Objects[key] = op
    op.execute(
        a_tensor, c_tensor, d_tensor, sfa_tensor, padded_offsets, alpha_tensor, b_tensor=b_tensor, sfb_tensor=sfb_tensor,
        bias_tensor=bias_tensor, b_ptrs=b_ptrs, sfb_ptrs=sfb_ptrs, d_col_tensor=d_col_tensor, sfd_row_tensor=sfd_row_tensor,
        sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor, norm_const_tensor=norm_const_tensor, prob_tensor=prob_tensor,
        current_stream=current_stream,
    )  # fmt: skip
    return out
