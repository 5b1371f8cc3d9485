"""FC1 with discrete (per-expert pointer) weights.

Same names, arguments and error behaviour as the reference's
``DiscreteGroupedGemmSwigluSm100`` / ``discrete_grouped_gemm_swiglu_wrapper_sm100``
(python/cudnn/discrete_grouped_gemm/discrete_grouped_gemm_swiglu/api.py:60-1050): every expert's
weight is its own ``(n, k)`` K-major allocation with its own 128x4 scale-factor tensor; their
device addresses arrive as two 1-D int64 CUDA tensors that are only ever read on the device.
``execute`` allocates nothing (descriptor workspace is created in ``compile``).

``act_func="geglu"`` and a fused bias ``(n, l)`` (stride ``(1, n)``) are supported as in the reference's
GLU kernel; ``b_major="n"`` takes per-expert ``[k][n]`` weights and ``use_dynamic_sched=True`` the
atomic-counter tile scheduler.
"""

from __future__ import annotations

import logging
import os
from typing import Optional, Tuple

import torch

from . import ops
from .api_base import OperatorBase, TensorSpec, TupleDict, as_packed_fp4, ceil_div, check_tile_and_cluster, packed_fp4_dtype, pick_tile_mode
from .grouped_gemm_quant import _require_pointer_tensor
from .grouped_gemm_swiglu import _SF_STRIDE_MSG, _alloc_sfd

_logger = logging.getLogger(__name__)


class DiscreteGroupedGemmSwigluSm100(OperatorBase):
    def __init__(
        self,
        sample_a: torch.Tensor,
        num_experts: int,
        b_shape: Tuple[int, ...],
        b_dtype: torch.dtype,
        sample_c: Optional[torch.Tensor],
        sample_d: torch.Tensor,
        sample_sfa: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_d_col: Optional[torch.Tensor],
        sample_bias: Optional[torch.Tensor] = None,
        sample_sfd_row: Optional[torch.Tensor] = None,
        sample_sfd_col: Optional[torch.Tensor] = None,
        sample_amax: Optional[torch.Tensor] = None,
        sample_norm_const: Optional[torch.Tensor] = None,
        sample_prob: Optional[torch.Tensor] = None,
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
        b_dtype = packed_fp4_dtype(b_dtype)
        super().__init__()
        self.a = TensorSpec.of(as_packed_fp4(sample_a), "sample_a")
        self.c = TensorSpec.of(sample_c, "sample_c")
        self.d = TensorSpec.of(sample_d, "sample_d")
        self.sfa = TensorSpec.of(sample_sfa, "sample_sfa")
        self.padded_offsets = TensorSpec.of(sample_padded_offsets, "sample_padded_offsets")
        self.alpha = TensorSpec.of(sample_alpha, "sample_alpha")
        self.d_col = TensorSpec.of(sample_d_col, "sample_d_col")
        self.bias = TensorSpec.of(sample_bias, "sample_bias")
        self.sfd_row = TensorSpec.of(sample_sfd_row, "sample_sfd_row")
        self.sfd_col = TensorSpec.of(sample_sfd_col, "sample_sfd_col")
        self.amax = TensorSpec.of(sample_amax, "sample_amax")
        self.norm_const = TensorSpec.of(sample_norm_const, "sample_norm_const")
        self.prob = TensorSpec.of(sample_prob, "sample_prob")
        self._value_error_if(not num_experts or num_experts <= 0, "num_experts must be > 0")
        self.expert_cnt = num_experts
        self.b_shape = tuple(b_shape)
        self.b_dtype = b_dtype
        self.acc_dtype = acc_dtype
        self.mma_tiler_mn = tuple(mma_tiler_mn)
        self.use_2cta_instrs = self.mma_tiler_mn[0] == 256
        self.cluster_shape_mn = tuple(cluster_shape_mn) if cluster_shape_mn is not None else ((2, 1) if self.use_2cta_instrs else (1, 1))
        self.sf_vec_size = sf_vec_size
        self.vector_f32 = vector_f32
        self.m_aligned = m_aligned
        self.discrete_col_sfd = discrete_col_sfd
        self.act_func = act_func
        self.b_major = b_major
        self.use_dynamic_sched = use_dynamic_sched
        self.num_cluster_overlap_margin = int(os.getenv("CUDNNFE_CLUSTER_OVERLAP_MARGIN", "0"))
        self._workspace = None

    def check_support(self) -> bool:
        sfd_parts = [self.sfd_row, self.sfd_col, self.norm_const]
        all_none = all(x is None for x in sfd_parts)
        all_provided = all(x is not None for x in sfd_parts)
        self._value_error_if(not (all_none or all_provided), "sfd_row_desc, sfd_col_desc, and norm_const_desc must be all None or all not None")
        self.generate_sfd = all_provided
        if self.discrete_col_sfd and not self.generate_sfd:
            self._logger.warning("discrete_col_sfd is True but generate_sfd is False, discrete_col_sfd will be ignored")
            self.discrete_col_sfd = False
        self._value_error_if(self.act_func not in ("swiglu", "geglu"), f"act_func must be 'swiglu' or 'geglu', got {self.act_func}")
        self._value_error_if(self.b_major not in ("k", "n"), f"b_major must be 'k' or 'n', got {self.b_major}")
        self._value_error_if(len(self.a.shape) != 3 or len(self.b_shape) < 2, "A must be (m, k, 1) and b_shape (n, k)")
        a_l = self.a.logical()  # FP4 operands: two elements per byte along K; b_shape counts elements
        tensor_m, k, _ = a_l.shape
        n, b_k = self.b_shape[0], self.b_shape[1]
        self._value_error_if(b_k != k, f"B K dimension ({b_k}) must match A K dimension ({k})")
        self._value_error_if(self.padded_offsets.shape[0] != self.expert_cnt, f"padded_offsets length ({self.padded_offsets.shape[0]}) must equal num_experts ({self.expert_cnt})")
        n_2 = n // 2
        l = self.expert_cnt
        self._check_shape(a_l, (tensor_m, k, 1), "A")
        self._check_shape(self.c, (tensor_m, n, 1), "C")
        self._check_shape(self.d, (tensor_m, n_2, 1), "D")
        self._check_shape(self.d_col, (tensor_m, n_2, 1), "D_col")
        rest_k = ceil_div(ceil_div(k, self.sf_vec_size), 4)
        self._check_shape(self.sfa, (32, 4, ceil_div(tensor_m, 128), 4, rest_k, 1), "SFA")
        self._check_shape(self.sfd_row, (32, 4, ceil_div(tensor_m, 128), 4, ceil_div(ceil_div(n_2, self.sf_vec_size), 4), 1), "SFD_row")
        self._check_shape(self.sfd_col, (32, 4, ceil_div(n_2, 128), 4, ceil_div(ceil_div(tensor_m, self.sf_vec_size), 4), 1), "SFD_col")
        self._check_shape(self.alpha, (l,), "alpha")
        self._check_shape(self.prob, (tensor_m, 1, 1), "prob")
        self._check_shape(self.bias, (n, l), "bias")
        self._check_shape(self.amax, (l, 1), "amax")
        self._check_shape(self.norm_const, (1,), "norm_const")
        self._check_stride(a_l, (k, 1, tensor_m * k), "A must have k-major layout")
        self._check_stride(self.c, (n, 1, tensor_m * n), "C must have n-major layout")
        self._check_stride(self.d, (n_2, 1, tensor_m * n_2), "D must have n-major layout")
        self._check_stride(self.d_col, (n_2, 1, tensor_m * n_2), "D_col must have n-major layout")
        for spec, mn, kk in ((self.sfa, tensor_m, k), (self.sfd_row, tensor_m, n_2), (self.sfd_col, n_2, tensor_m)):
            if spec is not None:
                self._check_stride(spec, ops.sf_shape_stride(mn, kk, 1, self.sf_vec_size)[1], _SF_STRIDE_MSG)
        self.ab_dtype = self._check_dtype(self.a, [torch.float4_e2m1fn_x2, torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn], "A/B")
        self._value_error_if(self.b_dtype != self.ab_dtype, f"b_dtype ({self.b_dtype}) must match A dtype ({self.ab_dtype})")
        self.sf_dtype = self._check_dtype(self.sfa, [torch.float8_e8m0fnu, torch.float8_e4m3fn], "SFA/SFD_row/SFD_col")
        self._check_dtype(self.sfd_row, self.sf_dtype, "SFD_row")
        self._check_dtype(self.sfd_col, self.sf_dtype, "SFD_col")
        self._value_error_if(self.sf_vec_size not in (16, 32), f"sf_vec_size must be 16 or 32, got {self.sf_vec_size}")
        self._value_error_if(self._is_fp8(self.ab_dtype) and self.sf_vec_size == 16, f"ab_dtype {self.ab_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._check_dtype(self.acc_dtype, torch.float32, "Accumulator", "Accumulator must be float32")
        self.c_dtype = self._check_dtype(self.c, [torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2], "C")
        self.d_dtype = self._check_dtype(self.d, [torch.float16, torch.bfloat16, torch.float32, torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2], "D")
        self._check_dtype(self.d_col, self.d_dtype, "D_col", "D_col must have the same dtype as D")
        fp4 = self._is_fp4x2(self.ab_dtype)
        self._value_error_if(self.sf_dtype == torch.float8_e4m3fn and self.sf_vec_size == 32, f"sf_dtype {self.sf_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._value_error_if(fp4 and self.d_dtype not in (torch.float16, torch.bfloat16, torch.float32), "D must be fp16, bf16, or float32 when ab_dtype is fp4")
        self._not_implemented_error_if(
            fp4 and self.sf_vec_size == 16 and self.d_dtype == torch.float32,
            "Invalid configuration: fp4 ab_dtype, sf_vec_size 16, d_dtype float32 is not supported",
        )
        self._value_error_if(fp4 and self.b_major != "k", "b_major must be 'k' when ab_dtype is fp4")
        self._check_dtype(self.padded_offsets, torch.int32, "padded_offsets")
        check_tile_and_cluster(self, self.mma_tiler_mn, self.cluster_shape_mn, self.m_aligned, only_n256=True)
        self._value_error_if(k % (32 if fp4 else 16) != 0 or n % 16 != 0, "Invalid tensor alignment: tensors must be 16B aligned")
        if self.expert_cnt > 1024:
            raise ValueError(f"expert_cnt must be <= 1024, got {self.expert_cnt}")

        if self.bias is not None:
            self._check_stride(self.bias, (1, n), "bias must have stride (1, n)")
            self._check_dtype(self.bias, [torch.bfloat16, torch.float16], "bias")
        self._not_implemented_error_if(self.sf_dtype == torch.float8_e4m3fn and not fp4, f"E4M3 scale factors go with FP4 operands, got {self.ab_dtype}")
        self._not_implemented_error_if(fp4 and k % 64 != 0, f"FP4 operands need k to be a multiple of 64, got {k}")
        self._not_implemented_error_if(fp4 and self.generate_sfd, "scale-factor generation is built for fp8 operands only")
        self._not_implemented_error_if(self.c is not None and self.c_dtype not in (torch.bfloat16, torch.float16), f"only bf16 and fp16 C are built, got {self.c_dtype}")
        self._not_implemented_error_if(
            self.d_dtype not in (torch.bfloat16, torch.float16, torch.float8_e4m3fn, torch.float8_e5m2) and not (fp4 and self.d_dtype == torch.float32),
            f"only bf16, fp16, E4M3 and E5M2 D (and float32 D with FP4 operands) are built, got {self.d_dtype}",
        )
        self._not_implemented_error_if(not self.generate_sfd and self.d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2), "FP8 D needs sfd_row, sfd_col and norm_const")
        self._value_error_if(n % 64 != 0, f"n must be a multiple of 64 (32-column gate / up blocks), got {n}")
        self._value_error_if(self.generate_sfd and self.d_col is None, "sample_d_col is required when scale factors are generated")
        self._n, self._k = n, k
        self._require_sm100()
        self._is_supported = True
        return True

    def compile(self) -> None:
        if not self._is_supported:
            self.check_support()
        ops._lib.load()
        if self._workspace is None:
            nbytes = ops.workspace_bytes(self.expert_cnt, True, bool(self.use_dynamic_sched))
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.a.device)
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        b_ptrs: torch.Tensor,
        c_tensor: Optional[torch.Tensor],
        d_tensor: torch.Tensor,
        sfa_tensor: torch.Tensor,
        sfb_ptrs: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        bias_tensor: Optional[torch.Tensor] = None,
        d_col_tensor: Optional[torch.Tensor] = None,
        sfd_row_tensor: Optional[torch.Tensor] = None,
        sfd_col_tensor: Optional[torch.Tensor] = None,
        amax_tensor: Optional[torch.Tensor] = None,
        norm_const_tensor: Optional[torch.Tensor] = None,
        prob_tensor: Optional[torch.Tensor] = None,
        current_stream=None,
    ) -> None:
        a_tensor = as_packed_fp4(a_tensor)
        self._ensure_compiled()
        tensor_m, k = a_tensor.shape[0], a_tensor.shape[1]
        if tensor_m == 0:
            return
        if (bias_tensor is not None) != (self.bias is not None):
            raise ValueError("bias fusion is fixed at construction: pass bias_tensor exactly when sample_bias was given")
        _require_pointer_tensor(b_ptrs, "b_ptrs", self.expert_cnt)
        _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", self.expert_cnt)
        fp8_out = d_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
        gen = bool(getattr(self, "generate_sfd", fp8_out)) and sfd_row_tensor is not None and norm_const_tensor is not None
        ops.grouped_gemm_op(
            "fc1",
            a=a_tensor,
            sfa=sfa_tensor,
            b_ptrs=b_ptrs,
            sfb_ptrs=sfb_ptrs,
            padded_offsets=padded_offsets,
            alpha=alpha_tensor,
            prob=prob_tensor,
            norm_const=norm_const_tensor if gen else None,
            c=c_tensor,
            d=d_tensor,
            d_col=d_col_tensor if gen and sfd_col_tensor is not None else None,
            amax=None if fp8_out or d_tensor.dtype == torch.float32 else amax_tensor,  # the reference has amax for a 16-bit D only
            sf_vec_size=self.sf_vec_size,
            sfd_row=sfd_row_tensor if gen else None,
            sfd_col=sfd_col_tensor if gen and d_col_tensor is not None else None,
            workspace=self._workspace,
            n=self._n,
            discrete_col_sfd=self.discrete_col_sfd,
            sm_margin=self.num_cluster_overlap_margin,
            tile_mode=pick_tile_mode(self.mma_tiler_mn, self.m_aligned),
            bias=bias_tensor,
            act_func=self.act_func,
            stream=current_stream,
            dynamic_sched=bool(self.use_dynamic_sched),
            b_nmajor=self.b_major == "n",
        )


_cache_of_DiscreteGroupedGemmSwigluSm100Objects = {}


def discrete_grouped_gemm_swiglu_wrapper_sm100(
    a_tensor: torch.Tensor,
    b_ptrs: torch.Tensor,
    sfa_tensor: torch.Tensor,
    sfb_ptrs: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha_tensor: torch.Tensor,
    n: int,
    b_dtype: torch.dtype,
    bias_tensor: Optional[torch.Tensor] = None,
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
    b_major: str = "k",
    use_dynamic_sched: bool = False,
    current_stream=None,
) -> TupleDict:
    """One-shot discrete-weight FC1.  Returns ``TupleDict(c_tensor, d_tensor, d_col_tensor,
    amax_tensor, sfd_row_tensor, sfd_col_tensor)``."""
    a_tensor = as_packed_fp4(a_tensor)
    b_dtype = packed_fp4_dtype(b_dtype)
    _require_pointer_tensor(b_ptrs, "b_ptrs")
    l = b_ptrs.shape[0]
    _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", l)
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    valid_m, k, _ = a_tensor.shape
    if a_tensor.dtype == torch.float4_e2m1fn_x2:
        k *= 2  # two elements per byte
    n_out = n // 2
    dev = a_tensor.device
    c_tensor = torch.empty_strided((valid_m, n, 1), (n, 1, valid_m * n), dtype=c_dtype, device=dev)
    d_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    sfd_row_tensor = sfd_col_tensor = amax_tensor = None
    fp8_in = a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and sfa_tensor.dtype in (torch.float8_e8m0fnu, torch.float8_e4m3fn)
    # as in the reference: fp8 inputs get scale-factor outputs whatever d_dtype is (here: whenever a
    # norm_const is given; a 16-bit d_dtype without one gives the plain D plus amax)
    if fp8_in and (d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2) or norm_const_tensor is not None):
        sfd_row_tensor = _alloc_sfd(valid_m, n_out, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n_out, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    if d_dtype in (torch.bfloat16, torch.float16):
        amax_tensor = torch.full((l, 1), float("-inf"), dtype=torch.float32, device=dev)
    result = TupleDict(c_tensor=c_tensor, d_tensor=d_tensor, d_col_tensor=d_col_tensor, amax_tensor=amax_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)
    if valid_m == 0:
        return result
    cache_key = (
        a_tensor.dtype, sfa_tensor.dtype, b_dtype, c_dtype, d_dtype, tuple(a_tensor.shape[1:]), n, l, acc_dtype,
        tuple(mma_tiler_mn), None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, vector_f32,
        m_aligned, discrete_col_sfd, act_func, b_major, use_dynamic_sched, prob_tensor is not None,
        norm_const_tensor is not None, bias_tensor is not None, str(dev),
    )  # fmt: skip
    op = _cache_of_DiscreteGroupedGemmSwigluSm100Objects.get(cache_key)
    if op is None:
        op = DiscreteGroupedGemmSwigluSm100(
            sample_a=a_tensor, num_experts=l, b_shape=(n, k), b_dtype=b_dtype, sample_c=c_tensor, sample_d=d_tensor,
            sample_sfa=sfa_tensor, sample_padded_offsets=padded_offsets, sample_alpha=alpha_tensor, sample_d_col=d_col_tensor,
            sample_bias=bias_tensor, sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor, sample_amax=amax_tensor,
            sample_norm_const=norm_const_tensor if sfd_row_tensor is not None else None, sample_prob=prob_tensor,
            acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size,
            vector_f32=vector_f32, m_aligned=m_aligned, discrete_col_sfd=discrete_col_sfd, act_func=act_func,
            b_major=b_major, use_dynamic_sched=use_dynamic_sched,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_DiscreteGroupedGemmSwigluSm100Objects[cache_key] = op
    op.execute(
        a_tensor=a_tensor, b_ptrs=b_ptrs, c_tensor=c_tensor, d_tensor=d_tensor, sfa_tensor=sfa_tensor, sfb_ptrs=sfb_ptrs,
        padded_offsets=padded_offsets, alpha_tensor=alpha_tensor, bias_tensor=bias_tensor, d_col_tensor=d_col_tensor,
        sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
        norm_const_tensor=norm_const_tensor, prob_tensor=prob_tensor, current_stream=current_stream,
    )  # fmt: skip
    return result
