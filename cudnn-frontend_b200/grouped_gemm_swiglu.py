"""FC1 of an MoE layer: contiguous block-scaled grouped GEMM with fused SwiGLU.

Same names, arguments and error behaviour as the reference's
``GroupedGemmSwigluSm100`` / ``grouped_gemm_swiglu_wrapper_sm100``
(python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:52-771, :780-1043); the kernel behind
``execute`` is the hand-written sm_100a grouped GEMM of libb200moe.so instead of a JIT-compiled
CuTe-DSL kernel, so ``compile()`` only fixes launch parameters.

Differences a caller can observe:
* groups may be padded to any multiple of 128 rows (``m_aligned`` 128, 256, ...); the
  reference accepts exactly 256;
* ``c_tensor=None`` in ``execute`` skips the bf16 pre-activation store (the reference always
  writes C);
* the wrapper allocates scale-factor outputs only for an fp8 ``d_dtype`` (see its docstring);
* operands are E4M3 / E5M2 with E8M0 scales per 32 elements (MXFP8) or ``float4_e2m1fn_x2`` (or, as in the
  reference, the same bytes as ``uint8``) with E8M0 scales per 32 (MXFP4) or E8M0 / E4M3 scales per 16 (NVFP4);
  FP4 / FP8 / float32 C, an FP4 D and k that is not a multiple of 64 with FP4 operands raise
  ``NotImplementedError``.
"""

from __future__ import annotations

import logging
import os
from typing import Optional, Tuple

import torch

from . import ops
from .api_base import OperatorBase, TensorSpec, TupleDict, as_packed_fp4, ceil_div, check_tile_and_cluster, packed_fp4_dtype, pick_tile_mode

_logger = logging.getLogger(__name__)

_SF_STRIDE_MSG = "scale-factor tensors must use the 128x4 layout (32, 4, rest_mn, 4, rest_k, l)"


class GroupedGemmSwigluSm100(OperatorBase):
    """``C = alpha_e (A SFA)(B_e SFB_e)^T``, ``D[:, 32j:32j+32] = up_j * silu(gate_j) * prob``
    with gate / up the even / odd 32-column blocks of C, per-expert amax (bf16 D) or row and
    column MXFP8 re-quantisation (E4M3 D)."""

    def __init__(
        self,
        sample_a: torch.Tensor,
        sample_b: torch.Tensor,
        sample_c: Optional[torch.Tensor],
        sample_d: torch.Tensor,
        sample_sfa: torch.Tensor,
        sample_sfb: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_d_col: Optional[torch.Tensor],
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
        sample_bias: Optional[torch.Tensor] = None,
        act_func: str = "swiglu",
    ):
        """The two trailing arguments are not in the reference's class of this name (its unified
        successor ``GroupedGemmGluSm100`` has them): a fused bias ``(n, l)`` with stride ``(1, n)``
        and ``act_func`` ``"swiglu"`` or ``"geglu"``."""
        super().__init__()
        self.bias = TensorSpec.of(sample_bias, "sample_bias")
        self.act_func = act_func
        self.a = TensorSpec.of(as_packed_fp4(sample_a), "sample_a")
        self.b = TensorSpec.of(as_packed_fp4(sample_b), "sample_b")
        self.c = TensorSpec.of(sample_c, "sample_c")
        self.d = TensorSpec.of(sample_d, "sample_d")
        self.sfa = TensorSpec.of(sample_sfa, "sample_sfa")
        self.sfb = TensorSpec.of(sample_sfb, "sample_sfb")
        self.padded_offsets = TensorSpec.of(sample_padded_offsets, "sample_padded_offsets")
        self.alpha = TensorSpec.of(sample_alpha, "sample_alpha")
        self.d_col = TensorSpec.of(sample_d_col, "sample_d_col")
        self.sfd_row = TensorSpec.of(sample_sfd_row, "sample_sfd_row")
        self.sfd_col = TensorSpec.of(sample_sfd_col, "sample_sfd_col")
        self.amax = TensorSpec.of(sample_amax, "sample_amax")
        self.norm_const = TensorSpec.of(sample_norm_const, "sample_norm_const")
        self.prob = TensorSpec.of(sample_prob, "sample_prob")
        self.expert_cnt = self.padded_offsets.shape[0]
        self.acc_dtype = acc_dtype
        self.mma_tiler_mn = tuple(mma_tiler_mn)
        self.use_2cta_instrs = self.mma_tiler_mn[0] == 256
        self.cluster_shape_mn = tuple(cluster_shape_mn) if cluster_shape_mn is not None else ((2, 1) if self.use_2cta_instrs else (1, 1))
        self.sf_vec_size = sf_vec_size
        self.vector_f32 = vector_f32
        self.m_aligned = m_aligned
        self.discrete_col_sfd = discrete_col_sfd
        # SMs left free for a concurrently running (e.g. NCCL) kernel, as in the reference
        self.num_cluster_overlap_margin = int(os.getenv("CUDNNFE_CLUSTER_OVERLAP_MARGIN", "0"))
        # the reference's dense FC1 class has a static scheduler only; its unified GLU front end
        # (grouped_gemm_glu.py) owns one of these objects and may switch the dynamic scheduler on
        self.use_dynamic_sched = False
        self._workspace = None

    # ------------------------------------------------------------------------------------
    def check_support(self) -> bool:
        sfd_parts = [self.sfd_row, self.sfd_col, self.norm_const]
        all_none = all(x is None for x in sfd_parts)
        none_none = all(x is not None for x in sfd_parts)
        self._value_error_if(not (all_none or none_none), "sfd_row_desc, sfd_col_desc, and norm_const_desc must be all None or all not None")
        self.generate_sfd = none_none
        if self.discrete_col_sfd and not self.generate_sfd:
            self._logger.warning("discrete_col_sfd is True but generate_sfd is False, discrete_col_sfd will be ignored")
            self.discrete_col_sfd = False

        self._value_error_if(len(self.a.shape) != 3 or len(self.b.shape) != 3, "A must be (m, k, 1) and B (n, k, l)")
        a_l, b_l = self.a.logical(), self.b.logical()  # FP4 operands: two elements per byte along K
        tensor_m, k, _ = a_l.shape
        n, _, l = b_l.shape
        n_2 = n // 2
        self._check_shape(a_l, (tensor_m, k, 1), "A")
        self._check_shape(b_l, (n, k, l), "B")
        self._check_shape(self.c, (tensor_m, n, 1), "C")
        self._check_shape(self.d, (tensor_m, n_2, 1), "D")
        self._check_shape(self.d_col, (tensor_m, n_2, 1), "D_col")
        rest_k = ceil_div(ceil_div(k, self.sf_vec_size), 4)
        self._check_shape(self.sfa, (32, 4, ceil_div(tensor_m, 128), 4, rest_k, 1), "SFA")
        self._check_shape(self.sfb, (32, 4, ceil_div(n, 128), 4, rest_k, l), "SFB")
        rest_n2 = ceil_div(ceil_div(n_2, self.sf_vec_size), 4)
        self._check_shape(self.sfd_row, (32, 4, ceil_div(tensor_m, 128), 4, rest_n2, 1), "SFD_row")
        rest_m = ceil_div(ceil_div(tensor_m, self.sf_vec_size), 4)
        self._check_shape(self.sfd_col, (32, 4, ceil_div(n_2, 128), 4, rest_m, 1), "SFD_col")
        self._check_shape(self.alpha, (l,), "alpha")
        self._check_shape(self.prob, (tensor_m, 1, 1), "prob")
        self._check_shape(self.amax, (l, 1), "amax")
        self._check_shape(self.norm_const, (1,), "norm_const")
        self._check_shape(self.padded_offsets, (l,), "padded_offsets")

        self._check_stride(a_l, (k, 1, tensor_m * k), "A must have k-major layout")
        self._check_stride(b_l, (k, 1, n * k), "B must have k-major layout")
        self._check_stride(self.c, (n, 1, tensor_m * n), "C must have n-major layout")
        self._check_stride(self.d, (n_2, 1, tensor_m * n_2), "D must have n-major layout")
        self._check_stride(self.d_col, (n_2, 1, tensor_m * n_2), "D_col must have n-major layout")
        for spec, mn, kk, ll in ((self.sfa, tensor_m, k, 1), (self.sfb, n, k, l), (self.sfd_row, tensor_m, n_2, 1), (self.sfd_col, n_2, tensor_m, 1)):
            if spec is not None:
                self._check_stride(spec, ops.sf_shape_stride(mn, kk, ll, self.sf_vec_size)[1], _SF_STRIDE_MSG)

        self.ab_dtype = self._check_dtype(self.a, [torch.float4_e2m1fn_x2, torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn], "A/B")
        self._check_dtype(self.b, self.ab_dtype, "B", "B must have the same dtype as A")
        self.sf_dtype = self._check_dtype(self.sfa, [torch.float8_e8m0fnu, torch.float8_e4m3fn], "SFA/SFB/SFD_row/SFD_col")
        for spec, label in ((self.sfb, "SFB"), (self.sfd_row, "SFD_row"), (self.sfd_col, "SFD_col")):
            self._check_dtype(spec, self.sf_dtype, label, f"{label} must have the same dtype as SFA")
        self._value_error_if(self.sf_vec_size not in (16, 32), f"sf_vec_size must be 16 or 32, got {self.sf_vec_size}")
        self._value_error_if(self.sf_dtype == torch.float8_e4m3fn and self.sf_vec_size == 32, f"sf_dtype {self.sf_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._value_error_if(self._is_fp8(self.ab_dtype) and self.sf_vec_size == 16, f"ab_dtype {self.ab_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._check_dtype(self.acc_dtype, torch.float32, "Accumulator", "Accumulator must be float32")
        self.c_dtype = self._check_dtype(
            self.c, [torch.float32, torch.float16, torch.bfloat16, torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2], "C"
        )
        self.d_dtype = self._check_dtype(
            self.d, [torch.float16, torch.bfloat16, torch.float32, torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2], "D"
        )
        self._check_dtype(self.d_col, self.d_dtype, "D_col", "D_col must have the same dtype as D")
        fp4 = self._is_fp4x2(self.ab_dtype)
        self._value_error_if(fp4 and self.d_dtype not in (torch.float16, torch.bfloat16, torch.float32), "D must be fp16, bf16, or float32 when ab_dtype is fp4")
        self._not_implemented_error_if(
            fp4 and self.sf_vec_size == 16 and self.d_dtype == torch.float32,
            "Invalid configuration: fp4 ab_dtype, sf_vec_size 16, d_dtype float32 is not supported. Please use sf_vec_size 32 or d_dtype bf16 instead",
        )
        self._check_dtype(self.padded_offsets, torch.int32, "padded_offsets")
        self._check_dtype(self.alpha, torch.float32, "alpha")
        self._check_dtype(self.prob, torch.float32, "prob")
        self._check_dtype(self.amax, torch.float32, "amax")
        self._check_dtype(self.norm_const, torch.float32, "norm_const")

        check_tile_and_cluster(self, self.mma_tiler_mn, self.cluster_shape_mn, self.m_aligned, only_n256=False)
        self._value_error_if(k % (32 if fp4 else 16) != 0 or n % 16 != 0, "Invalid tensor alignment: tensors must be 16B aligned")
        if self.expert_cnt > 1024:
            raise ValueError(f"expert_cnt must be <= 1024, got {self.expert_cnt}")
        self._not_implemented_error_if(
            self._is_fp8(self.ab_dtype) and self.mma_tiler_mn[1] == 128 and self._is_fp8(self.d_dtype),
            "Invalid configuration: fp8 ab_dtype and sf_vec_size 32 with mma_tiler_mn[1] == 128 and fp8 d_dtype is not supported. Please use mma_tiler_mn[1] == 256 instead",
        )

        self._not_implemented_error_if(fp4 and self.c is not None and self.c_dtype not in (torch.float16, torch.bfloat16), f"Invalid configuration: for fp4 ab_dtype, c_dtype must be float16 or bfloat16, got {self.c_dtype}")

        # what this build implements of the reference's surface
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
        self._value_error_if(self.act_func not in ("swiglu", "geglu"), f"act_func must be 'swiglu' or 'geglu', got {self.act_func}")
        if self.bias is not None:
            self._check_shape(self.bias, (n, l), "bias")
            self._check_stride(self.bias, (1, n), "bias must have stride (1, n)")
            self._check_dtype(self.bias, [torch.bfloat16, torch.float16, torch.float32], "bias")

        self._require_sm100()
        self._is_supported = True
        return True

    def compile(self) -> None:
        if not self._is_supported:
            self.check_support()
        ops._lib.load()  # fails loudly when the CUDA library is missing
        nbytes = ops.workspace_bytes(self.b.shape[2], False, bool(self.use_dynamic_sched))
        if nbytes and self._workspace is None:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.a.device)
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        b_tensor: torch.Tensor,
        c_tensor: Optional[torch.Tensor],
        d_tensor: torch.Tensor,
        sfa_tensor: torch.Tensor,
        sfb_tensor: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        d_col_tensor: Optional[torch.Tensor] = None,
        sfd_row_tensor: Optional[torch.Tensor] = None,
        sfd_col_tensor: Optional[torch.Tensor] = None,
        amax_tensor: Optional[torch.Tensor] = None,
        norm_const_tensor: Optional[torch.Tensor] = None,
        prob_tensor: Optional[torch.Tensor] = None,
        current_stream=None,
        bias_tensor: Optional[torch.Tensor] = None,
        expert_range: Optional[Tuple[int, int]] = None,
        offsets_have_prev: bool = False,
    ) -> None:
        """Launch on ``current_stream`` (``None`` = torch's current stream).  Allocates nothing and
        does not synchronise; ``amax_tensor`` is only ever raised (atomic max).  ``expert_range = (lo, hi)``
        (not in the reference) computes experts ``lo .. hi - 1`` only, on the same full tensors; ``offsets_have_prev`` (not in the
        reference either) says that ``padded_offsets`` is a view one element into a longer array whose element
        before it is the first row of expert 0."""
        a_tensor = as_packed_fp4(a_tensor)
        b_tensor = as_packed_fp4(b_tensor)
        self._ensure_compiled()
        tensor_m = a_tensor.shape[0]
        if tensor_m == 0:
            return
        if (bias_tensor is not None) != (self.bias is not None):
            raise ValueError("bias fusion is fixed at construction: pass bias_tensor exactly when sample_bias was given")
        n, l = b_tensor.shape[0], b_tensor.shape[2]
        fp8_out = d_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
        gen = bool(getattr(self, "generate_sfd", fp8_out)) and sfd_row_tensor is not None and norm_const_tensor is not None
        ops.grouped_gemm_op(
            "fc1",
            a=a_tensor,
            sfa=sfa_tensor,
            b=b_tensor,
            sfb=sfb_tensor,
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
            n=n,
            discrete_col_sfd=self.discrete_col_sfd,
            sm_margin=self.num_cluster_overlap_margin,
            tile_mode=pick_tile_mode(self.mma_tiler_mn, self.m_aligned),
            bias=bias_tensor,
            act_func=self.act_func,
            stream=current_stream,
            workspace=self._workspace,
            dynamic_sched=bool(self.use_dynamic_sched),
            expert_range=expert_range,
            offsets_have_prev=offsets_have_prev,
        )


_cache_of_GroupedGemmSwigluSm100Objects = {}


def _alloc_sfd(mn: int, k: int, sf_vec_size: int, dtype, device) -> torch.Tensor:
    """(1, rest_mn, rest_k, 32, 4, 4) contiguous, viewed as (32, 4, rest_mn, 4, rest_k, 1)."""
    shape = (1, ceil_div(mn, 128), ceil_div(ceil_div(k, sf_vec_size), 4), 32, 4, 4)
    return torch.empty(shape, dtype=dtype, device=device).permute(3, 4, 1, 5, 2, 0)


def grouped_gemm_swiglu_wrapper_sm100(
    a_tensor: torch.Tensor,
    b_tensor: torch.Tensor,
    sfa_tensor: torch.Tensor,
    sfb_tensor: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha_tensor: torch.Tensor,
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
    current_stream=None,
) -> TupleDict:
    """One-shot FC1: allocates the outputs, reuses a cached operator object per configuration and
    launches.  Returns ``TupleDict(c_tensor, d_tensor, d_col_tensor, amax_tensor, sfd_row_tensor,
    sfd_col_tensor)``.  As in the reference (api.py:880-911), fp8 inputs get row and column scale-factor
    outputs whatever ``d_dtype`` is: with a 16-bit ``d_dtype`` D and D_col then hold the scaled values
    (block maximum mapped to 1) in that type, and amax is produced too.  The reference demands
    ``norm_const_tensor`` in that case; here a 16-bit ``d_dtype`` without ``norm_const_tensor`` gives the
    plain bf16 / fp16 D plus amax instead of an error.  As in the reference, the amax buffer of a
    cached configuration is reused across calls: it holds a running maximum until the caller
    resets it."""
    a_tensor = as_packed_fp4(a_tensor)
    b_tensor = as_packed_fp4(b_tensor)
    valid_m, k, _ = a_tensor.shape
    n, _, l = b_tensor.shape
    n_out = n // 2
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    dev = a_tensor.device
    c_tensor = torch.empty_strided((valid_m, n, 1), (n, 1, valid_m * n), dtype=c_dtype, device=dev)
    d_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    sfd_row_tensor = sfd_col_tensor = amax_tensor = None
    fp8_in = a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and sfa_tensor.dtype in (torch.float8_e8m0fnu, torch.float8_e4m3fn)
    if fp8_in and (d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2) or norm_const_tensor is not None):
        sfd_row_tensor = _alloc_sfd(valid_m, n_out, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n_out, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    if valid_m == 0:
        if d_dtype in (torch.bfloat16, torch.float16):
            amax_tensor = torch.full((l, 1), float("-inf"), dtype=torch.float32, device=dev)
        return TupleDict(c_tensor=c_tensor, d_tensor=d_tensor, d_col_tensor=d_col_tensor, amax_tensor=amax_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)

    cache_key = (
        a_tensor.dtype, b_tensor.dtype, sfa_tensor.dtype, c_dtype, d_dtype, cd_major, acc_dtype,
        tuple(a_tensor.shape[1:]), tuple(b_tensor.shape), tuple(mma_tiler_mn),
        None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, vector_f32, m_aligned,
        discrete_col_sfd, prob_tensor is not None, norm_const_tensor is not None, str(dev),
    )  # fmt: skip
    hit = _cache_of_GroupedGemmSwigluSm100Objects.get(cache_key)
    if hit is None:
        if d_dtype in (torch.bfloat16, torch.float16):
            amax_tensor = torch.full((l, 1), float("-inf"), dtype=torch.float32, device=dev)
        op = GroupedGemmSwigluSm100(
            sample_a=a_tensor, sample_b=b_tensor, sample_c=c_tensor, sample_d=d_tensor, sample_sfa=sfa_tensor,
            sample_sfb=sfb_tensor, sample_padded_offsets=padded_offsets, sample_alpha=alpha_tensor,
            sample_d_col=d_col_tensor, sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor,
            sample_amax=amax_tensor, sample_norm_const=norm_const_tensor if sfd_row_tensor is not None else None,
            sample_prob=prob_tensor,
            acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn,
            sf_vec_size=sf_vec_size, vector_f32=vector_f32, m_aligned=m_aligned, discrete_col_sfd=discrete_col_sfd,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_GroupedGemmSwigluSm100Objects[cache_key] = (op, amax_tensor)
    else:
        op, amax_tensor = hit
    op.execute(
        a_tensor=a_tensor, b_tensor=b_tensor, c_tensor=c_tensor, d_tensor=d_tensor, sfa_tensor=sfa_tensor,
        sfb_tensor=sfb_tensor, padded_offsets=padded_offsets, alpha_tensor=alpha_tensor, d_col_tensor=d_col_tensor,
        sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
        norm_const_tensor=norm_const_tensor, prob_tensor=prob_tensor, current_stream=current_stream,
    )  # fmt: skip
    return TupleDict(c_tensor=c_tensor, d_tensor=d_tensor, d_col_tensor=d_col_tensor, amax_tensor=amax_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)
