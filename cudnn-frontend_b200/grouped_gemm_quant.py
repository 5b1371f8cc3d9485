"""FC2 of an MoE layer: block-scaled grouped GEMM, per-row gating and MXFP8 re-quantisation.

Same names, arguments and error behaviour as the reference's ``GroupedGemmQuantSm100`` /
``grouped_gemm_quant_wrapper_sm100`` (python/cudnn/grouped_gemm/grouped_gemm_quant/api.py:57-1089,
:1098-1500), for both weight layouts: dense ``b_tensor (n, k, l)`` or discrete per-expert
pointers ``b_ptrs`` / ``sfb_ptrs`` (int64 device arrays).  In discrete mode the per-expert TMA
descriptors are built on the device from the pointer arrays into a workspace the object
allocates in ``compile()``, so ``execute()`` allocates nothing and never reads the pointers on
the host.

B may be K-major or, as in the reference for FP8 operands, N-major: a dense ``b_tensor`` with
strides ``(1, n, n*k)``, or ``b_major="n"`` with discrete pointers (each expert one ``[k][n]``
allocation).  ``use_dynamic_sched=True`` hands tiles out through an atomic counter (the reference's
dynamic MoE scheduler, python/cudnn/grouped_gemm/moe_persistent_scheduler.py:838-893); results are
bit-identical to the static schedule.

Not built (``NotImplementedError``): inputs other than MXFP8 (E4M3 / E5M2 with E8M0 scales per
32), D other than bf16 / fp16 / E4M3 / E5M2.
"""

from __future__ import annotations

import logging
import os
from typing import Optional, Tuple

import torch

from . import ops
from .api_base import OperatorBase, TensorSpec, TupleDict, as_packed_fp4, ceil_div, check_tile_and_cluster, packed_fp4_dtype, pick_tile_mode
from .grouped_gemm_swiglu import _SF_STRIDE_MSG, _alloc_sfd

_logger = logging.getLogger(__name__)


def _require_pointer_tensor(t: torch.Tensor, name: str, expected_len: Optional[int] = None) -> None:
    """Pointer arrays are 1-D contiguous int64 CUDA tensors
    (python/cudnn/discrete_grouped_gemm/discrete_grouped_gemm_swiglu/discrete_kernel_utils.py:73-83)."""
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name} must be a torch.Tensor of device addresses")
    if t.dtype != torch.int64 or t.dim() != 1 or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f"{name} must be a 1-D contiguous int64 CUDA tensor, got dtype={t.dtype} shape={tuple(t.shape)} device={t.device}")
    if expected_len is not None and t.shape[0] != expected_len:
        raise ValueError(f"{name} must have {expected_len} entries, got {t.shape[0]}")


class GroupedGemmQuantSm100(OperatorBase):
    """``D = quant(alpha_e (A SFA)(B_e SFB_e)^T * prob)``: bf16 D with per-expert amax, or E4M3 D
    with row and column E8M0 scale factors."""

    def __init__(
        self,
        sample_a: torch.Tensor,
        sample_sfa: torch.Tensor,
        sample_padded_offsets: torch.Tensor,
        sample_alpha: torch.Tensor,
        sample_d: torch.Tensor,
        sample_d_col: Optional[torch.Tensor] = None,
        sample_b: Optional[torch.Tensor] = None,
        sample_sfb: Optional[torch.Tensor] = None,
        sample_bias: Optional[torch.Tensor] = None,
        num_experts: Optional[int] = None,
        b_shape: Optional[Tuple[int, ...]] = None,
        b_dtype: Optional[torch.dtype] = None,
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
        b_major: str = "k",
        use_dynamic_sched: bool = False,
    ):
        super().__init__()
        self.a = TensorSpec.of(as_packed_fp4(sample_a), "sample_a")
        self.sfa = TensorSpec.of(sample_sfa, "sample_sfa")
        self.padded_offsets = TensorSpec.of(sample_padded_offsets, "sample_padded_offsets")
        self.alpha = TensorSpec.of(sample_alpha, "sample_alpha")
        self.d = TensorSpec.of(sample_d, "sample_d")
        self.d_col = TensorSpec.of(sample_d_col, "sample_d_col")
        self.bias = TensorSpec.of(sample_bias, "sample_bias")
        self.sfd_row = TensorSpec.of(sample_sfd_row, "sample_sfd_row")
        self.sfd_col = TensorSpec.of(sample_sfd_col, "sample_sfd_col")
        self.amax = TensorSpec.of(sample_amax, "sample_amax")
        self.norm_const = TensorSpec.of(sample_norm_const, "sample_norm_const")
        self.prob = TensorSpec.of(sample_prob, "sample_prob")
        self.discrete = not (sample_b is not None and num_experts is None)
        if not self.discrete:
            self.b = TensorSpec.of(as_packed_fp4(sample_b), "sample_b")
            self.sfb = TensorSpec.of(sample_sfb, "sample_sfb")
            self.expert_cnt = self.padded_offsets.shape[0]
        else:
            self._value_error_if(num_experts is None or num_experts == 0, "num_experts must be > 0")
            self._value_error_if(b_shape is None or b_dtype is None, "b_shape and b_dtype are required in discrete mode")
            self.b = self.sfb = None
            self.expert_cnt = num_experts
            self.b_shape = tuple(b_shape)
            self.b_dtype = packed_fp4_dtype(b_dtype)
            self._value_error_if(
                self.padded_offsets.shape[0] != self.expert_cnt,
                f"padded_offsets length ({self.padded_offsets.shape[0]}) must equal num_experts ({self.expert_cnt})",
            )
        self.b_major = b_major
        self.acc_dtype = acc_dtype
        self.mma_tiler_mn = tuple(mma_tiler_mn)
        self.use_2cta_instrs = self.mma_tiler_mn[0] == 256
        self.cluster_shape_mn = tuple(cluster_shape_mn) if cluster_shape_mn is not None else ((2, 1) if self.use_2cta_instrs else (1, 1))
        self.sf_vec_size = sf_vec_size
        self.vector_f32 = vector_f32
        self.m_aligned = m_aligned
        self.discrete_col_sfd = discrete_col_sfd
        self.use_dynamic_sched = use_dynamic_sched
        self.num_cluster_overlap_margin = int(os.getenv("CUDNNFE_CLUSTER_OVERLAP_MARGIN", "0"))
        self._workspace = None

    def check_support(self) -> bool:
        sfd_parts = [self.sfd_row, self.sfd_col, self.norm_const]
        all_none = all(x is None for x in sfd_parts)
        all_provided = all(x is not None for x in sfd_parts)
        self._value_error_if(not (all_none or all_provided), "sfd_row_desc, sfd_col_desc, and norm_const_desc must be all None or all not None")
        self.generate_sfd = all_provided
        self._value_error_if(self.generate_sfd and self.d_col is None, "sample_d_col is required when SFD outputs are generated")
        if self.discrete_col_sfd and not self.generate_sfd:
            self._logger.warning("discrete_col_sfd is True but generate_sfd is False, discrete_col_sfd will be ignored")
            self.discrete_col_sfd = False

        self._value_error_if(len(self.a.shape) != 3, "A must be (m, k, 1)")
        a_l = self.a.logical()  # FP4 operands: two elements per byte along K
        b_l = None if self.b is None else self.b.logical()
        tensor_m, k, _ = a_l.shape
        if not self.discrete:
            self._value_error_if(len(self.b.shape) != 3, "B must be (n, k, l)")
            n, _, l = b_l.shape
        else:
            n, b_k = self.b_shape[0], self.b_shape[1]
            self._value_error_if(b_k != k, f"B K dimension ({b_k}) must match A K dimension ({k})")
            l = self.expert_cnt
        self._check_shape(a_l, (tensor_m, k, 1), "A")
        self._check_shape(b_l, (n, k, l), "B")
        self._check_shape(self.d, (tensor_m, n, 1), "D")
        self._check_shape(self.d_col, (tensor_m, n, 1), "D_col")
        rest_k = ceil_div(ceil_div(k, self.sf_vec_size), 4)
        self._check_shape(self.sfa, (32, 4, ceil_div(tensor_m, 128), 4, rest_k, 1), "SFA")
        self._check_shape(self.sfb, (32, 4, ceil_div(n, 128), 4, rest_k, l), "SFB")
        rest_n = ceil_div(ceil_div(n, self.sf_vec_size), 4)
        self._check_shape(self.sfd_row, (32, 4, ceil_div(tensor_m, 128), 4, rest_n, 1), "SFD_row")
        rest_m = ceil_div(ceil_div(tensor_m, self.sf_vec_size), 4)
        self._check_shape(self.sfd_col, (32, 4, ceil_div(n, 128), 4, rest_m, 1), "SFD_col")
        self._check_shape(self.alpha, (self.expert_cnt,), "alpha")
        self._value_error_if(
            self.prob is None,
            "prob_tensor is required: the kernel unconditionally multiplies output by per-row gating probability. "
            "Pass a tensor of ones with shape (valid_m, 1, 1) if no gating is needed.",
        )
        self._check_shape(self.prob, (tensor_m, 1, 1), "prob")
        self._check_shape(self.bias, (n, l), "bias")
        self._check_shape(self.amax, (self.expert_cnt, 1), "amax")
        self._check_shape(self.norm_const, (1,), "norm_const")
        self._check_shape(self.padded_offsets, (self.expert_cnt,), "padded_offsets")

        self._check_stride(a_l, (k, 1, tensor_m * k), "A must have k-major layout")
        self._value_error_if(self.b_major not in ("k", "n"), f"b_major must be 'k' or 'n', got {self.b_major}")
        self._b_nmajor = self.b_major == "n"
        if self.b is not None:
            # dense weights: the strides say which way B is stored (the reference accepts both for fp8)
            if n > 1 and k > 1 and self.b.stride[0] == 1 and self.b.stride[1] == n and not self._is_fp4x2(self.b.dtype):
                self._check_stride(self.b, (1, n, n * k), "For fp8 ab_dtype, B must have k- or n-major layout")
                self._b_nmajor = True
            else:
                self._check_stride(b_l, (k, 1, n * k), "For fp4 ab_dtype, B must have k-major layout" if self._is_fp4x2(self.b.dtype) else "For fp8 ab_dtype, B must have k- or n-major layout")
                self._b_nmajor = False
        self._check_stride(self.d, (n, 1, tensor_m * n), "D must have n-major layout")
        self._check_stride(self.d_col, (n, 1, tensor_m * n), "D_col must have n-major layout")
        for spec, mn, kk, ll in ((self.sfa, tensor_m, k, 1), (self.sfb, n, k, l), (self.sfd_row, tensor_m, n, 1), (self.sfd_col, n, tensor_m, 1)):
            if spec is not None:
                self._check_stride(spec, ops.sf_shape_stride(mn, kk, ll, self.sf_vec_size)[1], _SF_STRIDE_MSG)

        self.ab_dtype = self._check_dtype(self.a, [torch.float4_e2m1fn_x2, torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn], "A/B")
        if self.b is not None:
            self._check_dtype(self.b, self.ab_dtype, "B", "B must have the same dtype as A")
        else:
            self._value_error_if(self.b_dtype != self.ab_dtype, f"b_dtype ({self.b_dtype}) must match A dtype ({self.ab_dtype})")
        self.sf_dtype = self._check_dtype(self.sfa, [torch.float8_e8m0fnu, torch.float8_e4m3fn], "SFA/SFB/SFD_row/SFD_col")
        for spec, label in ((self.sfb, "SFB"), (self.sfd_row, "SFD_row"), (self.sfd_col, "SFD_col")):
            self._check_dtype(spec, self.sf_dtype, label, f"{label} must have the same dtype as SFA")
        self._value_error_if(self.sf_vec_size not in (16, 32), f"sf_vec_size must be 16 or 32, got {self.sf_vec_size}")
        self._value_error_if(self.sf_dtype == torch.float8_e4m3fn and self.sf_vec_size == 32, f"sf_dtype {self.sf_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._value_error_if(self._is_fp8(self.ab_dtype) and self.sf_vec_size == 16, f"ab_dtype {self.ab_dtype} and sf_vec_size {self.sf_vec_size} combination is not supported")
        self._check_dtype(self.acc_dtype, torch.float32, "Accumulator", "Accumulator must be float32")
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
        self._value_error_if(fp4 and self.b_major != "k", "b_major must be 'k' when ab_dtype is fp4")
        self._check_dtype(self.padded_offsets, torch.int32, "padded_offsets")
        self._check_dtype(self.alpha, torch.float32, "alpha")
        self._check_dtype(self.prob, torch.float32, "prob")
        self._check_dtype(self.amax, torch.float32, "amax")
        self._check_dtype(self.norm_const, torch.float32, "norm_const")

        check_tile_and_cluster(self, self.mma_tiler_mn, self.cluster_shape_mn, self.m_aligned, only_n256=True)
        self._value_error_if(k % (32 if fp4 else 16) != 0 or n % 16 != 0, "Invalid tensor alignment: tensors must be 16B aligned")
        if self.expert_cnt > 1024:
            raise ValueError(f"expert_cnt must be <= 1024, got {self.expert_cnt}")

        if self.bias is not None:
            # (n, l) with stride (1, n), as the reference demands
            self._check_stride(self.bias, (1, n), "bias must have stride (1, n)")
            self._check_dtype(self.bias, [torch.bfloat16, torch.float16, torch.float32], "bias")
        self._not_implemented_error_if(self.sf_dtype == torch.float8_e4m3fn and not fp4, f"E4M3 scale factors go with FP4 operands, got {self.ab_dtype}")
        self._not_implemented_error_if(fp4 and k % 64 != 0, f"FP4 operands need k to be a multiple of 64, got {k}")
        self._not_implemented_error_if(fp4 and self.generate_sfd, "scale-factor generation is built for fp8 operands only")
        self._not_implemented_error_if(
            self.d_dtype not in (torch.bfloat16, torch.float16, torch.float8_e4m3fn, torch.float8_e5m2) and not (fp4 and self.d_dtype == torch.float32),
            f"only bf16, fp16, E4M3 and E5M2 D (and float32 D with FP4 operands) are built, got {self.d_dtype}",
        )
        self._not_implemented_error_if(not self.generate_sfd and self.d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2), "FP8 D needs sfd_row, sfd_col and norm_const")
        self._value_error_if(n % 32 != 0, f"n must be a multiple of 32, got {n}")
        self._n, self._k = n, k

        self._require_sm100()
        self._is_supported = True
        return True

    def compile(self) -> None:
        """Fix launch parameters and, in discrete mode, allocate the descriptor workspace (the
        reference allocates its workspace here too, grouped_gemm_quant/api.py:566-567)."""
        if not self._is_supported:
            self.check_support()
        ops._lib.load()
        nbytes = ops.workspace_bytes(self.expert_cnt, self.discrete, bool(self.use_dynamic_sched))
        if nbytes and self._workspace is None:
            self._workspace = torch.empty(nbytes, dtype=torch.uint8, device=self.a.device)
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        sfa_tensor: torch.Tensor,
        padded_offsets: torch.Tensor,
        alpha_tensor: torch.Tensor,
        d_tensor: torch.Tensor,
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
        d_row_map: Optional[torch.Tensor] = None,
        d_peer_ptrs: Optional[torch.Tensor] = None,
        d_peer_slots: int = 0,
        expert_range: Optional[Tuple[int, int]] = None,
        offsets_have_prev: bool = False,
    ) -> None:
        """Launch on ``current_stream``; allocates nothing.  ``d_row_map`` (int32 ``[M]``, not in the
        reference) stores row ``r`` of a bf16 result at row ``d_row_map[r]`` of ``d_tensor`` (negative:
        not stored), so a caller can receive the rows in another order, e.g. all-to-all order.  With
        ``d_peer_ptrs`` (int64 device tensor of G buffer addresses, each ``[d_peer_slots, N]`` bf16) a map
        value ``v`` addresses row ``v % d_peer_slots`` of rank ``v // d_peer_slots``'s buffer: the epilogue
        stores over NVLink into the ranks the rows came from.  ``expert_range = (lo, hi)`` (not in the
        reference) computes experts ``lo .. hi - 1`` only, on the same full tensors; ``offsets_have_prev`` (not in the
        reference either) says that ``padded_offsets`` is a view one element into a longer array whose element
        before it is the first row of expert 0."""
        a_tensor = as_packed_fp4(a_tensor)
        b_tensor = as_packed_fp4(b_tensor)
        self._ensure_compiled()
        tensor_m, k = a_tensor.shape[0], a_tensor.shape[1]
        if tensor_m == 0:
            return
        if (bias_tensor is not None) != (self.bias is not None):
            raise ValueError("bias fusion is fixed at construction: pass bias_tensor exactly when sample_bias was given")
        if self.discrete:
            if b_ptrs is None or sfb_ptrs is None:
                raise ValueError("discrete mode needs b_ptrs and sfb_ptrs")
            _require_pointer_tensor(b_ptrs, "b_ptrs", self.expert_cnt)
            _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", self.expert_cnt)
        elif b_tensor is None or sfb_tensor is None:
            raise ValueError("dense mode needs b_tensor and sfb_tensor")
        if prob_tensor is None:
            raise ValueError("prob_tensor is required")
        fp8_out = d_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2)
        gen = bool(getattr(self, "generate_sfd", fp8_out)) and sfd_row_tensor is not None and norm_const_tensor is not None
        ops.grouped_gemm_op(
            "fc2",
            a=a_tensor,
            sfa=sfa_tensor,
            b=None if self.discrete else b_tensor,
            sfb=None if self.discrete else sfb_tensor,
            b_ptrs=b_ptrs if self.discrete else None,
            sfb_ptrs=sfb_ptrs if self.discrete else None,
            padded_offsets=padded_offsets,
            alpha=alpha_tensor,
            prob=prob_tensor,
            norm_const=norm_const_tensor if gen else None,
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
            d_row_map=d_row_map,
            d_peer_ptrs=d_peer_ptrs,
            d_peer_slots=d_peer_slots,
            bias=bias_tensor,
            stream=current_stream,
            dynamic_sched=bool(self.use_dynamic_sched),
            b_nmajor=self._b_nmajor,
            expert_range=expert_range,
            offsets_have_prev=offsets_have_prev,
        )


_cache_of_GroupedGemmQuantSm100Objects = {}


def grouped_gemm_quant_wrapper_sm100(
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
    d_dtype: torch.dtype = torch.bfloat16,
    cd_major: str = "n",
    mma_tiler_mn: Tuple[int, int] = (256, 256),
    cluster_shape_mn: Optional[Tuple[int, int]] = None,
    sf_vec_size: int = 16,
    vector_f32: bool = False,
    m_aligned: int = 256,
    discrete_col_sfd: bool = False,
    use_dynamic_sched: bool = False,
    current_stream=None,
) -> TupleDict:
    """One-shot FC2.  Returns ``TupleDict(d_tensor, d_col_tensor, amax_tensor, sfd_row_tensor,
    sfd_col_tensor)``; amax (bf16 D) is allocated per call and starts at -inf."""
    a_tensor = as_packed_fp4(a_tensor)
    b_tensor = as_packed_fp4(b_tensor)
    b_dtype = packed_fp4_dtype(b_dtype)
    is_dense = b_tensor is not None
    is_discrete = b_ptrs is not None
    if is_dense and is_discrete:
        raise ValueError("Provide either (b_tensor, sfb_tensor) or (b_ptrs, sfb_ptrs), not both")
    if not is_dense and not is_discrete:
        raise ValueError("Must provide either (b_tensor, sfb_tensor) or (b_ptrs, sfb_ptrs)")
    valid_m, k, _ = a_tensor.shape
    if a_tensor.dtype == torch.float4_e2m1fn_x2:
        k *= 2  # two elements per byte (grouped_gemm_quant/api.py:1204)
    if is_dense:
        n_out, _, l = b_tensor.shape
    else:
        _require_pointer_tensor(b_ptrs, "b_ptrs")
        l = b_ptrs.shape[0]
        _require_pointer_tensor(sfb_ptrs, "sfb_ptrs", l)
        if n is None or b_dtype is None:
            raise ValueError("n and b_dtype are required for discrete mode")
        n_out = n
    if bias_tensor is not None and tuple(bias_tensor.shape) != (n_out, l):
        raise ValueError(f"bias_tensor must have shape {(n_out, l)}, got {tuple(bias_tensor.shape)}")
    if cd_major != "n":
        raise ValueError(f"cd_major must be 'n', got {cd_major}")
    dev = a_tensor.device
    fp8_in = a_tensor.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and sfa_tensor.dtype in (torch.float8_e8m0fnu, torch.float8_e4m3fn)
    low_out = d_dtype in (torch.float8_e4m3fn, torch.float8_e5m2, torch.float4_e2m1fn_x2)
    d_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev)
    d_col_tensor = torch.empty_strided((valid_m, n_out, 1), (n_out, 1, valid_m * n_out), dtype=d_dtype, device=dev) if low_out else None
    sfd_row_tensor = sfd_col_tensor = amax_tensor = None
    if fp8_in and low_out and norm_const_tensor is None:
        raise ValueError(
            "norm_const_tensor is required when FP8 inputs are used with FP8 output. "
            "Pass a tensor with shape (1,), e.g. torch.tensor([0.01], dtype=torch.float32, device=a_tensor.device)."
        )
    if not low_out:
        norm_const_tensor = None
    if fp8_in and low_out:
        sfd_row_tensor = _alloc_sfd(valid_m, n_out, sf_vec_size, sfa_tensor.dtype, dev)
        sfd_col_tensor = _alloc_sfd(n_out, valid_m, sf_vec_size, sfa_tensor.dtype, dev)
    if d_dtype in (torch.bfloat16, torch.float16):
        amax_tensor = torch.full((l, 1), float("-inf"), dtype=torch.float32, device=dev)
    if prob_tensor is None:
        raise ValueError(
            "prob_tensor is required: the kernel unconditionally multiplies output by per-row gating probability. "
            "Pass a tensor of ones with shape (valid_m, 1, 1) if no gating is needed."
        )
    result = TupleDict(d_tensor=d_tensor, d_col_tensor=d_col_tensor, amax_tensor=amax_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor)
    if valid_m == 0:
        return result

    cache_key = (
        is_dense, a_tensor.dtype, sfa_tensor.dtype, d_dtype, tuple(a_tensor.shape[1:]),
        (tuple(b_tensor.shape), tuple(b_tensor.stride())) if is_dense else (n, l, b_dtype), b_major, acc_dtype, tuple(mma_tiler_mn),
        None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, vector_f32, m_aligned,
        discrete_col_sfd, use_dynamic_sched, norm_const_tensor is not None, bias_tensor is not None, str(dev),
    )  # fmt: skip
    op = _cache_of_GroupedGemmQuantSm100Objects.get(cache_key)
    if op is None:
        op = GroupedGemmQuantSm100(
            sample_a=a_tensor, sample_sfa=sfa_tensor, sample_padded_offsets=padded_offsets, sample_alpha=alpha_tensor,
            sample_d=d_tensor, sample_d_col=d_col_tensor, sample_b=b_tensor, sample_sfb=sfb_tensor, sample_bias=bias_tensor,
            num_experts=None if is_dense else l, b_shape=None if is_dense else (n, k), b_dtype=None if is_dense else b_dtype,
            sample_sfd_row=sfd_row_tensor, sample_sfd_col=sfd_col_tensor, sample_amax=amax_tensor,
            sample_norm_const=norm_const_tensor, sample_prob=prob_tensor, acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn,
            cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size, vector_f32=vector_f32, m_aligned=m_aligned,
            discrete_col_sfd=discrete_col_sfd, b_major=b_major, use_dynamic_sched=use_dynamic_sched,
        )  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_GroupedGemmQuantSm100Objects[cache_key] = op
    op.execute(
        a_tensor=a_tensor, sfa_tensor=sfa_tensor, padded_offsets=padded_offsets, alpha_tensor=alpha_tensor, d_tensor=d_tensor,
        b_tensor=b_tensor, sfb_tensor=sfb_tensor, bias_tensor=bias_tensor, b_ptrs=b_ptrs, sfb_ptrs=sfb_ptrs,
        d_col_tensor=d_col_tensor, sfd_row_tensor=sfd_row_tensor, sfd_col_tensor=sfd_col_tensor, amax_tensor=amax_tensor,
        norm_const_tensor=norm_const_tensor, prob_tensor=prob_tensor, current_stream=current_stream,
    )  # fmt: skip
    return result
