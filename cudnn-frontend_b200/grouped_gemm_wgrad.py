"""Weight gradient of the MoE grouped GEMMs: the experts partition the contraction dimension.

Same names, arguments and error behaviour as the reference's ``GroupedGemmWgradSm100`` /
``grouped_gemm_wgrad_wrapper_sm100`` (python/cudnn/grouped_gemm/grouped_gemm_wgrad/api.py:47-557, :559-672).
``A (m, T)`` and ``B (T, n)`` are both contiguous along the tokens ``T`` (``B`` is stored ``[n, T]``); expert ``e``
owns tokens ``[offsets[e-1], offsets[e])`` and its own 128x4 block of scale factors inside ``SFA (round_up(m, 128),
cols)`` / ``SFB (round_up(n, 128), cols)``; ``wgrad[e] = gs_a[e] gs_b[e] (A_e SFA_e)(B_e SFB_e)^T``, shape ``(E, m,
n)`` in bf16 / fp16 / float32, overwritten or (``accumulate_on_output``) added to.

Dense output mode writes one ``(E, m, n)`` tensor, discrete output mode one ``(m, n)`` allocation per expert behind the
int64 pointer tensor ``wgrad_ptrs``.

Differences a caller can observe: every expert's token count must be a multiple of 32 (the reference's scale shape
rule already implies a multiple of ``4 * sf_vec_size``); the per-expert allocations of the discrete mode must be
contiguous ``(m, n)`` and 16-byte aligned.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import ops
from .api_base import OperatorBase, TensorSpec, TupleDict, as_packed_fp4, ceil_div, is_power_of_2


def _round_up(a: int, b: int) -> int:
    return ceil_div(a, b) * b


class GroupedGemmWgradSm100(OperatorBase):
    def __init__(
        self,
        sample_a: torch.Tensor,
        sample_b: torch.Tensor,
        sample_sfa: torch.Tensor,
        sample_sfb: torch.Tensor,
        sample_offsets: torch.Tensor,
        sample_wgrad: Optional[torch.Tensor] = None,
        sample_wgrad_expert: Optional[torch.Tensor] = None,
        num_experts: Optional[int] = None,
        wgrad_shape: Optional[Tuple[int, int]] = None,
        wgrad_dtype: Optional[torch.dtype] = None,
        sample_global_scale_a: Optional[torch.Tensor] = None,
        sample_global_scale_b: Optional[torch.Tensor] = None,
        acc_dtype: torch.dtype = torch.float32,
        mma_tiler_mn: Tuple[int, int] = (256, 256),
        cluster_shape_mn: Optional[Tuple[int, int]] = None,
        sf_vec_size: int = 16,
        accumulate_on_output: bool = False,
    ):
        super().__init__()
        if sample_wgrad is not None and num_experts is None:
            self.discrete = False
        elif sample_wgrad is None and num_experts is not None:
            self.discrete = True
            if wgrad_shape is None or wgrad_dtype is None:
                raise ValueError("wgrad_shape and wgrad_dtype are required in discrete mode")
        else:
            raise ValueError("Provide either sample_wgrad for dense mode or (num_experts, wgrad_shape, wgrad_dtype) for discrete mode, but not both")
        self.a = TensorSpec.of(as_packed_fp4(sample_a), "sample_a")
        self.b = TensorSpec.of(as_packed_fp4(sample_b), "sample_b")
        self.sfa = TensorSpec.of(sample_sfa, "sample_sfa")
        self.sfb = TensorSpec.of(sample_sfb, "sample_sfb")
        self.offsets = TensorSpec.of(sample_offsets, "sample_offsets")
        self.wgrad = TensorSpec.of(sample_wgrad, "sample_wgrad")
        self.wgrad_expert = TensorSpec.of(sample_wgrad_expert, "sample_wgrad_expert")
        self.wgrad_shape = tuple(wgrad_shape) if wgrad_shape is not None else None
        self.gs_a = TensorSpec.of(sample_global_scale_a, "sample_global_scale_a")
        self.gs_b = TensorSpec.of(sample_global_scale_b, "sample_global_scale_b")
        self.expert_cnt = num_experts if self.discrete else self.wgrad.shape[0]
        self.wgrad_dtype = wgrad_dtype if self.discrete else self.wgrad.dtype
        self.sf_vec_size = sf_vec_size
        self.acc_dtype = acc_dtype
        self.mma_tiler_mn = tuple(mma_tiler_mn)
        self.use_2cta_instrs = self.mma_tiler_mn[0] == 256
        self.cluster_shape_mn = tuple(cluster_shape_mn) if cluster_shape_mn is not None else ((2, 1) if self.use_2cta_instrs else (1, 1))
        self.accumulate_on_output = accumulate_on_output

    def check_support(self) -> bool:
        self._value_error_if(len(self.a.shape) != 2 or len(self.b.shape) != 2, "sample_a must be (m, tokens) and sample_b (tokens, n)")
        a_l, b_l = self.a.logical(), self.b.logical()  # FP4 operands: two elements per byte along the tokens
        m, tokens = a_l.shape
        tokens_b, n = b_l.shape
        self._value_error_if(tokens != tokens_b, f"sample_a and sample_b token dimensions must match, got {tokens} and {tokens_b}")
        self._check_stride(a_l, (tokens, 1), "sample_a must be contiguous along the tokens")
        self._check_stride(b_l, (1, tokens), "sample_b must be contiguous along the tokens (stored [n, tokens])")
        scale_cols = _round_up(ceil_div(tokens, self.sf_vec_size), 4)
        self._check_shape(self.sfa, (_round_up(m, 128), scale_cols), "sample_sfa")
        self._check_shape(self.sfb, (_round_up(n, 128), scale_cols), "sample_sfb")
        self._check_stride(self.sfa, (scale_cols, 1), "sample_sfa must be contiguous")
        self._check_stride(self.sfb, (scale_cols, 1), "sample_sfb must be contiguous")
        self._check_shape(self.offsets, (self.expert_cnt,), "sample_offsets")
        dtype = self._check_dtype(self.a, [torch.float4_e2m1fn_x2, torch.uint8, torch.float8_e5m2, torch.float8_e4m3fn, torch.bfloat16], "sample_a")
        self._check_dtype(self.b, dtype, "sample_b", "sample_b must have the same dtype as sample_a")
        sf_dtype = self._check_dtype(self.sfa, [torch.float8_e8m0fnu, torch.float8_e4m3fn], "sample_sfa", "sample_sfa must have dtype float8_e8m0fnu or float8_e4m3fn")
        self._check_dtype(self.sfb, sf_dtype, "sample_sfb", "sample_sfb must have the same dtype as sample_sfa")
        self._check_dtype(self.offsets, torch.int32, "sample_offsets", "sample_offsets must be int32")
        self._check_dtype(self.wgrad_dtype, [torch.bfloat16, torch.float16, torch.float32], "wgrad_dtype", "wgrad_dtype must be bfloat16, float16, or float32")
        if not self.discrete:
            self._check_shape(self.wgrad, (self.expert_cnt, m, n), "sample_wgrad")
            self._check_stride(self.wgrad, (m * n, n, 1), "sample_wgrad must be contiguous")
        else:
            self._value_error_if(self.wgrad_shape != (m, n), f"wgrad_shape must be {(m, n)}, got {self.wgrad_shape}")
            self._check_shape(self.wgrad_expert, (m, n), "single_expert_wgrad")
            self._check_stride(self.wgrad_expert, (n, 1), "sample_wgrad_expert must be contiguous")
            self._check_dtype(self.wgrad_expert, self.wgrad_dtype, "sample_wgrad_expert", "sample_wgrad_expert must have the same dtype as wgrad_dtype")
        self._value_error_if(self.mma_tiler_mn[0] not in (128, 256), f"mma_tiler_mn[0] must be 128 or 256, got {self.mma_tiler_mn[0]}")
        self._value_error_if(self.mma_tiler_mn[1] not in (128, 256), f"mma_tiler_mn[1] must be 128 or 256, got {self.mma_tiler_mn[1]}")
        cm, cn = self.cluster_shape_mn
        self._value_error_if(cm % (2 if self.use_2cta_instrs else 1) != 0, f"cluster_shape_mn[0] must be divisible by 2 when use_2cta_instrs=True, got {cm}")
        self._value_error_if(cm * cn > 16, f"cluster shape product must be <= 16, got {self.cluster_shape_mn}")
        self._value_error_if(not (is_power_of_2(cm) and is_power_of_2(cn)), f"cluster shape values must be powers of 2, got {self.cluster_shape_mn}")
        has_gs = self.gs_a is not None or self.gs_b is not None
        if has_gs:
            self._value_error_if(self.gs_a is None or self.gs_b is None, "sample_global_scale_a and sample_global_scale_b must be provided together")
            self._check_shape(self.gs_a, (self.expert_cnt,), "sample_global_scale_a")
            self._check_shape(self.gs_b, (self.expert_cnt,), "sample_global_scale_b")
            self._check_dtype(self.gs_a, torch.float32, "sample_global_scale_a")
            self._check_dtype(self.gs_b, torch.float32, "sample_global_scale_b")
        fp4 = self._is_fp4x2(dtype)
        self._value_error_if(fp4 and self.sf_vec_size == 16 and sf_dtype == torch.float8_e4m3fn and not has_gs, "NVFP4 wgrad requires sample_global_scale_a and sample_global_scale_b")
        self._value_error_if(self.sf_vec_size not in (16, 32), f"sf_vec_size must be 16 or 32, got {self.sf_vec_size}")
        self._value_error_if(self._is_fp8(dtype) and self.sf_vec_size != 32, f"fp8 operands take sf_vec_size 32, got {self.sf_vec_size}")

        # what this build implements of the reference's surface
        self._not_implemented_error_if(dtype in (torch.uint8, torch.bfloat16), f"operands of dtype {dtype} are not built (float8 and float4_e2m1fn_x2 are)")
        self._value_error_if(tokens % 32 != 0 or n % 32 != 0, f"tokens ({tokens}) and n ({n}) must be multiples of 32")
        self._m, self._n, self._tokens = m, n, tokens
        self._require_sm100()
        self._is_supported = True
        return True

    def compile(self) -> None:
        if not self._is_supported:
            self.check_support()
        ops._lib.load()  # fails loudly when the CUDA library is missing
        self._is_compiled = True

    def execute(
        self,
        a_tensor: torch.Tensor,
        b_tensor: torch.Tensor,
        sfa_tensor: torch.Tensor,
        sfb_tensor: torch.Tensor,
        offsets_tensor: torch.Tensor,
        wgrad_tensor: Optional[torch.Tensor] = None,
        wgrad_ptrs: Optional[torch.Tensor] = None,
        global_scale_a: Optional[torch.Tensor] = None,
        global_scale_b: Optional[torch.Tensor] = None,
        current_stream=None,
    ) -> None:
        """Launch on ``current_stream``; allocates nothing.  The token count may differ from the sample's (it is read
        from ``a_tensor``)."""
        a_tensor = as_packed_fp4(a_tensor)
        b_tensor = as_packed_fp4(b_tensor)
        self._ensure_compiled()
        if not self.discrete and wgrad_tensor is None:
            raise ValueError("wgrad_tensor is required in dense mode")
        if self.discrete:
            if wgrad_ptrs is None:
                raise ValueError("wgrad_ptrs is required in discrete mode")
            if wgrad_ptrs.dtype != torch.int64 or wgrad_ptrs.dim() != 1 or wgrad_ptrs.shape[0] != self.expert_cnt or not wgrad_ptrs.is_cuda:
                raise ValueError(f"wgrad_ptrs must be a 1-D int64 CUDA tensor of {self.expert_cnt} addresses")
        tokens = a_tensor.shape[1] * (2 if a_tensor.dtype == torch.float4_e2m1fn_x2 else 1)
        ops.launch_wgrad(a=a_tensor, b=b_tensor, sfa=sfa_tensor, sfb=sfb_tensor, offsets=offsets_tensor,
                         wgrad=None if self.discrete else wgrad_tensor, wgrad_ptrs=wgrad_ptrs if self.discrete else None, wgrad_dtype=self.wgrad_dtype,
                         m=self._m, n=self._n, tokens=tokens, sf_vec_size=self.sf_vec_size, scale_a=global_scale_a, scale_b=global_scale_b,
                         accumulate=self.accumulate_on_output, stream=current_stream)  # fmt: skip


_cache_of_GroupedGemmWgradSm100Objects = {}


def grouped_gemm_wgrad_wrapper_sm100(
    a_tensor: torch.Tensor,
    b_tensor: torch.Tensor,
    sfa_tensor: torch.Tensor,
    sfb_tensor: torch.Tensor,
    offsets_tensor: torch.Tensor,
    output_mode: str = "dense",
    wgrad_tensor: Optional[torch.Tensor] = None,
    wgrad_ptrs: Optional[torch.Tensor] = None,
    global_scale_a: Optional[torch.Tensor] = None,
    global_scale_b: Optional[torch.Tensor] = None,
    acc_dtype: torch.dtype = torch.float32,
    wgrad_dtype: torch.dtype = torch.bfloat16,
    mma_tiler_mn: Tuple[int, int] = (256, 256),
    cluster_shape_mn: Optional[Tuple[int, int]] = None,
    sf_vec_size: int = 16,
    accumulate_on_output: bool = False,
    current_stream=None,
) -> TupleDict:
    """One-shot weight gradient.  Returns ``TupleDict(wgrad_tensor)``; the output is allocated here when the caller
    passes none (zeros with ``accumulate_on_output``, as in the reference, api.py:587-592)."""
    a_tensor = as_packed_fp4(a_tensor)
    b_tensor = as_packed_fp4(b_tensor)
    if output_mode not in ("dense", "discrete"):
        raise ValueError(f"output_mode must be 'dense' or 'discrete', got {output_mode}")
    hidden = a_tensor.shape[0]
    intermediate = b_tensor.shape[1]
    e = offsets_tensor.shape[0]
    if output_mode == "discrete":
        if wgrad_ptrs is None:
            raise ValueError("wgrad_ptrs is required in discrete output mode")
        key = ("discrete", a_tensor.dtype, sfa_tensor.dtype, hidden, intermediate, e, wgrad_dtype, tuple(mma_tiler_mn), sf_vec_size, accumulate_on_output,
               global_scale_a is not None, str(a_tensor.device))  # fmt: skip
        op = _cache_of_GroupedGemmWgradSm100Objects.get(key)
        if op is None:
            op = GroupedGemmWgradSm100(a_tensor, b_tensor, sfa_tensor, sfb_tensor, offsets_tensor, num_experts=e, wgrad_shape=(hidden, intermediate),
                                       wgrad_dtype=wgrad_dtype, sample_global_scale_a=global_scale_a, sample_global_scale_b=global_scale_b,
                                       acc_dtype=acc_dtype, mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size,
                                       accumulate_on_output=accumulate_on_output)  # fmt: skip
            assert op.check_support(), "Unsupported configuration"
            op.compile()
            _cache_of_GroupedGemmWgradSm100Objects[key] = op
        op.execute(a_tensor, b_tensor, sfa_tensor, sfb_tensor, offsets_tensor, wgrad_ptrs=wgrad_ptrs, global_scale_a=global_scale_a,
                   global_scale_b=global_scale_b, current_stream=current_stream)  # fmt: skip
        return TupleDict(wgrad_tensor=None)
    if wgrad_tensor is None:
        alloc = torch.zeros if accumulate_on_output else torch.empty
        wgrad_tensor = alloc((e, hidden, intermediate), dtype=wgrad_dtype, device=a_tensor.device)
    key = (a_tensor.dtype, sfa_tensor.dtype, hidden, intermediate, e, wgrad_tensor.dtype, acc_dtype, tuple(mma_tiler_mn),
           None if cluster_shape_mn is None else tuple(cluster_shape_mn), sf_vec_size, accumulate_on_output, global_scale_a is not None,
           str(a_tensor.device))  # fmt: skip
    op = _cache_of_GroupedGemmWgradSm100Objects.get(key)
    if op is None:
        op = GroupedGemmWgradSm100(a_tensor, b_tensor, sfa_tensor, sfb_tensor, offsets_tensor, sample_wgrad=wgrad_tensor,
                                   sample_global_scale_a=global_scale_a, sample_global_scale_b=global_scale_b, acc_dtype=acc_dtype,
                                   mma_tiler_mn=mma_tiler_mn, cluster_shape_mn=cluster_shape_mn, sf_vec_size=sf_vec_size,
                                   accumulate_on_output=accumulate_on_output)  # fmt: skip
        assert op.check_support(), "Unsupported configuration"
        op.compile()
        _cache_of_GroupedGemmWgradSm100Objects[key] = op
    op.execute(a_tensor, b_tensor, sfa_tensor, sfb_tensor, offsets_tensor, wgrad_tensor=wgrad_tensor, global_scale_a=global_scale_a,
               global_scale_b=global_scale_b, current_stream=current_stream)  # fmt: skip
    return TupleDict(wgrad_tensor=wgrad_tensor)
