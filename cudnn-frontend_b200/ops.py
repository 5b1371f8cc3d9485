"""Thin launchers: torch tensors in, C-ABI calls of libb200moe.so out, plus the torch custom-op
registrations.  Nothing here computes on the host; without the CUDA library these functions
raise.

The custom ops (``b200moe::fc1_swiglu``, ``b200moe::fc2_quant``, ``b200moe::quantize_mxfp8``)
mutate caller-provided outputs, like the reference's compiled kernels do
(python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:706-771), and carry fake
implementations so they trace under ``torch.compile`` / ``torch.export``; the in-repo precedent
for that registration style is python/cudnn/experimental/ops/moe_grouped_matmul.py:259-362.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _lib

_FP8_BYTES = (torch.float8_e4m3fn, torch.uint8)
_SF_BYTES = (torch.float8_e8m0fnu, torch.uint8, torch.int8)


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def sf_shape_stride(mn: int, k: int, l: int = 1, sf_vec: int = 32) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """Shape and strides of a scale-factor tensor in the reference's 128x4 layout
    (python/cudnn/grouped_gemm/grouped_gemm_swiglu/api.py:205-215, :513-517)."""
    rm, rk = ceil_div(mn, 128), ceil_div(ceil_div(k, sf_vec), 4)
    return (32, 4, rm, 4, rk, l), (16, 4, rk * 512, 1, 512, rm * rk * 512)


def empty_sf(mn: int, k: int, l: int = 1, device="cuda", dtype=torch.float8_e8m0fnu, zero: bool = False, sf_vec: int = 32) -> torch.Tensor:
    """Allocate a scale-factor tensor for an (mn, k) operand: 6-D view over a flat byte buffer."""
    shape, stride = sf_shape_stride(mn, k, l, sf_vec)
    n = l * shape[2] * shape[4] * 512
    flat = (torch.zeros if zero else torch.empty)(n, dtype=torch.uint8, device=device)
    return torch.as_strided(flat.view(dtype), shape, stride)


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream_ptr(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, torch.cuda.Stream):
        return stream.cuda_stream
    return int(stream)  # raw CUstream handle


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("all tensors must live on a CUDA device")


def quantize_mxfp8_out(x: torch.Tensor, q: torch.Tensor, sf: torch.Tensor, stream=None) -> None:
    """bf16 ``x [rows, cols]`` -> E4M3 ``q [rows, cols]`` and E8M0 ``sf`` (128x4 layout)."""
    _require_cuda(x, q, sf)
    if x.dim() != 2 or x.dtype != torch.bfloat16 or x.stride(1) != 1:
        raise ValueError("x must be a 2-D bf16 tensor with contiguous rows")
    rows, cols = x.shape
    if tuple(q.shape) != (rows, cols) or q.dtype not in _FP8_BYTES or not q.is_contiguous():
        raise ValueError("q must be a contiguous [rows, cols] float8_e4m3fn/uint8 tensor")
    need = ceil_div(rows, 128) * ceil_div(ceil_div(cols, 32), 4) * 512
    if sf.dtype not in _SF_BYTES or sf.numel() < need:
        raise ValueError(f"sf must hold at least {need} E8M0 bytes")
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_quantize_mxfp8(
            x.data_ptr(), rows, cols, x.stride(0), q.data_ptr(), sf.data_ptr(), _stream_ptr(stream)
        )
    _lib.check(rc)


def quantize_mxfp8(x: torch.Tensor, stream=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Allocate outputs and quantise.  Returns (q float8_e4m3fn [rows, cols], sf 6-D E8M0)."""
    rows, cols = x.shape
    q = torch.empty((rows, cols), dtype=torch.float8_e4m3fn, device=x.device)
    sf = empty_sf(rows, cols, 1, device=x.device)
    quantize_mxfp8_out(x, q, sf, stream)
    return q, sf


def launch_grouped_gemm(
    kind: str,
    *,
    a: torch.Tensor,
    sfa: torch.Tensor,
    padded_offsets: torch.Tensor,
    alpha: torch.Tensor,
    d: torch.Tensor,
    m_rows: int,
    n: int,
    k: int,
    num_experts: int,
    b: Optional[torch.Tensor] = None,
    sfb: Optional[torch.Tensor] = None,
    b_ptrs: Optional[torch.Tensor] = None,
    sfb_ptrs: Optional[torch.Tensor] = None,
    prob: Optional[torch.Tensor] = None,
    norm_const: Optional[torch.Tensor] = None,
    c: Optional[torch.Tensor] = None,
    d_col: Optional[torch.Tensor] = None,
    amax: Optional[torch.Tensor] = None,
    sfd_row: Optional[torch.Tensor] = None,
    sfd_col: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    discrete_col_sfd: bool = False,
    sm_margin: int = 0,
    tile_mode: Optional[str] = None,
    d_row_map: Optional[torch.Tensor] = None,
    d_peer_ptrs: Optional[torch.Tensor] = None,
    d_peer_slots: int = 0,
    bias: Optional[torch.Tensor] = None,
    act_func: str = "swiglu",
    stream=None,
    dynamic_sched: bool = False,
    b_nmajor: bool = False,
    expert_range: Optional[Tuple[int, int]] = None,
    wait_limit_ms: int = 0,
    light_m_tiles: Optional[int] = None,
    test_skip_b_loads: bool = False,
    stream_m_tiles: Optional[int] = None,
    offsets_have_prev: bool = False,
    sf_vec_size: int = 32,
    beta: Optional[torch.Tensor] = None,
    dprob: Optional[torch.Tensor] = None,
) -> None:
    """Fill the C struct and call b200moe_fc1_swiglu / b200moe_fc2_quant / b200moe_dswiglu (``kind`` "fc1", "fc2",
    "dswiglu"; for the last ``c`` is the forward pre-activation, an input, ``beta`` its per-expert scale and
    ``dprob`` the float32 ``[m_rows]`` accumulator of the gate-probability gradient).

    ``tile_mode``: ``"single"`` (128 x 256 tiles, one CTA), ``"pair"`` (256 x 256 tiles on CTA pairs)
    or ``None`` / ``"auto"`` (the library picks from the average group size).  The environment
    variable ``B200MOE_TILE_MODE`` overrides ``None``.

    ``dynamic_sched``: tiles are drawn from an atomic counter (needs ``workspace`` with room for it,
    see :func:`workspace_bytes`).  ``b_nmajor``: ``b`` is stored ``[E][k][n]`` (or one ``[k][n]``
    allocation per expert behind ``b_ptrs``).  ``expert_range = (lo, hi)``: run experts ``lo .. hi - 1``
    only; all per-expert tensors are still the full ones, rows of the other experts are left alone
    (``lo > 0`` reads ``padded_offsets[lo - 1]`` as the slice's first row).  ``light_m_tiles``: experts with at
    most that many row tiles are interleaved with the larger ones in the tile schedule (``None`` = the
    library's default or ``B200MOE_LIGHT_M_TILES``, ``-1`` = experts in order); ``stream_m_tiles``: weight tiles of
    experts with at most that many row tiles are read with an evict-first L2 hint (``None`` = default or
    ``B200MOE_STREAM_M_TILES``, ``-1`` = no hints).  ``wait_limit_ms`` and
    ``test_skip_b_loads`` drive the bounded-wait test hook.  ``k`` counts elements: with ``float4_e2m1fn_x2``
    operands (two per byte) it is twice the byte width of ``a``; ``sf_vec_size`` is 32, or 16 with FP4 operands,
    and the scale-factor type (E8M0 or E4M3) is taken from ``sfa``.  ``offsets_have_prev``: ``padded_offsets`` is a view that
    starts one element into a longer int32 array whose element before it is the first row of expert 0 (a
    layer that runs row ranges of its expert groups passes clamped offsets this way)."""
    _require_cuda(a, sfa, padded_offsets, alpha, d, b, sfb, b_ptrs, sfb_ptrs, prob, norm_const, c, d_col, amax, sfd_row, sfd_col)
    args = _lib.GemmArgs()
    args.a, args.sfa = _ptr(a), _ptr(sfa)
    args.b, args.sfb = _ptr(b), _ptr(sfb)
    args.b_ptrs, args.sfb_ptrs = _ptr(b_ptrs), _ptr(sfb_ptrs)
    args.padded_offsets, args.alpha = _ptr(padded_offsets), _ptr(alpha)
    args.prob, args.norm_const = _ptr(prob), _ptr(norm_const)
    args.c, args.d, args.d_col = _ptr(c), _ptr(d), _ptr(d_col)
    args.amax, args.sfd_row, args.sfd_col = _ptr(amax), _ptr(sfd_row), _ptr(sfd_col)
    args.workspace = _ptr(workspace)
    args.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    args.m_rows, args.n, args.k, args.num_experts = m_rows, n, k, num_experts
    extra_flags = 0
    if expert_range is not None:
        lo, hi = int(expert_range[0]), int(expert_range[1])
        if not (0 <= lo < hi <= num_experts):
            raise ValueError(f"expert_range {expert_range} outside [0, {num_experts}]")
        # the slice's per-expert entries start at expert lo; its rows stay where they are
        args.num_experts = hi - lo
        args.padded_offsets = padded_offsets.data_ptr() + 4 * lo
        args.alpha = alpha.data_ptr() + 4 * lo
        if amax is not None:
            args.amax = amax.data_ptr() + 4 * lo
        if b is not None:
            rest_k = ceil_div(ceil_div(k, 32), 4)
            args.b = b.data_ptr() + lo * n * k
            args.sfb = sfb.data_ptr() + lo * ceil_div(n, 128) * rest_k * 512
        else:
            args.b_ptrs = b_ptrs.data_ptr() + 8 * lo
            args.sfb_ptrs = sfb_ptrs.data_ptr() + 8 * lo
        if lo > 0:
            extra_flags |= _lib.FLAG_OFFSETS_HAVE_PREV
    if offsets_have_prev:
        # padded_offsets is a view one element into a longer array: the element before it is the first row
        extra_flags |= _lib.FLAG_OFFSETS_HAVE_PREV
    if dynamic_sched:
        extra_flags |= _lib.FLAG_DYNAMIC_SCHED
    if b_nmajor:
        extra_flags |= _lib.FLAG_B_NMAJOR
    if test_skip_b_loads:
        extra_flags |= _lib.FLAG_TEST_SKIP_B_LOADS
    args.wait_limit_ms = int(wait_limit_ms)
    if light_m_tiles is None:
        light_m_tiles = int(os.environ.get("B200MOE_LIGHT_M_TILES", "0"))
    args.sched_light_m_tiles = int(light_m_tiles)
    if stream_m_tiles is None:
        stream_m_tiles = int(os.environ.get("B200MOE_STREAM_M_TILES", "0"))
    args.l2_stream_m_tiles = int(stream_m_tiles)
    if d.dtype not in _D_DTYPES:
        raise NotImplementedError(f"D dtype {d.dtype} is not built (bf16, fp16, float32, E4M3, E5M2 are)")
    args.d_dtype = _D_DTYPES[d.dtype]
    c_types = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16}
    if kind == "dswiglu":
        c_types.update({torch.float8_e4m3fn: _lib.DTYPE_E4M3, torch.float8_e5m2: _lib.DTYPE_E5M2})
    if c is not None and c.dtype not in c_types:
        raise NotImplementedError(f"C dtype {c.dtype} is not built ({', '.join(str(t) for t in c_types)} are)")
    args.c_dtype = _lib.DTYPE_BF16 if c is None else c_types[c.dtype]
    args.beta, args.dprob = _ptr(beta), _ptr(dprob)
    args.flags = _lib.FLAG_DISCRETE_COL_SFD if discrete_col_sfd else 0
    mode = tile_mode or os.environ.get("B200MOE_TILE_MODE", "auto")
    if mode not in ("auto", "single", "pair"):
        raise ValueError(f"tile_mode must be 'auto', 'single' or 'pair', got {mode!r}")
    args.flags |= {"auto": 0, "single": _lib.FLAG_TILE_SINGLE, "pair": _lib.FLAG_TILE_PAIR}[mode]
    args.flags |= extra_flags
    args.sm_margin = sm_margin
    args.d_row_map = _ptr(d_row_map)
    args.d_peer_ptrs = _ptr(d_peer_ptrs)
    args.d_peer_slots = int(d_peer_slots)
    args.bias = _ptr(bias)
    if bias is not None:
        if bias.dtype not in _BIAS_DTYPES:
            raise NotImplementedError(f"bias dtype {bias.dtype} is not built (bf16, f16, f32 are)")
        args.bias_dtype = _BIAS_DTYPES[bias.dtype]
        if expert_range is not None:
            args.bias = bias.data_ptr() + int(expert_range[0]) * n * bias.element_size()
    if act_func not in ("swiglu", "geglu"):
        raise ValueError(f"act_func must be 'swiglu' or 'geglu', got {act_func!r}")
    args.act_func = _lib.ACT_GEGLU if act_func == "geglu" else _lib.ACT_SWIGLU
    if a.dtype in (torch.float8_e5m2, torch.float4_e2m1fn_x2):
        other = b.dtype if b is not None else a.dtype  # discrete weights: the caller vouches for the pointers
        if other != a.dtype:
            raise ValueError("A and B must have the same element type")
        args.ab_dtype = _lib.DTYPE_E5M2 if a.dtype == torch.float8_e5m2 else _lib.DTYPE_E2M1
    else:
        args.ab_dtype = _lib.DTYPE_E4M3
    args.sf_vec_size = int(sf_vec_size)
    args.sf_dtype = _lib.DTYPE_E4M3 if sfa.dtype == torch.float8_e4m3fn else 0
    lib = _lib.load()
    fn = {"fc1": lib.b200moe_fc1_swiglu, "fc2": lib.b200moe_fc2_quant, "dswiglu": lib.b200moe_dswiglu}[kind]
    with torch.cuda.device(a.device):
        rc = fn(ctypes.byref(args), _stream_ptr(stream))
    _lib.check(rc)


def launch_wgrad(
    *, a: torch.Tensor, b: torch.Tensor, sfa: torch.Tensor, sfb: torch.Tensor, offsets: torch.Tensor, wgrad: Optional[torch.Tensor], m: int, n: int,
    tokens: int, wgrad_ptrs: Optional[torch.Tensor] = None, wgrad_dtype: Optional[torch.dtype] = None, sf_vec_size: int = 32, scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None, accumulate: bool = False,
    sm_margin: int = 0, stream=None, tile_mode: Optional[str] = None,
) -> None:  # fmt: skip
    """Call b200moe_wgrad: ``a [m, tokens]`` and ``b`` stored ``[n, tokens]`` (both contiguous along the tokens),
    ``offsets [E]`` int32 token END offsets, ``wgrad [E, m, n]`` bf16 / fp16 / float32 — or ``wgrad_ptrs``, an int64
    device tensor of E addresses of per-expert ``[m, n]`` allocations of ``wgrad_dtype``."""
    _require_cuda(a, b, sfa, sfb, offsets, wgrad, scale_a, scale_b, wgrad_ptrs)
    args = _lib.GemmArgs()
    args.a, args.b, args.sfa, args.sfb = _ptr(a), _ptr(b), _ptr(sfa), _ptr(sfb)
    args.padded_offsets = _ptr(offsets)
    args.alpha, args.beta = _ptr(scale_a), _ptr(scale_b)
    args.d = _ptr(wgrad)
    args.d_peer_ptrs = _ptr(wgrad_ptrs)
    out_dtype = wgrad.dtype if wgrad is not None else wgrad_dtype
    if out_dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError(f"wgrad dtype must be bfloat16, float16 or float32, got {out_dtype}")
    args.d_dtype = _D_DTYPES[out_dtype]
    args.m_rows, args.n, args.k, args.num_experts = m, n, tokens, offsets.shape[0]
    args.ab_dtype = {torch.float8_e5m2: _lib.DTYPE_E5M2, torch.float4_e2m1fn_x2: _lib.DTYPE_E2M1}.get(a.dtype, _lib.DTYPE_E4M3)
    args.sf_vec_size = int(sf_vec_size)
    args.sf_dtype = _lib.DTYPE_E4M3 if sfa.dtype == torch.float8_e4m3fn else 0
    args.flags = _lib.FLAG_ACCUMULATE if accumulate else 0
    mode = tile_mode or os.environ.get("B200MOE_TILE_MODE", "auto")
    args.flags |= {"auto": 0, "single": _lib.FLAG_TILE_SINGLE, "pair": _lib.FLAG_TILE_PAIR}[mode]
    args.sm_margin = sm_margin
    with torch.cuda.device(a.device):
        rc = _lib.load().b200moe_wgrad(ctypes.byref(args), _stream_ptr(stream))
    _lib.check(rc)


_D_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16, torch.float8_e4m3fn: _lib.DTYPE_E4M3,
             torch.uint8: _lib.DTYPE_E4M3, torch.float8_e5m2: _lib.DTYPE_E5M2, torch.float32: _lib.DTYPE_F32}
_BIAS_DTYPES = {torch.bfloat16: _lib.DTYPE_BF16, torch.float16: _lib.DTYPE_F16, torch.float32: _lib.DTYPE_F32}


def workspace_bytes(num_experts: int, discrete: bool, dynamic_sched: bool = False) -> int:
    """Bytes of workspace a launch needs: per-expert descriptors (discrete weights) plus the tile
    counter of the dynamic scheduler."""
    mode = (_lib.WORKSPACE_DISCRETE if discrete else 0) | (_lib.WORKSPACE_DYNAMIC_SCHED if dynamic_sched else 0)
    return int(_lib.load().b200moe_workspace_bytes(num_experts, mode))


def device_status(clear: bool = False) -> int:
    """Device-side status word (0 unless a bounded wait inside a kernel gave up)."""
    return int(_lib.load().b200moe_device_status(1 if clear else 0))


# ---------------------------------------------------------------------------------------------
# torch custom ops: the C-ABI launches as first-class PyTorch operators (schema, fake kernels for
# tracing, mutation annotations).  Outputs are caller-provided and mutated in place, as with the
# reference's compiled kernels; optional tensors are passed as None.
# ---------------------------------------------------------------------------------------------
_T = Optional[torch.Tensor]


@torch.library.custom_op("b200moe::quantize_mxfp8", mutates_args=("q", "sf"), device_types="cuda")
def _quantize_mxfp8_op(x: torch.Tensor, q: torch.Tensor, sf: torch.Tensor) -> None:
    quantize_mxfp8_out(x, q, sf)


@_quantize_mxfp8_op.register_fake
def _(x, q, sf) -> None:
    return None


@torch.library.custom_op(
    "b200moe::fc1_swiglu", mutates_args=("c", "d", "d_col", "amax", "sfd_row", "sfd_col", "workspace"), device_types="cuda"
)
def _fc1_swiglu_op(
    a: torch.Tensor, sfa: torch.Tensor, b: _T, sfb: _T, b_ptrs: _T, sfb_ptrs: _T, padded_offsets: torch.Tensor,
    alpha: torch.Tensor, prob: _T, norm_const: _T, c: _T, d: torch.Tensor, d_col: _T, amax: _T, sfd_row: _T,
    sfd_col: _T, workspace: _T, bias: _T, n: int, discrete_col_sfd: bool, sm_margin: int, tile_mode: str, act_func: str,
    dynamic_sched: bool = False, b_nmajor: bool = False,
) -> None:  # fmt: skip
    launch_grouped_gemm(
        "fc1", a=a, sfa=sfa, b=b, sfb=sfb, b_ptrs=b_ptrs, sfb_ptrs=sfb_ptrs, padded_offsets=padded_offsets, alpha=alpha,
        prob=prob, norm_const=norm_const, c=c, d=d, d_col=d_col, amax=amax, sfd_row=sfd_row, sfd_col=sfd_col,
        workspace=workspace, m_rows=a.shape[0], n=n, k=a.shape[1], num_experts=padded_offsets.shape[0],
        discrete_col_sfd=discrete_col_sfd, sm_margin=sm_margin, tile_mode=tile_mode or None, bias=bias, act_func=act_func or "swiglu",
        dynamic_sched=dynamic_sched, b_nmajor=b_nmajor,
    )  # fmt: skip


@_fc1_swiglu_op.register_fake
def _(a, sfa, b, sfb, b_ptrs, sfb_ptrs, padded_offsets, alpha, prob, norm_const, c, d, d_col, amax, sfd_row, sfd_col,
      workspace, bias, n, discrete_col_sfd, sm_margin, tile_mode, act_func, dynamic_sched=False, b_nmajor=False) -> None:  # fmt: skip
    return None


@torch.library.custom_op(
    "b200moe::fc2_quant", mutates_args=("d", "d_col", "amax", "sfd_row", "sfd_col", "workspace"), device_types="cuda"
)
def _fc2_quant_op(
    a: torch.Tensor, sfa: torch.Tensor, b: _T, sfb: _T, b_ptrs: _T, sfb_ptrs: _T, padded_offsets: torch.Tensor,
    alpha: torch.Tensor, prob: torch.Tensor, norm_const: _T, d: torch.Tensor, d_col: _T, amax: _T, sfd_row: _T,
    sfd_col: _T, workspace: _T, d_row_map: _T, d_peer_ptrs: _T, d_peer_slots: int, bias: _T, n: int, discrete_col_sfd: bool,
    sm_margin: int, tile_mode: str, dynamic_sched: bool = False, b_nmajor: bool = False,
) -> None:  # fmt: skip
    launch_grouped_gemm(
        "fc2", a=a, sfa=sfa, b=b, sfb=sfb, b_ptrs=b_ptrs, sfb_ptrs=sfb_ptrs, padded_offsets=padded_offsets, alpha=alpha,
        prob=prob, norm_const=norm_const, d=d, d_col=d_col, amax=amax, sfd_row=sfd_row, sfd_col=sfd_col,
        workspace=workspace, m_rows=a.shape[0], n=n, k=a.shape[1], num_experts=padded_offsets.shape[0],
        discrete_col_sfd=discrete_col_sfd, sm_margin=sm_margin, tile_mode=tile_mode or None, d_row_map=d_row_map,
        d_peer_ptrs=d_peer_ptrs, d_peer_slots=d_peer_slots, bias=bias, dynamic_sched=dynamic_sched, b_nmajor=b_nmajor,
    )  # fmt: skip


@_fc2_quant_op.register_fake
def _(a, sfa, b, sfb, b_ptrs, sfb_ptrs, padded_offsets, alpha, prob, norm_const, d, d_col, amax, sfd_row, sfd_col, workspace,
      d_row_map, d_peer_ptrs, d_peer_slots, bias, n, discrete_col_sfd, sm_margin, tile_mode, dynamic_sched=False,
      b_nmajor=False) -> None:  # fmt: skip
    return None


_FORCE_CUSTOM_OP = os.environ.get("B200MOE_FORCE_CUSTOM_OP", "0") == "1"


def grouped_gemm_op(kind: str, *, stream=None, **kw) -> None:
    """Launch FC1 / FC2.  While ``torch.compile`` traces (or with ``B200MOE_FORCE_CUSTOM_OP=1``) the
    launch goes through the registered custom op (``torch.ops.b200moe.fc1_swiglu`` / ``fc2_quant``),
    so the graph sees one opaque op; in eager mode it calls the C ABI directly.  An explicit
    ``stream`` is honoured in both (the custom op makes it current for the call: custom ops take
    tensors and plain scalars only)."""
    if not (torch.compiler.is_compiling() or _FORCE_CUSTOM_OP):
        # eager fast path: the same C-ABI launch without the dispatcher round trip (about 15 us of
        # host time per call, which is most of a small problem's latency)
        a = kw["a"]
        launch_grouped_gemm(
            kind, a=a, sfa=kw["sfa"], padded_offsets=kw["padded_offsets"], alpha=kw["alpha"], d=kw["d"], m_rows=a.shape[0], n=kw["n"],
            k=a.shape[1] * (2 if a.dtype == torch.float4_e2m1fn_x2 else 1), sf_vec_size=int(kw.get("sf_vec_size", 32)), num_experts=kw["padded_offsets"].shape[0], b=kw.get("b"), sfb=kw.get("sfb"), b_ptrs=kw.get("b_ptrs"),
            sfb_ptrs=kw.get("sfb_ptrs"), prob=kw.get("prob"), norm_const=kw.get("norm_const"), c=kw.get("c") if kind != "fc2" else None,
            beta=kw.get("beta"), dprob=kw.get("dprob"),
            d_col=kw.get("d_col"), amax=kw.get("amax"), sfd_row=kw.get("sfd_row"), sfd_col=kw.get("sfd_col"),
            workspace=kw.get("workspace"), discrete_col_sfd=bool(kw.get("discrete_col_sfd", False)), sm_margin=int(kw.get("sm_margin", 0)),
            tile_mode=kw.get("tile_mode") or None, d_row_map=kw.get("d_row_map"), d_peer_ptrs=kw.get("d_peer_ptrs"),
            d_peer_slots=int(kw.get("d_peer_slots", 0)), bias=kw.get("bias"), act_func=kw.get("act_func") or "swiglu", stream=stream,
            dynamic_sched=bool(kw.get("dynamic_sched", False)), b_nmajor=bool(kw.get("b_nmajor", False)),
            expert_range=kw.get("expert_range"), wait_limit_ms=int(kw.get("wait_limit_ms", 0)), light_m_tiles=kw.get("light_m_tiles"),
            test_skip_b_loads=bool(kw.get("test_skip_b_loads", False)), stream_m_tiles=kw.get("stream_m_tiles"),
            offsets_have_prev=bool(kw.get("offsets_have_prev", False)),
        )  # fmt: skip
        return
    ctx = torch.cuda.stream(stream) if isinstance(stream, torch.cuda.Stream) else None
    if stream is not None and ctx is None:
        ctx = torch.cuda.stream(torch.cuda.ExternalStream(int(stream)))
    common = (kw["a"], kw["sfa"], kw.get("b"), kw.get("sfb"), kw.get("b_ptrs"), kw.get("sfb_ptrs"), kw["padded_offsets"],
              kw["alpha"], kw.get("prob"), kw.get("norm_const"))  # fmt: skip
    if kw.get("expert_range") is not None or kw.get("test_skip_b_loads") or kw.get("offsets_have_prev"):
        raise NotImplementedError("expert_range and the test hook are eager-only launch options")
    if kw["a"].dtype == torch.float4_e2m1fn_x2 or kind == "dswiglu":
        raise NotImplementedError("FP4 operands and the dSwiGLU kernel are launched eagerly only (no custom-op schema is registered for them)")
    tail = (kw["n"], bool(kw.get("discrete_col_sfd", False)), int(kw.get("sm_margin", 0)), kw.get("tile_mode") or "")
    sched = (bool(kw.get("dynamic_sched", False)), bool(kw.get("b_nmajor", False)))
    outs = (kw["d"], kw.get("d_col"), kw.get("amax"), kw.get("sfd_row"), kw.get("sfd_col"), kw.get("workspace"))

    def call():
        if kind == "fc1":
            torch.ops.b200moe.fc1_swiglu(*common, kw.get("c"), *outs, kw.get("bias"), *tail, kw.get("act_func") or "swiglu", *sched)
        else:
            torch.ops.b200moe.fc2_quant(*common, *outs, kw.get("d_row_map"), kw.get("d_peer_ptrs"), int(kw.get("d_peer_slots", 0)),
                                        kw.get("bias"), *tail, *sched)  # fmt: skip

    if ctx is None:
        call()
    else:
        with ctx:
            call()
