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


def empty_sf(mn: int, k: int, l: int = 1, device="cuda", dtype=torch.float8_e8m0fnu, zero: bool = False) -> torch.Tensor:
    """Allocate a scale-factor tensor for an (mn, k) operand: 6-D view over a flat byte buffer."""
    shape, stride = sf_shape_stride(mn, k, l)
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
    stream=None,
) -> None:
    """Fill the C struct and call b200moe_fc1_swiglu / b200moe_fc2_quant.

    ``tile_mode``: ``"single"`` (128 x 256 tiles, one CTA), ``"pair"`` (256 x 256 tiles on CTA pairs)
    or ``None`` / ``"auto"`` (the library picks from the average group size).  The environment
    variable ``B200MOE_TILE_MODE`` overrides ``None``."""
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
    args.d_dtype = _lib.DTYPE_E4M3 if d.dtype in _FP8_BYTES else _lib.DTYPE_BF16
    args.flags = _lib.FLAG_DISCRETE_COL_SFD if discrete_col_sfd else 0
    mode = tile_mode or os.environ.get("B200MOE_TILE_MODE", "auto")
    if mode not in ("auto", "single", "pair"):
        raise ValueError(f"tile_mode must be 'auto', 'single' or 'pair', got {mode!r}")
    args.flags |= {"auto": 0, "single": _lib.FLAG_TILE_SINGLE, "pair": _lib.FLAG_TILE_PAIR}[mode]
    args.sm_margin = sm_margin
    args.d_row_map = _ptr(d_row_map)
    lib = _lib.load()
    fn = lib.b200moe_fc1_swiglu if kind == "fc1" else lib.b200moe_fc2_quant
    with torch.cuda.device(a.device):
        rc = fn(ctypes.byref(args), _stream_ptr(stream))
    _lib.check(rc)


def workspace_bytes(num_experts: int, discrete: bool) -> int:
    return int(_lib.load().b200moe_workspace_bytes(num_experts, 1 if discrete else 0))


def device_status(clear: bool = False) -> int:
    """Device-side status word (0 unless a bounded wait inside a kernel gave up)."""
    return int(_lib.load().b200moe_device_status(1 if clear else 0))
