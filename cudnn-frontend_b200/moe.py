"""Routing side of the MoE layer: expert grouping, padded END offsets, row scatter, combine.

The reference has no counterpart (its tests build the offsets on the host,
test/python/fe_api/test_grouped_gemm_swiglu_utils.py:270-312); these launch the integer kernels of
libb200moe.so and are exact: rows of one expert keep their original order (a stable sort).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .ops import _stream_ptr


def route(expert_ids: torch.Tensor, num_experts: int, m_aligned: int = 128, stream=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``expert_ids`` (int32, any shape, token-major) -> ``(counts [E], padded_offsets [E],
    dst_row [R])``: rows per expert, END offsets with every group rounded up to ``m_aligned``
    rows, and for every routed row its row in the expert-grouped padded buffer."""
    if expert_ids.dtype != torch.int32 or not expert_ids.is_cuda:
        raise ValueError("expert_ids must be an int32 CUDA tensor")
    ids = expert_ids.contiguous().view(-1)
    r = ids.numel()
    dev = ids.device
    lib = _lib.load()
    counts = torch.empty(num_experts, dtype=torch.int32, device=dev)
    offsets = torch.empty(num_experts, dtype=torch.int32, device=dev)
    dst = torch.empty(r, dtype=torch.int32, device=dev)
    scratch = torch.empty(max(int(lib.b200moe_route_scratch_bytes(r, num_experts)) // 4, 1), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.b200moe_route(ids.data_ptr(), r, num_experts, m_aligned, counts.data_ptr(), offsets.data_ptr(), dst.data_ptr(), scratch.data_ptr(), _stream_ptr(stream))
    _lib.check(rc)
    return counts, offsets, dst


def scatter_rows(
    x: torch.Tensor,
    dst_row: torch.Tensor,
    out: torch.Tensor,
    rows_per_src: int = 1,
    in_prob: Optional[torch.Tensor] = None,
    out_prob: Optional[torch.Tensor] = None,
    stream=None,
) -> None:
    """``out[dst_row[r]] = x[r // rows_per_src]`` for bf16 rows (top-k replication when
    ``rows_per_src = k``); optionally ``out_prob[dst_row[r]] = in_prob[r]``."""
    if x.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or not x.is_contiguous() or not out.is_contiguous():
        raise ValueError("x and out must be contiguous bf16 tensors")
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_scatter_rows(
            x.data_ptr(), dst_row.data_ptr(), dst_row.numel(), rows_per_src, x.shape[-1], out.data_ptr(),
            None if in_prob is None else in_prob.data_ptr(), None if out_prob is None else out_prob.data_ptr(), _stream_ptr(stream),
        )  # fmt: skip
    _lib.check(rc)


def gather_rows(x: torch.Tensor, src_row: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """``out[r] = x[src_row[r]]`` for bf16 rows (a negative index gives a zero row)."""
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 tensor")
    if out is None:
        out = torch.empty((src_row.numel(), x.shape[-1]), dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_gather_rows(x.data_ptr(), src_row.data_ptr(), src_row.numel(), x.shape[-1], out.data_ptr(), _stream_ptr(stream))
    _lib.check(rc)
    return out


def zero_pad_rows(buf: torch.Tensor, counts: torch.Tensor, padded_offsets: torch.Tensor, prob: Optional[torch.Tensor] = None, stream=None) -> None:
    """Zero the padding rows of every expert group of a bf16 ``[M, cols]`` buffer."""
    with torch.cuda.device(buf.device):
        rc = _lib.load().b200moe_zero_pad_rows(
            buf.data_ptr(), counts.data_ptr(), padded_offsets.data_ptr(), counts.numel(), buf.shape[-1],
            None if prob is None else prob.data_ptr(), _stream_ptr(stream),
        )  # fmt: skip
    _lib.check(rc)


def combine_rows(y: torch.Tensor, dst_row: torch.Tensor, num_tokens: int, topk: int, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """``out[t] = sum_j y[dst_row[t * topk + j]]`` (bf16 in, float32 accumulate, bf16 out)."""
    if y.dtype != torch.bfloat16 or not y.is_contiguous():
        raise ValueError("y must be a contiguous bf16 tensor")
    if out is None:
        out = torch.empty((num_tokens, y.shape[-1]), dtype=torch.bfloat16, device=y.device)
    with torch.cuda.device(y.device):
        rc = _lib.load().b200moe_combine_rows(y.data_ptr(), dst_row.data_ptr(), num_tokens, topk, y.shape[-1], out.data_ptr(), _stream_ptr(stream))
    _lib.check(rc)
    return out


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[..., I, K]`` gate and up projection weights -> ``[..., 2I, K]`` in the order FC1 consumes:
    rows ``64j .. 64j+31`` are gate block ``j`` and rows ``64j+32 .. 64j+63`` up block ``j`` (the
    reference's kernels pair even and odd 32-column blocks of the GEMM output,
    test/python/fe_api/test_grouped_gemm_swiglu_utils.py:543-560).  For callers that hold
    ``[gate | up]`` halves."""
    i, k = w_gate.shape[-2], w_gate.shape[-1]
    if i % 32 != 0 or w_up.shape != w_gate.shape:
        raise ValueError("gate and up must have equal shapes with the intermediate size a multiple of 32")
    lead = w_gate.shape[:-2]
    g = w_gate.reshape(*lead, i // 32, 1, 32, k)
    u = w_up.reshape(*lead, i // 32, 1, 32, k)
    return torch.cat([g, u], dim=-3).reshape(*lead, 2 * i, k)
