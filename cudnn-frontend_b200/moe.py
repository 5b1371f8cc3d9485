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


def dispatch_quantize(x: torch.Tensor, send_pos: torch.Tensor, topk: int, topk_prob: Optional[torch.Tensor] = None, stream=None):
    """Fused dispatch-side pass: every token row of ``x [T, H]`` (bf16) is read once, quantised to
    MXFP8 and written to its ``topk`` positions ``send_pos[t * topk + j]`` of the send buffers.
    Returns ``(q [R, H] uint8 E4M3, sf [R, H/32] uint8 E8M0 row-major, prob [R] f32)``."""
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 tensor")
    t, h = x.shape
    r = t * topk
    dev = x.device
    q = torch.empty((r, h), dtype=torch.uint8, device=dev)
    sf = torch.empty((r, h // 32), dtype=torch.uint8, device=dev)
    prob = torch.empty((r,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().b200moe_dispatch_quantize(
            x.data_ptr(), send_pos.data_ptr(), None if topk_prob is None else topk_prob.data_ptr(), t, topk, h,
            q.data_ptr(), sf.data_ptr(), prob.data_ptr(), _stream_ptr(stream),
        )  # fmt: skip
    _lib.check(rc)
    return q, sf, prob


def place_quantized_rows(q_in, sf_in, prob_in, dst_row, m_rows: int, counts=None, padded_offsets=None, stream=None):
    """Receive-side pass: arrival-order MXFP8 rows -> expert-grouped GEMM operand.  Returns
    ``(a (M, H, 1) float8_e4m3fn, sfa 6-D E8M0 in the 128x4 layout, prob (M, 1, 1) f32)``; with
    ``counts`` / ``padded_offsets`` the padding rows of every group are zeroed."""
    from .ops import empty_sf

    h = q_in.shape[1]
    dev = q_in.device
    a = torch.empty((m_rows, h), dtype=torch.uint8, device=dev)
    sfa = empty_sf(m_rows, h, 1, device=dev)
    prob = torch.empty((m_rows,), dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.b200moe_place_quantized_rows(
            q_in.data_ptr(), sf_in.data_ptr(), prob_in.data_ptr(), dst_row.data_ptr(), dst_row.numel(), h,
            a.data_ptr(), sfa.data_ptr(), prob.data_ptr(), _stream_ptr(stream),
        )  # fmt: skip
        _lib.check(rc)
        if counts is not None:
            # an E4M3 row of H bytes is zeroed as H/2 bf16 elements
            rc = lib.b200moe_zero_pad_rows(a.data_ptr(), counts.data_ptr(), padded_offsets.data_ptr(), counts.numel(), h // 2,
                                           prob.data_ptr(), _stream_ptr(stream))  # fmt: skip
            _lib.check(rc)
    return a.view(torch.float8_e4m3fn).view(m_rows, h, 1), sfa, prob.view(m_rows, 1, 1)


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


def dispatch_record_pitch(cols: int) -> int:
    """Bytes of one dispatch record (scales + gate probability + return address) for rows of ``cols``."""
    return int(_lib.load().b200moe_dispatch_record_pitch(cols))


def dispatch_quantize_peer(x: torch.Tensor, topk_ids: torch.Tensor, local_row: torch.Tensor, delta: torch.Tensor,
                           topk_prob: Optional[torch.Tensor], experts_per_rank: int, num_ranks: int, my_rank: int,
                           slot_capacity: int, row_capacity: int, peer_q: torch.Tensor, peer_rec: torch.Tensor, stream=None,
                           row_bounds: Optional[torch.Tensor] = None, chunk: int = 0, max_blocks: int = 0) -> None:  # fmt: skip
    """Fused quantise + dispatch over peer memory: token rows of ``x [T, H]`` are quantised to MXFP8 and
    stored straight into the expert-grouped GEMM operand of the rank that owns each slot's expert,
    each with a record of its scales, gate probability and return address
    (see ``b200moe_dispatch_quantize_peer`` in include/b200moe.h).  ``peer_*`` are int64 device tensors
    of ``num_ranks`` base addresses.  With ``row_bounds`` (int32 ``[num_ranks, C + 1]``: first row of every
    chunk on every rank, the rank's row count last) only the slots whose destination row lies in chunk
    ``chunk`` of its rank are moved; ``max_blocks`` bounds the grid for a launch that runs beside a GEMM."""
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("x must be a contiguous bf16 tensor")
    t, h = x.shape
    k = topk_ids.shape[1]
    num_chunks = 0
    if row_bounds is not None:
        if row_bounds.dtype != torch.int32 or not row_bounds.is_contiguous() or row_bounds.dim() != 2 or row_bounds.shape[0] != num_ranks:
            raise ValueError("row_bounds must be a contiguous int32 tensor [num_ranks, chunks + 1]")
        num_chunks = row_bounds.shape[1] - 1
    for name, ten in (("topk_ids", topk_ids), ("local_row", local_row), ("delta", delta)):
        if ten.dtype != torch.int32 or not ten.is_contiguous():
            raise ValueError(f"{name} must be a contiguous int32 tensor")
    with torch.cuda.device(x.device):
        rc = _lib.load().b200moe_dispatch_quantize_peer_chunk(
            x.data_ptr(), topk_ids.data_ptr(), local_row.data_ptr(), delta.data_ptr(),
            None if topk_prob is None else topk_prob.data_ptr(), t, k, h, experts_per_rank, num_ranks, my_rank, slot_capacity,
            row_capacity, peer_q.data_ptr(), peer_rec.data_ptr(), None if row_bounds is None else row_bounds.data_ptr(), num_chunks, int(chunk),
            int(max_blocks), _stream_ptr(stream))  # fmt: skip
    _lib.check(rc)


def copy_segments(dst, src, nbytes, stream=None) -> None:
    """One asynchronous device-to-device copy per segment on ``stream`` (copy engines, no SM):
    ``dst`` / ``src`` are sequences of device addresses (peer-mapped ones included), ``nbytes`` their sizes."""
    import ctypes

    n = len(dst)
    if n == 0:
        return
    arr = ctypes.c_int64 * n
    rc = _lib.load().b200moe_copy_segments(n, arr(*[int(v) for v in dst]), arr(*[int(v) for v in src]), arr(*[int(v) for v in nbytes]),
                                           _stream_ptr(stream))  # fmt: skip
    _lib.check(rc)


def unpack_dispatch_records(rec: torch.Tensor, m_rows: int, cols: int, sfa: torch.Tensor, prob: torch.Tensor, row_map: torch.Tensor,
                            stream=None) -> None:  # fmt: skip
    """Records of the first ``m_rows`` received rows -> swizzled scale tensor, gate probabilities and
    FC2 return addresses (``b200moe_unpack_dispatch_records``)."""
    with torch.cuda.device(rec.device):
        rc = _lib.load().b200moe_unpack_dispatch_records(rec.data_ptr(), m_rows, cols, sfa.data_ptr(), prob.data_ptr(),
                                                         row_map.data_ptr(), _stream_ptr(stream))  # fmt: skip
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
