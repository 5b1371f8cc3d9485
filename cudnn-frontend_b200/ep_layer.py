"""Expert-parallel MoE layer: experts sharded over the ranks of a process group, tokens
dispatched and combined with all-to-all (NCCL over NVLink on GPUs).

    route -> sort rows by (destination rank, expert) -> exchange counts
    -> fused [read token row once, MXFP8 quantise, write to its k send positions]
    -> all-to-all dispatch of E4M3 rows + E8M0 scales + gate probabilities (half the bytes of bf16;
       row-wise quantisation commutes with the row permutation, so results equal quantising after)
    -> regroup by local expert (padded to 128) straight into the GEMM operand / swizzled scale layout
    -> FC1 (+SwiGLU, MXFP8 out) -> FC2 (x gating probability; its epilogue stores every row at its
       all-to-all arrival index) -> all-to-all combine -> un-permute and sum each token's k rows

The reference has no multi-GPU code at all; this is the layer its kernels are meant to sit in.
Expert ``e`` lives on rank ``e // (E / G)``.

Two parts:
* :func:`plan_dispatch` - pure integer index maths plus the tiny count exchange.  It only uses
  device-agnostic torch ops and ``torch.distributed``, so the same code runs on CUDA/NCCL and on
  CPU/Gloo ranks (the latter is how the multi-rank logic is tested without GPUs).
* :class:`ExpertParallelMoE` - holds this rank's expert weights and runs the CUDA path (row
  movement kernels, quantiser, grouped GEMMs).  CUDA only; there is no CPU implementation.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist


@dataclass
class DispatchPlan:
    num_tokens: int
    topk: int
    send_pos: torch.Tensor  # [R] int32: routed row r -> position in the send buffer
    in_splits: List[int]  # rows sent to each rank
    out_splits: List[int]  # rows received from each rank
    recv_dst: torch.Tensor  # [R_recv] int32: received row i -> row of the padded expert-grouped buffer
    row_map: torch.Tensor  # [m_rows] int32: row of the grouped buffer -> arrival index (-1 for padding rows)
    counts_local: torch.Tensor  # [E_local] int32 rows per local expert
    padded_offsets: torch.Tensor  # [E_local] int32 END offsets (groups padded to m_aligned)
    m_rows: int  # padded_offsets[-1]

    @property
    def rows_sent(self) -> int:
        return sum(self.in_splits)

    @property
    def rows_received(self) -> int:
        return sum(self.out_splits)


def _all_to_all_counts(counts_by_rank: torch.Tensor, group) -> torch.Tensor:
    """[G, E_local] rows I send to (rank, expert) -> [G, E_local] rows I receive from (rank, expert)."""
    if group is None or dist.get_world_size(group) == 1:
        return counts_by_rank.clone()
    recv = torch.empty_like(counts_by_rank)
    dist.all_to_all_single(recv, counts_by_rank.contiguous(), group=group)
    return recv


def plan_dispatch(topk_ids: torch.Tensor, num_experts: int, group=None, m_aligned: int = 128) -> DispatchPlan:
    """Index maths of one dispatch.  ``topk_ids [T, k]`` holds global expert ids.

    Send order = stable sort of the routed rows by expert id (experts are contiguous per rank, so
    this is also sorted by destination rank).  A receiver sees rows ordered by (source rank, local
    expert, original order) and regroups them by local expert with a second stable sort.  One host
    synchronisation reads the split sizes (needed by ``all_to_all_single``) and the padded row count.
    """
    world = 1 if group is None else dist.get_world_size(group)
    if num_experts % world != 0:
        raise ValueError(f"num_experts ({num_experts}) must be divisible by the group size ({world})")
    e_local = num_experts // world
    t, k = topk_ids.shape
    dev = topk_ids.device
    flat = topk_ids.reshape(-1).to(torch.int64)
    r = flat.numel()
    order = torch.argsort(flat, stable=True)
    send_pos = torch.empty(r, dtype=torch.int64, device=dev)
    send_pos[order] = torch.arange(r, device=dev)
    counts = torch.bincount(flat, minlength=num_experts).to(torch.int32).view(world, e_local)
    recv_counts = _all_to_all_counts(counts, group)  # [src rank, local expert]
    counts_local = recv_counts.sum(0)
    padded = ((counts_local + m_aligned - 1) // m_aligned) * m_aligned
    offsets = torch.cumsum(padded, 0)
    host = torch.cat([counts.sum(1), recv_counts.sum(1), offsets[-1:]]).cpu().tolist()  # the one sync
    in_splits, out_splits, m_rows = host[:world], host[world : 2 * world], int(host[-1])
    r_recv = sum(out_splits)
    # expert of every received row: rows arrive as (src, expert, j)
    expert_of_slot = torch.arange(e_local, device=dev).repeat(world)
    ids_recv = torch.repeat_interleave(expert_of_slot, recv_counts.reshape(-1).to(torch.int64), output_size=r_recv)
    order2 = torch.argsort(ids_recv, stable=True)
    first = torch.cumsum(counts_local.to(torch.int64), 0) - counts_local
    starts = (offsets - padded).to(torch.int64)
    sorted_ids = ids_recv[order2]
    rank_in_expert = torch.arange(r_recv, device=dev) - first[sorted_ids]
    recv_dst = torch.empty(r_recv, dtype=torch.int64, device=dev)
    recv_dst[order2] = starts[sorted_ids] + rank_in_expert
    row_map = torch.full((m_rows,), -1, dtype=torch.int32, device=dev)
    row_map[recv_dst] = torch.arange(r_recv, device=dev, dtype=torch.int32)
    return DispatchPlan(t, k, send_pos.to(torch.int32), in_splits, out_splits, recv_dst.to(torch.int32), row_map,
                        counts_local.to(torch.int32), offsets.to(torch.int32), m_rows)  # fmt: skip


@dataclass
class FusedPlan:
    """Index plan of the peer-memory path, identical inputs give identical plans on every rank."""

    delta: torch.Tensor  # [E] int32: destination row = delta[e] + compact local row of the routed slot
    padded_offsets: torch.Tensor  # [E_local] int32 END offsets of this rank's expert groups
    m_rows_all: torch.Tensor  # [G] int64 padded rows every rank will hold
    rows_all: torch.Tensor  # [G] int64 true rows every rank receives
    group_starts: Optional[torch.Tensor] = None  # [G, E_local] int64 first padded row of every expert group on its rank


def plan_fused(counts_all: torch.Tensor, rank: int, m_aligned: int = 128) -> FusedPlan:
    """``counts_all [G, E]``: rows source rank s routes to global expert e (the all-gathered
    per-rank histograms).  Expert e lives on rank ``e // (E / G)``; its group there holds the rows of
    source rank 0 first, then rank 1, ..., each in the sender's own (stable) order, and starts at the
    padded end of the previous local expert.  Pure integer torch ops: runs on any device."""
    g, e = counts_all.shape
    e_local = e // g
    c = counts_all.to(torch.int64)
    total = c.sum(0)  # rows of every expert over all sources
    padded = ((total + m_aligned - 1) // m_aligned) * m_aligned
    ends = torch.cumsum(padded.view(g, e_local), dim=1)  # END offsets on the owning rank
    group_start = (ends - padded.view(g, e_local)).reshape(e)
    before = torch.cumsum(c, dim=0) - c  # rows of earlier source ranks inside each group
    compact_start = torch.cumsum(c[rank], 0) - c[rank]  # this rank's route(m_aligned=1) starts
    delta = group_start + before[rank] - compact_start
    return FusedPlan(delta.to(torch.int32), ends[rank].to(torch.int32), ends[:, -1].contiguous(), total.view(g, e_local).sum(1),
                     group_start.view(g, e_local))


def chunk_weights(chunks: int):
    """Relative sizes of the chunks of the chunked peer path: equal, except that the last two are 0.6 and
    0.4 of a share, because the return of the last chunk's rows is the one transfer nothing hides."""
    if chunks < 3:
        return [10] * chunks
    return [10] * (chunks - 2) + [6, 4]


def chunk_row_bounds(rows_per_rank: torch.Tensor, weights) -> torch.Tensor:
    """Row ranges of the chunks of every rank: ``rows_per_rank [G]`` (padded rows, multiples of 128) ->
    int64 ``[G, C + 1]`` with ``bounds[r, c] = rows_r * sum(weights[:c]) // sum(weights)`` rounded down to a
    multiple of 128, ``bounds[r, 0] = 0`` and ``bounds[r, C] = rows_r``.  Chunks cut through expert groups:
    an expert that holds half of a rank's rows is spread over several chunks.  Integer arithmetic only, so
    every rank computes the same table from the all-gathered histogram on any device and the host can
    repeat it with the same numbers."""
    total = int(sum(weights))
    rows = rows_per_rank.to(torch.int64).view(-1, 1)
    cum = torch.tensor([0] + [int(v) for v in torch.tensor(list(weights)).cumsum(0).tolist()], dtype=torch.int64, device=rows.device).view(1, -1)
    bounds = ((rows * cum) // total) // 128 * 128
    bounds[:, -1] = rows.view(-1)
    return bounds


def chunk_offsets(padded_ends: torch.Tensor, bounds_row: torch.Tensor) -> torch.Tensor:
    """END offsets of one rank's expert groups restricted to each chunk's row range: ``padded_ends
    [E_local]``, ``bounds_row [C + 1]`` -> int32 ``[C, 1 + E_local]``; row c is ``[first row of chunk c,
    ends clamped to the chunk's range]``.  A GEMM launch for chunk c takes ``out[c, 1:]`` as its
    padded_offsets with the flag that the element before the view is the first row: experts before the
    chunk get no rows, the expert the chunk starts in begins at the chunk's first row."""
    lo = bounds_row[:-1].to(torch.int64).view(-1, 1)
    hi = bounds_row[1:].to(torch.int64).view(-1, 1)
    ends = torch.minimum(torch.maximum(padded_ends.to(torch.int64).view(1, -1), lo), hi)
    return torch.cat([lo, ends], dim=1).to(torch.int32).contiguous()


def return_segments(counts_host, padded_ends, rank: int, row_lo: int, row_hi: int):
    """Row blocks that rank ``rank`` returns for the rows ``row_lo .. row_hi - 1`` of its expert-grouped
    buffer.

    ``counts_host [G, E]`` (host integers): rows source rank s routes to physical expert e;
    ``padded_ends [E_local]``: END offsets of this rank's expert groups.  The group of local expert j holds
    the rows of source 0 first, then source 1, ...; source s keeps its result rows sorted by expert, expert
    e starting at the exclusive prefix of its own histogram.  Returns a list of
    ``(source rank, first row in the source's result buffer, first row here, rows)``, the sources rotated
    to start behind this rank so that the ranks do not all send to the same destination at once."""
    import numpy as np

    cnt = np.asarray(counts_host, dtype=np.int64)
    g, e = cnt.shape
    el = e // g
    ends = np.asarray(padded_ends, dtype=np.int64)
    starts = np.concatenate([[0], ends[:-1]])
    before = np.cumsum(cnt, axis=0) - cnt
    compact = np.cumsum(cnt, axis=1) - cnt
    # local experts whose groups touch the row range
    j_lo = int(np.searchsorted(ends, row_lo, "right"))
    j_hi = int(np.searchsorted(starts, row_hi, "left"))
    out = []
    for i in range(g):
        s_ = (rank + 1 + i) % g
        for j in range(j_lo, min(j_hi, el)):
            e_glob = rank * el + j
            a = int(starts[j]) + int(before[s_, e_glob])  # this source's rows of expert j: [a, b)
            b = a + int(cnt[s_, e_glob])
            a2, b2 = max(a, row_lo), min(b, row_hi)
            if b2 > a2:
                out.append((s_, int(compact[s_, e_glob]) + (a2 - a), a2, b2 - a2))
    return out


def balanced_placement(rows_per_expert, num_ranks: int):
    """Placement of E experts on G ranks, E / G per rank, that evens out the rows per rank: experts in
    order of decreasing load, each onto the least-loaded rank that still has a free slot (ties: lower
    rank).  ``rows_per_expert``: E numbers (e.g. routed rows per expert summed over ranks and over some
    steps).  Returns ``slot_of_expert`` (list of E ints): expert e lives in physical slot p, i.e. on rank
    ``p // (E / G)`` as its local expert ``p % (E / G)``.  Deterministic: every rank computes the same."""
    loads = [float(v) for v in rows_per_expert]
    e = len(loads)
    if e % num_ranks != 0:
        raise ValueError(f"{e} experts cannot be split evenly over {num_ranks} ranks")
    per = e // num_ranks
    rank_load = [0.0] * num_ranks
    rank_used = [0] * num_ranks
    slot = [0] * e
    for ex in sorted(range(e), key=lambda i: (-loads[i], i)):
        r = min((r for r in range(num_ranks) if rank_used[r] < per), key=lambda r: (rank_load[r], r))
        slot[ex] = r * per + rank_used[r]
        rank_used[r] += 1
        rank_load[r] += loads[ex]
    return slot


def exchange_rows(send: torch.Tensor, out_rows: int, in_splits, out_splits, group) -> torch.Tensor:
    """All-to-all of whole rows (first dimension split)."""
    if group is None or dist.get_world_size(group) == 1:
        return send
    recv = torch.empty((out_rows,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send, output_split_sizes=list(out_splits), input_split_sizes=list(in_splits), group=group)
    return recv


def exchange_rows_async(send: torch.Tensor, out_rows: int, in_splits, out_splits, group):
    """As :func:`exchange_rows`, but returns ``(recv, work)`` without making the caller's stream wait:
    the exchange runs on the process group's own stream (it starts once the kernels already queued on
    the caller's stream have produced ``send``) and ``work.wait()`` later orders the caller's stream
    behind it.  ``work`` is None for a single rank."""
    if group is None or dist.get_world_size(group) == 1:
        return send, None
    recv = torch.empty((out_rows,) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    work = dist.all_to_all_single(recv, send, output_split_sizes=list(out_splits), input_split_sizes=list(in_splits), group=group,
                                  async_op=True)  # fmt: skip
    return recv, work


class ExpertParallelMoE:
    """One MoE layer with this rank's ``E / G`` experts resident in HBM as MXFP8.

    ``w1 (2I, H, E_local)`` is the FC1 weight in the 32-row interleaved gate/up order, ``w2 (H, I,
    E_local)`` the FC2 weight, both float8_e4m3fn K-major with E8M0 scales in the 128x4 layout
    (as produced by ``synthetic.make_weights`` or by quantising real weights with
    ``quantize_mxfp8``)."""

    def __init__(self, w1, sfw1, w2, sfw2, num_experts: int, group=None, m_aligned: int = 128, overlap_sm_margin: int = 16):
        if not w1.is_cuda:
            raise RuntimeError("ExpertParallelMoE runs on CUDA devices only")
        from . import grouped_gemm_quant, grouped_gemm_swiglu  # noqa: F401  (fails loudly without the CUDA library)

        self.w1, self.sfw1, self.w2, self.sfw2 = w1, sfw1, w2, sfw2
        self.num_experts = num_experts
        self.group = group
        self.world = 1 if group is None else dist.get_world_size(group)
        self.e_local = num_experts // self.world
        self.m_aligned = m_aligned
        self.hidden = w1.shape[1]
        self.inter = w2.shape[1]
        assert w1.shape[0] == 2 * self.inter and w2.shape[0] == self.hidden and w1.shape[2] == self.e_local
        dev = w1.device
        self.alpha = torch.ones(self.e_local, dtype=torch.float32, device=dev)
        self.norm = torch.ones(1, dtype=torch.float32, device=dev)
        self._ops = {}
        # logical expert id -> physical slot (rank = slot // e_local); None = identity (contiguous sharding)
        self.slot_of_expert: Optional[torch.Tensor] = None
        self._slot_host: Optional[List[int]] = None
        self.last_plan: Optional[DispatchPlan] = None
        self.last_rows_received = 0
        # SMs the GEMMs leave to the all-to-all kernels that run beside them in the pipelined path
        self.overlap_sm_margin = overlap_sm_margin if self.world > 1 else 0
        # chunked peer path: SMs the GEMMs leave to the quantise-and-dispatch launch (and the barrier
        # kernels) that run beside them, and the persistent blocks of that launch
        import os

        self.chunk_sm_margin = int(os.environ.get("B200MOE_EP_SM_MARGIN", "8")) if self.world > 1 else 0
        self.dispatch_blocks = int(os.environ.get("B200MOE_EP_DISPATCH_BLOCKS", "256"))

    def _fc_ops(self, m_rows: int, bufs, sm_margin: int = 0):
        """Operator objects are cached per padded row count (shapes are part of their samples)."""
        from .grouped_gemm_quant import GroupedGemmQuantSm100
        from .grouped_gemm_swiglu import GroupedGemmSwigluSm100

        key = (m_rows, sm_margin)
        if key not in self._ops:
            a, sfa, h8, sfh, y, prob, offs = bufs
            y = torch.empty((m_rows, self.hidden, 1), dtype=torch.bfloat16, device="meta")  # shape sample only
            fc1 = GroupedGemmSwigluSm100(a, self.w1, None, h8, sfa, self.sfw1, offs, self.alpha, h8, sample_sfd_row=sfh,
                                         sample_sfd_col=_dummy_sf_col(self.inter, m_rows, a.device), sample_norm_const=self.norm,
                                         sf_vec_size=32, m_aligned=self.m_aligned)  # fmt: skip
            fc2 = GroupedGemmQuantSm100(h8, sfh, offs, self.alpha, y, sample_b=self.w2, sample_sfb=self.sfw2, sample_prob=prob,
                                        sf_vec_size=32, m_aligned=self.m_aligned)  # fmt: skip
            assert fc1.check_support() and fc2.check_support()
            fc1.compile()
            fc2.compile()
            fc1.num_cluster_overlap_margin = fc2.num_cluster_overlap_margin = sm_margin
            self._ops[key] = (fc1, fc2)
        return self._ops[key]

    def _experts(self, plan: DispatchPlan, recv_q, recv_sf, recv_p, sm_margin: int = 0) -> torch.Tensor:
        """Received rows -> regroup by local expert -> FC1 -> FC2 -> result rows in arrival order."""
        from . import moe, ops

        h, dev, m = self.hidden, recv_q.device, plan.m_rows
        y_recv = torch.empty((plan.rows_received, h), dtype=torch.bfloat16, device=dev)
        if m > 0:
            a, sfa, prob3 = moe.place_quantized_rows(recv_q, recv_sf, recv_p, plan.recv_dst, m, plan.counts_local, plan.padded_offsets)
            h8 = torch.empty((m, self.inter, 1), dtype=torch.float8_e4m3fn, device=dev)
            sfh = ops.empty_sf(m, self.inter, 1, device=dev)
            fc1, fc2 = self._fc_ops(m, (a, sfa, h8, sfh, y_recv.view(-1, h, 1), prob3, plan.padded_offsets), sm_margin)
            fc1.execute(a, self.w1, None, h8, sfa, self.sfw1, plan.padded_offsets, self.alpha, sfd_row_tensor=sfh, norm_const_tensor=self.norm)
            fc2.execute(h8, sfh, plan.padded_offsets, self.alpha, y_recv.view(-1, h, 1), b_tensor=self.w2, sfb_tensor=self.sfw2,
                        prob_tensor=prob3, d_row_map=plan.row_map)  # fmt: skip
        return y_recv

    # ------------------------------------------------------------------------------------------
    # expert placement
    # ------------------------------------------------------------------------------------------
    def _physical_ids(self, topk_ids: torch.Tensor) -> torch.Tensor:
        """Logical expert ids of the router -> physical slots of the current placement."""
        if self.slot_of_expert is None:
            return topk_ids
        return self.slot_of_expert[topk_ids.long()]

    def rebalance(self, rows_per_expert: torch.Tensor) -> List[int]:
        """Re-shard the experts so that every rank gets about the same number of rows, and move the
        weights accordingly (collective: every rank calls it with the same ``rows_per_expert [E]``, e.g.
        the routing histogram summed over ranks and over a few steps).  Afterwards ``forward*`` maps the
        router's expert ids to the new slots; results do not change, only which rank computes them.
        Returns the new ``slot_of_expert`` list."""
        loads = rows_per_expert.detach().to("cpu", torch.float64).tolist()
        new = balanced_placement(loads, self.world)
        old = self._slot_host if self._slot_host is not None else list(range(self.num_experts))
        if new != old:
            self._move_weights(old, new)
        self._slot_host = new
        self.slot_of_expert = torch.tensor(new, dtype=torch.int32, device=self.w1.device)
        return new

    def _move_weights(self, old: List[int], new: List[int]) -> None:
        """Weights of logical expert e move from slot old[e] to slot new[e].  One all-to-all per weight
        tensor over whole experts; both sides order the experts they exchange by destination slot."""
        el, g = self.e_local, self.world
        rank = 0 if self.group is None else dist.get_rank(self.group)
        # experts I hold now, by destination rank then destination slot; experts I will hold, by source
        # rank then destination slot: the same order on the sending and the receiving side
        mine = [e for e in range(self.num_experts) if old[e] // el == rank]
        send = sorted(mine, key=lambda e: (new[e] // el, new[e]))
        recv = sorted((e for e in range(self.num_experts) if new[e] // el == rank), key=lambda e: (old[e] // el, new[e]))
        in_splits = [sum(1 for e in send if new[e] // el == d) for d in range(g)]
        out_splits = [sum(1 for e in recv if old[e] // el == s_) for s_ in range(g)]
        send_idx = torch.tensor([old[e] % el for e in send], dtype=torch.int64, device=self.w1.device)
        recv_idx = torch.tensor([new[e] % el for e in recv], dtype=torch.int64, device=self.w1.device)

        def move(per_expert: torch.Tensor) -> torch.Tensor:
            """``per_expert [E_local, bytes]`` uint8 -> the same shape in the new placement."""
            staged = per_expert.index_select(0, send_idx)
            if g > 1:
                got = torch.empty_like(staged)
                dist.all_to_all_single(got, staged, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)
            else:
                got = staged
            out = torch.empty_like(per_expert)
            out.index_copy_(0, recv_idx, got)
            return out

        def flat_sf(sf: torch.Tensor) -> torch.Tensor:
            t = sf.view(torch.uint8)
            return torch.as_strided(t, (t.numel(),), (1,)).view(el, -1)

        from . import ops

        n1, k1 = self.w1.shape[0], self.w1.shape[1]
        n2, k2 = self.w2.shape[0], self.w2.shape[1]
        w1 = move(self.w1.permute(2, 0, 1).contiguous().view(torch.uint8).view(el, -1)).view(torch.float8_e4m3fn).view(el, n1, k1)
        w2 = move(self.w2.permute(2, 0, 1).contiguous().view(torch.uint8).view(el, -1)).view(torch.float8_e4m3fn).view(el, n2, k2)
        sf1 = move(flat_sf(self.sfw1).contiguous())
        sf2 = move(flat_sf(self.sfw2).contiguous())
        self.w1, self.w2 = w1.permute(1, 2, 0), w2.permute(1, 2, 0)
        shape, stride = ops.sf_shape_stride(n1, k1, el)
        self.sfw1 = torch.as_strided(sf1.view(-1).view(torch.float8_e8m0fnu), shape, stride)
        shape, stride = ops.sf_shape_stride(n2, k2, el)
        self.sfw2 = torch.as_strided(sf2.view(-1).view(torch.float8_e8m0fnu), shape, stride)
        self._ops = {}  # operator objects hold samples of the old weight tensors

    # ------------------------------------------------------------------------------------------
    # peer-memory path: no all-to-all of rows at all
    # ------------------------------------------------------------------------------------------
    def _peer_setup(self, tokens: int, topk: int, capacity_factor: float):
        """Peer-addressable buffers, allocated once per (tokens, topk): the expert-grouped GEMM operand
        of this rank (E4M3 rows, swizzled scales, gate probabilities, return addresses) that every
        rank's dispatch kernel stores into, and the [T * k, H] result buffer that every rank's FC2
        epilogue stores into."""
        from .peer_memory import PeerBuffer

        # One set of buffers per (tokens, topk).  A step that needed more rows than the caller's factor
        # gives has grown them; later calls with the smaller factor keep the grown buffers instead of
        # shrinking and growing again on every step.
        key = (tokens, topk)
        slots = tokens * topk
        # rows this rank may receive: its fair share times the factor, plus the padding of every group
        cap = int(slots * capacity_factor) + self.e_local * self.m_aligned
        cap = ((cap + 127) // 128) * 128
        if getattr(self, "_peer_key", None) == key and self._peer["cap"] >= cap:
            return self._peer
        if getattr(self, "_peer", None) is not None:
            self.release_peer_buffers()
        h = self.hidden
        rest_k = (h // 32 + 3) // 4
        from . import moe

        pitch = moe.dispatch_record_pitch(h)
        bufs = {
            "q": PeerBuffer(cap * h, self.group),  # E4M3 rows of this rank's expert groups
            "rec": PeerBuffer(cap * pitch, self.group),  # per row: scales, gate probability, return address
            "back": PeerBuffer(slots * h * 2, self.group),  # result rows, slot order
        }
        dev = self.w1.device
        local = {
            "sf": torch.empty((cap // 128) * rest_k * 512, dtype=torch.uint8, device=dev),
            "prob": torch.empty(cap, dtype=torch.float32, device=dev),
            "map": torch.empty(cap, dtype=torch.int32, device=dev),
        }
        self._peer = dict(bufs=bufs, local=local, cap=cap, slots=slots, pitch=pitch, identity=torch.arange(slots, dtype=torch.int32, device=self.w1.device))
        self._peer_key = key
        return self._peer

    def release_peer_buffers(self) -> None:
        """Unmap and free the peer buffers (every rank, after the last step; ends with a barrier)."""
        peer = getattr(self, "_peer", None)
        if peer is None:
            return
        # Three phases, the ranks in step: (1) nobody still computes on or stores into a buffer; (2) every
        # rank unmaps its views of the others' buffers; (3) only then does an owner free its allocation
        # (freeing memory that another process still has mapped is undefined).
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        for b in peer["bufs"].values():
            b.unmap_peers()
        if self.world > 1:
            dist.barrier(group=self.group)
        for b in peer["bufs"].values():
            b.free_own()
        self._peer, self._peer_key = None, None

    def _rank_barrier(self):
        """Orders the ranks on the device: kernels queued after it start only when every rank has
        finished the kernels it queued before it (a one-element all-reduce on the compute stream;
        the host does not wait)."""
        if self.world > 1:
            dist.all_reduce(self._token, group=self.group)

    def default_chunks(self) -> int:
        """Chunks :meth:`forward_fused` uses when none are given (0 = the direct form)."""
        import os

        if self.world <= 1:
            return 0
        return int(os.environ.get("B200MOE_EP_CHUNKS", "0" if self.world <= 2 else "8"))

    def forward_fused(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_prob: torch.Tensor, capacity_factor: float = 2.0,
                      chunks: Optional[int] = None) -> torch.Tensor:
        """The peer-memory path.  On one rank: :meth:`forward_fused_direct`.  On several ranks:
        :meth:`forward_fused_chunked`, which overlaps the NVLink traffic with the GEMMs (``chunks``
        expert chunks; ``chunks=0`` selects the direct form on any number of ranks).  Default, unless the
        environment variable ``B200MOE_EP_CHUNKS`` says otherwise: the direct form on two ranks (half of the
        rows stay local and FC2's peer stores hide behind its MMAs: 26.9 ms against 27.7 ms with 5 chunks), 8
        chunks on more (4 GPUs: 29.5 / 30.2 / 28.9 / 31.0 ms per step with 3 / 5 / 8 / 12 chunks, 30.4 direct;
        8 GPUs: 33.0 against 36.7)."""
        if chunks is None:
            chunks = self.default_chunks()
        if chunks <= 0:
            return self.forward_fused_direct(x, topk_ids, topk_prob, capacity_factor)
        return self.forward_fused_chunked(x, topk_ids, topk_prob, capacity_factor, chunks)

    def forward_fused_direct(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_prob: torch.Tensor, capacity_factor: float = 2.0) -> torch.Tensor:
        """Same result as :meth:`forward`, without any all-to-all of rows: the dispatch kernel stores
        quantised rows straight into the owning rank's GEMM operand over NVLink, and the FC2 epilogue
        stores result rows straight into the source rank's result buffer.

            histogram of my slots -> all-gather of the histograms (G x E ints) -> plan (same on every rank)
            -> [quantise + dispatch + regroup] one kernel, peer stores -> barrier
            -> FC1 -> FC2 (epilogue: peer stores to the slot the row came from) -> barrier -> top-k sum

        One host synchronisation reads every rank's padded row count.  ``capacity_factor`` sizes the
        buffers (rows a rank may receive, times its fair share); when a step needs more, all ranks
        reallocate larger ones together."""
        from . import moe, ops

        if not x.is_cuda:
            raise RuntimeError("ExpertParallelMoE.forward_fused needs CUDA tensors")
        t, k = topk_ids.shape
        h, dev, g = self.hidden, x.device, self.world
        rank = 0 if self.group is None else dist.get_rank(self.group)
        if not hasattr(self, "_token"):
            self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        peer = self._peer_setup(t, k, capacity_factor)
        bufs, cap, slots = peer["bufs"], peer["cap"], peer["slots"]

        ids = self._physical_ids(topk_ids).contiguous()
        counts, _, local_row = moe.route(ids.view(-1), self.num_experts, 1)
        bufs["rec"].local.fill_(0xFF)  # a record nobody writes reads as "padding row, returns nowhere"
        if g > 1:
            counts_all = torch.empty((g, self.num_experts), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(counts_all, counts, group=self.group)
        else:
            counts_all = counts.view(1, -1)
        plan = plan_fused(counts_all, rank, self.m_aligned)
        host = torch.cat([plan.m_rows_all, plan.rows_all]).cpu().tolist()  # the one host synchronisation
        m_all = host[:g]
        m = int(m_all[rank])
        self.last_rows_received = int(host[g + rank])
        if max(m_all) > cap:
            # every rank sees the same row counts, so every rank takes this branch together: new, larger
            # buffers, their maps reset, and a barrier so that no rank stores before every reset is done
            if max(m_all) > 64 * slots:
                raise RuntimeError(f"a rank would receive {max(m_all)} padded rows from {slots} slots per rank")
            peer = self._peer_setup(t, k, 1.25 * max(m_all) / slots)
            bufs, cap = peer["bufs"], peer["cap"]
            bufs["rec"].local.fill_(0xFF)
            self._rank_barrier()
        # (otherwise the all-gather above already ordered this step's stores behind every rank's map reset)
        moe.dispatch_quantize_peer(x, ids, local_row, plan.delta, topk_prob.reshape(t * k).contiguous(), self.e_local, g, rank,
                                   slots, cap, bufs["q"].ptrs_dev, bufs["rec"].ptrs_dev)  # fmt: skip
        self._rank_barrier()
        if m > 0:
            loc = peer["local"]
            moe.unpack_dispatch_records(bufs["rec"].local, m, h, loc["sf"], loc["prob"], loc["map"])
            a = torch.as_strided(bufs["q"].view(torch.float8_e4m3fn, (m, h)), (m, h, 1), (h, 1, m * h))
            shape, stride = ops.sf_shape_stride(m, h, 1)
            sfa = torch.as_strided(loc["sf"].view(torch.float8_e8m0fnu), shape, stride)
            prob3 = loc["prob"][:m].view(m, 1, 1)
            row_map = loc["map"][:m]
            back_local = bufs["back"].view(torch.bfloat16, (slots, h))
            h8 = torch.empty((m, self.inter, 1), dtype=torch.float8_e4m3fn, device=dev)
            sfh = ops.empty_sf(m, self.inter, 1, device=dev)
            fc1, fc2 = self._fc_ops(m, (a, sfa, h8, sfh, None, prob3, plan.padded_offsets))
            fc1.execute(a, self.w1, None, h8, sfa, self.sfw1, plan.padded_offsets, self.alpha, sfd_row_tensor=sfh, norm_const_tensor=self.norm)
            fc2.execute(h8, sfh, plan.padded_offsets, self.alpha, back_local.view(slots, h, 1),
                        b_tensor=self.w2, sfb_tensor=self.sfw2, prob_tensor=prob3, d_row_map=row_map,
                        d_peer_ptrs=bufs["back"].ptrs_dev, d_peer_slots=slots)  # fmt: skip
        self._rank_barrier()
        return moe.combine_rows(bufs["back"].view(torch.bfloat16, (slots, h)), peer["identity"], t, k)

    # ------------------------------------------------------------------------------------------
    # peer-memory path in expert chunks: transfers run beside the GEMMs
    # ------------------------------------------------------------------------------------------
    def _side_streams(self):
        if getattr(self, "_streams", None) is None:
            self._streams = dict(disp=torch.cuda.Stream(), copy=[torch.cuda.Stream(), torch.cuda.Stream()])
        return self._streams

    def forward_fused_chunked(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_prob: torch.Tensor, capacity_factor: float = 2.0,
                              chunks: int = 4) -> torch.Tensor:
        """Same result as :meth:`forward_fused_direct`, with the local experts run in ``chunks`` slices so
        that the result rows return over NVLink while later slices still compute:

            plan (as forward_fused_direct: histogram all-gather, one host synchronisation)
            chunks = row ranges of this rank's expert-grouped buffer (they cut through large expert groups)
            quantise + dispatch of every row over NVLink (one kernel, all SMs) -> barrier
            for every chunk c:   FC1(c), FC2(c) on the compute stream (FC2 stores bf16 rows locally, in
                                 expert-grouped order: full-speed stores, no row map)
                                 | return of chunk c - 1 by the copy engines: every (expert, source rank)
                                 |   block of result rows is one contiguous device-to-device copy into the
                                 |   source rank's result buffer, which holds its rows in its own
                                 |   expert-sorted order
            barrier -> top-k sum (each token gathers its k rows through its sorted positions)

        Only the dispatch and the return of the last chunk are exposed; the copy engines cost the GEMMs
        nothing.  With ``B200MOE_EP_OVERLAP_DISPATCH=1`` only chunk 0 is dispatched ahead and the dispatch
        of chunk c + 1 runs on a side stream beside the GEMMs of chunk c, with ``chunk_sm_margin`` SMs left
        to it and a barrier after it (measured slower: the comment at the switch below).  All tables of
        the copies come from the all-gathered histogram, which the host reads in the plan's one
        synchronisation."""
        import numpy as np

        from . import moe, ops

        if not x.is_cuda:
            raise RuntimeError("ExpertParallelMoE.forward_fused_chunked needs CUDA tensors")
        t, k = topk_ids.shape
        h, dev, g, el = self.hidden, x.device, self.world, self.e_local
        rank = 0 if self.group is None else dist.get_rank(self.group)
        if not hasattr(self, "_token"):
            self._token = torch.zeros(1, dtype=torch.float32, device=dev)
        peer = self._peer_setup(t, k, capacity_factor)
        bufs, cap, slots = peer["bufs"], peer["cap"], peer["slots"]
        main = torch.cuda.current_stream()
        streams = self._side_streams()
        # step breakdown: when ``self.step_events`` is a list, a timing event is recorded on the caller's
        # stream at every phase boundary and appended as (label, event)
        rec = getattr(self, "step_events", None)

        def mark(label):
            if rec is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(main)
                rec.append((label, ev))

        mark("start")
        ids = self._physical_ids(topk_ids).contiguous()
        counts, _, local_row = moe.route(ids.view(-1), self.num_experts, 1)
        bufs["rec"].local.fill_(0xFF)  # a record nobody writes reads as "padding row"
        if g > 1:
            counts_all = torch.empty((g, self.num_experts), dtype=torch.int32, device=dev)
            dist.all_gather_into_tensor(counts_all, counts, group=self.group)
        else:
            counts_all = counts.view(1, -1)
        plan = plan_fused(counts_all, rank, self.m_aligned)
        host = torch.cat([plan.m_rows_all, plan.rows_all, plan.padded_offsets.to(torch.int64), counts_all.reshape(-1).to(torch.int64)]).cpu().numpy()
        m_all = host[:g]
        m = int(m_all[rank])
        self.last_rows_received = int(host[g + rank])
        ends = host[2 * g : 2 * g + el]  # padded END offsets of my expert groups
        cnt = host[2 * g + el :].reshape(g, self.num_experts)  # rows source s routes to (physical) expert e
        if int(m_all.max()) > cap:
            if int(m_all.max()) > 64 * slots:
                raise RuntimeError(f"a rank would receive {int(m_all.max())} padded rows from {slots} slots per rank")
            peer = self._peer_setup(t, k, 1.25 * float(m_all.max()) / slots)
            bufs, cap = peer["bufs"], peer["cap"]
            bufs["rec"].local.fill_(0xFF)
            self._rank_barrier()
        ev_plan = torch.cuda.Event()
        ev_plan.record(main)
        mark("route + plan (one host synchronisation)")

        # chunks = row ranges of about equal size on every rank: a table on the device for the dispatch
        # kernel (it covers every rank), the same numbers on the host for this rank's launches and copies,
        # and per chunk the expert END offsets clamped to the chunk's rows for the GEMM launches
        chunks = max(1, int(chunks))
        weights = chunk_weights(chunks)
        bounds_dev = chunk_row_bounds(plan.m_rows_all, weights)
        bounds_i32 = bounds_dev.to(torch.int32).contiguous()
        offs_c = chunk_offsets(plan.padded_offsets, bounds_dev[rank])
        cum = np.concatenate([[0], np.cumsum(weights)])
        row_bounds = [int(v) for v in ((m * cum) // int(sum(weights))) // 128 * 128]
        row_bounds[-1] = m
        flat_prob = topk_prob.reshape(t * k).contiguous()

        def dispatch(c, max_blocks):
            moe.dispatch_quantize_peer(x, ids, local_row, plan.delta, flat_prob, el, g, rank, slots, cap, bufs["q"].ptrs_dev,
                                       bufs["rec"].ptrs_dev, row_bounds=bounds_i32, chunk=c, max_blocks=max_blocks)  # fmt: skip

        # The quantise + dispatch kernel beside a GEMM shares the GEMM's SMs (its small blocks fit next to a GEMM
        # CTA) and slows FC1 and FC2 by more than it takes alone (one GPU, 5 chunks: FC1 13.4 -> 16.6 ms, FC2
        # 7.2 -> 9.7 ms for a kernel of 2.3 ms), while the copy engines' result copies cost the GEMMs nothing.  So
        # by default every row is dispatched before the first chunk and only the return runs beside the GEMMs
        # (4 GPUs: 27.8 against 29.7 ms per step, 8 GPUs: 30.7 against 34.4 ms);
        # ``B200MOE_EP_OVERLAP_DISPATCH=1`` selects the chunk-by-chunk dispatch on the side stream instead.
        import os

        overlap_dispatch = os.environ.get("B200MOE_EP_OVERLAP_DISPATCH", "0") == "1"

        row_bytes = h * 2
        back_ptrs = bufs["back"].ptrs

        loc = peer["local"]
        rest_k = (h // 32 + 3) // 4
        pitch = peer["pitch"]
        y = h8 = sfh = None
        if m > 0:
            a = torch.as_strided(bufs["q"].view(torch.float8_e4m3fn, (m, h)), (m, h, 1), (h, 1, m * h))
            shape, stride = ops.sf_shape_stride(m, h, 1)
            sfa = torch.as_strided(loc["sf"].view(torch.float8_e8m0fnu), shape, stride)
            prob3 = loc["prob"][:m].view(m, 1, 1)
            h8 = torch.empty((m, self.inter, 1), dtype=torch.float8_e4m3fn, device=dev)
            sfh = ops.empty_sf(m, self.inter, 1, device=dev)
            y = torch.empty((m, h, 1), dtype=torch.bfloat16, device=dev)
            fc1, fc2 = self._fc_ops(m, (a, sfa, h8, sfh, None, prob3, plan.padded_offsets), self.chunk_sm_margin if overlap_dispatch else 0)

        if overlap_dispatch:
            dispatch(0, 0)
        else:
            moe.dispatch_quantize_peer(x, ids, local_row, plan.delta, flat_prob, el, g, rank, slots, cap, bufs["q"].ptrs_dev, bufs["rec"].ptrs_dev)
        self._rank_barrier()
        mark("dispatch of chunk 0 + barrier" if overlap_dispatch else "dispatch of all rows + barrier")
        ev_disp = [None] * chunks
        ev_fc2 = [None] * chunks
        for c in range(chunks):
            if c > 0 and overlap_dispatch:
                main.wait_event(ev_disp[c])
                mark(f"wait for the dispatch of chunk {c}")
            r0, r1 = row_bounds[c], row_bounds[c + 1]
            offs = offs_c[c, 1:]  # the element before this view is the chunk's first row
            if r1 > r0:
                moe.unpack_dispatch_records(bufs["rec"].local[r0 * pitch :], r1 - r0, h, loc["sf"][(r0 // 128) * rest_k * 512 :], loc["prob"][r0:],
                                            loc["map"][r0:])  # fmt: skip
                fc1.execute(a, self.w1, None, h8, sfa, self.sfw1, offs, self.alpha, sfd_row_tensor=sfh, norm_const_tensor=self.norm,
                            offsets_have_prev=True)  # fmt: skip
            mark(f"unpack + FC1 of chunk {c}")
            if c + 1 < chunks and overlap_dispatch:
                # the next chunk's rows travel while this chunk computes
                with torch.cuda.stream(streams["disp"]):
                    if c == 0:
                        streams["disp"].wait_event(ev_plan)
                    dispatch(c + 1, self.dispatch_blocks)
                    self._rank_barrier()
                    ev_disp[c + 1] = torch.cuda.Event()
                    ev_disp[c + 1].record(streams["disp"])
            if r1 > r0:
                fc2.execute(h8, sfh, offs, self.alpha, y, b_tensor=self.w2, sfb_tensor=self.sfw2, prob_tensor=prob3, offsets_have_prev=True)
            ev_fc2[c] = torch.cuda.Event()
            ev_fc2[c].record(main)
            mark(f"FC2 of chunk {c}")
            # return of this chunk's result rows: one copy per (expert, source rank) block inside the chunk,
            # destinations rotated so that the ranks do not all send to the same one at the same time
            if y is not None and r1 > r0:
                y_ptr = y.data_ptr()
                seg = [[], []]
                for s_, dst_row, src_row, n_rows in return_segments(cnt, ends, rank, r0, r1):
                    seg[s_ % 2].append((back_ptrs[s_] + dst_row * row_bytes, y_ptr + src_row * row_bytes, n_rows * row_bytes))
                for cs, lane_ in zip(streams["copy"], seg):
                    if lane_:
                        cs.wait_event(ev_fc2[c])
                        moe.copy_segments([v[0] for v in lane_], [v[1] for v in lane_], [v[2] for v in lane_], stream=cs)
        for cs in streams["copy"]:
            main.wait_stream(cs)
        main.wait_stream(streams["disp"])
        self._rank_barrier()  # every rank's copies into my result buffer are complete
        mark("last result copies + barrier")
        out = moe.combine_rows(bufs["back"].view(torch.bfloat16, (slots, h)), local_row, t, k)
        mark("top-k sum")
        return out

    def forward_pipelined(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_prob: torch.Tensor, micro_batches: int = 4) -> torch.Tensor:
        """Same result as :meth:`forward`, computed as ``micro_batches`` slices of the tokens in a
        software pipeline: while the GEMMs of slice i run on the caller's stream, the dispatch
        all-to-all of slice i + 1 and the combine all-to-all of slice i - 1 run on the process group's
        stream.  All index plans (and their host synchronisations) come first, so no host wait sits
        between the stages.  Exchanges are issued in the same order on every rank:
        d0, d1, c0, d2, c1, ... ; the GEMMs leave ``overlap_sm_margin`` SMs to the exchange kernels.
        Every token's result depends on its own row only, so slicing changes nothing numerically."""
        from . import moe

        if not x.is_cuda:
            raise RuntimeError("ExpertParallelMoE.forward needs CUDA tensors")
        topk_ids = self._physical_ids(topk_ids)
        t, k = topk_ids.shape
        n = max(1, min(micro_batches, t))
        bounds = [(i * t // n, (i + 1) * t // n) for i in range(n)]
        plans = [plan_dispatch(topk_ids[lo:hi], self.num_experts, self.group, self.m_aligned) for lo, hi in bounds]
        self.last_plan = plans[-1]
        self.last_rows_received = sum(p.rows_received for p in plans)
        flat_prob = topk_prob.reshape(t * k).contiguous()
        sends = [moe.dispatch_quantize(x[lo:hi], p.send_pos, k, flat_prob[lo * k : hi * k]) for (lo, hi), p in zip(bounds, plans)]

        def start_dispatch(i):
            p = plans[i]
            return [exchange_rows_async(buf, p.rows_received, p.in_splits, p.out_splits, self.group) for buf in sends[i]]

        out = torch.empty((t, self.hidden), dtype=torch.bfloat16, device=x.device)
        inflight = start_dispatch(0)
        backs = []
        for i in range(n):
            nxt = start_dispatch(i + 1) if i + 1 < n else None
            for _, work in inflight:
                if work is not None:
                    work.wait()
            y_recv = self._experts(plans[i], *(buf for buf, _ in inflight), sm_margin=self.overlap_sm_margin)
            backs.append(exchange_rows_async(y_recv, plans[i].rows_sent, plans[i].out_splits, plans[i].in_splits, self.group))
            inflight = nxt
        for (lo, hi), p, (back, work) in zip(bounds, plans, backs):
            if work is not None:
                work.wait()
            moe.combine_rows(back, p.send_pos, hi - lo, k, out=out[lo:hi])
        return out

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_prob: torch.Tensor) -> torch.Tensor:
        """``x [T, H]`` bf16, ``topk_ids [T, k]`` int32 global expert ids, ``topk_prob [T, k]`` f32
        -> ``[T, H]`` bf16 = sum over the token's k experts of prob * FC2(SwiGLU(FC1(x)))."""
        from . import moe, ops

        if not x.is_cuda:
            raise RuntimeError("ExpertParallelMoE.forward needs CUDA tensors")
        topk_ids = self._physical_ids(topk_ids)
        t, k = topk_ids.shape
        h = self.hidden
        dev = x.device
        plan = plan_dispatch(topk_ids, self.num_experts, self.group, self.m_aligned)
        self.last_plan = plan
        self.last_rows_received = plan.rows_received
        # dispatch: each token row is read once, quantised, and written to its k send positions
        # (E4M3 + row-major scales + gate probability travel together: half the bytes of bf16)
        send_q, send_sf, send_p = moe.dispatch_quantize(x, plan.send_pos, k, topk_prob.reshape(-1).contiguous())
        recv_q = exchange_rows(send_q, plan.rows_received, plan.in_splits, plan.out_splits, self.group)
        recv_sf = exchange_rows(send_sf, plan.rows_received, plan.in_splits, plan.out_splits, self.group)
        recv_p = exchange_rows(send_p, plan.rows_received, plan.in_splits, plan.out_splits, self.group)
        m = plan.m_rows
        y_recv = torch.empty((plan.rows_received, h), dtype=torch.bfloat16, device=dev)
        if m > 0:
            # regroup by local expert straight into the GEMM operand layout (scales swizzled here)
            a, sfa, prob3 = moe.place_quantized_rows(recv_q, recv_sf, recv_p, plan.recv_dst, m, plan.counts_local, plan.padded_offsets)
            h8 = torch.empty((m, self.inter, 1), dtype=torch.float8_e4m3fn, device=dev)
            sfh = ops.empty_sf(m, self.inter, 1, device=dev)
            fc1, fc2 = self._fc_ops(m, (a, sfa, h8, sfh, y_recv.view(-1, h, 1), prob3, plan.padded_offsets))
            fc1.execute(a, self.w1, None, h8, sfa, self.sfw1, plan.padded_offsets, self.alpha, sfd_row_tensor=sfh, norm_const_tensor=self.norm)
            # FC2 stores every result row at its arrival index: y_recv is already in all-to-all order
            fc2.execute(h8, sfh, plan.padded_offsets, self.alpha, y_recv.view(-1, h, 1), b_tensor=self.w2, sfb_tensor=self.sfw2,
                        prob_tensor=prob3, d_row_map=plan.row_map)  # fmt: skip
        back = exchange_rows(y_recv, plan.rows_sent, plan.out_splits, plan.in_splits, self.group)
        return moe.combine_rows(back, plan.send_pos, t, k)

    __call__ = forward


def _dummy_sf_col(n_out: int, m_rows: int, device):
    """Column scale factors are not produced inside the layer, but the operator's validation
    wants a sample of the right shape; a meta tensor costs no memory."""
    from . import ops

    shape, stride = ops.sf_shape_stride(n_out, m_rows, 1)
    return torch.empty_strided(shape, stride, dtype=torch.float8_e8m0fnu, device="meta")
