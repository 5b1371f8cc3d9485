"""Expert-parallel MoE layer on GPUs: one rank against the layer oracle, and (when the box has
two GPUs) two NCCL ranks against the single-rank result."""

import os
import socket

import numpy as np
import pytest
import torch

from oracle import mxfp8_oracle as orc
from tests import helpers as H

pytestmark = pytest.mark.gpu

T, HID, INTER, E, K = 384, 256, 128, 8, 2


def _inputs(seed, device):
    from cudnn_frontend_b200 import synthetic

    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(T, HID, generator=g, device=device).to(torch.bfloat16)
    ids = torch.multinomial(torch.ones(T, E, device=device), K, generator=g).to(torch.int32)
    prob = torch.softmax(torch.randn(T, K, generator=g, device=device), -1)
    w1, sfw1 = synthetic.make_weights(E, 2 * INTER, HID, seed + 1, device, std=0.05)
    w2, sfw2 = synthetic.make_weights(E, HID, INTER, seed + 2, device, std=0.05)
    return x, ids, prob, w1, sfw1, w2, sfw2


def test_single_rank_layer_matches_oracle():
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    x, ids, prob, w1, sfw1, w2, sfw2 = _inputs(3, "cuda")
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    torch.cuda.synchronize()
    ref = orc.moe_layer_reference(
        x.float().cpu().numpy(), ids.cpu().numpy(), prob.cpu().numpy(),
        w1.permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(), H.sf_to_numpy(sfw1, 2 * INTER, HID // 32, E),
        w2.permute(2, 0, 1).contiguous().view(torch.uint8).cpu().numpy(), H.sf_to_numpy(sfw2, HID, INTER // 32, E), 128,
    )  # fmt: skip
    assert H.rel_fro(y.float().cpu().numpy(), ref) <= 2e-2


@pytest.mark.parametrize("micro_batches", [1, 3, 4])
def test_pipelined_layer_equals_the_plain_layer(micro_batches):
    """Slicing the tokens into micro-batches changes nothing: every token's result depends on its own row."""
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    x, ids, prob, w1, sfw1, w2, sfw2 = _inputs(4, "cuda")
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    yp = layer.forward_pipelined(x, ids, prob, micro_batches=micro_batches)
    torch.cuda.synchronize()
    assert torch.equal(y, yp)
    assert layer.last_rows_received == T * K


def test_peer_memory_layer_equals_the_plain_layer():
    """One rank: the fused quantise + dispatch kernel and the FC2 epilogue address this rank's own
    buffers through the same pointer tables the multi-rank path uses."""
    from cudnn_frontend_b200 import ops
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    x, ids, prob, w1, sfw1, w2, sfw2 = _inputs(5, "cuda")
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    yf = layer.forward_fused(x, ids, prob)
    yf2 = layer.forward_fused(x, ids, prob)  # buffers are reused from step to step
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    assert torch.equal(y, yf) and torch.equal(y, yf2)
    layer.release_peer_buffers()


@pytest.mark.parametrize("overlap_dispatch", ["0", "1"])
@pytest.mark.parametrize("chunks", [1, 3, 8])
def test_chunked_peer_path_equals_the_plain_layer(chunks, overlap_dispatch, monkeypatch):
    """The chunked form of the peer path (experts in slices, result rows returned by device-to-device copies
    in the sources' sorted order; every row dispatched ahead of the first slice, or the next slice's rows
    dispatched on a side stream) on one rank: the same bytes as the plain layer, step after step."""
    from cudnn_frontend_b200 import ops
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    monkeypatch.setenv("B200MOE_EP_OVERLAP_DISPATCH", overlap_dispatch)
    x, ids, prob, w1, sfw1, w2, sfw2 = _inputs(7, "cuda")
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    yc = layer.forward_fused(x, ids, prob, chunks=chunks)
    x2, ids2, prob2, *_ = _inputs(8, "cuda")
    y2 = layer(x2, ids2, prob2)
    yc2 = layer.forward_fused(x2, ids2, prob2, chunks=chunks)  # buffers and streams are reused
    torch.cuda.synchronize()
    assert ops.device_status(clear=True) == 0
    assert torch.equal(y, yc) and torch.equal(y2, yc2)
    layer.release_peer_buffers()


def test_peer_buffers_grow_when_a_step_needs_more_rows():
    """A capacity factor far too small for the step: the layer reallocates larger peer buffers (all
    ranks together in the multi-rank case) and still returns the plain layer's result."""
    from cudnn_frontend_b200 import ops, synthetic
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    t = 2048
    g = torch.Generator(device="cuda").manual_seed(21)
    x = torch.randn(t, HID, generator=g, device="cuda").to(torch.bfloat16)
    ids = torch.multinomial(torch.ones(t, E, device="cuda"), K, generator=g).to(torch.int32)
    prob = torch.softmax(torch.randn(t, K, generator=g, device="cuda"), -1)
    w1, sfw1 = synthetic.make_weights(E, 2 * INTER, HID, 31, "cuda", std=0.05)
    w2, sfw2 = synthetic.make_weights(E, HID, INTER, 32, "cuda", std=0.05)
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    yf = layer.forward_fused(x, ids, prob, capacity_factor=0.1)
    torch.cuda.synchronize()
    assert layer._peer["cap"] >= layer.last_plan.m_rows if layer.last_plan is not None else True
    assert ops.device_status(clear=True) == 0
    assert torch.equal(y, yf)
    layer.release_peer_buffers()


def test_rebalanced_layer_computes_the_same_function():
    """Moving experts to other slots (here within one rank) changes where rows are computed, not what."""
    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    x, ids, prob, w1, sfw1, w2, sfw2 = _inputs(6, "cuda")
    layer = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
    y = layer(x, ids, prob)
    counts = torch.bincount(ids.reshape(-1).long(), minlength=E)
    counts[3] += 1000  # make the order of the placement differ from the identity
    slot = layer.rebalance(counts)
    assert sorted(slot) == list(range(E)) and slot != list(range(E))
    y2 = layer(x, ids, prob)
    y3 = layer.forward_fused(x, ids, prob)
    torch.cuda.synchronize()
    assert torch.equal(y, y2) and torch.equal(y, y3)
    layer.release_peer_buffers()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

        # every rank builds the same global weights, keeps its shard; tokens differ per rank
        _, _, _, w1, sfw1, w2, sfw2 = _inputs(3, dev)
        x, ids, prob, *_ = _inputs(10 + rank, dev)
        e_local = E // world
        sl = slice(rank * e_local, (rank + 1) * e_local)
        sf1 = torch.as_strided(sfw1.view(torch.uint8), (sfw1.numel(),), (1,)).view(E, -1)[sl].contiguous()
        sf2 = torch.as_strided(sfw2.view(torch.uint8), (sfw2.numel(),), (1,)).view(E, -1)[sl].contiguous()
        from cudnn_frontend_b200 import ops

        def as_sf(flat, mn, kk):
            shape, stride = ops.sf_shape_stride(mn, kk, e_local)
            return torch.as_strided(flat.view(-1).view(torch.float8_e8m0fnu), shape, stride)

        w1l = w1.permute(2, 0, 1)[sl].contiguous().permute(1, 2, 0)
        w2l = w2.permute(2, 0, 1)[sl].contiguous().permute(1, 2, 0)
        layer = ExpertParallelMoE(w1l, as_sf(sf1, 2 * INTER, HID), w2l, as_sf(sf2, HID, INTER), E, dist.group.WORLD)
        y = layer(x, ids, prob)
        # same tokens through a single-rank layer that owns all experts
        full = ExpertParallelMoE(w1, sfw1, w2, sfw2, E)
        y1 = full(x, ids, prob)
        yp = layer.forward_pipelined(x, ids, prob, micro_batches=3)
        yf = layer.forward_fused(x, ids, prob, chunks=0)  # rows cross NVLink by peer stores, no all-to-all
        yf2 = layer.forward_fused(x, ids, prob)  # the default form for this number of ranks
        yc2 = layer.forward_fused(x, ids, prob, chunks=2)
        os.environ["B200MOE_EP_OVERLAP_DISPATCH"] = "1"  # the next slice's rows dispatched beside the GEMMs
        yc3 = layer.forward_fused(x, ids, prob, chunks=3)
        os.environ["B200MOE_EP_OVERLAP_DISPATCH"] = "0"
        # re-shard by load (weights cross ranks) and run again: same function
        counts = torch.bincount(ids.reshape(-1).long(), minlength=E).float()
        dist.all_reduce(counts)
        counts[1] += 500
        layer.rebalance(counts)
        yr = layer.forward_fused(x, ids, prob)
        yr2 = layer(x, ids, prob)
        torch.cuda.synchronize()
        from cudnn_frontend_b200 import ops as _ops

        status = _ops.device_status(clear=True)
        layer.release_peer_buffers()
        # row order inside an expert group differs between the runs, the per-row maths does not
        ret[rank] = bool(torch.equal(y, y1)) and bool(torch.equal(yp, y1)) and bool(torch.equal(yf, y1)) and bool(torch.equal(yf2, y1)) and bool(torch.equal(yc2, y1)) and bool(torch.equal(yc3, y1)) and bool(torch.equal(yr, y1)) and bool(torch.equal(yr2, y1)) and status == 0
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_equal_single_rank():
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ep_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert all(ret.get(r) for r in range(2)), dict(ret)
