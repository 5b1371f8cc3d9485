"""World-size-2 checks of the expert-parallel dispatch plan on CPU ranks (Gloo): the index maths
and the sequence of collectives, with a stand-in expert function instead of the CUDA GEMMs."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cudnn_frontend_b200.ep_layer import exchange_rows, plan_dispatch

        experts, t, k, h = 8, 50 + 13 * rank, 2, 16
        g = torch.Generator().manual_seed(5 + rank)
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(t)]).to(torch.int32)
        ids[ids == 3] = 4  # expert 3 never used: an empty local group on rank 0
        x = torch.randn(t, h, generator=g)
        p = torch.rand(t, k, generator=g)
        plan = plan_dispatch(ids, experts, dist.group.WORLD, m_aligned=128)
        e_local = experts // world
        # --- dispatch with plain indexing (stand-in for the CUDA row kernels)
        send = torch.empty(t * k, h)
        send[plan.send_pos.long()] = x.repeat_interleave(k, 0)
        send_e = torch.empty(t * k, dtype=torch.int64)
        send_e[plan.send_pos.long()] = ids.reshape(-1).long()
        send_p = torch.empty(t * k)
        send_p[plan.send_pos.long()] = p.reshape(-1)
        assert torch.equal(send_e, torch.sort(send_e).values)  # send buffer sorted by expert = by rank
        recv = exchange_rows(send, plan.rows_received, plan.in_splits, plan.out_splits, dist.group.WORLD)
        recv_e = exchange_rows(send_e, plan.rows_received, plan.in_splits, plan.out_splits, dist.group.WORLD)
        recv_p = exchange_rows(send_p, plan.rows_received, plan.in_splits, plan.out_splits, dist.group.WORLD)
        assert ((recv_e // e_local) == rank).all()  # only my experts arrive
        # --- regroup by local expert, padded
        m = plan.m_rows
        assert m % 128 == 0 and m == int(plan.padded_offsets[-1])
        grouped_e = torch.full((m,), -1, dtype=torch.int64)
        grouped_e[plan.recv_dst.long()] = recv_e - rank * e_local
        xg = torch.zeros(m, h)
        xg[plan.recv_dst.long()] = recv
        pg = torch.zeros(m)
        pg[plan.recv_dst.long()] = recv_p
        start = 0
        for e in range(e_local):
            end = int(plan.padded_offsets[e])
            cnt = int(plan.counts_local[e])
            assert (end - start) % 128 == 0 and cnt <= end - start
            assert (grouped_e[start : start + cnt] == e).all() and (grouped_e[start + cnt : end] == -1).all()
            start = end
        assert len(torch.unique(plan.recv_dst)) == plan.rows_received
        # --- stand-in expert: y = x * (global expert + 1) * prob
        ge = torch.where(grouped_e >= 0, grouped_e + rank * e_local + 1, torch.zeros_like(grouped_e)).float()
        yg = xg * ge[:, None] * pg[:, None]
        y_recv = yg[plan.recv_dst.long()]
        back = exchange_rows(y_recv, plan.rows_sent, plan.out_splits, plan.in_splits, dist.group.WORLD)
        out = back[plan.send_pos.long()].view(t, k, h).sum(1)
        ref = (x[:, None, :] * (ids.float()[:, :, None] + 1) * p[:, :, None]).sum(1)
        ok = torch.allclose(out, ref, rtol=1e-5, atol=1e-5)
        # rows sent by everyone == rows received by everyone
        tot = torch.tensor([plan.rows_sent, plan.rows_received])
        dist.all_reduce(tot)
        ret[rank] = bool(ok) and int(tot[0]) == int(tot[1])
    finally:
        dist.destroy_process_group()


def test_dispatch_plan_round_trip_world_size_2():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_dispatch_plan_single_rank_matches_oracle_routing():
    from cudnn_frontend_b200.ep_layer import plan_dispatch
    from oracle import mxfp8_oracle as orc

    r = np.random.default_rng(0)
    ids = r.integers(0, 16, (200, 4)).astype(np.int32)
    plan = plan_dispatch(torch.from_numpy(ids), 16, None, 128)
    counts, offs, dst = orc.route_rows(ids.reshape(-1), 16, 128)
    np.testing.assert_array_equal(plan.counts_local.numpy(), counts)
    np.testing.assert_array_equal(plan.padded_offsets.numpy(), offs)
    # single rank: send order then regroup == direct stable grouping
    composed = plan.recv_dst[plan.send_pos.long()].numpy()
    np.testing.assert_array_equal(composed, dst)
    assert plan.in_splits == [800] and plan.out_splits == [800] and plan.m_rows == int(offs[-1])


def test_plan_rejects_indivisible_expert_count():
    from cudnn_frontend_b200.ep_layer import plan_dispatch

    class FakeGroup:
        pass

    with pytest.raises(ValueError):
        # 7 experts cannot be sharded over 2 ranks; checked before any collective
        import unittest.mock as mock

        with mock.patch("torch.distributed.get_world_size", return_value=2):
            plan_dispatch(torch.zeros((4, 1), dtype=torch.int32), 7, FakeGroup(), 128)
