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


def _peer_worker(rank, world, port, ret):
    """The peer-memory path's index logic on CPU ranks: peer stores are emulated by exchanging
    (destination rank, row, payload) lists; everything else is the code the CUDA path runs."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cudnn_frontend_b200.ep_layer import plan_fused
        from oracle import mxfp8_oracle as orc

        experts, t, k, h, m_aligned = 8, 40 + 9 * rank, 2, 8, 16
        e_local = experts // world
        g = torch.Generator().manual_seed(11 + rank)
        ids = torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(t)]).to(torch.int32)
        ids[ids == 5] = 6  # an expert nobody uses
        x = torch.randn(t, h, generator=g)
        p = torch.rand(t, k, generator=g)
        slots = 64 * k  # slot capacity, the same on every rank
        counts = torch.bincount(ids.reshape(-1).long(), minlength=experts).to(torch.int32)
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts)
        plan = plan_fused(torch.stack(gathered), rank, m_aligned)
        # compact local rows = stable grouping of my slots by expert (what b200moe_route(m_aligned=1) returns)
        _, _, local_row = orc.route_rows(ids.reshape(-1).numpy(), experts, 1)
        # "peer stores": (destination rank, destination row, payload row, prob, return address)
        msgs = []
        for slot in range(t * k):
            e = int(ids.reshape(-1)[slot])
            msgs.append((e // e_local, int(plan.delta[e]) + int(local_row[slot]), x[slot // k].clone(), float(p.reshape(-1)[slot]),
                         rank * slots + slot, e))
        everyone = [None] * world
        dist.all_gather_object(everyone, msgs)
        m = int(plan.m_rows_all[rank])
        assert m == int(plan.padded_offsets[-1]) and m % m_aligned == 0
        xg, pg = torch.zeros(m, h), torch.zeros(m)
        row_map = torch.full((m,), -1, dtype=torch.int64)
        expert_of_row = torch.full((m,), -1, dtype=torch.int64)
        for src in everyone:
            for d, row, payload, prob, ret_addr, e in src:
                if d != rank:
                    continue
                assert 0 <= row < m and row_map[row] == -1  # inside my buffer, written once
                xg[row], pg[row], row_map[row], expert_of_row[row] = payload, prob, ret_addr, e
        assert int((row_map >= 0).sum()) == int(plan.rows_all[rank])
        start = 0
        for el in range(e_local):  # every group holds its expert's rows first, then padding
            end = int(plan.padded_offsets[el])
            inside = expert_of_row[start:end]
            cnt = int((inside >= 0).sum())
            assert (inside[:cnt] == rank * e_local + el).all() and (inside[cnt:] == -1).all()
            start = end
        # stand-in expert, then "peer stores" of the result rows to (source rank, slot)
        yg = xg * (expert_of_row.clamp(min=0).float()[:, None] + 1) * pg[:, None]
        returns = [(int(a) // slots, int(a) % slots, yg[r].clone()) for r, a in enumerate(row_map.tolist()) if a >= 0]
        everyone = [None] * world
        dist.all_gather_object(everyone, returns)
        back = torch.zeros(slots, h)
        for src in everyone:
            for d, slot, row in src:
                if d == rank:
                    back[slot] = row
        out = back[: t * k].view(t, k, h).sum(1)
        ref = (x[:, None, :] * (ids.float()[:, :, None] + 1) * p[:, :, None]).sum(1)
        ret[rank] = bool(torch.allclose(out, ref, rtol=1e-5, atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_peer_memory_plan_round_trip_world_size_2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_peer_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def _move_worker(rank, world, port, ret):
    """Weight movement of ExpertParallelMoE.rebalance on CPU ranks: every expert's weight bytes carry
    its logical id, so after the move each slot can be checked against the new placement."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cudnn_frontend_b200 import ops
        from cudnn_frontend_b200.ep_layer import ExpertParallelMoE, balanced_placement

        experts, el = 8, 8 // world
        n1, k1, n2, k2 = 256, 128, 128, 128
        layer = object.__new__(ExpertParallelMoE)  # the constructor wants CUDA tensors; only the movement is under test
        layer.group, layer.world, layer.e_local, layer.num_experts = dist.group.WORLD, world, el, experts
        layer._ops = {}

        def weights(n, k, tag):
            w = torch.empty((el, n, k), dtype=torch.uint8)
            sf_shape, sf_stride = ops.sf_shape_stride(n, k, el)
            per = (n // 128) * ((k // 32 + 3) // 4) * 512
            sf = torch.empty(el * per, dtype=torch.uint8)
            for i in range(el):
                w[i] = rank * el + i + tag
                sf[i * per : (i + 1) * per] = 100 + rank * el + i + tag
            return w.view(torch.float8_e4m3fn).permute(1, 2, 0), torch.as_strided(sf.view(torch.float8_e8m0fnu), sf_shape, sf_stride), per

        layer.w1, layer.sfw1, per1 = weights(n1, k1, 0)
        layer.w2, layer.sfw2, per2 = weights(n2, k2, 50)
        old = list(range(experts))
        new = balanced_placement([5, 1, 9, 2, 7, 3, 8, 4], world)
        layer._move_weights(old, new)
        ok = True
        for e in range(experts):
            if new[e] // el != rank:
                continue
            slot = new[e] % el
            ok &= bool((layer.w1.permute(2, 0, 1)[slot].view(torch.uint8) == e).all())
            ok &= bool((layer.w2.permute(2, 0, 1)[slot].view(torch.uint8) == e + 50).all())
            f1 = torch.as_strided(layer.sfw1.view(torch.uint8), (layer.sfw1.numel(),), (1,)).view(el, per1)
            f2 = torch.as_strided(layer.sfw2.view(torch.uint8), (layer.sfw2.numel(),), (1,)).view(el, per2)
            ok &= bool((f1[slot] == 100 + e).all()) and bool((f2[slot] == 150 + e).all())
        # and back again
        layer._move_weights(new, old)
        for i in range(el):
            ok &= bool((layer.w1.permute(2, 0, 1)[i].view(torch.uint8) == rank * el + i).all())
        ret[rank] = ok
    finally:
        dist.destroy_process_group()


def test_rebalance_moves_every_expert_to_its_new_slot_world_size_2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_move_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_return_segments_put_every_row_where_its_source_expects_it():
    """The chunked peer path returns result rows as contiguous blocks, one per (expert, source rank) and
    chunk.  Emulated on the host for 4 ranks: every rank labels the rows of its expert groups with (source,
    expert, index), applies its segments to the sources' result buffers chunk by chunk (row ranges that cut
    through expert groups), and every source must find its rows in its own expert-sorted order."""
    from cudnn_frontend_b200.ep_layer import chunk_row_bounds, chunk_weights, return_segments

    g, e, m_aligned = 4, 12, 128
    el = e // g
    rng = np.random.default_rng(3)
    cnt = rng.integers(0, 400, (g, e))
    cnt[:, 5] = 0  # an expert nobody routes to
    cnt[2, :] = 0  # a rank without tokens
    cnt[0, 1] = 3000  # one expert holds most rows of its rank: chunks must cut through it
    total = cnt.sum(0)
    padded = (total + m_aligned - 1) // m_aligned * m_aligned
    back = [np.full((int(cnt[s].sum()), 3), -1, dtype=np.int64) for s in range(g)]
    rows_per_rank = torch.tensor([int(padded[r * el : (r + 1) * el].sum()) for r in range(g)])
    bounds = chunk_row_bounds(rows_per_rank, chunk_weights(5)).numpy()
    for rank in range(g):
        ends = np.cumsum(padded[rank * el : (rank + 1) * el])
        starts = np.concatenate([[0], ends[:-1]])
        y = np.full((int(ends[-1]), 3), -1, dtype=np.int64)
        for j_ in range(el):
            eg = rank * el + j_
            row = int(starts[j_])
            for s in range(g):
                for i_ in range(int(cnt[s, eg])):
                    y[row] = (s, eg, i_)
                    row += 1
        b = bounds[rank]
        assert b[0] == 0 and b[-1] == ends[-1] and (np.diff(b) >= 0).all() and (b % 128 == 0).all()
        written = 0
        for c in range(len(b) - 1):
            for s, dst_row, src_row, rows in return_segments(cnt, ends, rank, int(b[c]), int(b[c + 1])):
                assert b[c] <= src_row and src_row + rows <= b[c + 1]
                assert (back[s][dst_row : dst_row + rows] == -1).all()  # nothing is written twice
                back[s][dst_row : dst_row + rows] = y[src_row : src_row + rows]
                written += rows
        assert written == int(total[rank * el : (rank + 1) * el].sum())
    for s in range(g):
        expect = [(s, eg, i_) for eg in range(e) for i_ in range(int(cnt[s, eg]))]
        assert back[s].tolist() == [list(v) for v in expect]


def _teardown_worker(rank, world, port, log):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import time

        from cudnn_frontend_b200 import _lib, ep_layer, peer_memory

        class FakeLib:
            def b200moe_peer_close(self, p):
                log.append((rank, "unmap", int(p)))
                return 0

            def b200moe_peer_free(self, p):
                log.append((rank, "free", int(p)))
                return 0

        _lib.load = lambda: FakeLib()
        bufs = {}
        for name in ("q", "rec", "back"):
            b = peer_memory.PeerBuffer.__new__(peer_memory.PeerBuffer)
            b.group, b.world, b.rank, b.device = dist.group.WORLD, world, rank, torch.device("cpu")
            b._own, b._opened, b.local = 1000 + rank, [2000 + r for r in range(world) if r != rank], None
            bufs[name] = b
        layer = ep_layer.ExpertParallelMoE.__new__(ep_layer.ExpertParallelMoE)
        layer.world, layer.group = world, dist.group.WORLD
        layer._peer, layer._peer_key = dict(bufs=bufs), ("x",)
        ep_layer.torch.cuda.synchronize = lambda *a, **k: None  # CPU ranks
        if rank == 1:
            time.sleep(0.3)  # a slow rank: the others must not free before it has unmapped
        layer.release_peer_buffers()
        assert layer._peer is None
    finally:
        dist.destroy_process_group()


def test_peer_buffers_are_freed_only_after_every_rank_unmapped_them():
    """Teardown order of the peer buffers on 2 CPU ranks with a stand-in library that logs the calls: every
    'free' comes after every rank's 'unmap' (freeing memory another process still maps is undefined)."""
    mgr = mp.Manager()
    log = mgr.list()
    mp.spawn(_teardown_worker, args=(2, _free_port(), log), nprocs=2, join=True)
    events = list(log)
    assert sum(1 for e in events if e[1] == "unmap") == 2 * 3 and sum(1 for e in events if e[1] == "free") == 2 * 3
    last_unmap = max(i for i, e in enumerate(events) if e[1] == "unmap")
    first_free = min(i for i, e in enumerate(events) if e[1] == "free")
    assert last_unmap < first_free, events


def test_chunk_offsets_restrict_every_expert_group_to_the_chunk():
    """Per chunk, the expert END offsets clamped to the chunk's row range (what a GEMM launch of the chunk
    gets): over all chunks every row of every group is covered exactly once, and the host's restatement of
    the bounds agrees with the device table."""
    from cudnn_frontend_b200.ep_layer import chunk_offsets, chunk_row_bounds, chunk_weights

    gen = torch.Generator().manual_seed(1)
    padded = torch.randint(0, 6, (3, 10), generator=gen) * 128
    padded[1, 2] = 128 * 40  # a group larger than any chunk
    padded[2] = 0
    ends = torch.cumsum(padded, 1)
    rows = ends[:, -1]
    for chunks in (1, 2, 5, 7):
        w = chunk_weights(chunks)
        bounds = chunk_row_bounds(rows, w)
        for r in range(3):
            m = int(rows[r])
            cum = np.concatenate([[0], np.cumsum(w)])
            host = ((m * cum) // int(sum(w))) // 128 * 128
            host[-1] = m
            assert bounds[r].tolist() == host.tolist()
            offs = chunk_offsets(ends[r], bounds[r]).numpy()
            assert offs.shape == (chunks, 11)
            covered = np.zeros(m, dtype=np.int64)
            starts_full = np.concatenate([[0], ends[r].numpy()[:-1]])
            for c in range(chunks):
                assert offs[c, 0] == bounds[r, c] and (np.diff(offs[c]) >= 0).all() and offs[c, -1] <= bounds[r, c + 1]
                for j_ in range(10):
                    lo, hi = int(offs[c, j_]), int(offs[c, j_ + 1])
                    if hi > lo:
                        assert lo >= starts_full[j_] and hi <= int(ends[r, j_])  # rows of group j only
                        covered[lo:hi] += 1
            assert (covered == 1).all()


def test_default_form_of_the_peer_path_by_world_size(monkeypatch):
    """One rank and two ranks take the direct form (no chunks), more ranks take eight chunks; the environment
    variable overrides the choice on several ranks and never on one."""
    from types import SimpleNamespace

    from cudnn_frontend_b200.ep_layer import ExpertParallelMoE

    monkeypatch.delenv("B200MOE_EP_CHUNKS", raising=False)
    picks = {w: ExpertParallelMoE.default_chunks(SimpleNamespace(world=w)) for w in (1, 2, 4, 8)}
    assert picks == {1: 0, 2: 0, 4: 8, 8: 8}
    monkeypatch.setenv("B200MOE_EP_CHUNKS", "3")
    assert ExpertParallelMoE.default_chunks(SimpleNamespace(world=2)) == 3
    assert ExpertParallelMoE.default_chunks(SimpleNamespace(world=8)) == 3
    assert ExpertParallelMoE.default_chunks(SimpleNamespace(world=1)) == 0
