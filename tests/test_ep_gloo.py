"""Expert-parallel host logic (dispatch plan, count exchange, all-to-all, un-permute, reduce) on
CPU: two gloo ranks with a stand-in for the expert kernels.  No GPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ane_fieldfare_b200.parallel import (ExpertParallelMoE, balanced_placement, contiguous_placement,
                                         dispatch_plan)

E, K, D, T_PER_RANK = 8, 3, 16, 11


def test_dispatch_plan_orders_routes_by_destination_keeping_token_order():
    ids = torch.tensor([[5, 0, 7], [1, 6, 2], [4, 3, 0]], dtype=torch.int32)
    plan = dispatch_plan(ids, experts_per_rank=4, world=2)
    # rank 0 owns experts 0..3, rank 1 owns 4..7; routes are (token*K + rank)
    assert plan.send_counts.tolist() == [5, 4]
    assert plan.order.tolist() == [1, 3, 5, 7, 8, 0, 2, 4, 6]
    assert plan.local_expert.tolist() == [0, 1, 2, 3, 0, 1, 3, 2, 0]
    assert plan.token.tolist() == [0, 1, 1, 2, 2, 0, 0, 1, 2]
    empty = dispatch_plan(torch.zeros((0, 3), dtype=torch.int32), 4, 2)
    assert empty.send_counts.tolist() == [0, 0] and empty.order.numel() == 0
    with pytest.raises(ValueError, match="out of range"):
        dispatch_plan(torch.tensor([[9, 1, 2]], dtype=torch.int32), 4, 2)


def test_balanced_placement_evens_out_a_skewed_prior():
    load = [1.0 / (r + 1) ** 1.1 for r in range(16)]  # Zipf over experts 0..15
    naive = contiguous_placement(16, 4)
    smart = balanced_placement(load, 4)
    def rank_loads(p):
        return [sum(load[e] for e in p.experts_of(r)) for r in range(4)]
    assert all(len(smart.experts_of(r)) == 4 for r in range(4))
    assert sorted(e for r in range(4) for e in smart.experts_of(r)) == list(range(16))
    assert max(rank_loads(smart)) < 0.6 * max(rank_loads(naive))
    # local ids follow the order in which a rank loads its blobs
    for r in range(4):
        assert [int(smart.local_of[e]) for e in smart.experts_of(r)] == [0, 1, 2, 3]
    ids = torch.tensor([[0, 5, 9]], dtype=torch.int32)
    plan = dispatch_plan(ids, 4, 4, smart)
    assert sorted(plan.order.tolist()) == [0, 1, 2]
    for pos, route in enumerate(plan.order.tolist()):
        e = int(ids.reshape(-1)[route])
        assert int(plan.local_expert[pos]) == int(smart.local_of[e])


def _tokens(rank):
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn((T_PER_RANK, D), generator=g)
    ids = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T_PER_RANK)]).to(torch.int32)
    if rank == 1:
        ids[:4] = torch.tensor([4, 5, 6], dtype=torch.int32)  # skew: these rows stay on rank 1
    w = torch.rand((T_PER_RANK, K), generator=g)
    return x, ids, w


def _expected(rank):
    x, ids, w = _tokens(rank)
    y = 0.5 * x
    for t in range(T_PER_RANK):
        for k in range(K):
            y[t] += w[t, k] * (float(ids[t, k]) + 1.0) * x[t]
    return y


def _worker(rank, world, port, results, chunks=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, ids, w = _tokens(rank)
        epr = E // world

        def experts_fn(rows, local):
            glob = local.to(torch.float32) + float(rank * epr) + 1.0
            return rows * glob[:, None]

        def reduce_fn(partials, weights, residual):
            p = partials.reshape(T_PER_RANK, K, D)
            return residual + (weights[:, :, None] * p).sum(dim=1)

        layer = ExpertParallelMoE(E, K, lambda v: (ids, w), lambda v: 0.5 * v, experts_fn, reduce_fn,
                                  chunks=chunks)
        layer.count_experts = True
        y = layer.forward(x)
        assert int(layer.last_expert_counts.sum()) == T_PER_RANK * K
        # every route arrives somewhere: received rows over the ranks == routes over the ranks
        total = torch.tensor([layer.last_recv_rows], dtype=torch.int64)
        dist.all_reduce(total)
        results[rank] = (torch.allclose(y, _expected(rank), rtol=1e-5, atol=1e-5), int(total.item()),
                         layer.last_recv_rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_expert_parallel_layer_two_gloo_ranks(chunks):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results, chunks), nprocs=2, join=True)
    assert results[0][0] and results[1][0]
    assert results[0][1] == 2 * T_PER_RANK * K
    assert results[0][2] != results[1][2]  # the skewed routing loads the ranks unevenly
