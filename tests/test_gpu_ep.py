"""Expert parallelism on real GPUs: two NCCL ranks, experts split over them (contiguous blocks, and
a load-balanced placement with the tokens cut into chunks whose exchanges overlap the GEMMs, and
the same placement with the rows moved by peer stores into symmetric memory, per route and once
per token and destination),
compared bit for bit with the single-GPU layer on the same tokens.  Needs two GPUs; skipped
otherwise."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SHAPE = dict(experts=16, d=128, f=64, sharedF=192, topK=8)
TOKENS = 40


def _worker(rank, world, port, results):
    import torch.distributed as dist
    from ane_fieldfare_b200 import hotpath, parallel, workload
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        L = workload.make_layer(0xE9, 0, router_bias="zipf", **SHAPE)
        epr = SHAPE["experts"] // world
        full = hotpath.HotpathContext(layers=1, maxTokens=TOKENS, device=rank, **SHAPE)
        workload.load_layer(full, 0, L)
        home = hotpath.HotpathContext(layers=1, maxTokens=TOKENS, device=rank, **SHAPE)
        home.loadShared(0, *L.shared_projections())
        home.loadRouter(0, L.routerW, logitBias=L.logitBias)
        local = hotpath.HotpathContext(layers=2, experts=epr, d=SHAPE["d"], f=SHAPE["f"], sharedF=0, topK=1,
                                       maxTokens=TOKENS * SHAPE["topK"] * world, device=rank)
        local.loadLayer(0, L.blobs[rank * epr:(rank + 1) * epr], L.layout.stride, L.layout.offsets,
                        expertCount=epr)
        x = hotpath.bf16_tensor(workload.make_tokens(0xE9 + rank, "ep.x", TOKENS, SHAPE["d"]), full.device)
        block = parallel.ExpertParallelMoE(SHAPE["experts"], SHAPE["topK"],
                                           *parallel.cuda_layer_fns(home, local, 0))
        y = block.forward(x)
        want = full.moeLayer(0, x)
        torch.cuda.synchronize()
        same = bool(torch.equal(y, want))
        rows = int(block.last_recv_rows)
        # a placement that balances a skewed load (experts interleaved over the ranks), the tokens in
        # three chunks: the same bits
        load = [1.0 / (e + 1) ** 1.1 for e in range(SHAPE["experts"])]
        placement = parallel.balanced_placement(load, world)
        local.loadLayer(1, np.ascontiguousarray(L.blobs[placement.experts_of(rank)]), L.layout.stride,
                        L.layout.offsets, expertCount=epr)
        balanced = parallel.ExpertParallelMoE(SHAPE["experts"], SHAPE["topK"],
                                              *parallel.cuda_layer_fns(home, local, 0, expert_layer=1),
                                              placement=placement, chunks=3,
                                              route_sorter=parallel.cuda_route_sorter(home))
        y2 = balanced.forward(x)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(y2, want))
        # rows moved by peer stores into symmetric memory instead of the collective: the same bits,
        # twice over the same buffers (the second pass checks the reuse barriers)
        buffers = parallel.PeerBuffers(TOKENS * SHAPE["topK"] * world, SHAPE["d"], torch.bfloat16, full.device)
        peer = parallel.ExpertParallelMoE(SHAPE["experts"], SHAPE["topK"],
                                          *parallel.cuda_layer_fns(home, local, 0, expert_layer=1),
                                          placement=placement, peer=buffers)
        for _ in range(2):
            y3 = peer.forward(x)
            torch.cuda.synchronize()
            same = same and bool(torch.equal(y3, want))
        # one row per (token, destination rank): the expert context takes K routes per row
        wide = hotpath.HotpathContext(layers=1, experts=epr, d=SHAPE["d"], f=SHAPE["f"], sharedF=0,
                                      topK=SHAPE["topK"], maxTokens=TOKENS * world, device=rank)
        wide.loadLayer(0, np.ascontiguousarray(L.blobs[placement.experts_of(rank)]), L.layout.stride,
                       L.layout.offsets, expertCount=epr)
        buffers_k = parallel.PeerBuffers(TOKENS * SHAPE["topK"] * world, SHAPE["d"], torch.bfloat16, full.device,
                                         ids_width=SHAPE["topK"])
        once = parallel.ExpertParallelMoE(SHAPE["experts"], SHAPE["topK"],
                                          *parallel.cuda_layer_fns(home, wide, 0, expert_layer=0),
                                          placement=placement, peer=buffers_k, one_row_per_token=True,
                                          route_sorter=parallel.cuda_route_sorter(home))
        for _ in range(2):
            y4 = once.forward(x)
            torch.cuda.synchronize()
            same = same and bool(torch.equal(y4, want))
        flags = wide.info().deviceErrorFlag | home.info().deviceErrorFlag | local.info().deviceErrorFlag | full.info().deviceErrorFlag
        results[rank] = (same, int(flags), rows)
        for c in (full, home, local, wide):
            c.close()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_matches_single_gpu_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    for rank in (0, 1):
        same, flags, rows = results[rank]
        assert same, f"rank {rank}: expert-parallel output differs from the single-GPU layer"
        assert flags == 0
    assert results[0][2] + results[1][2] == 2 * TOKENS * SHAPE["topK"]
