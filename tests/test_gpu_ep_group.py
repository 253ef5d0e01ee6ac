"""Expert parallelism behind the C ABI (`ff_ep_create` / `ff_ep_moe_layer`): one process drives every
GPU of the group, the rows travel as stores into the destination's memory and come back as peer
copies.  Compared bit for bit with the one-device layer holding all experts.  A group of one rank
runs the whole path (sort by destination, send kernel, grouped experts on received rows, indexed
combine) on a single GPU; the two-rank case needs two GPUs and is skipped otherwise."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SHAPE = dict(experts=16, d=128, f=64, sharedF=192, topK=8)
TOKENS = 40


def _contexts(world, L, with_shared=True):
    from ane_fieldfare_b200 import hotpath
    epr = SHAPE["experts"] // world
    home, expert = [], []
    for r in range(world):
        h = hotpath.HotpathContext(layers=1, maxTokens=TOKENS, device=r, **SHAPE)
        if with_shared:
            h.loadShared(0, *L.shared_projections())
        h.loadRouter(0, L.routerW, logitBias=L.logitBias)
        e = hotpath.HotpathContext(layers=1, experts=epr, d=SHAPE["d"], f=SHAPE["f"], sharedF=0, topK=1,
                                   maxTokens=TOKENS * SHAPE["topK"] * world, device=r)
        e.loadLayer(0, np.ascontiguousarray(L.blobs[r * epr:(r + 1) * epr]), L.layout.stride, L.layout.offsets,
                    expertCount=epr)
        home.append(h)
        expert.append(e)
    return home, expert


@pytest.mark.parametrize("world", [1, 2])
def test_group_matches_the_one_device_layer(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from ane_fieldfare_b200 import hotpath, workload
    L = workload.make_layer(0xE9, 0, router_bias="zipf", **SHAPE)
    home, expert = _contexts(world, L)
    group = hotpath.ExpertParallelGroup(home, expert)
    xs, wants, fulls = [], [], []
    for r in range(world):
        full = hotpath.HotpathContext(layers=1, maxTokens=TOKENS, device=r, **SHAPE)
        workload.load_layer(full, 0, L)
        x = hotpath.bf16_tensor(workload.make_tokens(0xE9 + r, "ep.x", TOKENS, SHAPE["d"]), full.device)
        with torch.cuda.device(r):
            want = full.moeLayer(0, x)
            torch.cuda.synchronize(r)
        xs.append(x)
        wants.append(want)
        fulls.append(full)
    for _ in range(2):  # twice over the same buffers
        ys = group.moeLayer(0, xs)
        for r in range(world):
            assert torch.equal(ys[r].cpu(), wants[r].cpu()), f"rank {r} differs from the one-device layer"
    # every route whose expert lives on another rank crossed once
    ids = [np.empty((TOKENS, SHAPE["topK"]), np.uint32) for _ in range(world)]
    away = 0
    for r in range(world):
        with torch.cuda.device(r):
            i = torch.empty((TOKENS, SHAPE["topK"]), dtype=torch.int32, device=xs[r].device)
            w = torch.empty((TOKENS, SHAPE["topK"]), dtype=torch.bfloat16, device=xs[r].device)
            hotpath.PrefillRouter(home[r]).encodeGemma4Block(None, 0, xs[r], i, w, TOKENS)
            torch.cuda.synchronize(r)
        away += int((i.cpu().numpy() // (SHAPE["experts"] // world) != r).sum())
    assert group.lastRowsSent == away
    for c in home + expert + fulls:
        assert c.info().deviceErrorFlag == 0
    group.close()
    for c in home + expert + fulls:
        c.close()


@pytest.mark.parametrize("rows", [TOKENS, 300])
@pytest.mark.parametrize("world", [1, 2])
def test_group_stack_with_a_balanced_placement(world, rows):
    """Two layers (the second with its experts placed to even out the Zipf load), RMSNorm between:
    the bits of ff_moe_stack on one device holding everything.  At 300 rows the shared FFN runs in
    two parts on its own stream."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from ane_fieldfare_b200 import hotpath, parallel, workload
    layers = [workload.make_layer(0xEA, i, router_bias="zipf", **SHAPE) for i in range(2)]
    epr = SHAPE["experts"] // world
    load = [1.0 / (e + 1) ** 1.1 for e in range(SHAPE["experts"])]
    placements = [parallel.contiguous_placement(SHAPE["experts"], world), parallel.balanced_placement(load, world)]
    home, expert, fulls, xs, wants = [], [], [], [], []
    for r in range(world):
        h = hotpath.HotpathContext(layers=2, maxTokens=rows, device=r, **SHAPE)
        e = hotpath.HotpathContext(layers=2, experts=epr, d=SHAPE["d"], f=SHAPE["f"], sharedF=0, topK=1,
                                   maxTokens=rows * SHAPE["topK"] * world, device=r)
        full = hotpath.HotpathContext(layers=2, maxTokens=rows, device=r, **SHAPE)
        for i, L in enumerate(layers):
            h.loadShared(i, *L.shared_projections())
            h.loadRouter(i, L.routerW, logitBias=L.logitBias)
            e.loadLayer(i, np.ascontiguousarray(L.blobs[placements[i].experts_of(r)]), L.layout.stride,
                        L.layout.offsets, expertCount=epr)
            workload.load_layer(full, i, L)
        x = hotpath.bf16_tensor(workload.make_tokens(0xEA + r, "ep.x", rows, SHAPE["d"]), full.device)
        with torch.cuda.device(r):
            want = torch.empty_like(x)
            full.moeStack(0, 2, x, 1e-6, want)
            torch.cuda.synchronize(r)
        home.append(h); expert.append(e); fulls.append(full); xs.append(x); wants.append(want)
    group = hotpath.ExpertParallelGroup(home, expert)
    group.setPlacement(1, placements[1].rank_of.numpy(), placements[1].local_of.numpy())
    with pytest.raises(hotpath.FieldfareError, match="share slot"):
        group.setPlacement(0, np.zeros(SHAPE["experts"]), np.zeros(SHAPE["experts"]))
    for _ in range(2):
        ys = group.moeStack(0, 2, xs, 1e-6)
        for r in range(world):
            assert torch.equal(ys[r].cpu(), wants[r].cpu()), f"rank {r} differs from the one-device stack"
    # a traced call: the same bits, and every rank reports its ten phases
    group.setTracing(True)
    ys = group.moeStack(0, 2, xs, 1e-6)
    group.setTracing(False)
    phases = group.phaseTimes()
    assert len(phases) == world and all(set(p) == set(group.PHASES) for p in phases)
    assert all(v >= 0.0 for p in phases for v in p.values()) and all(p["experts"] > 0.0 for p in phases)
    for r in range(world):
        assert torch.equal(ys[r].cpu(), wants[r].cpu())
    group.close()
    for c in home + expert + fulls:
        assert c.info().deviceErrorFlag == 0
        c.close()


def test_group_refuses_what_it_cannot_run():
    from ane_fieldfare_b200 import hotpath, workload
    from ane_fieldfare_b200.binding import FieldfareError
    L = workload.make_layer(0xE9, 0, router_bias="zipf", **SHAPE)
    home, expert = _contexts(1, L)
    # an expert context that takes K routes per row
    wide = hotpath.HotpathContext(layers=1, experts=SHAPE["experts"], d=SHAPE["d"], f=SHAPE["f"], sharedF=0,
                                  topK=SHAPE["topK"], maxTokens=TOKENS * SHAPE["topK"], device=0)
    with pytest.raises(FieldfareError, match="topK = 1"):
        hotpath.ExpertParallelGroup(home, [wide])
    # an expert context too small for the capacity
    small = hotpath.HotpathContext(layers=1, experts=SHAPE["experts"], d=SHAPE["d"], f=SHAPE["f"], sharedF=0,
                                   topK=1, maxTokens=TOKENS, device=0)
    with pytest.raises(FieldfareError, match="capacity"):
        hotpath.ExpertParallelGroup(home, [small])
    # two ranks on one device
    with pytest.raises(FieldfareError, match="share device"):
        hotpath.ExpertParallelGroup(home + home, expert + expert)
    group = hotpath.ExpertParallelGroup(home, expert)
    x = hotpath.bf16_tensor(workload.make_tokens(1, "ep.x", TOKENS + 1, SHAPE["d"]), home[0].device)
    with pytest.raises(FieldfareError, match="exceed"):
        group.moeLayer(0, [x])
    group.close()
    for c in home + expert + [wide, small]:
        c.close()
