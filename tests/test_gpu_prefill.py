"""Prefill path (device permute + grouped INT4 tensor-core GEMMs) against the CPU oracle."""
import numpy as np
import pytest

from ane_fieldfare_b200 import synth, workload
from conftest import ELEMENTWISE_TOL, LAYER_ELEMENTWISE_TOL, assert_layer_close, oracle_layer

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _hp():
    from ane_fieldfare_b200 import hotpath
    return hotpath


def make_ctx(L, max_tokens):
    ctx = _hp().HotpathContext(layers=1, experts=L.experts, d=L.d, f=L.f, sharedF=L.sharedF,
                               topK=L.topK, maxTokens=max_tokens)
    workload.load_layer(ctx, 0, L)
    return ctx


def dev(bits, ctx):
    return _hp().bf16_tensor(bits, ctx.device)


@pytest.fixture(scope="module")
def tiny():
    L = workload.make_layer(0x9F1, 0, experts=16, d=128, f=64, sharedF=192, topK=8, router_bias="zipf")
    ctx = make_ctx(L, 700)
    yield L, ctx
    ctx.close()


@pytest.fixture(scope="module")
def full():
    """Benchmark shape with the Zipf-skewed router of the prefill configuration."""
    L = workload.make_layer(0xB203, 0, router_bias="zipf")
    ctx = make_ctx(L, 4096)
    yield L, ctx
    ctx.close()


@pytest.mark.parametrize("tokens", [17, 40, 300])
def test_router_rows_bit_exact(tiny, full, oracle, tokens):
    hp = _hp()
    for L, ctx in (tiny, full):
        x = workload.make_tokens(101, f"pr{tokens}", tokens, L.d)
        ids = torch.zeros((tokens, L.topK), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((tokens, L.topK), dtype=torch.bfloat16, device=ctx.device)
        logits = torch.zeros((tokens, L.experts), dtype=torch.float32, device=ctx.device)
        hp.PrefillRouter(ctx).encodeGemma4Block(None, 0, dev(x, ctx), ids, w, tokens, outLogits=logits)
        torch.cuda.synchronize()
        ref_ids, ref_w, ref_logits = oracle.router_topk(oracle_layer(oracle, L), x)
        assert logits.cpu().numpy().view(np.uint32).tobytes() == ref_logits.view(np.uint32).tobytes()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        assert np.abs(oracle.bf16_to_float(hp.bf16_numpy(w)) - oracle.bf16_to_float(ref_w)).max() < 5e-3


@pytest.mark.parametrize("tokens", [17, 40, 300, 700])
def test_device_permute_equals_reference_sort(tiny, oracle, tokens):
    """The device counting sort reproduces PrefillMoEGrouping's (expert, token, rank) order
    (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110) exactly."""
    hp = _hp()
    L, ctx = tiny
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(102, f"perm{tokens}", tokens, L.d)
    ref_ids, ref_w, _ = oracle.router_topk(ld, x)
    ids = torch.from_numpy(ref_ids.astype(np.int32)).to(ctx.device)
    partials = torch.zeros((tokens * L.topK, L.d), dtype=torch.bfloat16, device=ctx.device)
    routed = hp.PrefillGroupedRoutedMoE(ctx)
    routed.encodeStreamedBatched(None, 0, dev(x, ctx), ids, partials, tokens)
    pairs, offsets = routed.lastRoutes(tokens * L.topK)
    assert ctx.info().deviceErrorFlag == 0
    ref_pairs, n = oracle.make_pairs(ref_ids, ref_w, tokens, L.topK)
    sp, groups, _ = oracle.group_pairs(ref_pairs, n, tokens, L.topK, L.experts, 16)
    assert [(p.token, p.expert, p.rank) for p in pairs] == [(p.token, p.expert, p.rank) for p in sp]
    want = np.zeros(L.experts + 1, dtype=np.uint32)
    for g in groups:
        want[g.expert + 1] = g.pair_count
    assert np.array_equal(offsets, np.cumsum(want).astype(np.uint32))


@pytest.mark.parametrize("tokens", [17, 40, 300])
def test_prefill_partials_tiny(tiny, oracle, tokens):
    """Per-route partial rows; 40 rows = tiles of 32 + 8 in the reference's own test
    (Tests/.../Kernels/Prefill/PrefillGroupedRoutedMoETests+Execution.swift:106-228)."""
    hp = _hp()
    L, ctx = tiny
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(103, f"part{tokens}", tokens, L.d)
    ref_ids, ref_w, _ = oracle.router_topk(ld, x)
    ids = torch.from_numpy(ref_ids.astype(np.int32)).to(ctx.device)
    partials = torch.full((tokens * L.topK, L.d), -99.0, dtype=torch.bfloat16, device=ctx.device)
    hp.PrefillGroupedRoutedMoE(ctx).encodeStreamedBatched(None, 0, dev(x, ctx), ids, partials, tokens)
    torch.cuda.synchronize()
    assert ctx.info().deviceErrorFlag == 0
    ref_pairs, n = oracle.make_pairs(ref_ids, ref_w, tokens, L.topK)
    want = oracle.route_partials(ld, x, ref_pairs, n, tokens)
    assert_layer_close(hp.bf16_numpy(partials), want, oracle, f"prefill partials T={tokens}")
    # against the oracle that multiplies the same bf16-rounded weights: element by element
    want16 = oracle.route_partials(ld, x, ref_pairs, n, tokens, bf16_weights=True)
    assert_layer_close(hp.bf16_numpy(partials), want16, oracle, f"prefill partials T={tokens} vs bf16 weights",
                       elementwise_tol=ELEMENTWISE_TOL)


@pytest.mark.parametrize("tokens,experts_used", [(1, 8), (3, 8), (192, 8), (193, 8), (400, 8), (401, 9)])
def test_prefill_partials_with_chosen_routes(tiny, oracle, tokens, experts_used):
    """Row tiles at their edges: every token routed to the same eight experts (each expert then has
    exactly `tokens` rows: one row, a full tile of 192, 192 + 1, two tiles + 16, and the other
    experts none), and a ninth expert taking one route of the last token (a one-row expert behind
    full ones).  Routes are handed in, as `PrefillGroupedRoutedMoE.encodeStreamedBatched` takes them
    (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:275-326)."""
    hp = _hp()
    L, ctx = tiny
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(105, f"chosen{tokens}", tokens, L.d)
    ids_np = np.tile(np.arange(2, 2 + L.topK, dtype=np.uint32), (tokens, 1))
    if experts_used == 9:
        ids_np[-1, -1] = 12
    w_np = np.tile(synth.bf16_bits(np.full(L.topK, 1.0 / L.topK, dtype=np.float32)), (tokens, 1))
    ids = torch.from_numpy(ids_np.astype(np.int32)).to(ctx.device)
    partials = torch.full((tokens * L.topK, L.d), -99.0, dtype=torch.bfloat16, device=ctx.device)
    hp.PrefillGroupedRoutedMoE(ctx).encodeStreamedBatched(None, 0, dev(x, ctx), ids, partials, tokens)
    torch.cuda.synchronize()
    assert ctx.info().deviceErrorFlag == 0
    pairs, n = oracle.make_pairs(ids_np, w_np, tokens, L.topK)
    want16 = oracle.route_partials(ld, x, pairs, n, tokens, bf16_weights=True)
    assert_layer_close(hp.bf16_numpy(partials), want16, oracle, f"chosen routes T={tokens}",
                       elementwise_tol=ELEMENTWISE_TOL)


@pytest.mark.parametrize("tokens,groups", [(17, 2), (300, 5), (700, 16)])
def test_sort_routes_by_any_group_id(tiny, tokens, groups):
    """ff_sort_routes: the device permute on its own, by an arbitrary group id (the expert-parallel
    dispatch sorts by destination rank with it).  Against a stable sort on the host: (group, token,
    rank) order, as PrefillMoEGrouping.groupTokenExpertPairs gives it
    (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:49-110); ids past `groups` are dropped."""
    hp = _hp()
    L, ctx = tiny
    rng = np.random.default_rng(tokens)
    ids = rng.integers(0, groups + 1, size=(tokens, L.topK)).astype(np.int32)   # `groups` itself: dropped
    pairs, offsets = hp.PrefillGroupedRoutedMoE(ctx).sortRoutesOnDevice(
        None, torch.from_numpy(ids).to(ctx.device), groups)
    torch.cuda.synchronize()
    flat = ids.reshape(-1)
    keep = np.flatnonzero(flat < groups)
    order = keep[np.argsort(flat[keep], kind="stable")]
    want_offsets = np.concatenate([[0], np.cumsum(np.bincount(flat[keep], minlength=groups))])
    assert np.array_equal(offsets.cpu().numpy(), want_offsets.astype(np.int32))
    got = pairs.cpu().numpy()[:order.size]
    assert np.array_equal(got[:, 0], order // L.topK)
    assert np.array_equal(got[:, 1], flat[order])
    assert np.array_equal(got[:, 2], order % L.topK)


@pytest.mark.parametrize("tokens", [20, 300])
def test_prefill_shared_ffn(tiny, full, oracle, tokens):
    hp = _hp()
    for L, ctx in (tiny, full):
        x = workload.make_tokens(104, f"sh{tokens}", tokens, L.d)
        y = torch.zeros((tokens, L.d), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillSharedExpert(ctx).encodeBlock(None, 0, dev(x, ctx), y, tokens)
        torch.cuda.synchronize()
        assert ctx.info().deviceErrorFlag == 0
        want = oracle.shared_ffn(oracle_layer(oracle, L), x)
        assert_layer_close(hp.bf16_numpy(y), want, oracle, f"prefill shared T={tokens}")
        want16 = oracle.shared_ffn(oracle_layer(oracle, L), x, bf16_weights=True)
        assert_layer_close(hp.bf16_numpy(y), want16, oracle, f"prefill shared T={tokens} vs bf16 weights",
                           elementwise_tol=ELEMENTWISE_TOL)


@pytest.mark.parametrize("tokens", [17, 130, 700])
def test_prefill_layer_tiny(tiny, oracle, tokens):
    hp = _hp()
    L, ctx = tiny
    x = workload.make_tokens(105, f"lay{tokens}", tokens, L.d)
    ids = torch.zeros((tokens, L.topK), dtype=torch.int32, device=ctx.device)
    y = ctx.moeLayer(0, dev(x, ctx), ids=ids)
    torch.cuda.synchronize()
    assert ctx.info().deviceErrorFlag == 0
    want, _, ref_ids, _ = oracle.moe_layer(oracle_layer(oracle, L), x, oracle.MODE_PARTIALS)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
    assert_layer_close(hp.bf16_numpy(y), want, oracle, f"prefill layer T={tokens}")
    want16, _, _, _ = oracle.moe_layer(oracle_layer(oracle, L), x, oracle.MODE_PARTIALS | oracle.MODE_BF16_WEIGHTS)
    assert_layer_close(hp.bf16_numpy(y), want16, oracle, f"prefill layer T={tokens} vs bf16 weights",
                       elementwise_tol=LAYER_ELEMENTWISE_TOL)


def test_prefill_layer_full_shape(full, oracle):
    """Benchmark configuration 3 (4096 tokens, Zipf-skewed routing): 512 tokens against the oracle
    directly; the full 4096 through properties that do not need the oracle at full size — rows are
    independent, so a row's result in the 4096-row call equals its result in a 512-row call."""
    hp = _hp()
    L, ctx = full
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(106, "cfg3", 4096, L.d)
    xd = dev(x, ctx)
    ids = torch.zeros((4096, L.topK), dtype=torch.int32, device=ctx.device)
    y = ctx.moeLayer(0, xd, ids=ids)
    torch.cuda.synchronize()
    info = ctx.info()
    assert info.deviceErrorFlag == 0
    counts = np.bincount(ids.cpu().numpy().reshape(-1), minlength=L.experts)
    assert counts.sum() == 4096 * L.topK and counts.max() > 4 * counts[counts > 0].min()
    y512 = ctx.moeLayer(0, xd[:512].contiguous())
    torch.cuda.synchronize()
    assert torch.equal(y512, y[:512])
    want, _, ref_ids, _ = oracle.moe_layer(ld, x[:512], oracle.MODE_PARTIALS)
    assert np.array_equal(ids[:512].cpu().numpy().astype(np.uint32), ref_ids)
    rel, literal, peak = assert_layer_close(hp.bf16_numpy(y512), want, oracle, "cfg3 rows 0..511")
    want16, _, _, _ = oracle.moe_layer(ld, x[:512], oracle.MODE_PARTIALS | oracle.MODE_BF16_WEIGHTS)
    assert_layer_close(hp.bf16_numpy(y512), want16, oracle, "cfg3 rows 0..511 vs bf16 weights",
                       elementwise_tol=LAYER_ELEMENTWISE_TOL)
    # scattered rows of the full batch against the oracle
    pick = np.arange(0, 4096, 64)
    want_pick, _, _, _ = oracle.moe_layer(ld, x[pick], oracle.MODE_PARTIALS)
    assert_layer_close(hp.bf16_numpy(y)[pick], want_pick, oracle, "cfg3 sampled rows")
    assert np.isfinite(oracle.bf16_to_float(hp.bf16_numpy(y))).all()


def test_guest_plugin_contract(tiny, oracle):
    """CudaRoutedPrefillGuest.runLayer writes every (token, rank) row named by the routes
    (Runtime/Supervisor/DeviceSupervisor.swift:14-22) and leaves other memory alone."""
    hp = _hp()
    L, ctx = tiny
    tokens = 50
    x = workload.make_tokens(107, "guest", tokens, L.d)
    ref_ids, ref_w, _ = oracle.router_topk(oracle_layer(oracle, L), x)
    ids = torch.from_numpy(ref_ids.astype(np.int32)).to(ctx.device)
    partials = torch.full((tokens * L.topK + 4, L.d), -99.0, dtype=torch.bfloat16, device=ctx.device)
    guest = hp.CudaRoutedPrefillGuest(ctx)
    guest.runLayer(0, dev(x, ctx), partials, ids, tokens)
    torch.cuda.synchronize()
    assert guest.profile == {"layers": 1, "pairs": tokens * L.topK}
    assert (partials[tokens * L.topK:] == -99.0).all()
    assert not (partials[:tokens * L.topK] == -99.0).all(dim=1).any()
