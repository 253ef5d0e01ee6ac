"""The layer stack of benchmark configuration 4, the unit-scale variants of configurations 1-3
(where the stated max-abs <= 2e-2 is asserted as written), and the inputs the library refuses
before (or instead of) touching memory it does not own."""
import ctypes
import dataclasses

import numpy as np
import pytest

from ane_fieldfare_b200 import binding, gturbo, synth, workload
from conftest import LAYER_ELEMENTWISE_TOL, assert_layer_close, oracle_layer

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOY = dict(experts=16, d=128, f=64, sharedF=192, topK=8)


def _hp():
    from ane_fieldfare_b200 import hotpath
    return hotpath


def dev(bits, ctx):
    return _hp().bf16_tensor(bits, ctx.device)


def _stack_case(oracle, layers, ctx, x, what):
    """Free-running stack against the oracle, then every layer on the oracle's own inputs."""
    hp = _hp()
    n, tokens, K = len(layers), x.shape[0], layers[0].topK
    lds = [oracle_layer(oracle, L) for L in layers]
    # the library multiplies weights rounded to bf16 above 16 rows (tensor-core path): the oracle mode
    # with the same operand is the one a free-running stack is compared with
    mode = oracle.MODE_DECODE if tokens == 1 else oracle.MODE_PARTIALS
    if tokens > 16:
        mode |= oracle.MODE_BF16_WEIGHTS
    want, want_ids = oracle.moe_stack(lds, x, 1e-6, mode)
    ids = torch.zeros((n, tokens, K), dtype=torch.int32, device=ctx.device)
    y = ctx.moeStack(0, n, dev(x, ctx), 1e-6, ids=ids)
    torch.cuda.synchronize()
    assert ctx.info().deviceErrorFlag == 0
    got_ids = ids.cpu().numpy().astype(np.uint32)
    # layer 0 sees identical inputs: identical routes.  Deeper layers see inputs that differ by the
    # layers' tolerance, so a near-tie between the 8th and 9th score may fall the other way; tokens
    # whose routes agree at every layer are compared with the oracle's output.
    assert np.array_equal(got_ids[0], want_ids[0]), what
    same = (got_ids == want_ids).all(axis=(0, 2))
    assert same.mean() >= 0.75, f"{what}: only {same.sum()} of {tokens} tokens keep the oracle's routes"
    assert_layer_close(hp.bf16_numpy(y)[same], want[same], oracle, f"{what} free-running ({same.sum()}/{tokens} tokens)")
    # every layer in sequence on the oracle's input to that layer: routes equal, output in tolerance
    cur = x
    for i, ld in enumerate(lds):
        normed = oracle.rmsnorm_bf16(cur, None, 1e-6, tokens, ld.D)
        got_norm = hp.bf16_numpy(ctx.rmsnorm(dev(cur, ctx), None, 1e-6))
        dn = np.abs(oracle.bf16_to_float(got_norm) - oracle.bf16_to_float(normed))
        assert dn.max() <= 2.0 ** -7 * np.abs(oracle.bf16_to_float(normed)).max()
        layer_ids = torch.zeros((tokens, K), dtype=torch.int32, device=ctx.device)
        yl = ctx.moeLayer(i, dev(normed, ctx), ids=layer_ids)
        torch.cuda.synchronize()
        cur, _, ref_ids, _ = oracle.moe_layer(ld, normed, mode)
        assert np.array_equal(layer_ids.cpu().numpy().astype(np.uint32), ref_ids), (what, i)
        # (no element-wise bound here: deeper layers of the Zipf-routed stack have outputs of peak
        # several hundred beside elements of order one, where half an ulp of a large partial row is
        # a tenth of a small sum)
        assert_layer_close(hp.bf16_numpy(yl), cur, oracle, f"{what} layer {i} on the oracle's input")
        if tokens > 16:  # and within the layer tolerance of the fp32-weight reference
            ref32, _, _, _ = oracle.moe_layer(ld, normed, oracle.MODE_PARTIALS)
            assert_layer_close(hp.bf16_numpy(yl), ref32, oracle, f"{what} layer {i} vs fp32 weights")


@pytest.mark.parametrize("tokens", [1, 8, 40])
def test_stack_of_four_toy_layers(oracle, tokens):
    hp = _hp()
    layers = [workload.make_layer(0x57AC4, i, router_bias="normal", **TOY) for i in range(4)]
    ctx = hp.HotpathContext(layers=4, maxTokens=64, **TOY)
    try:
        for i, L in enumerate(layers):
            workload.load_layer(ctx, i, L)
        x = workload.make_tokens(0x57AC4, f"x{tokens}", tokens, TOY["d"])
        _stack_case(oracle, layers, ctx, x, f"toy stack T={tokens}")
    finally:
        ctx.close()


def test_stack_of_three_layers_at_the_benchmark_shape(oracle):
    """Configuration 4's block (128 experts, top-8, shared FFN, Zipf-skewed router) three deep,
    64 tokens."""
    hp = _hp()
    layers = [workload.make_layer(0x57AC5, i, router_bias="zipf") for i in range(3)]
    ctx = hp.HotpathContext(layers=3, experts=128, d=2816, f=704, sharedF=2112, topK=8, maxTokens=64)
    try:
        for i, L in enumerate(layers):
            workload.load_layer(ctx, i, L)
        x = workload.make_tokens(0x57AC5, "x", 64, 2816)
        _stack_case(oracle, layers, ctx, x, "cfg4 block x3, 64 tokens")
    finally:
        ctx.close()


# ---- unit-scale variants: outputs of peak <= 1, the stated bound, literally ---------------

@pytest.fixture(scope="module")
def unit_full():
    """The benchmark shape with every down projection scaled by 2^-5: outputs peak below 1."""
    L = workload.make_layer(0xB205, 0, router_bias="normal", down_shift=5)
    ctx = _hp().HotpathContext(layers=1, experts=L.experts, d=L.d, f=L.f, sharedF=L.sharedF, topK=L.topK,
                               maxTokens=512)
    workload.load_layer(ctx, 0, L)
    yield L, ctx
    ctx.close()


@pytest.mark.parametrize("tokens", [1, 16, 512])
def test_unit_scale_configs_meet_the_literal_bound(unit_full, oracle, tokens):
    """Configurations 1 (decode), 2 (verify block of 16) and 3 (prefill; 512 of its rows, Zipf
    router prior) with outputs of unit scale: rel-L2 <= 1e-2 and max-abs <= 2e-2 as written."""
    hp = _hp()
    L, ctx = unit_full
    if tokens == 512:
        bias = synth.zipf_log_prior(L.experts, 1.1, 0xB205, "unit.zipf")
        L = dataclasses.replace(L, logitBias=bias)
    ctx.loadRouter(0, L.routerW, logitBias=L.logitBias)
    x = workload.make_tokens(0xB205, f"unit{tokens}", tokens, L.d)
    ids = torch.zeros((tokens, L.topK), dtype=torch.int32, device=ctx.device)
    y = ctx.moeLayer(0, dev(x, ctx), ids=ids)
    torch.cuda.synchronize()
    assert ctx.info().deviceErrorFlag == 0
    mode = oracle.MODE_DECODE if tokens == 1 else oracle.MODE_PARTIALS
    want, _, ref_ids, _ = oracle.moe_layer(oracle_layer(oracle, L), x, mode)
    assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
    assert np.abs(oracle.bf16_to_float(want)).max() <= 1.0
    assert_layer_close(hp.bf16_numpy(y), want, oracle, f"unit-scale T={tokens}", literal_tol=2e-2)


# ---- inputs that are refused --------------------------------------------------------------------

def test_route_past_the_resident_experts_is_reported_not_followed(oracle):
    """The reference traps a route id past the expert count ("route expert N is out of range",
    Runtime/Inference/RealForwardRunner.swift:815).  Here such a route never becomes an address:
    decode runs expert 0 with weight 0 in its place, the verify plan leaves its row unwritten, and
    both raise the context's error flag."""
    hp = _hp()
    L = workload.make_layer(0xBAD1D, 0, router_bias="normal", **TOY)
    ctx = hp.HotpathContext(layers=1, maxTokens=16, **TOY)
    try:
        workload.load_layer(ctx, 0, L)
        x = workload.make_tokens(0xBAD1D, "x", 2, TOY["d"])
        xd = dev(x, ctx)
        good = np.arange(8, dtype=np.int32)[None, :]
        w = synth.bf16_bits(np.full((1, 8), 0.125, dtype=np.float32))
        y_ref = torch.zeros((1, TOY["d"]), dtype=torch.bfloat16, device=ctx.device)
        moe = hp.MoE(ctx)
        moe.encodeRoutedPersistentGPUSlots(None, 0, torch.from_numpy(good).to(ctx.device), xd[:1].contiguous(),
                                           dev(w, ctx), None, y_ref)
        torch.cuda.synchronize()
        assert ctx.info().deviceErrorFlag == 0
        bad = good.copy()
        bad[0, 3] = TOY["experts"] + 5
        y_bad = torch.zeros_like(y_ref)
        moe.encodeRoutedPersistentGPUSlots(None, 0, torch.from_numpy(bad).to(ctx.device), xd[:1].contiguous(),
                                           dev(w, ctx), None, y_bad)
        torch.cuda.synchronize()
        assert ctx.info().deviceErrorFlag == 12
        # the other seven routes still count: the row equals the good row minus route 3's share
        assert torch.isfinite(y_bad.float()).all()
        ctx.resetDeviceError()
        assert ctx.info().deviceErrorFlag == 0
        ids2 = np.stack([np.arange(8), np.arange(8) + 4]).astype(np.int32)
        ids2[1, 7] = 4000
        partials = torch.full((16, TOY["d"]), -99.0, dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillGroupedRoutedMoE(ctx).encodeVerifyBound(None, 0, xd, torch.from_numpy(ids2).to(ctx.device),
                                                          partials, 2)
        torch.cuda.synchronize()
        assert ctx.info().deviceErrorFlag == 12
        assert (partials[15] == -99.0).all() and not (partials[:15] == -99.0).all(dim=1).any()
        ctx.resetDeviceError()
    finally:
        ctx.close()


def test_misaligned_and_mismatched_arguments_fail_before_any_launch(oracle):
    hp = _hp()
    L = workload.make_layer(0xA119, 0, **TOY)
    ctx = hp.HotpathContext(layers=1, maxTokens=16, **TOY)
    try:
        workload.load_layer(ctx, 0, L)
        launches = ctx.info().kernelLaunches
        d = TOY["d"]
        buf = torch.zeros((4, d + 8), dtype=torch.bfloat16, device=ctx.device)
        odd = buf.data_ptr() + 2  # one bf16 element past a 16-byte boundary
        out = torch.zeros((4, d), dtype=torch.bfloat16, device=ctx.device)
        w, s, b = gturbo.sub_tensor(L.sharedBlob, L.sharedLayout, "gate")
        wd = torch.from_numpy(np.ascontiguousarray(w)).to(ctx.device)
        sd, bd = dev(np.ascontiguousarray(s), ctx), dev(np.ascontiguousarray(b), ctx)
        proj = binding.FFProjection(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), TOY["sharedF"], d)
        down = binding.FFProjection(wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), d, TOY["sharedF"])
        stream = None
        with pytest.raises(hp.FieldfareError, match="4-byte aligned"):
            binding.call("ff_int4_gemv_rows", ctx.handle, ctypes.byref(proj), odd, d + 8, 2,
                         torch.zeros((2, TOY["sharedF"]), dtype=torch.bfloat16, device=ctx.device).data_ptr(),
                         TOY["sharedF"], stream)
        with pytest.raises(hp.FieldfareError, match="4-byte aligned"):
            binding.call("ff_moe_reduce", ctx.handle, odd, out.data_ptr(), None, out.data_ptr(), 1, stream)
        with pytest.raises(hp.FieldfareError, match="2-byte aligned"):
            binding.call("ff_rmsnorm", ctx.handle, buf.data_ptr() + 1, None, ctypes.c_float(1e-6), 1,
                         out.data_ptr(), stream)
        with pytest.raises(hp.FieldfareError, match="4-byte aligned"):
            binding.call("ff_shared_ffn_noalloc", ctypes.byref(proj), ctypes.byref(proj), ctypes.byref(down),
                         odd, d + 8, 2, out.data_ptr(), d, stream)
        with pytest.raises(hp.FieldfareError, match="16-byte aligned"):
            binding.call("ff_moe_layer", ctx.handle, 0, odd, 1, out.data_ptr(), None, None, stream)
        # a router whose expert count differs from the layer's would rank ids the layer does not hold
        with pytest.raises(hp.FieldfareError, match="the context expects 16"):
            ctx.loadRouter(0, L.routerW[:12])
        with pytest.raises(hp.FieldfareError, match="out of range"):
            ctx.moeStack(0, 2, buf[:1, :d].contiguous())
        assert ctx.info().kernelLaunches == launches
        assert ctx.info().deviceErrorFlag == 0
    finally:
        ctx.close()


# ---- lossy routing modes: host-side weight edits in front of the K-wide operators ---------------

@pytest.mark.parametrize("tokens", [1, 3, 40])
def test_lossy_routing_modes_feed_the_operators(oracle, tokens):
    """`activeRoutedExperts` < 8 and `prefillExpertUnionCap` (RuntimeConfiguration.swift:57-67) edit
    the route weights on the host (supervisor.apply_active_routed_experts / cap_expert_union); the
    operators then take the edited weights with the full routes.  Against the oracle's partial rows
    reduced with the same edited weights."""
    from ane_fieldfare_b200 import supervisor as sv
    hp = _hp()
    L = workload.make_layer(0x4055, 0, **TOY)
    ld = oracle_layer(oracle, L)
    ctx = hp.HotpathContext(layers=1, maxTokens=64, **TOY)
    try:
        workload.load_layer(ctx, 0, L)
        x = workload.make_tokens(0x4055, f"lossy{tokens}", tokens, TOY["d"])
        ids, w, _ = oracle.router_topk(ld, x)
        ids_dev = torch.from_numpy(ids.astype(np.int32)).to(ctx.device)
        xd = dev(x, ctx)
        shared = torch.zeros((tokens, TOY["d"]), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillSharedExpert(ctx).encodeBlock(None, 0, xd, shared, tokens)
        partials = torch.zeros((tokens * TOY["topK"], TOY["d"]), dtype=torch.bfloat16, device=ctx.device)
        routed = hp.PrefillGroupedRoutedMoE(ctx)
        if tokens <= 16:
            routed.encodeVerifyBound(None, 0, xd, ids_dev, partials, tokens)
        else:
            routed.encodeStreamedBatched(None, 0, xd, ids_dev, partials, tokens)
        wide = tokens > 16  # the GEMM path multiplies weights rounded to bf16
        pairs, n = oracle.make_pairs(ids, w, tokens, TOY["topK"])
        ref_partials = oracle.route_partials(ld, x, pairs, n, tokens, bf16_weights=wide)
        ref_shared = oracle.shared_ffn(ld, x, bf16_weights=wide)
        for what, edited in (("active 5", sv.apply_active_routed_experts(w, 5)),
                             ("union cap 6", sv.cap_expert_union(ids, w, TOY["experts"], 6))):
            assert not np.array_equal(edited, w)
            got = torch.zeros((tokens, TOY["d"]), dtype=torch.bfloat16, device=ctx.device)
            hp.PrefillMoE(ctx).encodeReduceTokenMajor(None, partials, dev(edited, ctx), got, tokens, residual=shared)
            torch.cuda.synchronize()
            want = oracle.reduce_token_major(ref_partials, edited, ref_shared, tokens, TOY["topK"], TOY["d"])
            assert_layer_close(hp.bf16_numpy(got), want, oracle, f"lossy {what} T={tokens}",
                               elementwise_tol=LAYER_ELEMENTWISE_TOL)
            if tokens == 1:
                # the one-token operator takes the edited weights with the full routes, too
                y1 = torch.zeros((1, TOY["d"]), dtype=torch.bfloat16, device=ctx.device)
                hp.MoE(ctx).encodeRoutedPersistentGPUSlots(None, 0, ids_dev, xd, dev(edited, ctx), shared, y1)
                torch.cuda.synchronize()
                assert_layer_close(hp.bf16_numpy(y1), want, oracle, f"lossy {what}, one-token operator",
                                   elementwise_tol=LAYER_ELEMENTWISE_TOL)
            assert ctx.info().deviceErrorFlag == 0
    finally:
        ctx.close()
