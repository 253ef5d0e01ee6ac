"""The INT8 affine router of the shipped checkpoints (Runtime/Inference/Model.swift:473-475, kernel
body Metal/MoE/moe.metal:65-103) against the oracle: logits and indices bit for bit at 1..300
rows, with the per-input scale and per-expert gain, and the fused operators taking the INT8 router
in place of the bf16 one."""
import numpy as np
import pytest

from ane_fieldfare_b200 import synth, workload

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _hp():
    from ane_fieldfare_b200 import hotpath
    return hotpath


def int8_router(seed, experts, d, spread=1.0):
    """Seeded INT8 router: codes, bf16 scales and biases such that w = q*s + b lies in about
    [-spread, spread] / sqrt(d), with every expert row offset a little (distinct scores)."""
    codes = (synth.uniform(seed, experts * d, 0.0, 256.0).astype(np.int64).clip(0, 255)).astype(np.uint8)
    codes = codes.reshape(experts, d)
    groups = d // 64
    amp = np.float32(spread / np.sqrt(d))
    scales = synth.uniform(seed + 1, experts * groups, 0.5, 1.5).reshape(experts, groups) * (2 * amp / 255)
    biases = -amp * synth.uniform(seed + 2, experts * groups, 0.8, 1.2).reshape(experts, groups) + \
        (np.arange(experts, dtype=np.float32) * np.float32(1e-3 / np.sqrt(d)))[:, None]
    return codes, synth.bf16_bits(scales.astype(np.float32)), synth.bf16_bits(biases.astype(np.float32))


def dev(bits, ctx):
    return _hp().bf16_tensor(bits, ctx.device)


SHAPES = [dict(experts=16, d=128, f=64, sharedF=192, topK=8), dict(experts=128, d=2816, f=704, sharedF=2112, topK=8)]


@pytest.mark.parametrize("shape", SHAPES, ids=["toy", "benchmark"])
@pytest.mark.parametrize("rows", [1, 3, 16, 40, 300])
def test_int8_router_logits_and_indices_are_bit_exact(oracle, shape, rows):
    hp = _hp()
    E, D, K = shape["experts"], shape["d"], shape["topK"]
    codes, scales, biases = int8_router(0x18, E, D)
    eff = synth.bf16_bits(synth.uniform(7, D, 0.5, 1.5))
    gain = synth.bf16_bits(synth.uniform(8, E, 0.6, 1.4))
    bias = synth.uniform(9, E, -0.2, 0.2)
    ctx = hp.HotpathContext(layers=1, maxTokens=max(rows, 17), **shape)
    try:
        ctx.loadRouterInt8(0, codes, scales, biases, effectiveScale=eff, perExpertScale=gain, logitBias=bias)
        x = workload.make_tokens(0x18, f"int8.x{rows}", rows, D)
        ids = torch.zeros((rows, K), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((rows, K), dtype=torch.bfloat16, device=ctx.device)
        logits = torch.zeros((rows, E), dtype=torch.float32, device=ctx.device)
        if rows <= 16:
            hp.MoE(ctx).encodeRouterRowsGemma4(None, 0, dev(x, ctx), D, rows, ids, w, logits)
        else:
            hp.PrefillRouter(ctx).encodeGemma4Block(None, 0, dev(x, ctx), ids, w, rows, outLogits=logits)
        torch.cuda.synchronize()
        ref_ids, ref_w, ref_logits = oracle.router_topk_int8(codes, scales, biases, x, K, effective_scale=eff,
                                                             logit_bias=bias, gain=gain)
        assert logits.cpu().numpy().view(np.uint32).tobytes() == ref_logits.view(np.uint32).tobytes()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        dw = np.abs(oracle.bf16_to_float(hp.bf16_numpy(w)) - oracle.bf16_to_float(ref_w))
        assert dw.max() < 5e-3
        assert ctx.info().deviceErrorFlag == 0
    finally:
        ctx.close()


@pytest.mark.parametrize("rows", [1, 5, 40])
def test_operators_take_the_int8_router(oracle, rows):
    """The one-token kernel, the 2..16-row block and the prefill layer with an INT8 router give the
    bits they give for the same routes handed in."""
    hp = _hp()
    shape = SHAPES[0]
    E, D, K = shape["experts"], shape["d"], shape["topK"]
    L = workload.make_layer(0x19, 0, **shape)
    codes, scales, biases = int8_router(0x19, E, D)
    ctx = hp.HotpathContext(layers=1, maxTokens=64, **shape)
    try:
        ctx.loadLayer(0, L.blobs, L.layout.stride, L.layout.offsets)
        ctx.loadShared(0, *L.shared_projections())
        ctx.loadRouterInt8(0, codes, scales, biases)
        x = workload.make_tokens(0x19, f"int8.layer{rows}", rows, D)
        xd = dev(x, ctx)
        y = ctx.moeLayer(0, xd)
        ref_ids, ref_w, _ = oracle.router_topk_int8(codes, scales, biases, x, K)
        ids = torch.zeros((rows, K), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((rows, K), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillRouter(ctx).encodeGemma4Block(None, 0, xd, ids, w, rows)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        # the same layer from its parts, the routes handed to the operators that take routes
        shared = torch.zeros((rows, D), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillSharedExpert(ctx).encodeBlock(None, 0, xd, shared, rows)
        given = torch.zeros((rows, D), dtype=torch.bfloat16, device=ctx.device)
        if rows == 1:
            hp.MoE(ctx).encodeRoutedPersistentGPUSlots(None, 0, ids, xd, w, shared, given)
        else:
            partials = torch.zeros((rows * K, D), dtype=torch.bfloat16, device=ctx.device)
            routed = hp.PrefillGroupedRoutedMoE(ctx)
            if rows <= 16:
                routed.encodeVerifyBound(None, 0, xd, ids, partials, rows)
            else:
                routed.encodeStreamedBatched(None, 0, xd, ids, partials, rows)
            hp.PrefillMoE(ctx).encodeReduceTokenMajor(None, partials, w, given, rows, residual=shared)
        torch.cuda.synchronize()
        assert torch.equal(y, given)
        assert ctx.info().deviceErrorFlag == 0
        # host entry: the same rows through host buffers
        hx = torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
        hy = torch.empty((rows, D), dtype=torch.bfloat16).pin_memory()
        ctx.moeLayerHost(0, hx, hy)
        assert torch.equal(hy, y.cpu())
    finally:
        ctx.close()


def test_int8_router_refusals():
    hp = _hp()
    shape = SHAPES[0]
    codes, scales, biases = int8_router(1, shape["experts"], shape["d"])
    ctx = hp.HotpathContext(layers=1, maxTokens=16, **shape)
    try:
        with pytest.raises(hp.FieldfareError, match="experts"):
            ctx.loadRouterInt8(0, codes[:8], scales[:8], biases[:8])
        with pytest.raises(hp.FieldfareError, match="out of range"):
            ctx.loadRouterInt8(3, codes, scales, biases)
    finally:
        ctx.close()


def int8_projection(seed, rows, cols, amp):
    codes = (synth.uniform(seed, rows * cols, 0.0, 256.0).astype(np.int64).clip(0, 255)).astype(np.uint8)
    groups = cols // 64
    scales = synth.uniform(seed + 1, rows * groups, 0.5, 1.5).reshape(rows, groups) * np.float32(2 * amp / 255)
    biases = -np.float32(amp) * synth.uniform(seed + 2, rows * groups, 0.8, 1.2).reshape(rows, groups)
    return (codes.reshape(rows, cols), synth.bf16_bits(scales.astype(np.float32)),
            synth.bf16_bits(biases.astype(np.float32)))


@pytest.mark.parametrize("shape", SHAPES, ids=["toy", "benchmark"])
@pytest.mark.parametrize("rows", [1, 5, 40])
def test_int8_shared_ffn(oracle, shape, rows):
    """The INT8 affine shared FFN (Kernels/MoE/SharedExpertInt8.swift) against the oracle (same
    defined order: equal except where the two tanh implementations round an activation apart), and
    the whole layer with it against the layer put together from its parts, bit for bit."""
    from conftest import ELEMENTWISE_TOL, assert_layer_close
    hp = _hp()
    D, Fs, K = shape["d"], shape["sharedF"], shape["topK"]
    amp = 0.5 / np.sqrt(D)
    gate, up = int8_projection(0x80, Fs, D, amp), int8_projection(0x83, Fs, D, amp)
    down = int8_projection(0x86, D, Fs, 0.5 / np.sqrt(Fs))
    L = workload.make_layer(0x1A, 0, **shape)
    ctx = hp.HotpathContext(layers=1, maxTokens=64, **shape)
    try:
        ctx.loadLayer(0, L.blobs, L.layout.stride, L.layout.offsets)
        ctx.loadRouter(0, L.routerW)
        ctx.loadSharedInt8(0, gate, up, down)
        x = workload.make_tokens(0x1A, f"int8.shared{rows}", rows, D)
        xd = dev(x, ctx)
        shared = torch.zeros((rows, D), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillSharedExpert(ctx).encodeBlock(None, 0, xd, shared, rows)
        torch.cuda.synchronize()
        want = oracle.shared_ffn_int8(gate, up, down, x)
        assert_layer_close(hp.bf16_numpy(shared), want, oracle, f"int8 shared rows={rows}",
                           elementwise_tol=ELEMENTWISE_TOL)
        assert np.mean(hp.bf16_numpy(shared) != want) < 2e-2
        # the layer = router + routed experts + this shared FFN, against its parts
        y = ctx.moeLayer(0, xd)
        ids = torch.zeros((rows, K), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((rows, K), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillRouter(ctx).encodeGemma4Block(None, 0, xd, ids, w, rows)
        parts = torch.zeros((rows, D), dtype=torch.bfloat16, device=ctx.device)
        if rows == 1:
            hp.MoE(ctx).encodeRoutedPersistentGPUSlots(None, 0, ids, xd, w, shared, parts)
        else:
            partials = torch.zeros((rows * K, D), dtype=torch.bfloat16, device=ctx.device)
            routed = hp.PrefillGroupedRoutedMoE(ctx)
            if rows <= 16:
                routed.encodeVerifyBound(None, 0, xd, ids, partials, rows)
            else:
                routed.encodeStreamedBatched(None, 0, xd, ids, partials, rows)
            hp.PrefillMoE(ctx).encodeReduceTokenMajor(None, partials, w, parts, rows, residual=shared)
        torch.cuda.synchronize()
        assert torch.equal(y, parts)
        hx = torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
        hy = torch.empty((rows, D), dtype=torch.bfloat16).pin_memory()
        ctx.moeLayerHost(0, hx, hy)
        assert torch.equal(hy, y.cpu())
        assert ctx.info().deviceErrorFlag == 0
    finally:
        ctx.close()
