"""Parity of the CUDA library (through the C ABI) with the CPU oracle on the same seeded inputs.

Bit-exact: dequantized weights, router logits, top-K indices, pair grouping.
Tolerance (bf16 outputs; conftest.assert_layer_close): relative L2 <= 1e-2; max-abs <= 2e-2 as
written for the unit-scale variants (outputs of peak <= 1), and in units of the output peak at the
benchmark configurations' own scale.
"""
import ctypes
import os

import numpy as np
import pytest

from ane_fieldfare_b200 import gturbo, synth, workload
from conftest import ELEMENTWISE_TOL, LAYER_ELEMENTWISE_TOL, assert_layer_close, oracle_layer

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _hp():
    from ane_fieldfare_b200 import hotpath
    return hotpath


def make_ctx(L, max_tokens=16, layers=1):
    hp = _hp()
    ctx = hp.HotpathContext(layers=layers, experts=L.experts, d=L.d, f=L.f, sharedF=L.sharedF,
                            topK=L.topK, maxTokens=max_tokens)
    workload.load_layer(ctx, 0, L)
    return ctx


@pytest.fixture(scope="module")
def tiny():
    L = workload.make_layer(0x604, 0, experts=16, d=128, f=64, sharedF=192, topK=8, router_bias="normal")
    ctx = make_ctx(L)
    yield L, ctx
    ctx.close()


@pytest.fixture(scope="module")
def full():
    """One layer at the benchmark shape (D=2816, F=704, Fs=2112, 128 experts, top-8)."""
    L = workload.make_layer(0xB200, 0, router_bias="normal")
    ctx = make_ctx(L)
    yield L, ctx
    ctx.close()


def dev(bits, ctx):
    return _hp().bf16_tensor(bits, ctx.device)


def test_dequant_probe_is_bit_exact(tiny, full, oracle):
    for L, ctx in (tiny, full):
        for expert in (0, L.experts - 1, -1):
            blob = L.sharedBlob if expert < 0 else L.blobs[expert]
            lay = L.sharedLayout if expert < 0 else L.layout
            for role, name in enumerate(gturbo.ROLES):
                w, s, b = gturbo.sub_tensor(blob, lay, name)
                rows, cols = lay.matrix_shape(name)
                got = ctx.dequantProbe(0, expert, role).cpu().numpy()
                want = oracle.dequant_int4(np.ascontiguousarray(w), np.ascontiguousarray(s),
                                           np.ascontiguousarray(b), rows, cols)
                assert got.view(np.uint32).tobytes() == want.view(np.uint32).tobytes(), (expert, name)
                got16 = _hp().bf16_numpy(ctx.dequantProbe(0, expert, role, bf16=True))
                want16 = oracle.dequant_int4(np.ascontiguousarray(w), np.ascontiguousarray(s),
                                             np.ascontiguousarray(b), rows, cols, bf16=True)
                assert np.array_equal(got16, want16), (expert, name)


def test_dequant_probe_adversarial_scales(oracle):
    """Denormal, negative and huge scales/biases (the adversarial cases of
    Tests/ANEFieldfareUpstreamTests/Kernels/TensorCore/MPPPrefillInt4QMMTests.swift:75-144)."""
    L = workload.make_layer(5, 0, experts=4, d=128, f=64, sharedF=0, topK=2)
    lay = L.layout
    blobs = L.blobs.copy()
    w, s, b = gturbo.sub_tensor(blobs[1], lay, "gate")
    vals = np.array([1e-40, -3.5, 2.0 ** -20, 1e30, -1e-3, 0.0], dtype=np.float32)
    s[:] = synth.bf16_bits(np.resize(vals, s.shape))
    b[:] = synth.bf16_bits(np.resize(vals[::-1] * np.float32(3.0), b.shape))
    L.blobs = blobs
    ctx = make_ctx(L)
    try:
        got = ctx.dequantProbe(0, 1, 0).cpu().numpy()
        want = oracle.dequant_int4(np.ascontiguousarray(w), np.ascontiguousarray(s),
                                   np.ascontiguousarray(b), 64, 128)
        assert got.view(np.uint32).tobytes() == want.view(np.uint32).tobytes()
        got16 = _hp().bf16_numpy(ctx.dequantProbe(0, 1, 0, bf16=True))
        want16 = oracle.dequant_int4(np.ascontiguousarray(w), np.ascontiguousarray(s),
                                     np.ascontiguousarray(b), 64, 128, bf16=True)
        assert np.array_equal(got16, want16)
    finally:
        ctx.close()


@pytest.mark.parametrize("rows", [1, 3, 16])
def test_router_logits_and_indices_are_bit_exact(tiny, full, oracle, rows):
    hp = _hp()
    for L, ctx in (tiny, full):
        x = workload.make_tokens(21, f"router{rows}", rows, L.d)
        ids = torch.zeros((rows, L.topK), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((rows, L.topK), dtype=torch.bfloat16, device=ctx.device)
        logits = torch.zeros((rows, L.experts), dtype=torch.float32, device=ctx.device)
        hp.MoE(ctx).encodeRouterRowsGemma4(None, 0, dev(x, ctx), L.d, rows, ids, w, logits)
        torch.cuda.synchronize()
        ref_ids, ref_w, ref_logits = oracle.router_topk(oracle_layer(oracle, L), x)
        assert logits.cpu().numpy().view(np.uint32).tobytes() == ref_logits.view(np.uint32).tobytes()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        # weights: same formula, different exp -> 5e-3 as the reference's RouterTopKTests.swift:39-43
        dw = np.abs(oracle.bf16_to_float(hp.bf16_numpy(w)) - oracle.bf16_to_float(ref_w))
        assert dw.max() < 5e-3


def test_router_with_effective_scale_and_gain(oracle):
    """Per-input scale and per-expert gain, as MoE.encodeRouterGemma4 takes them
    (Kernels/MoE/MoE.swift:168-180); rows offset by 0.01*expert as in RouterTopKTests.swift:17-24."""
    hp = _hp()
    E, D, K = 16, 128, 8
    wr = synth.uniform(1, E * D, -0.05, 0.05).reshape(E, D) + \
        (np.arange(E, dtype=np.float32) * np.float32(0.01))[:, None]
    scale = synth.uniform(2, D, 0.5, 1.5) / np.float32(np.sqrt(D))
    gain = synth.uniform(3, E, 0.6, 1.4)
    x = synth.bf16_bits(synth.uniform(4, D, -1, 1))[None, :]
    L = workload.make_layer(5, 0, experts=E, d=D, f=64, sharedF=0, topK=K)
    ctx = hp.HotpathContext(layers=1, experts=E, d=D, f=64, sharedF=0, topK=K, maxTokens=4)
    try:
        ctx.loadLayer(0, L.blobs, L.layout.stride, L.layout.offsets)
        ctx.loadRouter(0, synth.bf16_bits(wr), effectiveScale=synth.bf16_bits(scale),
                       perExpertScale=synth.bf16_bits(gain))
        ld = oracle.LayerData(experts=L.blobs, stride=L.layout.stride, off=L.layout.offsets.as_tuple(),
                              E=E, D=D, F=64, K=K, router_w=synth.bf16_bits(wr),
                              router_scale=synth.bf16_bits(scale), gain=synth.bf16_bits(gain))
        ids = torch.zeros((1, K), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((1, K), dtype=torch.bfloat16, device=ctx.device)
        hp.MoE(ctx).encodeRouterGemma4(None, 0, dev(x, ctx), ids, w, topK=K)
        torch.cuda.synchronize()
        ref_ids, ref_w, _ = oracle.router_topk(ld, x)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        assert np.abs(oracle.bf16_to_float(hp.bf16_numpy(w)) - oracle.bf16_to_float(ref_w)).max() < 5e-3
    finally:
        ctx.close()


@pytest.mark.parametrize("rows", [1, 2, 4, 7, 16])
def test_multi_row_gemv_matches_and_rows_are_bitwise_single_row(oracle, rows):
    """DequantInt4GEMV.encodeRows: fp32 reference within 5e-3 (peak-relative) and row r bitwise
    equal to the one-row call (Tests/.../Kernels/Quant/DequantInt4SmallBatchTests.swift:17-79)."""
    hp = _hp()
    M, N = 200, 704
    p, s, b = synth.int4_matrix(31, "gemv", 1, M, N)
    p, s, b = p.reshape(M, N // 2), s.reshape(M, N // 64), b.reshape(M, N // 64)
    x = synth.bf16_bits(synth.uniform(32, rows * N, -1, 1)).reshape(rows, N)
    ctx = hp.HotpathContext(layers=1, experts=8, d=N, f=64, sharedF=0, topK=2, maxTokens=16)
    try:
        proj = hp.SharedExpertProjection(
            torch.from_numpy(p.copy()).to(ctx.device),
            dev(s, ctx), dev(b, ctx), M, N)
        xd = dev(x, ctx)
        y = torch.zeros((rows, M), dtype=torch.bfloat16, device=ctx.device)
        gemv = hp.DequantInt4GEMV(ctx)
        gemv.encodeRows(None, proj, xd, N, rows, y, M)
        torch.cuda.synchronize()
        got = oracle.bf16_to_float(hp.bf16_numpy(y))
        want = oracle.int4_gemv_rows(p, s, b, M, N, oracle.bf16_to_float(x))
        assert np.abs(got - want).max() / np.abs(want).max() < 5e-3
        for r in range(rows):
            y1 = torch.zeros((1, M), dtype=torch.bfloat16, device=ctx.device)
            gemv.encodeRows(None, proj, xd[r:r + 1].contiguous(), N, 1, y1, M)
            torch.cuda.synchronize()
            assert torch.equal(y1[0], y[r]), r
    finally:
        ctx.close()


@pytest.mark.parametrize("rows", [1, 5, 16])
def test_shared_ffn(tiny, full, oracle, rows):
    hp = _hp()
    for L, ctx in (tiny, full):
        x = workload.make_tokens(41, f"shared{rows}", rows, L.d)
        y = torch.zeros((rows, L.d), dtype=torch.bfloat16, device=ctx.device)
        hp.SharedExpertInt4(ctx).encode(None, 0, dev(x, ctx), y, rows=rows)
        torch.cuda.synchronize()
        want = oracle.shared_ffn(oracle_layer(oracle, L), x)
        assert_layer_close(hp.bf16_numpy(y), want, oracle, f"shared rows={rows}", elementwise_tol=ELEMENTWISE_TOL)


def test_single_expert_decode_config0(full, oracle):
    """Benchmark configuration 0: one INT4 expert, batch 1: down(gelu_tanh(gate x) * (up x))."""
    hp = _hp()
    L, ctx = full
    x = workload.make_tokens(50, "cfg0", 1, L.d)
    for expert in (0, 77):
        # the other seven slots name distinct experts with weight 0 (a token's routes are distinct)
        others = [e for e in range(8) if e != expert][:7]
        ids = torch.tensor([[expert] + others], dtype=torch.int32, device=ctx.device)
        w = dev(synth.bf16_bits(np.array([[1.0] + [0.0] * 7], dtype=np.float32)), ctx)
        y = torch.zeros((1, L.d), dtype=torch.bfloat16, device=ctx.device)
        hp.MoE(ctx).encodeRoutedPersistentGPUSlots(None, 0, ids, dev(x, ctx), w, None, y)
        torch.cuda.synchronize()
        want = oracle.bf16_bits(oracle.expert_ffn(L.blobs[expert], L.layout.offsets.as_tuple(), L.d,
                                                  L.f, x))
        assert_layer_close(hp.bf16_numpy(y), want, oracle, f"cfg0 expert {expert}", elementwise_tol=ELEMENTWISE_TOL)


def test_decode_routed_with_residual_and_split_equals_fused(tiny, full, oracle):
    """Routed decode onto a residual, and the fused block == router + shared + routed operators
    called one by one, bit for bit (the reference's "full == split" check,
    Tests/.../Kernels/MoE/MoEFusedFFNTests.swift:143-145)."""
    hp = _hp()
    for L, ctx in (tiny, full):
        x = workload.make_tokens(60, "decode", 1, L.d)
        xd = dev(x, ctx)
        y_fused = ctx.moeLayer(0, xd)
        ids = torch.zeros((1, L.topK), dtype=torch.int32, device=ctx.device)
        w = torch.zeros((1, L.topK), dtype=torch.bfloat16, device=ctx.device)
        moe = hp.MoE(ctx)
        moe.encodeRouterGemma4(None, 0, xd, ids, w, topK=L.topK)
        h1 = torch.zeros((1, L.d), dtype=torch.bfloat16, device=ctx.device)
        hp.SharedExpertInt4(ctx).encode(None, 0, xd, h1)
        y_split = torch.zeros((1, L.d), dtype=torch.bfloat16, device=ctx.device)
        moe.encodeRoutedPersistentGPUSlots(None, 0, ids, xd, w, h1, y_split)
        torch.cuda.synchronize()
        assert torch.equal(y_fused, y_split)
        want, _, ref_ids, _ = oracle.moe_layer(oracle_layer(oracle, L), x, oracle.MODE_DECODE)
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
        assert_layer_close(hp.bf16_numpy(y_fused), want, oracle, "decode layer", elementwise_tol=LAYER_ELEMENTWISE_TOL)


@pytest.mark.parametrize("rows", [1, 2, 3, 8, 16])
def test_verify_partials_and_layer(tiny, full, oracle, rows):
    """Grouped GEMV for a verify block: per-route partial rows, then the block output."""
    hp = _hp()
    for L, ctx in (tiny, full):
        ld = oracle_layer(oracle, L)
        x = workload.make_tokens(70, f"verify{rows}", rows, L.d)
        xd = dev(x, ctx)
        ref_ids, ref_w, _ = oracle.router_topk(ld, x)
        ids = torch.from_numpy(ref_ids.astype(np.int32)).to(ctx.device)
        partials = torch.full((rows * L.topK, L.d), -99.0, dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillGroupedRoutedMoE(ctx).encodeVerifyBound(None, 0, xd, ids, partials, rows)
        torch.cuda.synchronize()
        pairs, n = oracle.make_pairs(ref_ids, ref_w, rows, L.topK)
        want_p = oracle.route_partials(ld, x, pairs, n, rows)
        assert_layer_close(hp.bf16_numpy(partials), want_p, oracle, f"partials rows={rows}", elementwise_tol=ELEMENTWISE_TOL)
        if rows == 8:
            # input rows with a stride wider than the hidden size give the same bits
            wide = torch.zeros((rows, L.d + 64), dtype=torch.bfloat16, device=ctx.device)
            wide[:, :L.d] = xd
            partials2 = torch.full_like(partials, -99.0)
            hp.PrefillGroupedRoutedMoE(ctx).encodeVerifyBound(None, 0, wide, ids, partials2, rows,
                                                              hiddenStrideElements=L.d + 64)
            torch.cuda.synchronize()
            assert torch.equal(partials2, partials)
        if rows > 1:
            y = ctx.moeLayer(0, xd)
            torch.cuda.synchronize()
            want, _, _, _ = oracle.moe_layer(ld, x, oracle.MODE_PARTIALS)
            assert_layer_close(hp.bf16_numpy(y), want, oracle, f"verify layer rows={rows}", elementwise_tol=LAYER_ELEMENTWISE_TOL)
            # rows of a block are independent: row r of the block == the same row run alone
            if rows == 3:
                y2 = ctx.moeLayer(0, xd[:2].contiguous())
                assert torch.equal(y2, y[:2])


def test_reduce_token_major(tiny, oracle):
    """PrefillMoE.encodeReduceTokenMajor against the CPU reduce
    (Tests/.../Kernels/Prefill/PrefillMoETests.swift:8-64), with and without a residual."""
    hp = _hp()
    L, ctx = tiny
    T, K, D = 7, L.topK, L.d
    p = synth.bf16_bits(synth.uniform(1, T * K * D, -2, 2)).reshape(T * K, D)
    w = synth.bf16_bits(synth.uniform(2, T * K, 0, 1)).reshape(T, K)
    r = synth.bf16_bits(synth.uniform(3, T * D, -1, 1)).reshape(T, D)
    for residual in (None, r):
        h2 = torch.zeros((T, D), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillMoE(ctx).encodeReduceTokenMajor(
            None, dev(p, ctx), dev(w, ctx), h2, T,
            residual=None if residual is None else dev(residual, ctx))
        torch.cuda.synchronize()
        want = oracle.reduce_token_major(p, w, residual, T, K, D)
        assert np.array_equal(hp.bf16_numpy(h2), want)
        # the same rows lying in another order, found through a row index: the same bits
        perm = np.random.default_rng(5).permutation(T * K)
        inverse = np.empty(T * K, dtype=np.int32)
        inverse[perm] = np.arange(T * K, dtype=np.int32)   # row of route i in the shuffled buffer
        h3 = torch.zeros((T, D), dtype=torch.bfloat16, device=ctx.device)
        hp.PrefillMoE(ctx).encodeReduceTokenMajor(
            None, dev(np.ascontiguousarray(p[perm]), ctx), dev(w, ctx), h3, T,
            residual=None if residual is None else dev(residual, ctx),
            rowIndex=torch.from_numpy(inverse).to(ctx.device))
        torch.cuda.synchronize()
        assert np.array_equal(hp.bf16_numpy(h3), want)


def test_rmsnorm(tiny, oracle):
    hp = _hp()
    L, ctx = tiny
    x = workload.make_tokens(90, "norm", 9, L.d)
    w = synth.bf16_bits(synth.uniform(91, L.d, 0.5, 1.5))
    for weight in (None, w):
        y = ctx.rmsnorm(dev(x, ctx), None if weight is None else dev(weight, ctx), 1e-6)
        torch.cuda.synchronize()
        want = oracle.rmsnorm_bf16(x, weight, 1e-6, 9, L.d)
        got = oracle.bf16_to_float(hp.bf16_numpy(y))
        assert np.abs(got - oracle.bf16_to_float(want)).max() <= 2.0 ** -7 * np.abs(got).max()


def test_golden_fixture_on_gpu(oracle):
    """The committed tiny-layer fixture through the library."""
    hp = _hp()
    z = np.load(os.path.join(GOLDEN, "tiny_layer.npz"))
    L = workload.make_layer(int(z["root"]), 0, experts=int(z["experts"]), d=int(z["d"]),
                            f=int(z["f"]), sharedF=int(z["sharedF"]), topK=int(z["topK"]),
                            router_bias="normal")
    ctx = make_ctx(L)
    try:
        xd = dev(z["x"], ctx)
        ids = torch.zeros(z["ids"].shape, dtype=torch.int32, device=ctx.device)
        y = ctx.moeLayer(0, xd, ids=ids)
        torch.cuda.synchronize()
        assert np.array_equal(ids.cpu().numpy().astype(np.uint32), z["ids"])
        assert_layer_close(hp.bf16_numpy(y), z["y_partials_mode"], oracle, "golden block")
        y1 = ctx.moeLayer(0, xd[:1].contiguous())
        assert_layer_close(hp.bf16_numpy(y1), z["y_decode_mode_row0"], oracle, "golden decode")
    finally:
        ctx.close()


def test_host_entry_point_and_errors(tiny, oracle):
    hp = _hp()
    L, ctx = tiny
    x = workload.make_tokens(95, "host", 4, L.d)
    hx = torch.from_numpy(x.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
    hy = torch.zeros((4, L.d), dtype=torch.bfloat16).pin_memory()
    ctx.moeLayerHost(0, hx, hy)
    y = ctx.moeLayer(0, dev(x, ctx))
    torch.cuda.synchronize()
    assert torch.equal(hy, y.cpu())
    # one token: the row travels in the kernel parameters and the kernel writes a pinned output
    # itself; a pageable output takes the copy path.  Both equal the device-buffer call bit for bit,
    # also when called again (the mailbox epoch moves on).
    y1 = ctx.moeLayer(0, dev(x[2:3], ctx))
    torch.cuda.synchronize()
    for attempt in range(3):
        hy1 = torch.full((1, L.d), 3.0, dtype=torch.bfloat16).pin_memory()
        ctx.moeLayerHost(0, hx[2:3], hy1)
        assert torch.equal(hy1, y1.cpu()), attempt
    pageable_x = torch.from_numpy(x[2:3].view(np.int16).copy()).view(torch.bfloat16)
    pageable_y = torch.full((1, L.d), 3.0, dtype=torch.bfloat16)
    ctx.moeLayerHost(0, pageable_x, pageable_y)
    assert torch.equal(pageable_y, y1.cpu())
    with pytest.raises(hp.FieldfareError, match="exceed the context's maxTokens"):
        ctx.moeLayer(0, torch.zeros((17, L.d), dtype=torch.bfloat16, device=ctx.device))
    with pytest.raises(hp.FieldfareError, match="out of range"):
        ctx.moeLayer(3, dev(x, ctx))
    with pytest.raises(hp.FieldfareError, match="hidden stride is too small"):
        hp.PrefillGroupedRoutedMoE(ctx).encodeVerifyBound(
            None, 0, dev(x, ctx), torch.zeros((4, 8), dtype=torch.int32, device=ctx.device),
            torch.zeros((32, L.d), dtype=torch.bfloat16, device=ctx.device), 4, hiddenStrideElements=64)
    bad = gturbo.MoEExpertOffsets(*[v + 2 for v in L.layout.offsets.as_tuple()])
    with pytest.raises(hp.FieldfareError, match="does not match the required schema"):
        ctx.loadLayer(0, L.blobs, L.layout.stride, bad)
    with pytest.raises(hp.FieldfareError, match="truncated"):
        ctx.loadLayer(0, L.blobs[:2], L.layout.stride, L.layout.offsets)
    assert ctx.info().kernelLaunches > 0 and ctx.info().smCount > 0


def test_decode_kernel_replays_in_a_cuda_graph_and_mixes_with_other_modes(full, oracle):
    """The one-token kernel keeps its grid-wide counters in device memory with no host-side state:
    a captured graph of steps replays to the same bits, also when launches of its other modes
    (shared FFN alone, routed with given routes) run on the same context in between."""
    hp = _hp()
    L, ctx = full
    xs = [dev(workload.make_tokens(300 + i, "graph", 1, L.d), ctx) for i in range(4)]
    eager = [ctx.moeLayer(0, x).clone() for x in xs]
    torch.cuda.synchronize()
    ys = [torch.zeros((1, L.d), dtype=torch.bfloat16, device=ctx.device) for _ in xs]
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        for x, y in zip(xs, ys):
            ctx.moeLayer(0, x, y)
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for x, y in zip(xs, ys):
                ctx.moeLayer(0, x, y)
    h1 = torch.zeros((1, L.d), dtype=torch.bfloat16, device=ctx.device)
    ids = torch.zeros((1, L.topK), dtype=torch.int32, device=ctx.device)
    w = torch.zeros((1, L.topK), dtype=torch.bfloat16, device=ctx.device)
    for replay in range(20):
        for y in ys:
            y.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(ys, eager):
            assert torch.equal(got, want), replay
        # other modes of the same kernel in between
        hp.SharedExpertInt4(ctx).encode(None, 0, xs[replay % 4], h1)
        hp.MoE(ctx).encodeRouterGemma4(None, 0, xs[replay % 4], ids, w, topK=L.topK)
        hp.MoE(ctx).encodeRoutedPersistentGPUSlots(None, 0, ids, xs[replay % 4], w, h1, ys[0])
        torch.cuda.synchronize()
        assert torch.equal(ys[0], eager[replay % 4]), replay
    assert ctx.info().deviceErrorFlag == 0


@pytest.mark.parametrize("rows", [1, 7, 300])
def test_fused_steps_either_side_of_the_block(tiny, full, oracle, rows):
    """`prefill_post_attn_setup_block` and `prefill_layer_tail_block`
    (Metal/Prefill/prefill.metal:244-399) against the oracle.  Only the order of the RMS sums
    differs (a CTA-wide reduction here, one chain there), so results agree except where a value sits
    on a rounding boundary: at most one 16-bit step of the terms involved, in under one element
    in a hundred."""
    hp = _hp()
    for L, ctx in (tiny, full):
        D, eps = L.d, 1e-6
        mk = lambda seed, lo, hi, n: synth.bf16_bits(synth.uniform(seed, n, lo, hi))
        hidden = mk(51, -2, 2, rows * D).reshape(rows, D)
        attn = mk(52, -4, 4, rows * D).reshape(rows, D)
        w = [mk(53 + i, 0.5, 1.5, D) for i in range(5)]
        hd, dense, routed, router = (dev(hidden, ctx), *[torch.zeros((rows, D), dtype=torch.bfloat16, device=ctx.device)
                                                         for _ in range(3)])
        glue = hp.PrefillLayerGlue(ctx)
        glue.encodePostAttnSetupBlock(None, hd, dev(attn, ctx), dev(w[0], ctx), dev(w[1], ctx), dev(w[2], ctx), eps,
                                      dense, routed, router)
        h2 = mk(60, -6, 6, rows * D).reshape(rows, D)
        h1 = mk(61, -2, 2, rows * D).reshape(rows, D)
        tail = dev(hidden, ctx)
        glue.encodeLayerTailBlock(None, dev(h2, ctx), dev(h1, ctx), tail, dev(w[3], ctx), dev(w[4], ctx), eps, 0.7071)
        torch.cuda.synchronize()
        want = list(oracle.post_attn_setup(hidden, attn, w[0], w[1], w[2], eps))
        want.append(oracle.layer_tail(h2, h1, hidden, w[3], w[4], eps, 0.7071))
        for name, got, ref in zip(("hidden", "dense_x", "routed_x", "router_x", "tail"),
                                  (hd, dense, routed, router, tail), want):
            g, r = oracle.bf16_to_float(hp.bf16_numpy(got)), oracle.bf16_to_float(ref)
            # one 16-bit step of the larger of the value and the terms it was summed from (the sums
            # `hidden + a` and `hidden + u` cancel, their terms are of order one)
            step = np.maximum(np.abs(r), 4.0) * 2.0 ** -7   # the normalized terms reach about 4 here
            assert np.all(np.abs(g - r) <= step * 1.01), (name, float(np.abs(g - r).max()))
            assert np.mean(g != r) < 1e-2, (name, float(np.mean(g != r)))
