"""Pins the CPU oracle against the known answers the reference's own tests hold for this path,
and against the committed golden fixtures.  No GPU."""
import ctypes
import math
import os

import numpy as np
import pytest

from ane_fieldfare_b200 import gturbo, synth, workload
from conftest import oracle_layer

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_bf16_encode_is_round_half_even_of_top_16_bits(oracle):
    # Sources/ANEFieldfareHotpath/Infrastructure/ModelIO/Quantization.swift:9-20
    L = oracle.lib()
    assert L.ffo_bf16_bits(1.0) == 0x3F80
    assert L.ffo_bf16_bits(-2.0) == 0xC000
    # 1 + 2^-8 is exactly halfway between 0x3F80 and 0x3F81 -> even (0x3F80)
    assert L.ffo_bf16_bits(1.0 + 2.0 ** -8) == 0x3F80
    # 1 + 3*2^-8 is halfway between 0x3F81 and 0x3F82 -> even (0x3F82)
    assert L.ffo_bf16_bits(1.0 + 3 * 2.0 ** -8) == 0x3F82
    assert L.ffo_bf16_bits(1.0 + 2.0 ** -8 + 2.0 ** -20) == 0x3F81
    assert L.ffo_bf16_to_float(0x3F80) == 1.0
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    assert (oracle.bf16_bits(x) == synth.bf16_bits(x)).all()
    assert (oracle.bf16_to_float(oracle.bf16_bits(x)) == synth.bf16_to_float(synth.bf16_bits(x))).all()
    # the ANE carrier test builds bf16 by truncation of exactly representable values
    # (Tests/ANEFieldfareHotpathTests/ANEQuantizedCarrierTests.swift:24-27): same bits here
    for g in range(9):
        scale = np.float32(1 + g % 3) / np.float32(512)
        assert L.ffo_bf16_bits(float(scale)) == (np.float32(scale).view(np.uint32) >> 16)


def test_splitmix64_matches_published_constants_and_numpy_port(oracle):
    # Tests/Support/Validation/PRNG/SplitMix64.swift:9-21; first outputs for seed 0 are the
    # published SplitMix64 test vector.
    got = oracle.splitmix64_fill(0, 3)
    assert [int(v) for v in got] == [0xE220A8397B1DCDAF, 0x6E789E6AA1B965F4, 0x06C45D188009454F]
    for seed in (0, 0xA5B61234, 2 ** 64 - 1):
        assert (oracle.splitmix64_fill(seed, 257) == synth.splitmix64(seed, 257)).all()
    assert (synth.splitmix64(9, 10, start=5) == synth.splitmix64(9, 15)[5:]).all()
    state = ctypes.c_uint64(77)
    u = [oracle.lib().ffo_splitmix64_uniform(ctypes.byref(state), -0.4, 0.4) for _ in range(64)]
    assert np.array_equal(np.array(u, dtype=np.float32), synth.uniform(77, 64, -0.4, 0.4))
    assert all(-0.4 <= v < 0.4 for v in u)


def test_seedtree_key_is_fnv1a_xor_root(oracle):
    # Tests/Support/Validation/PRNG/SeedTree.swift:12-19
    L = oracle.lib()
    assert L.ffo_seedtree_key(0, b"") == 0xCBF29CE484222325
    assert L.ffo_seedtree_key(0, b"a") == 0xAF63DC4C8601EC8C  # FNV-1a 64 of "a"
    for root, label in ((0x604, "shared-expert-int4"), (1, "layer0.routed.gate.q")):
        assert L.ffo_seedtree_key(root, label.encode()) == synth.seedtree_key(root, label)


def test_int4_nibble_order_and_quantizer_roundtrip(oracle):
    # Tests/ANEFieldfareUpstreamTests/Infrastructure/ModelIO/QuantizationAffineTests.swift:8-29
    row = np.array([0.10 + k * 0.01 for k in range(64)] + [-0.50 - k * 0.005 for k in range(64)],
                   dtype=np.float32)
    packed, scales, biases = oracle.quantize_int4_rows(row[None, :])
    assert packed.shape == (1, 64) and scales.shape == (1, 2) and biases.shape == (1, 2)
    back = oracle.dequant_int4(packed, scales, biases, 1, 128)[0]
    assert np.abs(back - row).max() < 0.025
    # low nibble = even index (Tests/Support/Validation/Reference/Quant/AffineQuantization.swift:15)
    w = np.zeros((1, 32), dtype=np.uint8)
    w[0, 0] = 0x21
    w[0, 1] = 0xF0
    one = synth.bf16_bits(np.array([[1.0]], dtype=np.float32))
    zero = synth.bf16_bits(np.array([[0.0]], dtype=np.float32))
    out = oracle.dequant_int4(w, one, zero, 1, 64)[0]
    assert list(out[:4]) == [1.0, 2.0, 0.0, 15.0]
    # constant group: scale 1, bias = value (AffineQuantization.swift:42-46)
    p, s, b = oracle.quantize_int4_rows(np.full((1, 64), 0.375, dtype=np.float32))
    assert oracle.bf16_to_float(s)[0, 0] == 1.0 and oracle.bf16_to_float(b)[0, 0] == 0.375
    assert (oracle.dequant_int4(p, s, b, 1, 64) == 0.375).all()


def test_expert_blob_offsets_match_reference_constants():
    # Tests/ANEFieldfareHotpathTests/ANEQuantizedCarrierTests.swift:10-11,18
    lay = gturbo.expert_layout(2816, 704)
    o = lay.offsets
    assert [o.gateWOff, o.upWOff, o.downWOff] == [0, 1_115_136, 2_230_272]
    assert [o.gateSOff, o.upSOff, o.downSOff] == [991_232, 2_106_368, 3_221_504]
    assert [o.gateBOff, o.upBOff, o.downBOff] == [1_053_184, 2_168_320, 3_283_456]
    assert lay.stride == 3_358_720 and lay.payload == 3_345_408
    assert ctypes.sizeof(gturbo.MoEExpertOffsets) == 36


def test_ane_carrier_expansion_formula(oracle):
    # Weights of Tests/ANEFieldfareHotpathTests/ANEQuantizedCarrierTests.swift:20-33 on a reduced
    # shape: code = (i/17 + i*7 + slot*3 + m*5) % 16, scale = (1 + (g+slot)%3)/512,
    # bias = scale*(-7 + ((g+m)%5)/4); the expansion must equal code*scale + bias exactly.
    d, f, slot, m = 128, 64, 1, 2
    n = d * f
    codes = np.array([(i // 17 + i * 7 + slot * 3 + m * 5) % 16 for i in range(n)], dtype=np.uint8)
    packed = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8)
    g = np.arange(n // 64)
    scale = ((1 + (g + slot) % 3).astype(np.float32) / np.float32(512))
    bias = scale * (np.float32(-7) + ((g + m) % 5).astype(np.float32) / np.float32(4))
    s_bits = (scale.view(np.uint32) >> 16).astype(np.uint16)
    b_bits = (bias.view(np.uint32) >> 16).astype(np.uint16)
    out = oracle.dequant_int4(packed, s_bits, b_bits, d, f).reshape(-1)
    expect = codes.astype(np.float32) * np.repeat(synth.bf16_to_float(s_bits), 64) + \
        np.repeat(synth.bf16_to_float(b_bits), 64)
    assert np.array_equal(out, expect.astype(np.float32))


def _pairs(oracle, rows):
    arr = (oracle.Pair * len(rows))()
    for i, (t, e, r, w) in enumerate(rows):
        arr[i] = oracle.Pair(t, e, r, w)
    return arr


def test_grouping_known_answers(oracle):
    # Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillMoEGroupingTests.swift:6-50
    rows = [(0, 3, 0, 10), (0, 1, 1, 11), (0, 4, 2, 12), (1, 1, 0, 13), (1, 3, 1, 14), (1, 2, 2, 15),
            (2, 4, 0, 16), (2, 3, 1, 17), (2, 1, 2, 18), (3, 5, 0, 19), (3, 1, 1, 20), (3, 4, 2, 21)]
    rows = rows[::-1]
    sp, groups, tiles = oracle.group_pairs(_pairs(oracle, rows), len(rows), 4, 3, 6, 2)
    assert [p.expert for p in sp] == [1, 1, 1, 1, 2, 3, 3, 3, 4, 4, 4, 5]
    assert [[p.token, p.rank] for p in sp] == [[0, 1], [1, 0], [2, 2], [3, 1], [1, 2], [0, 0], [1, 1],
                                               [2, 1], [0, 2], [2, 0], [3, 2], [3, 0]]
    assert [p.weight_bits for p in sp] == [11, 13, 18, 20, 15, 10, 14, 17, 12, 16, 21, 19]
    assert [(g.expert, g.pair_start, g.pair_count) for g in groups] == \
        [(1, 0, 4), (2, 4, 1), (3, 5, 3), (4, 8, 3), (5, 11, 1)]
    assert [(t.group_start, t.group_count, t.pair_start, t.pair_count) for t in tiles] == \
        [(0, 2, 0, 5), (2, 2, 5, 6), (4, 1, 11, 1)]


def test_grouping_with_expert_sort_keys_and_rejection(oracle):
    # PrefillMoEGroupingTests.swift:52-82 and :84-96
    rows = [(0, 1, 0, 10), (0, 2, 1, 20), (1, 3, 0, 30), (1, 1, 1, 11), (2, 2, 0, 21), (2, 3, 1, 31)]
    sp, groups, tiles = oracle.group_pairs(_pairs(oracle, rows), 6, 3, 2, 4, 2, [0, 30, 10, 20])
    assert [g.expert for g in groups] == [2, 3, 1]
    assert [p.expert for p in sp] == [2, 2, 3, 3, 1, 1]
    assert [(t.group_start, t.group_count, t.pair_start, t.pair_count) for t in tiles] == \
        [(0, 2, 0, 4), (2, 1, 4, 2)]
    with pytest.raises(ValueError, match="route expert 2 is out of range"):
        oracle.group_pairs(_pairs(oracle, [(0, 2, 0, 1)]), 1, 1, 1, 2, 1)


def test_make_pairs_is_token_major(oracle):
    # Sources/ANEFieldfareHotpath/Kernels/Prefill/MoE/PrefillRouter.swift:75-95
    ids = np.array([[5, 1], [0, 3]], dtype=np.uint32)
    w = np.array([[100, 101], [102, 103]], dtype=np.uint16)
    pairs, n = oracle.make_pairs(ids, w, 2, 2)
    assert n == 4
    assert [(p.token, p.expert, p.rank, p.weight_bits) for p in list(pairs)[:4]] == \
        [(0, 5, 0, 100), (0, 1, 1, 101), (1, 0, 0, 102), (1, 3, 1, 103)]


def test_router_topk_on_separated_logits(oracle):
    # The reference checks index equality on rows offset by 0.01*expert
    # (Tests/ANEFieldfareUpstreamTests/Kernels/MoE/RouterTopKTests.swift:17-44): the selection is
    # the eight largest in descending order, weights a softmax over them times the gain.
    E, D, K = 16, 128, 8
    seed = 0xA5B61234
    w = synth.uniform(seed, E * D, -0.05, 0.05).reshape(E, D) + \
        (np.arange(E, dtype=np.float32) * np.float32(0.01))[:, None]
    x = synth.uniform(seed ^ 1, D, -1.0, 1.0)
    gain = synth.uniform(seed ^ 2, E, 0.6, 1.4)
    wb, xb, gb = synth.bf16_bits(w), synth.bf16_bits(x), synth.bf16_bits(gain)
    dummy = np.zeros((1, 16384), dtype=np.uint8)
    layer = oracle.LayerData(experts=dummy, stride=16384, off=(0,) * 9, E=E, D=D, F=64, K=K,
                             router_w=wb, gain=gb)
    ids, weights, logits = oracle.router_topk(layer, xb[None, :])
    exact = synth.bf16_to_float(wb).astype(np.float64) @ synth.bf16_to_float(xb).astype(np.float64)
    assert np.abs(logits[0] - exact).max() < 1e-5
    order = sorted(range(E), key=lambda e: (-logits[0][e], e))[:K]
    assert list(ids[0]) == order
    sel = logits[0][order].astype(np.float64)
    soft = np.exp(sel - sel[0]) / np.exp(sel - sel[0]).sum() * synth.bf16_to_float(gb)[order]
    assert np.abs(oracle.bf16_to_float(weights)[0] - soft).max() < 5e-3


def test_topk_ties_take_the_lower_expert_and_skip_non_finite(oracle):
    # Sources/ANEFieldfareHotpath/Metal/MoE/moe.metal:286-303 (equal score -> lower id);
    # :196-201 (-inf is never taken; empty slots report expert 0)
    logits = np.array([1.0, 3.0, 3.0, -np.inf, 2.0, 3.0], dtype=np.float32)
    ids = np.zeros(4, dtype=np.uint32)
    w = np.zeros(4, dtype=np.uint16)
    oracle.lib().ffo_topk(logits.ctypes.data_as(ctypes.c_void_p), 6, None, 4,
                          ids.ctypes.data_as(ctypes.c_void_p), w.ctypes.data_as(ctypes.c_void_p), None)
    assert list(ids) == [1, 2, 5, 4]
    few = np.array([0.5, -np.inf, -np.inf], dtype=np.float32)
    ids3 = np.zeros(3, dtype=np.uint32)
    w3 = np.zeros(3, dtype=np.uint16)
    oracle.lib().ffo_topk(few.ctypes.data_as(ctypes.c_void_p), 3, None, 3,
                          ids3.ctypes.data_as(ctypes.c_void_p), w3.ctypes.data_as(ctypes.c_void_p), None)
    assert list(ids3) == [0, 0, 0] and oracle.bf16_to_float(w3)[0] == 1.0


def test_scalar_dot_and_rows_gemv_agree_bitwise(oracle):
    # Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillGroupedRoutedMoETests.swift:153-178
    p, s, b = synth.int4_matrix(3, "m", 1, 24, 192)
    p, s, b = p.reshape(24, 96), s.reshape(24, 3), b.reshape(24, 3)
    x = synth.uniform(5, 5 * 192, -1, 1).reshape(5, 192)
    y = oracle.int4_gemv_rows(p, s, b, 24, 192, x)
    for r in range(5):
        for o in (0, 7, 23):
            assert y[r, o] == np.float32(oracle.int4_dot(p, s, b, o, 192, x[r]))
    w = oracle.dequant_int4(p, s, b, 24, 192).astype(np.float64)
    assert np.abs(y - x.astype(np.float64) @ w.T).max() < 1e-4


def test_gelu_matches_closed_form(oracle):
    # Tests/Support/Validation/Reference/MoE/Moe.swift:13-24
    for v in (-6.0, -1.0, -0.1, 0.0, 0.3, 2.0, 9.0):
        want = 0.5 * v * (1 + math.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
        assert abs(oracle.lib().ffo_gelu_tanh(v) - want) < 1e-6 * max(1.0, abs(v))


def test_reduce_token_major_small(oracle):
    # Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillMoETests.swift:46-64
    T, K, D = 3, 4, 64
    p = synth.bf16_bits(synth.uniform(1, T * K * D, -2, 2)).reshape(T * K, D)
    w = synth.bf16_bits(synth.uniform(2, T * K, 0, 1)).reshape(T, K)
    out = oracle.bf16_to_float(oracle.reduce_token_major(p, w, None, T, K, D))
    want = np.einsum("tk,tkd->td", synth.bf16_to_float(w).astype(np.float64),
                     synth.bf16_to_float(p).reshape(T, K, D).astype(np.float64))
    # one bf16 rounding of the fp32 sum (the reference's 2e-3 bound is for fp16 outputs)
    assert (np.abs(out - want) <= 2.0 ** -8 * np.abs(want) + 1e-6).all()


def test_rmsnorm_reference(oracle):
    # Tests/Support/Validation/Reference/Primitives/RmsNorm.swift:8-39
    x = synth.uniform(3, 256, -2, 2)
    w = synth.uniform(4, 256, 0.5, 1.5)
    y = np.empty(256, dtype=np.float32)
    oracle.lib().ffo_rmsnorm(x.ctypes.data_as(ctypes.c_void_p), w.ctypes.data_as(ctypes.c_void_p),
                             ctypes.c_float(1e-6), 256, y.ctypes.data_as(ctypes.c_void_p))
    want = x.astype(np.float64) * w / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-6)
    assert np.abs(y - want).max() < 1e-5


def test_decode_and_partials_modes_agree_within_rounding(oracle):
    L = workload.make_layer(11, 0, experts=8, d=128, f=64, sharedF=128, topK=4)
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(11, "x", 5, 128)
    y0, y0f, ids0, w0 = oracle.moe_layer(ld, x, oracle.MODE_DECODE)
    y1, y1f, ids1, w1 = oracle.moe_layer(ld, x, oracle.MODE_PARTIALS)
    assert np.array_equal(ids0, ids1) and np.array_equal(w0, w1)
    assert np.abs(y0f - y1f).max() < 2e-3
    # split operators reproduce the fused layer bit for bit
    pairs, n = oracle.make_pairs(ids1, w1, 5, 4)
    partials = oracle.route_partials(ld, x, pairs, n, 5)
    h1 = oracle.shared_ffn(ld, x)
    assert np.array_equal(oracle.reduce_token_major(partials, w1, h1, 5, 4, 128), y1)


def _bf16_round64(v):
    """float64 array -> nearest bf16 (ties to even), returned as float64."""
    f = np.asarray(v, dtype=np.float64).astype(np.float32)
    return synth.bf16_to_float(synth.bf16_bits(f)).astype(np.float64)


def _dense(blob, lay, role):
    w, s, b = gturbo.sub_tensor(blob, lay, role)
    rows, cols = lay.matrix_shape(role)
    q = np.stack([w & 0x0F, w >> 4], axis=-1).reshape(rows, cols).astype(np.float64)
    return q * np.repeat(synth.bf16_to_float(s).astype(np.float64), 64, axis=1) + \
        np.repeat(synth.bf16_to_float(b).astype(np.float64), 64, axis=1)


def _ffn64(blob, lay, x, round_gate_up):
    g, u = _dense(blob, lay, "gate") @ x, _dense(blob, lay, "up") @ x
    if round_gate_up:
        g, u = _bf16_round64(g), _bf16_round64(u)
    gelu = 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    return _dense(blob, lay, "down") @ _bf16_round64(gelu * u)


def test_whole_layer_against_float64_model(oracle):
    """ffo_moe_layer end to end against an independent float64 statement of the same layer with the
    same rounding points (Tests/Support/Validation/Reference/MoE/Moe.swift:26-78 for the routed
    sum; shared FFN rounding as Metal/MoE/moe.metal:548-570): catches a misplaced rounding, a wrong
    slot order or weight pairing, which the per-function pins cannot see."""
    L = workload.make_layer(0x64, 0, experts=16, d=128, f=64, sharedF=192, topK=8, router_bias="normal")
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(0x64, "x", 4, 128)
    xf = synth.bf16_to_float(x).astype(np.float64)
    for mode in (oracle.MODE_DECODE, oracle.MODE_PARTIALS):
        y, y32, ids, w = oracle.moe_layer(ld, x, mode)
        wf = synth.bf16_to_float(w).astype(np.float64)
        want = np.zeros((4, 128))
        for t in range(4):
            h1 = _bf16_round64(_ffn64(L.sharedBlob, L.sharedLayout, xf[t], True))
            acc = h1.copy() if mode == oracle.MODE_DECODE else np.zeros(128)
            for r in range(8):
                v = _ffn64(L.blobs[ids[t, r]], L.layout, xf[t], False)
                acc += wf[t, r] * (v if mode == oracle.MODE_DECODE else _bf16_round64(v))
            want[t] = acc if mode == oracle.MODE_DECODE else acc + h1
        rel = np.linalg.norm(y32 - want) / np.linalg.norm(want)
        # fp32 accumulation against float64, plus the rare intermediate that rounds to the other
        # bf16 neighbour: a misplaced rounding point or a wrong slot pairing gives >= 1e-3
        assert rel < 3e-4, (mode, rel)
        assert np.abs(oracle.bf16_to_float(y) - _bf16_round64(want)).max() <= \
            2.0 ** -7 * np.abs(want).max(), mode


def test_stack_is_rmsnorm_then_layer_per_layer(oracle):
    """ffo_moe_stack == x <- moe_layer_l(rmsnorm(x)) composed from the pinned pieces, bit for bit,
    with every layer's routes reported."""
    layers = [workload.make_layer(0x57AC, i, experts=16, d=128, f=64, sharedF=192, topK=8,
                                  router_bias="normal") for i in range(3)]
    lds = [oracle_layer(oracle, L) for L in layers]
    for tokens, mode in ((1, oracle.MODE_DECODE), (5, oracle.MODE_PARTIALS)):
        x = workload.make_tokens(0x57AC, f"x{tokens}", tokens, 128)
        y, ids = oracle.moe_stack(lds, x, 1e-6, mode)
        cur = x
        for i, ld in enumerate(lds):
            normed = oracle.rmsnorm_bf16(cur, None, 1e-6, tokens, 128)
            cur, _, want_ids, _ = oracle.moe_layer(ld, normed, mode)
            assert np.array_equal(ids[i], want_ids)
        assert np.array_equal(y, cur)
        # the norm keeps every block's input at unit RMS
        assert abs(np.sqrt((oracle.bf16_to_float(normed).astype(np.float64) ** 2).mean()) - 1.0) < 1e-2


def test_down_shift_scales_the_layer_output_exactly(oracle):
    """workload.make_layer(down_shift=n) multiplies the outputs by 2^-n exactly (only exponents of
    the down projections' scales and biases change): the unit-scale variants of the benchmark
    configurations are the same arithmetic in other units."""
    kw = dict(experts=8, d=128, f=64, sharedF=128, topK=4)
    a = workload.make_layer(31, 0, **kw)
    b = workload.make_layer(31, 0, down_shift=5, **kw)
    x = workload.make_tokens(31, "x", 3, 128)
    ya, _, ida, _ = oracle.moe_layer(oracle_layer(oracle, a), x, oracle.MODE_PARTIALS)
    yb, _, idb, _ = oracle.moe_layer(oracle_layer(oracle, b), x, oracle.MODE_PARTIALS)
    assert np.array_equal(ida, idb)
    assert np.array_equal(oracle.bf16_to_float(ya), oracle.bf16_to_float(yb) * np.float32(32.0))


def test_bf16_weight_mode_multiplies_the_rounded_weights(oracle):
    """FFO_MODE_BF16_WEIGHTS = the same layer with every weight rounded once to bf16 (what
    ffo_dequant_int4_bf16 returns and the tensor-core prefill path multiplies): checked against a
    float64 product with those weights, and against the fp32-weight layer, from which it differs by
    the weights' rounding only (~2^-9 relative per weight)."""
    L = workload.make_layer(0x16B, 0, experts=8, d=128, f=64, sharedF=128, topK=4)
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(0x16B, "x", 6, 128)
    xf = synth.bf16_to_float(x).astype(np.float64)
    got = oracle.bf16_to_float(oracle.shared_ffn(ld, x, bf16_weights=True)).astype(np.float64)
    mats = {}
    for role in gturbo.ROLES:
        w, s, b = gturbo.sub_tensor(L.sharedBlob, L.sharedLayout, role)
        rows, cols = L.sharedLayout.matrix_shape(role)
        mats[role] = synth.bf16_to_float(oracle.dequant_int4(
            np.ascontiguousarray(w), np.ascontiguousarray(s), np.ascontiguousarray(b), rows, cols,
            bf16=True)).astype(np.float64)
    g, u = _bf16_round64(xf @ mats["gate"].T), _bf16_round64(xf @ mats["up"].T)
    act = _bf16_round64(0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * u)
    want = act @ mats["down"].T
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 3e-3  # bf16 output rounding
    y32, _, ids32, _ = oracle.moe_layer(ld, x, oracle.MODE_PARTIALS)
    y16, _, ids16, _ = oracle.moe_layer(ld, x, oracle.MODE_PARTIALS | oracle.MODE_BF16_WEIGHTS)
    assert np.array_equal(ids32, ids16)
    a, b = oracle.bf16_to_float(y32).astype(np.float64), oracle.bf16_to_float(y16).astype(np.float64)
    rel = np.linalg.norm(a - b) / np.linalg.norm(a)
    assert 1e-4 < rel < 1e-2, rel


def test_golden_fixture(oracle):
    """Committed oracle outputs for a tiny seeded layer (tests/golden/make_golden.py): guards the
    oracle itself against drift.  The reference holds no golden vectors for this path."""
    z = np.load(os.path.join(GOLDEN, "tiny_layer.npz"))
    L = workload.make_layer(int(z["root"]), 0, experts=int(z["experts"]), d=int(z["d"]),
                            f=int(z["f"]), sharedF=int(z["sharedF"]), topK=int(z["topK"]),
                            router_bias="normal")
    ld = oracle_layer(oracle, L)
    x = workload.make_tokens(int(z["root"]), "x", int(z["tokens"]), int(z["d"]))
    assert np.array_equal(x, z["x"])
    assert np.array_equal(L.blobs[:, :L.layout.payload], z["blobs"])
    y, _, ids, w = oracle.moe_layer(ld, x, oracle.MODE_PARTIALS)
    assert np.array_equal(ids, z["ids"]) and np.array_equal(w, z["weights"])
    assert np.array_equal(y, z["y_partials_mode"])
    y1, _, _, _ = oracle.moe_layer(ld, x[:1], oracle.MODE_DECODE)
    assert np.array_equal(y1, z["y_decode_mode_row0"])


def test_int8_router_against_float64(oracle):
    """ffo_router_logits_int8 (Metal/MoE/moe.metal:65-103) against a float64 evaluation of
    sum_k (q_k s_g + b_g) x_k e_k: equal within fp32 accumulation error, and the top-K indices
    agree wherever the float64 scores are separated by more than that error."""
    rng = np.random.default_rng(31)
    E, D, K = 32, 256, 8
    codes = rng.integers(0, 256, size=(E, D), dtype=np.uint8)
    scales = synth.bf16_bits((rng.uniform(0.5, 1.5, size=(E, D // 64)) * 2e-3).astype(np.float32))
    biases = synth.bf16_bits((-rng.uniform(0.2, 0.3, size=(E, D // 64))).astype(np.float32))
    eff = synth.bf16_bits(rng.uniform(0.5, 1.5, size=D).astype(np.float32))
    bias = rng.uniform(-0.1, 0.1, size=E).astype(np.float32)
    x = synth.bf16_bits(rng.uniform(-1, 1, size=(5, D)).astype(np.float32))
    ids, w, logits = oracle.router_topk_int8(codes, scales, biases, x, K, effective_scale=eff, logit_bias=bias)
    s64 = np.repeat(oracle.bf16_to_float(scales).astype(np.float64), 64, axis=1)
    b64 = np.repeat(oracle.bf16_to_float(biases).astype(np.float64), 64, axis=1)
    w64 = codes.astype(np.float64) * s64 + b64
    xe = oracle.bf16_to_float(x).astype(np.float64) * oracle.bf16_to_float(eff).astype(np.float64)[None, :]
    want = xe @ w64.T + bias.astype(np.float64)[None, :]
    scale = np.abs(xe) @ np.abs(w64).T
    assert np.all(np.abs(logits - want) <= 4e-6 * scale + 1e-6)
    for t in range(x.shape[0]):
        order = np.argsort(-want[t], kind="stable")
        gaps = np.abs(np.diff(want[t][order][:K + 1]))
        if gaps.min() > 1e-4:
            assert list(ids[t]) == list(order[:K])
    assert np.all(np.abs(oracle.bf16_to_float(w).sum(axis=1) - 1.0) < 2e-2)


def test_fused_glue_steps_against_float64(oracle):
    """ffo_post_attn_setup / ffo_layer_tail (Metal/Prefill/prefill.metal:244-399) against a float64
    evaluation of the same formulas with the same 16-bit rounding points: the RMS sums are the only
    place where precision differs, so every output agrees to within one 16-bit step of its value."""
    rng = np.random.default_rng(41)
    T, D, eps = 5, 256, 1e-6
    bits = lambda a: synth.bf16_bits(np.asarray(a, dtype=np.float32))
    f64 = lambda b: oracle.bf16_to_float(b).astype(np.float64)
    r16 = lambda a: f64(bits(a))
    hidden, attn = bits(rng.normal(0, 1, (T, D))), bits(rng.normal(0, 2, (T, D)))
    w = [bits(rng.uniform(0.5, 1.5, D)) for _ in range(5)]
    inv = lambda a: 1.0 / np.sqrt((a * a).mean(axis=1, keepdims=True) + eps)

    h, dense, routed, router = oracle.post_attn_setup(hidden, attn, w[0], w[1], w[2], eps)
    a = r16(f64(attn) * inv(f64(attn)) * f64(w[0]))
    h64 = r16(f64(hidden) + a)
    n = h64 * inv(h64)
    step = lambda ref: np.maximum(np.abs(ref), 1e-30) * 2.0 ** -7   # one bf16 step of the value
    for got, want in ((h, h64), (dense, n * f64(w[1])), (routed, n * f64(w[2])), (router, n)):
        assert np.all(np.abs(f64(got) - want) <= step(want))

    h2, h1 = bits(rng.normal(0, 3, (T, D))), bits(rng.normal(0, 1, (T, D)))
    out = oracle.layer_tail(h2, h1, hidden, w[3], w[4], eps, 0.7071)
    t = r16(f64(h2) * inv(f64(h2)) * f64(w[3]))
    h12 = r16(f64(h1) + t)
    u = r16(h12 * inv(h12) * f64(w[4]))
    want = r16(f64(hidden) + u) * f64(bits([0.7071]))[0]
    assert np.all(np.abs(f64(out) - want) <= 2 * step(want))


def test_int8_shared_ffn_against_float64(oracle):
    """ffo_shared_ffn_int8 (Kernels/MoE/SharedExpertInt8.swift; Metal/Quant/dequant_int8.metal:41-138)
    against float64 with the same 16-bit rounding points."""
    rng = np.random.default_rng(43)
    D, Fs, T = 128, 192, 4

    def proj(rows, cols, amp):
        codes = rng.integers(0, 256, size=(rows, cols), dtype=np.uint8)
        s = synth.bf16_bits((rng.uniform(0.5, 1.5, (rows, cols // 64)) * 2 * amp / 255).astype(np.float32))
        b = synth.bf16_bits((-amp * rng.uniform(0.8, 1.2, (rows, cols // 64))).astype(np.float32))
        return codes, s, b

    gate, up, down = proj(Fs, D, 0.2), proj(Fs, D, 0.2), proj(D, Fs, 0.2)
    x = synth.bf16_bits(rng.uniform(-1, 1, (T, D)).astype(np.float32))
    y = oracle.shared_ffn_int8(gate, up, down, x)
    f64 = lambda b: oracle.bf16_to_float(b).astype(np.float64)
    r16 = lambda a: f64(synth.bf16_bits(np.asarray(a, dtype=np.float32)))
    w = lambda p: p[0].astype(np.float64) * np.repeat(f64(p[1]), 64, axis=1) + np.repeat(f64(p[2]), 64, axis=1)
    g, u = r16(f64(x) @ w(gate).T), r16(f64(x) @ w(up).T)
    act = r16(0.5 * g * (1 + np.tanh(np.clip(0.7978845608028654 * (g + 0.044715 * g ** 3), -20, 20))) * u)
    want = act @ w(down).T
    got = f64(y)
    assert np.sqrt(((got - want) ** 2).sum() / (want ** 2).sum()) < 6e-3   # 16-bit outputs, twice-rounded chain
    assert np.abs(got - want).max() <= 2.0 ** -7 * max(1.0, np.abs(want).max())
