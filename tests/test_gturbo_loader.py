"""The `.gturbo` packed-experts reader: layout.json decode + validation (no GPU), and — on a GPU —
layer files into the HBM store and through the kernels.  Modelled on the reference's loader tests
(Tests/ANEFieldfareUpstreamTests/Infrastructure/ModelIO/ModelLoaderTests.swift:130-300: a toy model
directory, one rejection per rule) and its file -> kernel check
(Tests/ANEFieldfareUpstreamTests/Infrastructure/Streaming/StreamingKernelIntegrationTests.swift:84-161)."""
import copy
import json
import os

import numpy as np
import pytest

from ane_fieldfare_b200 import gturbo, hotpath, workload
from conftest import oracle_layer

D, F, E = 128, 64, 8


def _write(tmp_path, doc):
    os.makedirs(tmp_path / "packed_experts", exist_ok=True)
    (tmp_path / "packed_experts" / "layout.json").write_text(doc if isinstance(doc, str) else json.dumps(doc))
    return str(tmp_path)


def _good(layers=2, ranks=None):
    return json.loads(gturbo.layout_json(layers, E, gturbo.expert_layout(D, F), ranks))


def test_valid_layout_is_accepted_and_reports_the_reference_offsets(tmp_path):
    lay = gturbo.expert_layout(D, F)
    info = hotpath.validateGTurboLayout(_write(tmp_path, _good()), D, F)
    assert (info.expertStride, info.numLayers, info.expertsPerLayer) == (lay.stride, 2, E)
    assert info.offsets.as_tuple() == lay.offsets.as_tuple() and info.identityPlacement == 1
    # positional expert ids (no "expert" keys) are as good as explicit ones
    doc = json.loads(gturbo.layout_json(2, E, lay, explicit_ids=False))
    assert hotpath.validateGTurboLayout(_write(tmp_path, doc), D, F).identityPlacement == 1
    # a permuted placement is valid and reported
    ranks = [list(np.random.default_rng(l).permutation(E)) for l in range(2)]
    assert hotpath.validateGTurboLayout(_write(tmp_path, _good(ranks=ranks)), D, F).identityPlacement == 0
    # the real model's shapes: the nine offsets of Tests/ANEFieldfareHotpathTests/ANEQuantizedCarrierTests.swift:10-11
    big = gturbo.expert_layout(2816, 704)
    info = hotpath.validateGTurboLayout(_write(tmp_path, gturbo.layout_json(1, 2, big)), 2816, 704)
    assert info.offsets.as_tuple()[6:] == (2_230_272, 3_221_504, 3_283_456) and info.expertStride == 3_358_720


def _mutations():
    """(name, mutation of a good document, expected message) — one per rule of
    GTurboPackedExpertsLayoutV1.swift:75-162 and Model.swift:478-527."""
    def m(name, fn, message):
        return pytest.param(fn, message, id=name)

    def set_(path, value):
        def fn(doc):
            node = doc
            for key in path[:-1]:
                node = node[key]
            node[path[-1]] = value
        return fn

    def del_(path):
        def fn(doc):
            node = doc
            for key in path[:-1]:
                node = node[key]
            del node[path[-1]]
        return fn

    e0 = ["layers", 0, "experts", 0]
    stride = gturbo.expert_layout(D, F).stride

    def every_expert(fn):
        def apply(doc):
            for layer in doc["layers"]:
                for expert in layer["experts"]:
                    fn(expert)
        return apply

    return [
        m("stride-not-page-multiple", set_(["expertStride"], stride + 64), "layout: invalid dimensions or stride"),
        m("layer-count", set_(["numLayers"], 3), "layout: invalid dimensions or stride"),
        m("duplicate-layer", set_(["layers", 1, "layer"], 0), "layout.layers: duplicate or invalid layer"),
        m("file-with-directory", set_(["layers", 0, "file"], "packed_experts/layer_00.bin"), "expected basename"),
        m("file-dotdot", set_(["layers", 0, "file"], ".."), "non-canonical path"),
        m("file-absolute", set_(["layers", 0, "file"], "/etc/passwd"), "unsafe relative path"),
        m("file-reserved", set_(["layers", 0, "file"], "Layout.JSON"), "reserved packed-expert filename"),
        m("file-duplicate", set_(["layers", 1, "file"], "LAYER_00.bin"), "duplicate layer filename"),
        m("expert-count", lambda d: d["layers"][0]["experts"].pop(), "wrong expert count"),
        m("mixed-ids", del_(e0 + ["expert"]), "either all explicit or all positional"),
        m("duplicate-expert", lambda d: d["layers"][0]["experts"][0].update(expert=1, physicalRank=0),
          "duplicate or invalid expert mapping"),
        m("rank-out-of-range", set_(e0 + ["physicalRank"], E), "duplicate or invalid expert mapping"),
        m("offset-vs-rank", set_(e0 + ["offset"], 5 * stride + 16), "offset or size does not match physical rank"),
        m("size-not-stride", set_(e0 + ["size"], stride - 16384), "offset or size does not match physical rank"),
        m("bad-dtype", set_(e0 + ["tensors", "gate", "dtype"], "F16"), "invalid dtype or shape"),
        m("zero-shape", set_(e0 + ["tensors", "up", "shape"], [F, 0]), "invalid dtype or shape"),
        m("range-exceeds-blob", set_(e0 + ["tensors", "down_biases", "offset"], stride - 8), "range exceeds expert blob"),
        m("overlap", set_(e0 + ["tensors", "up", "offset"], 16), "overlapping ranges"),
        m("missing-role", every_expert(lambda e: e["tensors"].pop("down_scales")), "routed layer 0 is missing role down_scales"),
        m("wrong-bits", every_expert(lambda e: e["tensors"]["gate"].__setitem__("bits", 8)),
          "routed layer 0 role gate does not match the required schema"),
        m("wrong-shape", every_expert(lambda e: e["tensors"]["down"].__setitem__("shape", [D, F // 4])),
          "routed layer 0 role down does not match the required schema"),
        m("scales-carry-bits", every_expert(lambda e: e["tensors"]["up_scales"].__setitem__("bits", 16)),
          "routed layer 0 role up_scales does not match the required schema"),
        m("differs-across-experts", set_(["layers", 1, "experts", 3, "tensors", "up_biases", "size"],
                                         F * D // 32 - 2), "routed layer 1 role up_biases metadata differs across experts"),
        m("not-json", None, "packed_experts/layout.json"),
        m("missing-key", del_(["expertsPerLayer"]), 'packed_experts/layout.json: key "expertsPerLayer" not found'),
        m("negative-offset", set_(e0 + ["offset"], -1), "packed_experts/layout.json"),
    ]


@pytest.mark.parametrize("mutate,message", _mutations())
def test_each_validation_rule_rejects(tmp_path, mutate, message):
    if mutate is None:
        path = _write(tmp_path, '{"expertStride": 16384, "numLayers": ')
    else:
        doc = copy.deepcopy(_good())
        mutate(doc)
        path = _write(tmp_path, doc)
    with pytest.raises(hotpath.FieldfareError) as err:
        hotpath.validateGTurboLayout(path, D, F)
    assert message in str(err.value), str(err.value)


def test_widths_of_the_context_must_match_the_layout(tmp_path):
    path = _write(tmp_path, _good())
    with pytest.raises(hotpath.FieldfareError, match="does not match the required schema"):
        hotpath.validateGTurboLayout(path, D, 2 * F)
    with pytest.raises(hotpath.FieldfareError, match="layout.json"):
        hotpath.validateGTurboLayout(str(tmp_path / "nowhere"), D, F)


@pytest.mark.gpu
def test_model_directory_into_hbm_and_through_the_kernels(tmp_path, oracle):
    """Layer files with permuted physical ranks -> ff_load_model_dir -> the dequantization probe and
    a decode step, against the oracle on the logical blobs."""
    torch = pytest.importorskip("torch")
    kw = dict(experts=E, d=D, f=F, sharedF=128, topK=4)
    layers = [workload.make_layer(0x6710, i, router_bias="normal", **kw) for i in range(2)]
    ranks = [list(np.random.default_rng(10 + l).permutation(E)) for l in range(2)]
    gturbo.write_model_dir(str(tmp_path), [L.blobs for L in layers], layers[0].layout, ranks)
    ctx = hotpath.HotpathContext(layers=2, maxTokens=16, **kw)
    try:
        ctx.loadModelDir(str(tmp_path))
        for i, L in enumerate(layers):
            ctx.loadShared(i, *L.shared_projections())
            ctx.loadRouter(i, L.routerW, logitBias=L.logitBias)
            for expert in (0, 3, E - 1):
                w, s, b = gturbo.sub_tensor(L.blobs[expert], L.layout, "down")
                want = oracle.dequant_int4(np.ascontiguousarray(w), np.ascontiguousarray(s), np.ascontiguousarray(b), D, F)
                got = ctx.dequantProbe(i, expert, 2).cpu().numpy()
                assert got.view(np.uint32).tobytes() == want.view(np.uint32).tobytes(), (i, expert)
            x = workload.make_tokens(0x6710, f"x{i}", 1, D)
            ids = torch.zeros((1, 4), dtype=torch.int32, device=ctx.device)
            y = ctx.moeLayer(i, hotpath.bf16_tensor(x, ctx.device), ids=ids)
            torch.cuda.synchronize()
            want, _, ref_ids, _ = oracle.moe_layer(oracle_layer(oracle, L), x, oracle.MODE_DECODE)
            assert np.array_equal(ids.cpu().numpy().astype(np.uint32), ref_ids)
            assert np.abs(oracle.bf16_to_float(hotpath.bf16_numpy(y)) - oracle.bf16_to_float(want)).max() <= 2e-2
        # a truncated layer file is refused like the reference's manifest cross-check
        with open(tmp_path / "packed_experts" / "layer_01.bin", "r+b") as fh:
            fh.truncate(layers[0].layout.stride * (E - 1))
        with pytest.raises(hotpath.FieldfareError, match="missing or wrong layer size"):
            ctx.loadModelDir(str(tmp_path))
    finally:
        ctx.close()
