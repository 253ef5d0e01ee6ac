"""Host-side logic of the library and its Python mirror; no compute calls, no GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from ane_fieldfare_b200 import binding, gturbo, hotpath
from ane_fieldfare_b200.hotpath import (PrefillMoEGrouping, PrefillMoEGroupingError, PrefillRouter,
                                        PrefillTokenExpertPair)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = binding.load()
    header = open(os.path.join(ROOT, "include", "fieldfare_cuda.h")).read()
    declared = set(re.findall(r"\b(ff_[a-z0-9_]+)\s*\(", header))
    assert declared == set(binding.SIGNATURES), declared ^ set(binding.SIGNATURES)
    for name in declared:
        assert getattr(lib, name) is not None


def test_expert_parallel_group_refuses_bad_arguments_before_touching_a_device():
    lib = binding.load()
    err = ctypes.c_char_p()
    assert not lib.ff_ep_create(None, None, 2, 0, ctypes.byref(err))
    assert b"1...8 ranks" in err.value
    one = (ctypes.c_void_p * 1)(None)
    err = ctypes.c_char_p()
    assert not lib.ff_ep_create(one, one, 1, 0, ctypes.byref(err))
    assert b"null context for rank 0" in err.value
    nine = (ctypes.c_void_p * 9)()
    err = ctypes.c_char_p()
    assert not lib.ff_ep_create(nine, nine, 9, 0, ctypes.byref(err))
    assert b"1...8 ranks" in err.value
    err = ctypes.c_char_p()
    assert not lib.ff_ep_moe_layer(None, 0, None, 1, None, ctypes.byref(err))
    assert b"null argument" in err.value
    assert lib.ff_ep_last_rows_sent(None) == 0
    lib.ff_ep_destroy(None)


def test_struct_layouts_match_the_reference_structs():
    # MoEExpertOffsets: 9 x UInt32 (Kernels/MoE/MoE.swift:4-15); PrefillTokenExpertPair: 4 x UInt32
    # (Kernels/Prefill/MoE/PrefillRouter.swift:4-21); groups 3, tiles 4 (PrefillMoEGrouping.swift:4-29)
    assert ctypes.sizeof(gturbo.MoEExpertOffsets) == 36
    assert ctypes.sizeof(binding.FFTokenExpertPair) == 16
    assert ctypes.sizeof(binding.FFMoEGroup) == 12
    assert ctypes.sizeof(binding.FFMoETile) == 16


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_create_fails_loudly_without_a_gpu():
    with pytest.raises(hotpath.FieldfareError, match="no CUDA device"):
        hotpath.HotpathContext(layers=1, experts=8, d=128, f=64, sharedF=64, topK=4, maxTokens=4)


def _pair(t, e, r, w):
    return PrefillTokenExpertPair(t, e, r, w)


def test_grouping_sorts_pairs_and_builds_offsets_counts_and_tiles():
    # Tests/ANEFieldfareUpstreamTests/Kernels/Prefill/PrefillMoEGroupingTests.swift:6-50
    pairs = [_pair(0, 3, 0, 10), _pair(0, 1, 1, 11), _pair(0, 4, 2, 12), _pair(1, 1, 0, 13),
             _pair(1, 3, 1, 14), _pair(1, 2, 2, 15), _pair(2, 4, 0, 16), _pair(2, 3, 1, 17),
             _pair(2, 1, 2, 18), _pair(3, 5, 0, 19), _pair(3, 1, 1, 20), _pair(3, 4, 2, 21)][::-1]
    g = PrefillMoEGrouping.groupTokenExpertPairs(pairs, queryCount=4, topK=3, numExperts=6,
                                                 tileExpertCount=2)
    assert [p.expert for p in g.sortedPairs] == [1, 1, 1, 1, 2, 3, 3, 3, 4, 4, 4, 5]
    assert [[p.token, p.rank] for p in g.sortedPairs] == \
        [[0, 1], [1, 0], [2, 2], [3, 1], [1, 2], [0, 0], [1, 1], [2, 1], [0, 2], [2, 0], [3, 2], [3, 0]]
    assert [p.weightBitsAndReserved for p in g.sortedPairs] == [11, 13, 18, 20, 15, 10, 14, 17, 12, 16, 21, 19]
    assert [(x.expert, x.pairStart, x.pairCount) for x in g.groups] == \
        [(1, 0, 4), (2, 4, 1), (3, 5, 3), (4, 8, 3), (5, 11, 1)]
    assert [(t.groupStart, t.groupCount, t.pairStart, t.pairCount) for t in g.tiles] == \
        [(0, 2, 0, 5), (2, 2, 5, 6), (4, 1, 11, 1)]


def test_grouping_orders_tiles_by_expert_sort_keys():
    # PrefillMoEGroupingTests.swift:52-82
    pairs = [_pair(0, 1, 0, 10), _pair(0, 2, 1, 20), _pair(1, 3, 0, 30), _pair(1, 1, 1, 11),
             _pair(2, 2, 0, 21), _pair(2, 3, 1, 31)]
    g = PrefillMoEGrouping.groupTokenExpertPairs(pairs, 3, 2, 4, 2, expertSortKeys=[0, 30, 10, 20])
    assert [x.expert for x in g.groups] == [2, 3, 1]
    assert [p.expert for p in g.sortedPairs] == [2, 2, 3, 3, 1, 1]
    assert [(t.groupStart, t.groupCount, t.pairStart, t.pairCount) for t in g.tiles] == \
        [(0, 2, 0, 4), (2, 1, 4, 2)]
    for t in g.tiles:
        in_tile = {p.expert for p in g.sortedPairs[t.pairStart:t.pairStart + t.pairCount]}
        assert in_tile == {x.expert for x in g.groups[t.groupStart:t.groupStart + t.groupCount]}


def test_grouping_rejects_invalid_metadata():
    # PrefillMoEGroupingTests.swift:84-96
    with pytest.raises(PrefillMoEGroupingError, match="route expert 2 is out of range"):
        PrefillMoEGrouping.groupTokenExpertPairs([_pair(0, 2, 0, 1)], 1, 1, 2, 1)
    with pytest.raises(ValueError):
        PrefillMoEGrouping.groupTokenExpertPairs([], 1, 1, 2, 17)


def test_grouping_empty_and_ragged_inputs():
    g = PrefillMoEGrouping.groupTokenExpertPairs([], 4, 2, 8, 16)
    assert g.sortedPairs == [] and g.groups == [] and g.tiles == []
    # fewer pairs than queryCount*topK (zero-weight pairs dropped by the caller)
    g = PrefillMoEGrouping.groupTokenExpertPairs([_pair(3, 7, 1, 5), _pair(0, 7, 0, 6)], 4, 2, 8, 16)
    assert [(p.token, p.rank) for p in g.sortedPairs] == [(0, 0), (3, 1)]
    assert [(x.expert, x.pairStart, x.pairCount) for x in g.groups] == [(7, 0, 2)]


def test_make_token_expert_pairs_and_agreement_with_the_oracle(oracle):
    rng = np.random.default_rng(3)
    T, K, E = 37, 8, 128
    ids = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.uint32)
    w = rng.integers(0, 65536, size=(T, K)).astype(np.uint16)
    pairs = PrefillRouter.makeTokenExpertPairs(ids.reshape(-1), w.reshape(-1), T, K)
    ref_pairs, n = oracle.make_pairs(ids, w, T, K)
    assert n == len(pairs) == T * K
    assert all((a.token, a.expert, a.rank, a.weightBitsAndReserved) ==
               (b.token, b.expert, b.rank, b.weight_bits) for a, b in zip(pairs, list(ref_pairs)[:n]))
    g = PrefillMoEGrouping.groupTokenExpertPairs(pairs, T, K, E, 16)
    sp, groups, tiles = oracle.group_pairs(ref_pairs, n, T, K, E, 16)
    assert [(p.token, p.expert, p.rank) for p in g.sortedPairs] == [(p.token, p.expert, p.rank) for p in sp]
    assert [(x.expert, x.pairStart, x.pairCount) for x in g.groups] == \
        [(x.expert, x.pair_start, x.pair_count) for x in groups]
    assert [(t.groupStart, t.groupCount, t.pairStart, t.pairCount) for t in g.tiles] == \
        [(t.group_start, t.group_count, t.pair_start, t.pair_count) for t in tiles]
    with pytest.raises(ValueError, match="indices count mismatch"):
        PrefillRouter.makeTokenExpertPairs([1, 2, 3], [0, 0, 0], 2, 2)


def test_layout_json_has_the_reference_keys():
    # Sources/ANEFieldfareInstallCore/Format/GTurboJSON.swift:110-172
    import json
    lay = gturbo.expert_layout(2816, 704)
    doc = json.loads(gturbo.layout_json(2, 4, lay))
    assert doc["expertStride"] == 3_358_720 and doc["numLayers"] == 2 and doc["expertsPerLayer"] == 4
    e1 = doc["layers"][1]["experts"][1]
    # the file is a basename and an expert's size is the stride
    # (Sources/ANEFieldfareImportedFormat/GTurboPackedExpertsLayoutV1.swift:89,127-131)
    assert doc["layers"][1]["file"] == "layer_01.bin"
    assert e1["offset"] == 3_358_720 and e1["size"] == 3_358_720 and e1["expert"] == 1
    assert set(e1["tensors"]) == {"gate", "gate_scales", "gate_biases", "up", "up_scales",
                                  "up_biases", "down", "down_scales", "down_biases"}
    assert e1["tensors"]["down"] == {"offset": 2_230_272, "size": 991_232, "dtype": "U32",
                                     "shape": [2816, 88], "bits": 4}
    assert e1["tensors"]["up_biases"]["offset"] == 2_168_320


def test_product_code_never_touches_the_oracle():
    """The shipped package must not import, load or run anything under oracle/."""
    pkg = os.path.join(ROOT, "ane_fieldfare_b200")
    for dirpath, _, files in os.walk(pkg):
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, name)).read()
                assert "liboracle" not in text and "from oracle" not in text and \
                    "import oracle" not in text and "ffo_" not in text, name
