import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.build()
    return O


def oracle_layer(O, L):
    """oracle.LayerData for an ane_fieldfare_b200.workload.SyntheticLayer."""
    return O.LayerData(
        experts=L.blobs, stride=L.layout.stride, off=L.layout.offsets.as_tuple(), E=L.experts,
        D=L.d, F=L.f, K=L.topK, shared=L.sharedBlob,
        shared_off=L.sharedLayout.offsets.as_tuple() if L.sharedF else None, Fs=L.sharedF,
        router_w=L.routerW, logit_bias=L.logitBias)


def bf16_ulp(x: np.ndarray) -> np.ndarray:
    """Spacing of bf16 numbers at |x| (8 significant bits)."""
    a = np.maximum(np.abs(x.astype(np.float64)), 2.0 ** -126)
    return 2.0 ** (np.floor(np.log2(a)) - 7)


def layer_errors(got: np.ndarray, ref: np.ndarray):
    """(relative L2, worst absolute error beyond one bf16 ulp of the larger value, peak-relative
    max error as the reference's RelError.compute defines it)."""
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    diff = np.abs(got - ref)
    rel_l2 = float(np.sqrt((diff ** 2).sum()) / max(np.sqrt((ref ** 2).sum()), 1e-30))
    slack = bf16_ulp(np.maximum(np.abs(got), np.abs(ref)))
    beyond = float(np.maximum(diff - slack, 0.0).max()) if diff.size else 0.0
    literal = float(diff.max()) if diff.size else 0.0
    peak_rel = literal / max(float(np.abs(ref).max()), 1e-6) if diff.size else 0.0
    return rel_l2, beyond, literal, peak_rel


# Tolerances of the layer outputs (bf16): relative L2 <= 1e-2; max-abs <= 2e-2, where an error
# of one bf16 ulp of the value itself is not counted (outputs reach |y| ~ 16, where bf16 numbers
# are 0.0625 apart, so two correct roundings of nearly equal fp32 values can differ by more than
# 2e-2).
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2


def assert_layer_close(got_bits, ref_bits, O, what=""):
    got = O.bf16_to_float(np.asarray(got_bits, dtype=np.uint16))
    ref = O.bf16_to_float(np.asarray(ref_bits, dtype=np.uint16))
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    rel_l2, beyond, literal, peak_rel = layer_errors(got, ref)
    assert rel_l2 <= REL_L2_TOL, f"{what}: rel-L2 {rel_l2:.3e}"
    assert literal <= MAX_ABS_TOL or beyond == 0.0 or literal - beyond <= 0 or \
        (np.abs(got.astype(np.float64) - ref.astype(np.float64)) <=
         np.maximum(MAX_ABS_TOL, bf16_ulp(np.maximum(np.abs(got), np.abs(ref))))).all(), \
        f"{what}: max-abs {literal:.3e} (beyond one ulp: {beyond:.3e})"
    return rel_l2, literal, peak_rel
