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


# Tolerances of bf16 layer outputs against the CPU oracle (the target stated for this path: "rel-L2 <= 1e-2 and
# max-abs <= 2e-2 in bf16"):
#   relative L2 <= 1e-2, always;
#   literal max-abs <= 2e-2 wherever the outputs are of unit scale (peak <= 1): asserted as
#     written by the unit-scale variants of the benchmark configurations (down_shift = 5);
#   at the benchmark configurations' own scale (outputs of rms ~4, peak ~20, where neighbouring
#     bf16 numbers are 0.03..0.125 apart and one rounding to the other neighbour already exceeds a
#     fixed 2e-2) the same bound in units of the output peak: max|got - ref| <= 2e-2 * max(1, peak),
#     the reference's own error measure (RelError.compute,
#     Tests/Support/Validation/Tolerance/RelError.swift:7-17; tolerance 1e-2 for chained 16-bit
#     reductions, Tolerances.swift:13);
#   element by element: |got_i - ref_i| <= elementwise_tol * max(1, |ref_i|) where a caller asks
#     for it: ELEMENTWISE_TOL for the outputs of one expert's chain (partial rows, shared FFN rows),
#     LAYER_ELEMENTWISE_TOL for layer outputs, which add up to nine bf16-rounded rows of either
#     sign: where they cancel, one ulp of a large term is several percent of a small sum.
# Every call appends its figures to the file named by FF_PARITY_LOG (when set).
REL_L2_TOL = 1e-2
MAX_ABS_TOL = 2e-2
ELEMENTWISE_TOL = 2e-2
LAYER_ELEMENTWISE_TOL = 5e-2


def assert_layer_close(got_bits, ref_bits, O, what="", literal_tol=None, elementwise_tol=None):
    got = O.bf16_to_float(np.asarray(got_bits, dtype=np.uint16))
    ref = O.bf16_to_float(np.asarray(ref_bits, dtype=np.uint16))
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    rel_l2, scaled, literal, peak_rel = layer_errors(got, ref)
    ref_peak = float(np.abs(ref).max()) if ref.size else 0.0
    peak = max(1.0, ref_peak)
    line = (f"{what}: rel-L2 {rel_l2:.3e} max-abs {literal:.3e} element-wise {scaled:.3e} "
            f"peak {ref_peak:.3f} n {ref.size}")
    log = os.environ.get("FF_PARITY_LOG")
    if log:
        with open(log, "a") as fh:
            fh.write(line + "\n")
    assert rel_l2 <= REL_L2_TOL, line
    assert literal <= MAX_ABS_TOL * peak, line
    if literal_tol is not None:
        assert literal <= literal_tol, line
    if elementwise_tol is not None:
        assert scaled <= elementwise_tol, line
    return rel_l2, literal, peak_rel
