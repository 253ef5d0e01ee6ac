"""The device supervisor's fault policy and the two lossy routing modes, with host-only fake guests
in the manner of the reference's DeviceSupervisorPolicyTests and FaultAtLayerGuest
(Tests/ANEFieldfareUpstreamTests/Runtime/Supervisor/DeviceSupervisorFailoverTests.swift:31-81,
120-152).  No GPU: a fault is an exception raised on the host."""
import asyncio

import numpy as np
import pytest

from ane_fieldfare_b200 import supervisor as sv
from ane_fieldfare_b200 import synth


class NoGuest:
    profile = {}

    def runLayer(self, *args, **kwargs):
        pass


class Injected(Exception):
    pass


def test_evicts_only_under_failover():
    closed = sv.DeviceSupervisor(2, sv.RuntimeFaultPolicy.failClosed, NoGuest())
    with pytest.raises(Injected):
        closed.supervise(0, lambda: (_ for _ in ()).throw(Injected()))
    assert [f.action for f in closed.faults] == ["failed-closed"]
    assert closed.routedPrefill(1) is not None
    assert closed.routedPrefill(2) is None

    failover = sv.DeviceSupervisor(2, sv.RuntimeFaultPolicy.failoverMetal, NoGuest())
    assert failover.supervise(1, lambda: (_ for _ in ()).throw(Injected())) is False
    assert [f.action for f in failover.faults] == ["evicted-to-metal"]
    assert failover.routedPrefill(0) is None, "an evicted guest is never admitted again"
    with pytest.raises(asyncio.CancelledError):
        failover.supervise(0, lambda: (_ for _ in ()).throw(asyncio.CancelledError()))
    assert len(failover.faults) == 1, "cancellation is not a fault"
    assert sv.DeviceSupervisor(3, sv.RuntimeFaultPolicy.failClosed, None).guestLayers == 0
    assert failover.profile["evicted"] and failover.profile["fault_policy"] == "failover-metal"


class FaultAtLayerGuest:
    """Delegates to a working rail, then on `fault_layer` corrupts the partial rows and faults, as a
    device that lost its program in mid-layer would leave them."""
    profile = {"injected": True}

    def __init__(self, inner, fault_layer):
        self.inner, self.fault_layer = inner, fault_layer

    def runLayer(self, layer, partials):
        if layer != self.fault_layer:
            self.inner(layer, partials)
            return
        partials[layer][:] = np.nan
        raise RuntimeError(f"injected routed fault at layer {layer}")


def _rail(tag):
    def run(layer, partials):
        partials[layer][:] = np.float32(layer * 10 + tag)
    return run


@pytest.mark.parametrize("fault_layer", [0, 3])
def test_failover_leaves_the_output_of_the_prefix_placement(fault_layer):
    layers = 6
    guest_rail, host_rail = _rail(1), _rail(2)

    def run(supervisor):
        partials = np.zeros((layers, 4), dtype=np.float32)
        sv.run_routed_prefill(supervisor, layers, lambda g, l: g.runLayer(l, partials),
                              lambda l: host_rail(l, partials))
        return partials

    class Plain:
        profile = {}

        def runLayer(self, layer, partials):
            guest_rail(layer, partials)

    # the reference: a plan that placed only layers 0..fault_layer-1 on the guest
    want = run(sv.DeviceSupervisor(fault_layer, sv.RuntimeFaultPolicy.failClosed, Plain()))
    s = sv.DeviceSupervisor(layers, sv.RuntimeFaultPolicy.failoverMetal, FaultAtLayerGuest(guest_rail, fault_layer))
    got = run(s)
    assert np.array_equal(got, want) and np.isfinite(got).all()
    assert [f.layer for f in s.faults] == [fault_layer]
    assert [f.action for f in s.faults] == ["evicted-to-metal"]
    with pytest.raises(RuntimeError, match="injected routed fault"):
        run(sv.DeviceSupervisor(layers, sv.RuntimeFaultPolicy.failClosed, FaultAtLayerGuest(guest_rail, fault_layer)))


def _bits(values):
    return synth.bf16_bits(np.asarray(values, dtype=np.float32))


def _floats(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def test_active_routed_experts_rescales_the_kept_ranks():
    w = _bits([[0.5, 0.25, 0.125, 0.125], [0.25, 0.25, 0.25, 0.25]])
    out = _floats(sv.apply_active_routed_experts(w, 2))
    # row 0: full 1.0, kept 0.75 -> 0.5/0.75, 0.25/0.75 in bf16; inactive ranks zero
    assert np.array_equal(out[0], _floats(_bits([0.5 / 0.75, 0.25 / 0.75, 0.0, 0.0])))
    assert np.array_equal(out[1], np.array([0.5, 0.5, 0.0, 0.0], dtype=np.float32))
    assert np.array_equal(sv.apply_active_routed_experts(w, 4), w)
    with pytest.raises(ValueError):
        sv.apply_active_routed_experts(w, 0)


def test_cap_expert_union_keeps_the_heaviest_experts():
    ids = np.array([[0, 1, 2], [1, 2, 3], [2, 3, 4]], dtype=np.uint32)
    w = _bits([[0.5, 0.25, 0.25], [0.5, 0.25, 0.25], [0.5, 0.25, 0.25]])
    # mass: e0 .5, e1 .75, e2 1.0, e3 .5, e4 .25 -> cap 2 keeps experts 2 and 1
    out = _floats(sv.cap_expert_union(ids, w, 8, 2))
    assert np.array_equal(out[0], _floats(_bits([0.0, 0.5, 0.5])))          # kept .25 + .25 -> scale 2
    assert np.array_equal(out[1], _floats(_bits([0.5 / 0.75, 0.25 / 0.75, 0.0])))
    assert np.array_equal(out[2], np.array([1.0, 0.0, 0.0], dtype=np.float32))
    # ties go to the lower expert id: cap 3 keeps 2, 1 and then 0 (mass .5) before 3 (mass .5)
    out3 = _floats(sv.cap_expert_union(ids, w, 8, 3))
    assert out3[0, 0] > 0 and out3[1, 2] == 0 and out3[2, 1] == 0
    # a block within the cap is untouched; an id past the experts is refused
    assert np.array_equal(sv.cap_expert_union(ids, w, 8, 5), w)
    with pytest.raises(ValueError, match="past 4"):
        sv.cap_expert_union(ids, w, 4, 2)
