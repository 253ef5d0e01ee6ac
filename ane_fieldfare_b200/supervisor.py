"""Host-side policy around the routed-prefill plug-in: the fault policy of the reference's device
supervisor and its two lossy routing modes.  Host logic only (the reference's is host code too):
nothing here touches a GPU, the guest it supervises is any object with `runLayer(...)` and
`profile` — `hotpath.CudaRoutedPrefillGuest` in production, a fake in the tests.

Reference: Sources/ANEFieldfareHotpath/Runtime/Supervisor/DeviceSupervisor.swift:4-125 (policy,
faults, admission), Runtime/Configuration/RuntimeConfiguration.swift:57-80 (`activeRoutedExperts`,
`prefillExpertUnionCap`), Runtime/Inference/RealForwardRunner.swift:807-852 (`capExpertUnion`) and
:1952-1961 (weights of the kept ranks rescaled to the full total).
"""
from __future__ import annotations

import asyncio
import enum
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import numpy as np


class RuntimeFaultPolicy(enum.Enum):
    """What the supervisor does when the guest reports a fault (DeviceSupervisor.swift:4-12).  The
    raw values are the reference's configuration strings; its host rail is Metal, here it is
    whatever the caller runs when the guest is not admitted."""
    failClosed = "fail-closed"
    failoverMetal = "failover-metal"


@dataclass(frozen=True)
class GuestFault:
    """One guest fault the supervisor observed, and what it did about it (DeviceSupervisor.swift:26-35)."""
    layer: int
    message: str
    action: str  # "failed-closed" | "evicted-to-metal"


class DeviceSupervisor:
    """Owns the routed-prefill guest for one runner.  The guest runs the routed experts of layers
    0..guestLayers-1; the forward loop asks `routedPrefill(layer)` whether the guest is admitted
    and runs it through `supervise`, which applies the fault policy.  An evicted guest is never
    admitted again (DeviceSupervisor.swift:37-109)."""

    def __init__(self, guestLayers: int, faultPolicy: RuntimeFaultPolicy, guest: Optional[Any]):
        self.guestLayers = 0 if guest is None else int(guestLayers)
        self.faultPolicy = faultPolicy
        self._guest = guest
        self.evicted = False
        self.faults: List[GuestFault] = []

    def routedPrefill(self, layer: int) -> Optional[Any]:
        return self._guest if (not self.evicted and layer < self.guestLayers) else None

    def supervise(self, layer: int, body: Callable[[], None]) -> bool:
        """Runs the guest under the fault policy.  True when the guest completed, False when it
        was evicted and the host must execute the layer.  Fail-closed re-raises; cancellation
        (and a keyboard interrupt) always propagates without being recorded."""
        try:
            body()
            return True
        except (asyncio.CancelledError, KeyboardInterrupt):
            raise
        except Exception as error:  # noqa: BLE001 - every guest failure is a fault
            closed = self.faultPolicy is RuntimeFaultPolicy.failClosed
            self.faults.append(GuestFault(layer, str(error), "failed-closed" if closed else "evicted-to-metal"))
            if closed:
                raise
            self.evicted = True
            return False

    @property
    def routedPrefillProfile(self) -> Optional[Dict[str, Any]]:
        return None if self._guest is None else self._guest.profile

    @property
    def profile(self) -> Dict[str, Any]:
        return {
            "fault_policy": self.faultPolicy.value,
            "guest_layers": self.guestLayers,
            "evicted": self.evicted,
            "faults": [{"layer": f.layer, "message": f.message, "action": f.action} for f in self.faults],
            "claim_boundary": ("The guest was evicted; layers from the fault on ran on the host rail."
                               if self.evicted else "Placement as planned; no guest eviction."),
        }


def run_routed_prefill(supervisor: DeviceSupervisor, layers: int, guest_call: Callable[[Any, int], None],
                       host_call: Callable[[int], None]) -> None:
    """The forward loop's use of the supervisor for the routed experts of `layers` layers: the
    guest where it is admitted, the host rail otherwise and for the layer on which the guest was
    evicted (RealForwardRunner's prefill loop around `supervisor.routedPrefill(layer:)`)."""
    for layer in range(layers):
        guest = supervisor.routedPrefill(layer)
        if guest is not None and supervisor.supervise(layer, lambda: guest_call(guest, layer)):
            continue
        host_call(layer)


# ---- lossy routing modes -----------------------------------------------------------------------

def _f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _bf16(values: np.ndarray) -> np.ndarray:
    u = np.asarray(values, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def apply_active_routed_experts(weights: np.ndarray, active: int) -> np.ndarray:
    """`activeRoutedExperts` below the checkpoint's top-K (an explicit lossy mode): per row the
    first `active` weights are rescaled to the row's full total, fp32 sums in rank order, the
    result stored in 16 bits (RealForwardRunner.swift:1952-1961); the other ranks get weight 0, so
    a K-wide operator adds nothing for them.  `weights`: bf16 bit patterns [rows][K]."""
    w = np.array(weights, dtype=np.uint16, copy=True)
    rows, k = w.shape
    if not 1 <= active <= k:
        raise ValueError(f"active routed experts must be in 1...{k}")
    if active == k:
        return w
    f = _f32(w)
    for r in range(rows):
        full = np.float32(0)
        for i in range(k):
            full = np.float32(full + f[r, i])
        kept = np.float32(0)
        for i in range(active):
            kept = np.float32(kept + f[r, i])
        if kept != 0:
            w[r, :active] = _bf16(np.float32(f[r, :active] * full) / kept)
        w[r, active:] = 0
    return w


def cap_expert_union(ids: np.ndarray, weights: np.ndarray, num_experts: int, cap: int) -> np.ndarray:
    """`prefillExpertUnionCap`: keeps the `cap` experts with the most routed weight in a block
    (sum of |weight|, ties to the lower id) and rescales each row's kept weights to its original
    total; routes to other experts get weight 0 (RealForwardRunner.swift:826-852).  `ids` uint32
    [rows][K], `weights` bf16 bit patterns [rows][K]; returns the new weights."""
    ids = np.asarray(ids, dtype=np.uint32)
    w = np.array(weights, dtype=np.uint16, copy=True)
    if not 1 <= cap <= 128:
        raise ValueError("prefill expert union cap must be in 1...128")
    if int(ids.max(initial=0)) >= num_experts:
        raise ValueError(f"router wrote an expert past {num_experts}")
    if len(set(ids.reshape(-1).tolist())) <= cap:
        return w
    f = _f32(w)
    mass = np.zeros(num_experts, dtype=np.float32)
    for e, v in zip(ids.reshape(-1).tolist(), np.abs(f).reshape(-1)):
        mass[e] = np.float32(mass[e] + v)
    live = [e for e in range(num_experts) if mass[e] > 0]
    retained = set(sorted(live, key=lambda e: (-float(mass[e]), e))[:cap])
    rows, k = w.shape
    for r in range(rows):
        original = np.float32(0)
        kept = np.float32(0)
        for i in range(k):
            original = np.float32(original + f[r, i])
            if int(ids[r, i]) in retained:
                kept = np.float32(kept + f[r, i])
        scale = np.float32(original / kept) if kept != 0 else np.float32(0)
        for i in range(k):
            w[r, i] = _bf16(np.float32(f[r, i] * scale))[()] if int(ids[r, i]) in retained else 0
    return w
