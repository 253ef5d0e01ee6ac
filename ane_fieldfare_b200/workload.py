"""Seeded synthetic MoE layers in the benchmark configurations' shapes, as host arrays.

One `SyntheticLayer` holds what a layer needs on the host — the `.gturbo` expert blobs, the
shared FFN's three projections, the bf16 router and its optional logit bias — generated from a
root seed with synth.py.  bench.py and the tests load these into a `HotpathContext`; the tests
hand the same arrays to the CPU oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import gturbo, synth


@dataclass
class SyntheticLayer:
    layer: int
    experts: int
    d: int
    f: int
    sharedF: int
    topK: int
    layout: gturbo.ExpertLayout
    blobs: np.ndarray                 # uint8 [experts, stride]
    sharedLayout: Optional[gturbo.ExpertLayout]
    sharedBlob: Optional[np.ndarray]  # uint8 [sharedLayout.stride]
    routerW: np.ndarray               # bf16 bits [experts, d]
    logitBias: Optional[np.ndarray]   # fp32 [experts]

    def shared_projections(self):
        return [gturbo.sub_tensor(self.sharedBlob, self.sharedLayout, role) for role in gturbo.ROLES]


def make_layer(root: int, layer: int, *, experts: int = 128, d: int = 2816, f: int = 704,
               sharedF: int = 2112, topK: int = 8, router_bias: str = "none",
               router_std: float = 0.02, down_shift: int = 0) -> SyntheticLayer:
    """router_bias: "none" (decode), "normal" (verify: N(0,1) per expert), "zipf" (prefill:
    log of a Zipf(1.1) prior in a seeded expert order).  down_shift = n scales every down
    projection's scales and biases by 2^-n (exactly: only bf16 exponents change), which scales
    the layer's outputs by 2^-n; the benchmark configurations use 0."""
    lay = gturbo.expert_layout(d, f)
    blobs = gturbo.synthetic_experts(root, f"layer{layer}.routed", experts, d, f)
    shared_lay = shared_blob = None
    if sharedF:
        shared_lay = gturbo.expert_layout(d, sharedF)
        shared_blob = gturbo.synthetic_experts(root, f"layer{layer}.shared", 1, d, sharedF)[0]
    if down_shift:
        def shrink(blob2d, layout):
            _, s_off, b_off = layout.offsets.as_tuple()[6:9]
            n = layout.d * layout.f // 64 * 2
            for off in (s_off, b_off):
                bits = blob2d[:, off:off + n].view(np.uint16)
                assert ((bits >> 7) & 0xFF).min() > down_shift  # stays a normal number
                bits -= np.uint16(down_shift << 7)
        shrink(blobs, lay)
        if sharedF:
            shrink(shared_blob[None, :], shared_lay)
    router = synth.normal_bf16(root, f"layer{layer}.router", (experts, d), router_std)
    if router_bias == "none":
        bias = None
    elif router_bias == "normal":
        bias = synth.normal(synth.seedtree_key(root, f"layer{layer}.router.bias"), experts).astype(np.float32)
    elif router_bias == "zipf":
        bias = synth.zipf_log_prior(experts, 1.1, root, f"layer{layer}.router.zipf")
    else:
        raise ValueError(router_bias)
    return SyntheticLayer(layer, experts, d, f, sharedF, topK, lay, blobs, shared_lay, shared_blob,
                          router, bias)


def load_layer(ctx, slot: int, L: SyntheticLayer):
    """Copies one synthetic layer into slot `slot` of a HotpathContext."""
    ctx.loadLayer(slot, L.blobs, L.layout.stride, L.layout.offsets, expertCount=L.experts)
    if L.sharedF:
        ctx.loadShared(slot, *L.shared_projections())
    ctx.loadRouter(slot, L.routerW, logitBias=L.logitBias)


def make_tokens(root: int, label: str, tokens: int, d: int) -> np.ndarray:
    """bf16 bits [tokens, d] drawn from N(0, 1)."""
    return synth.normal_bf16(root, label, (tokens, d), 1.0)
