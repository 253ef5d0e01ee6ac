"""Host-side mirror of the reference's operator classes for the INT4 MoE path, over the C ABI.

The reference drives this path through Swift wrapper objects whose `encode...(commandBuffer:)`
methods enqueue Metal kernels (Sources/ANEFieldfareHotpath/Kernels/MoE/MoE.swift,
Kernels/MoE/SharedExpertInt4.swift, Kernels/Prefill/MoE/PrefillRouter.swift,
Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift, Kernels/Prefill/MoE/PrefillMoE.swift,
Kernels/Prefill/MoE/PrefillSharedExpert.swift, Kernels/Quant/DequantInt4GEMV.swift).  The
classes here keep those names, method names and argument meanings, with a CUDA stream in place
of the command buffer and torch CUDA tensors in place of (MTLBuffer, offset) pairs; torch only
supplies device memory and streams.  Runtime failures raise `FieldfareError` carrying the
library's message (the reference throws Swift errors with descriptions); programmer errors the
reference traps with `precondition` raise `ValueError`.

Expert weights are not passed per call: they are resident in HBM, loaded once per layer from the
`.gturbo` layer file bytes (`HotpathContext.loadLayer`), which replaces the reference's mmap
store and per-call blob binding.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import binding
from .binding import (FFConfig, FFMoEGroup, FFMoETile, FFProjection, FFTokenExpertPair,
                      FieldfareError, call)
from .gturbo import MoEExpertOffsets

__all__ = ["HotpathContext", "validateGTurboLayout", "MoE", "SharedExpertInt4", "SharedExpertProjection", "PrefillRouter",
           "PrefillMoEGrouping", "PrefillGroupedRoutedMoE", "PrefillMoE", "PrefillSharedExpert",
           "DequantInt4GEMV", "CudaRoutedPrefillGuest", "PrefillTokenExpertPair", "PrefillMoEGroup",
           "PrefillMoETile", "PrefillMoEGroupedRoutes", "PrefillMoEGroupingError", "FieldfareError",
           "bf16_tensor", "bf16_numpy"]


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("device operands must be contiguous CUDA tensors")
    return t.data_ptr()


def _stream(stream: Optional[torch.cuda.Stream]) -> Optional[int]:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream or None


def validateGTurboLayout(path: str, d: int, f: int) -> binding.FFGTurboLayoutInfo:
    """Checks `<path>/packed_experts/layout.json` (no GPU needed); raises FieldfareError with the
    reference's message on the first rule that fails."""
    info = binding.FFGTurboLayoutInfo()
    call("ff_gturbo_validate_layout", path.encode(), d, f, ctypes.byref(info))
    return info


def bf16_tensor(bits: np.ndarray, device) -> torch.Tensor:
    """bf16 bit patterns (uint16 numpy) -> torch.bfloat16 tensor on `device`."""
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(device).view(torch.bfloat16)


def bf16_numpy(t: torch.Tensor) -> np.ndarray:
    """torch.bfloat16 tensor -> bf16 bit patterns (uint16 numpy)."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


class HotpathContext:
    """Owns one FFContext: the resident weights of `layers` layers and the kernels' scratch.

    Plays the part of the reference's `MetalContext` + `Model` for this path
    (Infrastructure/Metal/MetalContext.swift, Runtime/Inference/Model.swift:231-312)."""

    def __init__(self, *, layers: int, experts: int, d: int, f: int, sharedF: int, topK: int = 8,
                 maxTokens: int = 16, device: int = 0):
        lib = binding.load()
        self.config = FFConfig(layers, experts, d, f, sharedF, topK, maxTokens)
        err = ctypes.c_char_p()
        self._handle = lib.ff_create(device, ctypes.byref(self.config), ctypes.byref(err))
        if not self._handle:
            raise FieldfareError(err.value.decode() if err.value else "ff_create failed")
        self.device = torch.device("cuda", device)
        self.layers, self.experts, self.d, self.f = layers, experts, d, f
        self.sharedF, self.topK, self.maxTokens = sharedF, topK, maxTokens

    @property
    def handle(self):
        if not self._handle:
            raise FieldfareError("context was destroyed")
        return self._handle

    def close(self):
        if getattr(self, "_handle", None):
            binding.load().ff_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> binding.FFInfo:
        return binding.load().ff_get_info(self.handle)

    def setTracing(self, enabled: bool):
        """CUDA-event timing of every kernel launch (the reference's GPU trace,
        Infrastructure/Metal/GPUTrace.swift:67-90)."""
        binding.load().ff_set_tracing(self.handle, enabled)

    def trace(self) -> dict:
        """{kernel name: (launches, total milliseconds)} since the last call; waits for the device."""
        entries = (binding.FFTraceEntry * 32)()
        n = binding.load().ff_get_trace(self.handle, entries, 32)
        return {entries[i].name.decode(): (entries[i].launches, entries[i].milliseconds) for i in range(n)}

    def decodePhaseTimes(self):
        """Microseconds of the six phases of the last traced one-token launch (see the header)."""
        out = (ctypes.c_double * 6)()
        call("ff_decode_phase_times", self.handle, out)
        return list(out)

    def decodeWarpTimes(self):
        """[cta 0/1][phase A/B/C][warp 0..15][issued, arrived, done] microseconds since kernel start of
        the last traced one-token launch; -1 where a warp had no work."""
        out = (ctypes.c_double * 288)()
        call("ff_decode_warp_times", self.handle, out)
        return np.array(list(out)).reshape(2, 3, 16, 3)

    # -- resident weights (replaces MappedExpertLayer / Model.routedExpertViews) ---------------

    def loadLayer(self, layer: int, blobs: np.ndarray, expertStride: int,
                  offsets: MoEExpertOffsets, expertCount: Optional[int] = None):
        """`blobs`: the bytes of `packed_experts/layer_%02d.bin` (uint8)."""
        data = np.ascontiguousarray(blobs, dtype=np.uint8).reshape(-1)
        count = self.experts if expertCount is None else expertCount
        call("ff_load_layer", self.handle, layer, data.ctypes.data, data.size, count, expertStride,
             ctypes.byref(offsets))

    def loadModelDir(self, path: str):
        """An installed model's `packed_experts/` (layout.json + layer files) into the layer slots,
        after the reference's validation (Infrastructure/ModelIO/PackedExpertsLayout.swift:55-90,
        Runtime/Inference/Model.swift:478-527)."""
        call("ff_load_model_dir", self.handle, path.encode())

    def loadShared(self, layer: int, gate, up, down):
        """Each projection: (packed uint8 [rows, cols/2], scales uint16, biases uint16) on the host."""
        keep, projs = [], []
        for packed, scales, biases in (gate, up, down):
            arrays = [np.ascontiguousarray(packed, dtype=np.uint8),
                      np.ascontiguousarray(scales, dtype=np.uint16),
                      np.ascontiguousarray(biases, dtype=np.uint16)]
            keep.append(arrays)
            rows, half = arrays[0].shape
            projs.append(FFProjection(arrays[0].ctypes.data, arrays[1].ctypes.data,
                                      arrays[2].ctypes.data, rows, half * 2))
        call("ff_load_shared", self.handle, layer, *[ctypes.byref(p) for p in projs])

    def loadSharedInt8(self, layer: int, gate, up, down):
        """The INT8 affine shared FFN of the shipped checkpoints: every projection a tuple
        (codes uint8 [rows][cols], scales bf16 bits [rows][cols/64], biases likewise)
        (Kernels/MoE/SharedExpertInt8.swift:7-29)."""
        keep, projs = [], []
        for codes, scales, biases in (gate, up, down):
            arrays = [np.ascontiguousarray(codes, dtype=np.uint8), np.ascontiguousarray(scales, dtype=np.uint16),
                      np.ascontiguousarray(biases, dtype=np.uint16)]
            keep.append(arrays)
            rows, cols = arrays[0].shape
            projs.append(FFProjection(arrays[0].ctypes.data, arrays[1].ctypes.data, arrays[2].ctypes.data, rows, cols))
        call("ff_load_shared_int8", self.handle, layer, *[ctypes.byref(p) for p in projs])

    def loadRouter(self, layer: int, weights: np.ndarray, effectiveScale=None, perExpertScale=None,
                   logitBias=None):
        w = np.ascontiguousarray(weights, dtype=np.uint16)
        es = None if effectiveScale is None else np.ascontiguousarray(effectiveScale, dtype=np.uint16)
        pe = None if perExpertScale is None else np.ascontiguousarray(perExpertScale, dtype=np.uint16)
        lb = None if logitBias is None else np.ascontiguousarray(logitBias, dtype=np.float32)
        call("ff_load_router", self.handle, layer, w.ctypes.data,
             None if es is None else es.ctypes.data, None if pe is None else pe.ctypes.data,
             None if lb is None else lb.ctypes.data, w.shape[0], w.shape[1])

    def loadRouterInt8(self, layer: int, codes: np.ndarray, scales: np.ndarray, biases: np.ndarray,
                       effectiveScale=None, perExpertScale=None, logitBias=None):
        """The INT8 affine router of the shipped checkpoints: codes uint8 [experts][d], scales and
        biases bf16 bits [experts][d/64] (Runtime/Inference/Model.swift:473-475)."""
        q = np.ascontiguousarray(codes, dtype=np.uint8)
        sc = np.ascontiguousarray(scales, dtype=np.uint16)
        bi = np.ascontiguousarray(biases, dtype=np.uint16)
        if sc.shape != (q.shape[0], q.shape[1] // 64) or bi.shape != sc.shape:
            raise FieldfareError("router scales/biases must be [experts][d/64]")
        es = None if effectiveScale is None else np.ascontiguousarray(effectiveScale, dtype=np.uint16)
        pe = None if perExpertScale is None else np.ascontiguousarray(perExpertScale, dtype=np.uint16)
        lb = None if logitBias is None else np.ascontiguousarray(logitBias, dtype=np.float32)
        call("ff_load_router_int8", self.handle, layer, q.ctypes.data, sc.ctypes.data, bi.ctypes.data,
             None if es is None else es.ctypes.data, None if pe is None else pe.ctypes.data,
             None if lb is None else lb.ctypes.data, q.shape[0], q.shape[1])

    def expertAddress(self, layer: int, expert: int) -> int:
        return binding.load().ff_expert_address(self.handle, layer, expert)

    # -- parity hook ---------------------------------------------------------------------------

    def dequantProbe(self, layer: int, expert: int, role: int, *, bf16: bool = False) -> torch.Tensor:
        f = self.sharedF if expert < 0 else self.f
        rows, cols = (self.d, f) if role == 2 else (f, self.d)
        out = torch.empty((rows, cols), dtype=torch.bfloat16 if bf16 else torch.float32,
                          device=self.device)
        call("ff_dequant_probe_bf16" if bf16 else "ff_dequant_probe", self.handle, layer, expert,
             role, _ptr(out), _stream(None))
        return out

    # -- the fused block -----------------------------------------------------------------------

    def moeLayer(self, layer: int, x: torch.Tensor, y: Optional[torch.Tensor] = None,
                 ids: Optional[torch.Tensor] = None, weights: Optional[torch.Tensor] = None,
                 stream=None) -> torch.Tensor:
        tokens = x.shape[0]
        if y is None:
            y = torch.empty((tokens, self.d), dtype=torch.bfloat16, device=x.device)
        call("ff_moe_layer", self.handle, layer, _ptr(x), tokens, _ptr(y), _ptr(ids), _ptr(weights),
             _stream(stream))
        return y

    def moeStack(self, firstLayer: int, layerCount: int, x: torch.Tensor, eps: float = 1e-6,
                 y: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None,
                 stream=None) -> torch.Tensor:
        """x <- moeLayer(l, rmsnorm(x)) for `layerCount` consecutive layers (benchmark configuration
        4's stack); `ids` int32 [layerCount, tokens, K] receives every layer's routes."""
        tokens = x.shape[0]
        if y is None:
            y = torch.empty((tokens, self.d), dtype=torch.bfloat16, device=x.device)
        call("ff_moe_stack", self.handle, firstLayer, layerCount, _ptr(x), tokens, eps, _ptr(y),
             _ptr(ids), _stream(stream))
        return y

    def resetDeviceError(self):
        call("ff_reset_device_error", self.handle)

    def moeLayerHost(self, layer: int, hostX: torch.Tensor, hostY: torch.Tensor):
        """Host buffers in, host buffers out (copies inside); blocks until done."""
        if hostX.is_cuda or hostY.is_cuda:
            raise ValueError("moeLayerHost takes host tensors")
        call("ff_moe_layer_host", self.handle, layer, hostX.data_ptr(), hostX.shape[0],
             hostY.data_ptr())

    def rmsnorm(self, x: torch.Tensor, w: Optional[torch.Tensor], eps: float,
                y: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        if y is None:
            y = torch.empty_like(x)
        call("ff_rmsnorm", self.handle, _ptr(x), _ptr(w), eps, x.shape[0], _ptr(y), _stream(stream))
        return y


class MoE:
    """Decode router and routed experts (Kernels/MoE/MoE.swift:31-496)."""

    maxStreamedExperts = 8

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodeRouterGemma4(self, stream, layer: int, hidden: torch.Tensor, outIndices: torch.Tensor,
                           outWeights: torch.Tensor, topK: int = 8,
                           outLogits: Optional[torch.Tensor] = None):
        """One row: logits, top-K, softmax, gain (MoE.swift:168-237).  Router weights, the
        effective scale and the per-expert scale are the resident ones of `layer`."""
        if topK != self.context.topK:
            raise ValueError("topK must equal the context's routes per token")
        call("ff_router_topk", self.context.handle, layer, _ptr(hidden), self.context.d, 1,
             _ptr(outIndices), _ptr(outWeights), _ptr(outLogits), _stream(stream))

    def encodeRouterRowsGemma4(self, stream, layer: int, hidden: torch.Tensor,
                               hiddenStrideElements: int, rows: int, outIndices: torch.Tensor,
                               outWeights: torch.Tensor, outLogits: Optional[torch.Tensor] = None):
        """Up to 16 rows (MoE.swift:249-300)."""
        if not 0 < rows <= 16:
            raise ValueError("rows must be in 1...16")
        call("ff_router_topk", self.context.handle, layer, _ptr(hidden), hiddenStrideElements, rows,
             _ptr(outIndices), _ptr(outWeights), _ptr(outLogits), _stream(stream))

    def encodeRoutedPersistentGPUSlots(self, stream, layer: int, indices: torch.Tensor,
                                       x: torch.Tensor, routingWeights: torch.Tensor,
                                       residual: Optional[torch.Tensor], y: torch.Tensor):
        """Gather slots + phase 1 (gate/up/GeGLU) + phase 2 (down, weighted sum onto the residual)
        for one row (MoE.swift:429-496)."""
        call("ff_moe_decode", self.context.handle, layer, _ptr(x), _ptr(indices),
             _ptr(routingWeights), _ptr(residual), _ptr(y), _stream(stream))


@dataclass
class SharedExpertProjection:
    """Device-resident affine INT4 matrix (Kernels/MoE/SharedExpertInt8.swift:7-29)."""
    weights: torch.Tensor   # uint8 [rows, cols/2]
    scales: torch.Tensor    # bf16 [rows, cols/64]
    biases: torch.Tensor
    rows: int
    cols: int

    def ff(self) -> FFProjection:
        return FFProjection(_ptr(self.weights), _ptr(self.scales), _ptr(self.biases), self.rows,
                            self.cols)


class SharedExpertInt4:
    """Shared INT4 FFN (Kernels/MoE/SharedExpertInt4.swift:22-88); weights resident per layer."""

    def __init__(self, context: HotpathContext):
        self.context = context

    def encode(self, stream, layer: int, x: torch.Tensor, y: torch.Tensor, rows: int = 1,
               xStrideElements: Optional[int] = None):
        call("ff_shared_ffn", self.context.handle, layer, _ptr(x),
             self.context.d if xStrideElements is None else xStrideElements, rows, _ptr(y),
             _stream(stream))


class PrefillSharedExpert(SharedExpertInt4):
    """Shared FFN over a block of rows (Kernels/Prefill/MoE/PrefillSharedExpert.swift:51-137)."""

    def encodeBlock(self, stream, layer: int, x: torch.Tensor, y: torch.Tensor, queryCount: int,
                    hiddenStrideElements: Optional[int] = None):
        self.encode(stream, layer, x, y, rows=queryCount, xStrideElements=hiddenStrideElements)


class DequantInt4GEMV:
    """Multi-row INT4 GEMV on explicit device projections
    (Kernels/Quant/DequantInt4GEMV.swift:72-117)."""

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodeRows(self, stream, projection: SharedExpertProjection, x: torch.Tensor, xStride: int,
                   rows: int, y: torch.Tensor, yStride: int):
        p = projection.ff()
        call("ff_int4_gemv_rows", self.context.handle, ctypes.byref(p), _ptr(x), xStride, rows,
             _ptr(y), yStride, _stream(stream))


# ---- prefill: pairs, grouping, routed experts, combine -------------------------------------

PrefillTokenExpertPair = FFTokenExpertPair
PrefillMoEGroup = FFMoEGroup
PrefillMoETile = FFMoETile


class PrefillMoEGroupingError(FieldfareError):
    """`PrefillMoEGroupingError.expertOutOfRange` (PrefillMoEGrouping.swift:37-46)."""


@dataclass
class PrefillMoEGroupedRoutes:
    sortedPairs: list
    groups: list
    tiles: list


class PrefillRouter:
    """Router over a block of rows (Kernels/Prefill/MoE/PrefillRouter.swift:23-95)."""

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodeGemma4Block(self, stream, layer: int, hidden: torch.Tensor, outIndices: torch.Tensor,
                          outWeights: torch.Tensor, queryCount: int,
                          hiddenStrideElements: Optional[int] = None,
                          outLogits: Optional[torch.Tensor] = None):
        if queryCount <= 0:
            raise ValueError("queryCount must be positive")
        stride = self.context.d if hiddenStrideElements is None else hiddenStrideElements
        if stride < self.context.d:
            raise ValueError("hidden stride is too small")
        call("ff_router_topk", self.context.handle, layer, _ptr(hidden), stride, queryCount,
             _ptr(outIndices), _ptr(outWeights), _ptr(outLogits), _stream(stream))

    @staticmethod
    def makeTokenExpertPairs(indices: Sequence[int], weights: Sequence[int], queryCount: int,
                             topK: int):
        """Token-major, rank-minor pair list (PrefillRouter.swift:75-95); weights are 16-bit
        patterns."""
        if queryCount < 0 or topK < 0:
            raise ValueError("queryCount and topK must be non-negative")
        if len(indices) != queryCount * topK:
            raise ValueError("indices count mismatch")
        if len(weights) != queryCount * topK:
            raise ValueError("weights count mismatch")
        ids = np.ascontiguousarray(indices, dtype=np.uint32)
        w = np.ascontiguousarray(weights, dtype=np.uint16)
        out = (FFTokenExpertPair * max(1, queryCount * topK))()
        n = binding.load().ff_make_token_expert_pairs(ids.ctypes.data, w.ctypes.data, queryCount,
                                                      topK, out)
        return list(out)[:n]


class PrefillMoEGrouping:
    """Host sort/group/tile of (token, expert) pairs
    (Kernels/Prefill/MoE/PrefillMoEGrouping.swift:48-110)."""

    @staticmethod
    def groupTokenExpertPairs(pairs, queryCount: int, topK: int, numExperts: int,
                              tileExpertCount: int, expertSortKeys=None) -> PrefillMoEGroupedRoutes:
        if not (queryCount >= 0 and topK > 0 and numExperts > 0 and 1 <= tileExpertCount <= 16):
            raise ValueError("invalid grouping parameters")
        if len(pairs) > queryCount * topK:
            raise ValueError("more pairs than queryCount * topK")
        if expertSortKeys is not None and len(expertSortKeys) != numExperts:
            raise ValueError("expertSortKeys must have numExperts entries")
        n = len(pairs)
        src = (FFTokenExpertPair * max(1, n))(*pairs)
        dst = (FFTokenExpertPair * max(1, n))()
        groups = (FFMoEGroup * max(1, min(numExperts, n)))()
        tiles = (FFMoETile * max(1, min(numExperts, n)))()
        ng, nt = ctypes.c_uint32(), ctypes.c_uint32()
        keys = None
        if expertSortKeys is not None:
            keys = np.ascontiguousarray(expertSortKeys, dtype=np.uint64)
        try:
            call("ff_group_token_expert_pairs", src, n, queryCount, topK, numExperts,
                 tileExpertCount, None if keys is None else keys.ctypes.data, dst, groups,
                 ctypes.byref(ng), tiles, ctypes.byref(nt))
        except FieldfareError as e:
            raise PrefillMoEGroupingError(str(e)) from None
        return PrefillMoEGroupedRoutes(list(dst)[:n], list(groups)[:ng.value], list(tiles)[:nt.value])


class PrefillGroupedRoutedMoE:
    """Routed experts for verify blocks and prefill chunks
    (Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:187-448).  Both entry points write
    `routePartials[(token*topK + rank)*d ...]` for every route, like the reference."""

    verifyMaxRows = 16

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodeVerifyBound(self, stream, layer: int, hidden: torch.Tensor, routeIDs: torch.Tensor,
                          routePartials: torch.Tensor, rows: int,
                          hiddenStrideElements: Optional[int] = None):
        """GPU-planned grouped GEMV for 1..16 rows (PrefillGroupedRoutedMoE.swift:383-448)."""
        if not 0 < rows <= self.verifyMaxRows:
            raise ValueError("rows must be in 1...16")
        stride = self.context.d if hiddenStrideElements is None else hiddenStrideElements
        call("ff_moe_verify", self.context.handle, layer, _ptr(hidden), stride, rows, _ptr(routeIDs),
             _ptr(routePartials), _stream(stream))

    def encodeStreamedBatched(self, stream, layer: int, hidden: torch.Tensor, routeIDs: torch.Tensor,
                              routePartials: torch.Tensor, queryCount: int,
                              hiddenStrideElements: Optional[int] = None):
        """Device permute + grouped tensor-core GEMMs (PrefillGroupedRoutedMoE.swift:275-326)."""
        stride = self.context.d if hiddenStrideElements is None else hiddenStrideElements
        call("ff_moe_prefill", self.context.handle, layer, _ptr(hidden), stride, queryCount,
             _ptr(routeIDs), _ptr(routePartials), _stream(stream))

    def sortRoutesOnDevice(self, stream, groupIds: torch.Tensor, groups: int):
        """The device permute on its own: routes [tokens][K] (int32 group ids; ids >= groups are
        dropped) sorted by (group, token, rank).  Returns (pairs int32 [tokens*K][4] with columns
        token, group, rank, 0 — rows past the kept routes are unwritten —, offsets int32 [groups+1]),
        both on the device; asynchronous on the stream."""
        tokens = groupIds.shape[0]
        pairs = torch.empty((tokens * self.context.topK, 4), dtype=torch.int32, device=groupIds.device)
        offsets = torch.empty(groups + 1, dtype=torch.int32, device=groupIds.device)
        call("ff_sort_routes", self.context.handle, _ptr(groupIds), tokens, groups, _ptr(pairs), _ptr(offsets),
             _stream(stream))
        return pairs, offsets

    def lastRoutes(self, pairCount: int):
        """Sorted pairs and per-expert offsets of the last encodeStreamedBatched (synchronizes)."""
        pairs = (FFTokenExpertPair * max(1, pairCount))()
        offsets = np.zeros(self.context.experts + 1, dtype=np.uint32)
        call("ff_last_prefill_routes", self.context.handle, pairs, offsets.ctypes.data)
        return list(pairs)[:pairCount], offsets


class PrefillLayerGlue:
    """The fused steps either side of the MoE block: `prefill_post_attn_setup_block` and
    `prefill_layer_tail_block` (Metal/Prefill/prefill.metal:244-399).  Rows [T][d] bf16, contiguous."""

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodePostAttnSetupBlock(self, stream, hidden: torch.Tensor, attn: torch.Tensor, wPostAttn: torch.Tensor,
                                 wPreFfn: torch.Tensor, wPreFfn2: torch.Tensor, eps: float, denseX: torch.Tensor,
                                 routedX: torch.Tensor, routerX: torch.Tensor):
        call("ff_post_attn_setup", self.context.handle, _ptr(hidden), _ptr(attn), _ptr(wPostAttn), _ptr(wPreFfn),
             _ptr(wPreFfn2), hidden.shape[0], eps, _ptr(denseX), _ptr(routedX), _ptr(routerX), _stream(stream))

    def encodeLayerTailBlock(self, stream, h2: torch.Tensor, h1: torch.Tensor, hidden: torch.Tensor,
                             wPostFfn2: torch.Tensor, wPostFfn: torch.Tensor, eps: float, layerScalar: float):
        call("ff_layer_tail", self.context.handle, _ptr(h2), _ptr(h1), _ptr(hidden), _ptr(wPostFfn2),
             _ptr(wPostFfn), hidden.shape[0], eps, layerScalar, _stream(stream))


class PrefillMoE:
    """Token-major weighted combine (Kernels/Prefill/MoE/PrefillMoE.swift:11-32)."""

    def __init__(self, context: HotpathContext):
        self.context = context

    def encodeReduceTokenMajor(self, stream, routePartials: torch.Tensor, routeWeights: torch.Tensor,
                               h2: torch.Tensor, queryCount: int,
                               residual: Optional[torch.Tensor] = None,
                               rowIndex: Optional[torch.Tensor] = None):
        """rowIndex (int32 [queryCount*K], optional): where each route's partial row lies in
        `routePartials`, for rows that are not in (token, rank) order."""
        if rowIndex is None:
            call("ff_moe_reduce", self.context.handle, _ptr(routePartials), _ptr(routeWeights),
                 _ptr(residual), _ptr(h2), queryCount, _stream(stream))
        else:
            call("ff_moe_reduce_indexed", self.context.handle, _ptr(routePartials), _ptr(rowIndex),
                 _ptr(routeWeights), _ptr(residual), _ptr(h2), queryCount, _stream(stream))


class CudaRoutedPrefillGuest:
    """The `RoutedPrefillGuest` plug-in (Runtime/Supervisor/DeviceSupervisor.swift:18-22) backed by
    this library: on return every (token, rank) row named by the routes is written in `partials`;
    on failure nothing of this guest is in flight, so the host may overwrite `partials`."""

    def __init__(self, context: HotpathContext):
        self.context = context
        self._routed = PrefillGroupedRoutedMoE(context)
        self.profile = {"layers": 0, "pairs": 0}

    def runLayer(self, layer: int, hidden: torch.Tensor, partials: torch.Tensor,
                 routes: torch.Tensor, queryCount: int, stream=None):
        try:
            self._routed.encodeStreamedBatched(stream, layer, hidden, routes, partials, queryCount)
        except FieldfareError:
            torch.cuda.synchronize(self.context.device)
            raise
        self.profile["layers"] += 1
        self.profile["pairs"] += queryCount * self.context.topK


class ExpertParallelGroup:
    """`ff_ep_*`: one process driving every GPU of an expert-parallel group.  `home[r]` holds rank
    r's router and shared FFN (experts = E, topK = K), `expert[r]` its E/world experts (topK = 1,
    maxTokens >= the capacity).  The reference runs on one device; this stands where its
    `PrefillMoE` block stands (Kernels/Prefill/MoE/PrefillMoE.swift:60-140) with the grouped experts
    spread over devices."""

    def __init__(self, home: List[HotpathContext], expert: List[HotpathContext], capacityRows: int = 0):
        if len(home) != len(expert) or not home:
            raise ValueError("one home and one expert context per rank")
        self.home, self.expert = list(home), list(expert)
        world = len(home)
        arr = ctypes.c_void_p * world
        err = ctypes.c_char_p()
        self._handle = binding.load().ff_ep_create(arr(*[c.handle for c in home]), arr(*[c.handle for c in expert]),
                                                   world, capacityRows, ctypes.byref(err))
        if not self._handle:
            raise FieldfareError(err.value.decode() if err.value else "ff_ep_create failed")

    def close(self):
        if getattr(self, "_handle", None):
            binding.load().ff_ep_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def moeLayer(self, layer: int, x: List[torch.Tensor]) -> List[torch.Tensor]:
        """x[r]: bf16 [tokens][d] on rank r's device, complete (the call runs on the group's own
        streams); returns every rank's output rows, complete."""
        world = len(self.home)
        if len(x) != world or any(t.shape != x[0].shape for t in x):
            raise ValueError("one tensor of the same shape per rank")
        for r, t in enumerate(x):
            if t.device != self.home[r].device:
                raise ValueError(f"rank {r}'s rows are on {t.device}, its contexts on {self.home[r].device}")
        y = [torch.empty_like(t) for t in x]
        arr = ctypes.c_void_p * world
        call("ff_ep_moe_layer", self._handle, layer, arr(*[_ptr(t) for t in x]), x[0].shape[0],
             arr(*[_ptr(t) for t in y]))
        return y

    def moeStack(self, firstLayer: int, layerCount: int, x: List[torch.Tensor], eps: float,
                 y: Optional[List[torch.Tensor]] = None) -> List[torch.Tensor]:
        """x <- block(l, rmsnorm(x)) over the layers, per rank; returns the last block's rows."""
        world = len(self.home)
        if y is None:
            y = [torch.empty_like(t) for t in x]
        arr = ctypes.c_void_p * world
        call("ff_ep_moe_stack", self._handle, firstLayer, layerCount, arr(*[_ptr(t) for t in x]), x[0].shape[0],
             eps, arr(*[_ptr(t) for t in y]))
        return y

    def setPlacement(self, layer: int, rankOf, localOf):
        """Expert e of `layer` lives on rank rankOf[e], slot localOf[e] of that rank's expert context."""
        r = np.ascontiguousarray(np.asarray(rankOf, dtype=np.uint32))
        l = np.ascontiguousarray(np.asarray(localOf, dtype=np.uint32))
        if r.shape != l.shape or r.ndim != 1 or r.size != self.home[0].experts:
            raise ValueError("one rank and one slot per expert")
        call("ff_ep_set_placement", self._handle, layer, r.ctypes.data, l.ctypes.data)

    PHASES = ("router", "plan", "host", "send", "wait_rows", "experts", "copies_home", "shared_ffn",
              "wait_partials", "reduce")

    def setTracing(self, enabled: bool):
        binding.load().ff_ep_set_tracing(self._handle, enabled)

    def phaseTimes(self) -> List[dict]:
        """Per rank, the last traced call's milliseconds per phase, summed over its layers."""
        world, n = len(self.home), len(self.PHASES)
        out = (ctypes.c_double * (world * n))()
        got = binding.load().ff_ep_get_phase_times(self._handle, out, world * n)
        return [dict(zip(self.PHASES, out[r * n:(r + 1) * n])) for r in range(got // n)]

    @property
    def lastRowsSent(self) -> int:
        return int(binding.load().ff_ep_last_rows_sent(self._handle))
