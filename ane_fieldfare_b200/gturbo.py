"""The `.gturbo` packed-expert layout for one layer, as the reference writes and reads it.

One expert blob holds nine sub-tensors back to back — gate, up, down, each as packed weights
(U32 words, 8 codes each), bf16 scales, bf16 biases — and is padded to a 16 KiB page
(Sources/ANEFieldfareInstallCore/Planning/RepackPlanner.swift:425-498).  A layer file
`packed_experts/layer_%02d.bin` is expertsPerLayer blobs `expertStride` apart
(Sources/ANEFieldfareImportedFormat/GTurboPackedExpertsLayoutV1.swift:3-72); the nine byte offsets
are the same for every expert of the layer (Runtime/Inference/ModelExpertIO.swift:11-30) and are
what `MoEExpertOffsets` carries to the kernels (Kernels/MoE/MoE.swift:4-29).
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass

import numpy as np

from . import synth

PAGE = 16384
ROLES = ("gate", "up", "down")


class MoEExpertOffsets(ctypes.Structure):
    """Layout-identical to the reference's `MoEExpertOffsets` (Kernels/MoE/MoE.swift:4-15)."""

    _fields_ = [(n, ctypes.c_uint32) for n in (
        "gateWOff", "gateSOff", "gateBOff", "upWOff", "upSOff", "upBOff",
        "downWOff", "downSOff", "downBOff")]

    def as_tuple(self):
        return tuple(getattr(self, n) for n, _ in self._fields_)


@dataclass(frozen=True)
class ExpertLayout:
    d: int            # model width (gate/up columns, down rows)
    f: int            # intermediate width (gate/up rows, down columns)
    offsets: MoEExpertOffsets
    payload: int      # bytes used by the nine sub-tensors
    stride: int       # payload rounded up to a 16 KiB page

    def matrix_shape(self, role: str):
        return (self.f, self.d) if role in ("gate", "up") else (self.d, self.f)


def expert_layout(d: int, f: int) -> ExpertLayout:
    if d % 64 or f % 64:
        raise ValueError("D and F must be multiples of the group size 64")
    cursor = 0
    values = []
    for _ in ROLES:
        w = d * f // 2
        s = d * f // 64 * 2
        values += [cursor, cursor + w, cursor + w + s]
        cursor += w + 2 * s
    stride = (cursor + PAGE - 1) // PAGE * PAGE
    return ExpertLayout(d, f, MoEExpertOffsets(*values), cursor, stride)


def synthetic_experts(root: int, label: str, count: int, d: int, f: int) -> np.ndarray:
    """`count` seeded expert blobs as one uint8 array [count, stride] (a layer file's bytes)."""
    lay = expert_layout(d, f)
    blobs = np.zeros((count, lay.stride), dtype=np.uint8)
    off = lay.offsets.as_tuple()
    for r, role in enumerate(ROLES):
        rows, cols = lay.matrix_shape(role)
        packed, scales, biases = synth.int4_matrix(root, f"{label}.{role}", count, rows, cols)
        w_off, s_off, b_off = off[3 * r: 3 * r + 3]
        blobs[:, w_off:w_off + packed.shape[1]] = packed
        blobs[:, s_off:s_off + scales.shape[1] * 2] = scales.view(np.uint8).reshape(count, -1)
        blobs[:, b_off:b_off + biases.shape[1] * 2] = biases.view(np.uint8).reshape(count, -1)
    return blobs


def sub_tensor(blob: np.ndarray, lay: ExpertLayout, role: str):
    """Views (packed uint8 [rows, cols/2], scales uint16 [rows, cols/64], biases likewise)."""
    r = ROLES.index(role)
    rows, cols = lay.matrix_shape(role)
    w_off, s_off, b_off = lay.offsets.as_tuple()[3 * r: 3 * r + 3]
    w = blob[w_off:w_off + rows * cols // 2].reshape(rows, cols // 2)
    s = blob[s_off:s_off + rows * cols // 32].view(np.uint16).reshape(rows, cols // 64)
    b = blob[b_off:b_off + rows * cols // 32].view(np.uint16).reshape(rows, cols // 64)
    return w, s, b


def layout_json(num_layers: int, experts: int, lay: ExpertLayout, physical_ranks=None,
                explicit_ids: bool = True) -> str:
    """`packed_experts/layout.json` with the reference's keys and conventions
    (Sources/ANEFieldfareInstallCore/Format/GTurboJSON.swift:110-172): `file` is the layer file's
    basename, an expert's `size` is the expert stride and its `offset` physicalRank * stride.
    `physical_ranks[layer][expert]` (default: identity) places expert blobs inside the layer file."""
    off = lay.offsets.as_tuple()

    def tensors():
        out = {}
        for r, role in enumerate(ROLES):
            rows, cols = lay.matrix_shape(role)
            w_off, s_off, b_off = off[3 * r: 3 * r + 3]
            out[role] = {"offset": w_off, "size": rows * cols // 2, "dtype": "U32",
                         "shape": [rows, cols // 8], "bits": 4}
            out[role + "_scales"] = {"offset": s_off, "size": rows * cols // 32, "dtype": "BF16",
                                     "shape": [rows, cols // 64]}
            out[role + "_biases"] = {"offset": b_off, "size": rows * cols // 32, "dtype": "BF16",
                                     "shape": [rows, cols // 64]}
        return out

    layers = []
    for layer in range(num_layers):
        entries = []
        for e in range(experts):
            rank = e if physical_ranks is None else int(physical_ranks[layer][e])
            entry = {"offset": rank * lay.stride, "size": lay.stride, "tensors": tensors()}
            if explicit_ids:
                entry["expert"] = e
            if rank != e:
                entry["physicalRank"] = rank
            entries.append(entry)
        layers.append({"layer": layer, "file": "layer_%02d.bin" % layer, "experts": entries})
    return json.dumps({"expertStride": lay.stride, "numLayers": num_layers,
                       "expertsPerLayer": experts, "layers": layers})


def write_model_dir(path: str, layer_blobs, lay: ExpertLayout, physical_ranks=None) -> None:
    """Writes `<path>/packed_experts/layout.json` and one `layer_%02d.bin` per entry of
    `layer_blobs` (uint8 [experts, stride] each, logical expert order); with `physical_ranks` the
    blob of expert e is stored at rank physical_ranks[layer][e] of its file."""
    import os
    out = os.path.join(path, "packed_experts")
    os.makedirs(out, exist_ok=True)
    experts = layer_blobs[0].shape[0]
    for layer, blobs in enumerate(layer_blobs):
        data = np.ascontiguousarray(blobs, dtype=np.uint8)
        if physical_ranks is not None:
            stored = np.empty_like(data)
            stored[np.asarray(physical_ranks[layer], dtype=np.int64)] = data
            data = stored
        data.tofile(os.path.join(out, "layer_%02d.bin" % layer))
    with open(os.path.join(out, "layout.json"), "w") as fh:
        fh.write(layout_json(len(layer_blobs), experts, lay, physical_ranks))
