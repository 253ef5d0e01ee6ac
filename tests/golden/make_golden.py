"""Writes tests/golden/tiny_layer.npz: inputs and CPU-oracle outputs of a tiny seeded MoE layer.

The reference stores no golden vectors for this path and cannot be run on Linux, so these
fixtures come from this repository's oracle (oracle/oracle.c); they pin the oracle and the
generator against drift and give the GPU tests a fixed small case.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from ane_fieldfare_b200 import workload  # noqa: E402
from conftest import oracle_layer  # noqa: E402
from oracle import oracle as O  # noqa: E402

cfg = dict(root=0x604, experts=16, d=128, f=64, sharedF=192, topK=8, tokens=6)
L = workload.make_layer(cfg["root"], 0, experts=cfg["experts"], d=cfg["d"], f=cfg["f"],
                        sharedF=cfg["sharedF"], topK=cfg["topK"], router_bias="normal")
ld = oracle_layer(O, L)
x = workload.make_tokens(cfg["root"], "x", cfg["tokens"], cfg["d"])
y, y32, ids, w = O.moe_layer(ld, x, O.MODE_PARTIALS)
y1, _, _, _ = O.moe_layer(ld, x[:1], O.MODE_DECODE)
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tiny_layer.npz"),
                    x=x, blobs=L.blobs[:, :L.layout.payload], ids=ids, weights=w,
                    y_partials_mode=y, y_decode_mode_row0=y1, **cfg)
print("wrote tiny_layer.npz", y.shape)
