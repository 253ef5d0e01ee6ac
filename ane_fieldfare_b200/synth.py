"""Seeded synthetic inputs for the INT4 MoE hot path, in the reference's formats.

The generator is the reference's test PRNG — SplitMix64 streams derived from one root by
FNV-1a label hashing (Tests/Support/Validation/PRNG/SplitMix64.swift:9-21,
Tests/Support/Validation/PRNG/SeedTree.swift:12-19) — vectorised with numpy: SplitMix64's state
is a counter, so output i is a pure function of (seed, i).

Weights follow the benchmark configurations: every 4-bit code uniform in 0..15, per group of 64
scale = bf16(0.002 + U(0, 0.01)) and bias = bf16(-scale * U(6, 10)), packed low-nibble-first
(8 codes per little-endian uint32) and laid out as `.gturbo` expert blobs (see gturbo.py).
Normals are Box-Muller over two 53-bit uniforms (the reference PRNG only has `uniform`).
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_MASK = (1 << 64) - 1


def seedtree_key(root: int, label: str) -> int:
    """SeedTree.key: FNV-1a 64 of the label's UTF-8 bytes, XOR the root."""
    h = 0xCBF29CE484222325
    for byte in label.encode("utf-8"):
        h ^= byte
        h = (h * 0x100000001B3) & _MASK
    return (root ^ h) & _MASK


def splitmix64(seed: int, n: int, start: int = 0) -> np.ndarray:
    """Outputs start..start+n of SplitMix64(seed) as uint64 (output 0 is the first next())."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + n + 1, dtype=np.uint64)
        z = np.uint64(seed & _MASK) + idx * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, lo: float, hi: float, start: int = 0) -> np.ndarray:
    """SplitMix64.uniform: lo + (hi - lo) * (next() >> 40) / 2^24, all in fp32."""
    u = (splitmix64(seed, n, start) >> np.uint64(40)).astype(np.float32) / np.float32(1 << 24)
    span = np.float32(hi) - np.float32(lo)
    return (np.float32(lo) + span * u).astype(np.float32)


def normal(seed: int, n: int, std: float = 1.0) -> np.ndarray:
    """Box-Muller: draws 2i and 2i+1 of the stream give sample i (float64)."""
    raw = splitmix64(seed, 2 * n)
    u1 = ((raw[0::2] >> np.uint64(11)).astype(np.float64) + 1.0) / float(1 << 53)
    u2 = (raw[1::2] >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    return std * np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """Quantization.bf16Bits (Infrastructure/ModelIO/Quantization.swift:9-16), vectorised."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    with np.errstate(over="ignore"):
        return ((u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_to_float(bits: np.ndarray) -> np.ndarray:
    """Quantization.bf16ToFloat (Quantization.swift:18-20)."""
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def int4_matrix(root: int, label: str, count: int, rows: int, cols: int):
    """`count` affine INT4 matrices [rows][cols]: (packed uint8 [count, rows*cols/2],
    scales uint16 [count, rows*cols/64], biases uint16 [count, rows*cols/64])."""
    assert cols % 64 == 0
    words = count * rows * cols // 16
    packed = splitmix64(seedtree_key(root, label + ".q"), words).view(np.uint8)
    groups = count * rows * cols // 64
    scale = np.float32(0.002) + uniform(seedtree_key(root, label + ".s"), groups, 0.0, 0.01)
    s_bits = bf16_bits(scale)
    spread = uniform(seedtree_key(root, label + ".b"), groups, 6.0, 10.0)
    b_bits = bf16_bits(-bf16_to_float(s_bits) * spread)
    return (packed.reshape(count, rows * cols // 2), s_bits.reshape(count, -1), b_bits.reshape(count, -1))


def normal_bf16(root: int, label: str, shape, std: float = 1.0) -> np.ndarray:
    n = int(np.prod(shape))
    return bf16_bits(normal(seedtree_key(root, label), n, std).astype(np.float32)).reshape(shape)


def zipf_log_prior(experts: int, s: float = 1.1, root: int | None = None, label: str = "zipf") -> np.ndarray:
    """log of a Zipf(s) prior over the experts, assigned to experts in a seeded shuffle."""
    ranks = np.arange(1, experts + 1, dtype=np.float64)
    p = ranks ** (-s)
    p /= p.sum()
    order = np.arange(experts)
    if root is not None:
        order = np.argsort(splitmix64(seedtree_key(root, label), experts), kind="stable")
    out = np.empty(experts, dtype=np.float32)
    out[order] = np.log(p).astype(np.float32)
    return out
