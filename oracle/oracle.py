"""ctypes wrapper of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE: imported only by tests/,
__graft_entry__.smoke() and bench.py's CPU-baseline legs — never by the shipped package."""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_uint16, c_uint32, c_uint64, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    src = [os.path.join(HERE, n) for n in ("oracle.c", "oracle.h", "Makefile")]
    if force or not os.path.exists(LIB) or any(os.path.getmtime(s) > os.path.getmtime(LIB) for s in src):
        subprocess.run(["make", "-C", HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return LIB


class Offsets(ctypes.Structure):
    _fields_ = [(n, c_uint32) for n in ("gate_w", "gate_s", "gate_b", "up_w", "up_s", "up_b",
                                        "down_w", "down_s", "down_b")]


class Pair(ctypes.Structure):
    _fields_ = [("token", c_uint32), ("expert", c_uint32), ("rank", c_uint32), ("weight_bits", c_uint32)]


class Group(ctypes.Structure):
    _fields_ = [("expert", c_uint32), ("pair_start", c_uint32), ("pair_count", c_uint32)]


class Tile(ctypes.Structure):
    _fields_ = [("group_start", c_uint32), ("group_count", c_uint32), ("pair_start", c_uint32),
                ("pair_count", c_uint32)]


class Layer(ctypes.Structure):
    _fields_ = [("experts", c_void_p), ("expert_stride", c_uint64), ("off", Offsets),
                ("shared", c_void_p), ("shared_off", Offsets), ("router_w", c_void_p),
                ("router_scale", c_void_p), ("gain", c_void_p), ("logit_bias", c_void_p),
                ("E", c_int32), ("D", c_int32), ("F", c_int32), ("Fs", c_int32), ("K", c_int32)]


MODE_DECODE, MODE_PARTIALS = 0, 1
MODE_BF16_WEIGHTS = 2  # or-ed onto a mode: weights rounded once to bf16 (the prefill GEMM's operand)
_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        L = _lib
        L.ffo_bf16_bits.restype = c_uint16
        L.ffo_bf16_bits.argtypes = [c_float]
        L.ffo_bf16_to_float.restype = c_float
        L.ffo_bf16_to_float.argtypes = [c_uint16]
        L.ffo_splitmix64_next.restype = c_uint64
        L.ffo_splitmix64_next.argtypes = [POINTER(c_uint64)]
        L.ffo_splitmix64_uniform.restype = c_float
        L.ffo_splitmix64_uniform.argtypes = [POINTER(c_uint64), c_float, c_float]
        L.ffo_seedtree_key.restype = c_uint64
        L.ffo_seedtree_key.argtypes = [c_uint64, c_char_p]
        L.ffo_int4_dot.restype = c_float
        L.ffo_gelu_tanh.restype = c_float
        L.ffo_gelu_tanh.argtypes = [c_float]
        L.ffo_make_pairs.restype = c_int64
        L.ffo_group_pairs.restype = c_int32
        L.ffo_num_threads.restype = c_int32
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(c_void_p)


def offsets_from(tup) -> Offsets:
    return Offsets(*tup)


class LayerData:
    """Keeps the numpy arrays of one layer alive and exposes the C struct."""

    def __init__(self, *, experts, stride, off, E, D, F, K, shared=None, shared_off=None, Fs=0,
                 router_w=None, router_scale=None, gain=None, logit_bias=None):
        self.arrays = dict(experts=experts, shared=shared, router_w=router_w,
                           router_scale=router_scale, gain=gain, logit_bias=logit_bias)
        self.c = Layer(_p(experts), stride, offsets_from(off), _p(shared),
                       offsets_from(shared_off if shared_off is not None else (0,) * 9),
                       _p(router_w), _p(router_scale), _p(gain), _p(logit_bias), E, D, F, Fs, K)
        self.E, self.D, self.F, self.Fs, self.K = E, D, F, Fs, K


def bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().ffo_bf16_bits_n(_p(x), _p(out), c_int64(x.size))
    return out


def bf16_to_float(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float32)
    lib().ffo_bf16_to_float_n(_p(b), _p(out), c_int64(b.size))
    return out


def splitmix64_fill(seed: int, n: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint64)
    lib().ffo_splitmix64_fill(c_uint64(seed), _p(out), c_int64(n))
    return out


def quantize_int4_rows(rows: np.ndarray):
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    m, n = rows.shape
    packed = np.zeros((m, n // 2), dtype=np.uint8)
    scales = np.zeros((m, n // 64), dtype=np.uint16)
    biases = np.zeros((m, n // 64), dtype=np.uint16)
    for r in range(m):
        lib().ffo_quantize_int4_row(_p(rows[r]), c_int32(n), _p(packed[r]), _p(scales[r]), _p(biases[r]))
    return packed, scales, biases


def dequant_int4(w, s, b, rows, cols, bf16=False):
    out = np.empty((rows, cols), dtype=np.uint16 if bf16 else np.float32)
    fn = lib().ffo_dequant_int4_bf16 if bf16 else lib().ffo_dequant_int4
    fn(_p(w), _p(s), _p(b), c_int32(rows), c_int32(cols), _p(out))
    return out


def int4_gemv_rows(w, s, b, rows, cols, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty((x.shape[0], rows), dtype=np.float32)
    lib().ffo_int4_gemv_rows(_p(w), _p(s), _p(b), c_int32(rows), c_int32(cols), _p(x),
                             c_int32(x.shape[0]), c_int32(x.shape[1]), _p(y), c_int32(rows))
    return y


def int4_dot(w, s, b, row, cols, x) -> float:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return float(lib().ffo_int4_dot(_p(w), _p(s), _p(b), c_int32(row), c_int32(cols), _p(x)))


def expert_ffn(blob, off, D, F, x_bits, round_gate_up=False, round_act=True):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x_bits.shape[0]
    out = np.empty((T, D), dtype=np.float32)
    o = offsets_from(off)
    lib().ffo_expert_ffn(_p(blob), ctypes.byref(o), c_int32(D), c_int32(F), _p(x_bits), c_int32(T),
                         c_int32(x_bits.shape[1]), c_int32(int(round_gate_up)), c_int32(int(round_act)),
                         _p(out), c_int32(D))
    return out


def post_attn_setup(hidden, attn, w_post_attn, w_pre_ffn, w_pre_ffn2, eps):
    """prefill_post_attn_setup_block (Metal/Prefill/prefill.metal:244-318) on bf16 bit patterns
    [T][D]: returns (hidden', dense_x, routed_x, router_x)."""
    h = np.array(hidden, dtype=np.uint16, copy=True)
    attn = np.ascontiguousarray(attn, dtype=np.uint16)
    T, D = h.shape
    ws = [np.ascontiguousarray(w, dtype=np.uint16) for w in (w_post_attn, w_pre_ffn, w_pre_ffn2)]
    outs = [np.empty((T, D), dtype=np.uint16) for _ in range(3)]
    lib().ffo_post_attn_setup(_p(h), _p(attn), _p(ws[0]), _p(ws[1]), _p(ws[2]), c_int32(T), c_int32(D),
                              c_float(eps), _p(outs[0]), _p(outs[1]), _p(outs[2]))
    return h, outs[0], outs[1], outs[2]


def layer_tail(h2, h1, hidden, w_postffn2, w_postffn, eps, layer_scalar):
    """prefill_layer_tail_block (Metal/Prefill/prefill.metal:321-399): returns hidden'."""
    h = np.array(hidden, dtype=np.uint16, copy=True)
    h2 = np.ascontiguousarray(h2, dtype=np.uint16)
    h1 = np.ascontiguousarray(h1, dtype=np.uint16)
    T, D = h.shape
    w2 = np.ascontiguousarray(w_postffn2, dtype=np.uint16)
    w1 = np.ascontiguousarray(w_postffn, dtype=np.uint16)
    lib().ffo_layer_tail(_p(h2), _p(h1), _p(h), _p(w2), _p(w1), c_int32(T), c_int32(D), c_float(eps),
                         c_float(layer_scalar))
    return h


def shared_ffn_int8(gate, up, down, x_bits):
    """INT8 affine shared FFN (Kernels/MoE/SharedExpertInt8.swift): gate/up/down = (codes uint8
    [rows][cols], scales, biases bf16 bits [rows][cols/64]); x bf16 bits [T][D] -> y bf16 bits."""
    arrs = []
    for codes, scales, biases in (gate, up, down):
        arrs += [np.ascontiguousarray(codes, dtype=np.uint8), np.ascontiguousarray(scales, dtype=np.uint16),
                 np.ascontiguousarray(biases, dtype=np.uint16)]
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T, D = x_bits.shape
    Fs = arrs[0].shape[0]
    y = np.empty((T, D), dtype=np.uint16)
    lib().ffo_shared_ffn_int8(*[_p(a) for a in arrs], c_int32(D), c_int32(Fs), _p(x_bits), c_int32(T), _p(y))
    return y


def router_topk_int8(codes, scales, biases, x_bits, K, effective_scale=None, logit_bias=None, gain=None):
    """INT8 affine router (Metal/MoE/moe.metal:65-103) + top-K: ids, 16-bit weights, logits."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint16)
    biases = np.ascontiguousarray(biases, dtype=np.uint16)
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    E, D = codes.shape
    T = x_bits.shape[0]
    es = None if effective_scale is None else np.ascontiguousarray(effective_scale, dtype=np.uint16)
    lb = None if logit_bias is None else np.ascontiguousarray(logit_bias, dtype=np.float32)
    gn = None if gain is None else np.ascontiguousarray(gain, dtype=np.uint16)
    ids = np.empty((T, K), dtype=np.uint32)
    w = np.empty((T, K), dtype=np.uint16)
    logits = np.empty((T, E), dtype=np.float32)
    lib().ffo_router_topk_int8(_p(codes), _p(scales), _p(biases), _p(es) if es is not None else None,
                               _p(lb) if lb is not None else None, _p(gn) if gn is not None else None,
                               c_int32(E), c_int32(D), c_int32(K), _p(x_bits), c_int32(T),
                               c_int32(x_bits.shape[1]), _p(ids), _p(w), _p(logits))
    return ids, w, logits


def router_topk(layer: LayerData, x_bits):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x_bits.shape[0]
    ids = np.empty((T, layer.K), dtype=np.uint32)
    w = np.empty((T, layer.K), dtype=np.uint16)
    logits = np.empty((T, layer.E), dtype=np.float32)
    lib().ffo_router_topk(ctypes.byref(layer.c), _p(x_bits), c_int32(T), c_int32(x_bits.shape[1]),
                          _p(ids), _p(w), _p(logits))
    return ids, w, logits


def make_pairs(ids, weights, T, K):
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    weights = np.ascontiguousarray(weights, dtype=np.uint16)
    pairs = (Pair * max(1, T * K))()
    n = lib().ffo_make_pairs(_p(ids), _p(weights), c_int32(T), c_int32(K), pairs)
    return pairs, int(n)


def group_pairs(pairs, n_pairs, T, K, E, tile_experts, sort_keys=None):
    sorted_pairs = (Pair * max(1, n_pairs))()
    groups = (Group * max(1, E))()
    tiles = (Tile * max(1, E))()
    ng, nt, bad = c_int32(), c_int32(), c_uint32()
    keys = None if sort_keys is None else np.ascontiguousarray(sort_keys, dtype=np.uint64)
    rc = lib().ffo_group_pairs(pairs, c_int64(n_pairs), c_int32(T), c_int32(K), c_int32(E),
                               c_int32(tile_experts), _p(keys), sorted_pairs, groups,
                               ctypes.byref(ng), tiles, ctypes.byref(nt), ctypes.byref(bad))
    if rc != 0:
        raise ValueError(f"route expert {bad.value} is out of range")
    return list(sorted_pairs)[:n_pairs], list(groups)[:ng.value], list(tiles)[:nt.value]


def route_partials(layer: LayerData, x_bits, pairs, n_pairs, T, bf16_weights=False):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    out = np.zeros((T * layer.K, layer.D), dtype=np.uint16)
    fn = lib().ffo_route_partials_bf16w if bf16_weights else lib().ffo_route_partials
    fn(ctypes.byref(layer.c), _p(x_bits), c_int32(x_bits.shape[1]), pairs, c_int64(n_pairs), _p(out))
    return out


def reduce_token_major(partials, weights, residual, T, K, D):
    out = np.empty((T, D), dtype=np.uint16)
    lib().ffo_reduce_token_major(_p(partials), _p(weights), _p(residual), c_int32(T), c_int32(K),
                                 c_int32(D), _p(out))
    return out


def rmsnorm_bf16(x_bits, w_bits, eps, T, n):
    out = np.empty((T, n), dtype=np.uint16)
    lib().ffo_rmsnorm_bf16(_p(x_bits), _p(w_bits), c_float(eps), c_int32(T), c_int32(n), _p(out))
    return out


def shared_ffn(layer: LayerData, x_bits, bf16_weights=False):
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x_bits.shape[0]
    y = np.empty((T, layer.D), dtype=np.uint16)
    fn = lib().ffo_shared_ffn_bf16w if bf16_weights else lib().ffo_shared_ffn
    fn(ctypes.byref(layer.c), _p(x_bits), c_int32(T), c_int32(x_bits.shape[1]), _p(y))
    return y


def moe_layer(layer: LayerData, x_bits, mode):
    """Returns (y bf16 bits, y fp32 before the last rounding, ids, route weights bf16 bits)."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x_bits.shape[0]
    y = np.empty((T, layer.D), dtype=np.uint16)
    y32 = np.empty((T, layer.D), dtype=np.float32)
    ids = np.empty((T, layer.K), dtype=np.uint32)
    w = np.empty((T, layer.K), dtype=np.uint16)
    lib().ffo_moe_layer(ctypes.byref(layer.c), _p(x_bits), c_int32(T), c_int32(mode), _p(y), _p(y32),
                        _p(ids), _p(w))
    return y, y32, ids, w


def moe_stack(layers, x_bits, eps, mode):
    """x <- layer_l(rmsnorm(x)) over the list of LayerData; returns (y bf16 bits, ids [layers, T, K])."""
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    T = x_bits.shape[0]
    n = len(layers)
    arr = (Layer * n)(*[l.c for l in layers])
    y = np.empty((T, layers[0].D), dtype=np.uint16)
    ids = np.empty((n, T, layers[0].K), dtype=np.uint32)
    lib().ffo_moe_stack(arr, c_int32(n), _p(x_bits), c_int32(T), c_float(eps), c_int32(mode), _p(y), _p(ids))
    return y, ids


def set_num_threads(n: int) -> None:
    lib().ffo_set_num_threads(c_int32(int(n)))


def num_threads() -> int:
    return int(lib().ffo_num_threads())
