"""ctypes binding of libfieldfare_cuda.so (the C ABI declared in include/fieldfare_cuda.h).

This is the acting caller in this repository; a Swift caller binds the same symbols through a
module map.  Loading fails loudly when the library has not been built: there is no fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, c_bool, c_char_p, c_float, c_int32, c_uint16, c_uint32, c_uint64,
                    c_void_p)

from .gturbo import MoEExpertOffsets

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libfieldfare_cuda.so")


class FieldfareError(RuntimeError):
    """A `false` return of the C ABI, carrying the library's message."""


class FFTokenExpertPair(ctypes.Structure):
    _fields_ = [("token", c_uint32), ("expert", c_uint32), ("rank", c_uint32),
                ("weightBitsAndReserved", c_uint32)]


class FFMoEGroup(ctypes.Structure):
    _fields_ = [("expert", c_uint32), ("pairStart", c_uint32), ("pairCount", c_uint32)]


class FFMoETile(ctypes.Structure):
    _fields_ = [("groupStart", c_uint32), ("groupCount", c_uint32), ("pairStart", c_uint32),
                ("pairCount", c_uint32)]


class FFProjection(ctypes.Structure):
    _fields_ = [("weights", c_void_p), ("scales", c_void_p), ("biases", c_void_p),
                ("rows", c_uint32), ("cols", c_uint32)]


class FFConfig(ctypes.Structure):
    _fields_ = [(n, c_uint32) for n in
                ("layers", "experts", "d", "f", "sharedF", "topK", "maxTokens")]


class FFInfo(ctypes.Structure):
    _fields_ = [("kernelLaunches", c_uint64), ("weightBytesResident", c_uint64),
                ("scratchBytes", c_uint64), ("lastActiveExperts", c_uint32),
                ("lastPrefillUnits", c_uint32), ("deviceOrdinal", c_uint32), ("smCount", c_uint32),
                ("deviceErrorFlag", c_uint32), ("reserved", c_uint32)]


class FFGTurboLayoutInfo(ctypes.Structure):
    _fields_ = [("expertStride", c_uint64), ("numLayers", c_uint32), ("expertsPerLayer", c_uint32),
                ("offsets", MoEExpertOffsets), ("identityPlacement", c_uint32)]


class FFTraceEntry(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char * 40), ("launches", c_uint64), ("milliseconds", ctypes.c_double)]


_ERR = POINTER(c_char_p)
_P = c_void_p

# name -> (restype, argtypes); every symbol include/fieldfare_cuda.h declares
SIGNATURES = {
    "ff_create": (c_void_p, [c_int32, POINTER(FFConfig), _ERR]),
    "ff_destroy": (None, [c_void_p]),
    "ff_string_free": (None, [c_void_p]),
    "ff_get_info": (FFInfo, [c_void_p]),
    "ff_set_tracing": (None, [c_void_p, c_bool]),
    "ff_get_trace": (c_uint32, [c_void_p, POINTER(FFTraceEntry), c_uint32]),
    "ff_decode_phase_times": (c_bool, [c_void_p, POINTER(ctypes.c_double), _ERR]),
    "ff_decode_warp_times": (c_bool, [c_void_p, POINTER(ctypes.c_double), _ERR]),
    "ff_load_layer": (c_bool, [c_void_p, c_uint32, _P, c_uint64, c_uint32, c_uint64,
                               POINTER(MoEExpertOffsets), _ERR]),
    "ff_gturbo_validate_layout": (c_bool, [c_char_p, c_uint32, c_uint32, POINTER(FFGTurboLayoutInfo), _ERR]),
    "ff_load_model_dir": (c_bool, [c_void_p, c_char_p, _ERR]),
    "ff_load_shared": (c_bool, [c_void_p, c_uint32, POINTER(FFProjection), POINTER(FFProjection),
                                POINTER(FFProjection), _ERR]),
    "ff_load_shared_int8": (c_bool, [c_void_p, c_uint32, POINTER(FFProjection), POINTER(FFProjection),
                                     POINTER(FFProjection), _ERR]),
    "ff_load_router": (c_bool, [c_void_p, c_uint32, _P, _P, _P, _P, c_uint32, c_uint32, _ERR]),
    "ff_load_router_int8": (c_bool, [c_void_p, c_uint32, _P, _P, _P, _P, _P, _P, c_uint32, c_uint32, _ERR]),
    "ff_expert_address": (c_uint64, [c_void_p, c_uint32, c_uint32]),
    "ff_dequant_probe": (c_bool, [c_void_p, c_uint32, c_int32, c_uint32, _P, _P, _ERR]),
    "ff_dequant_probe_bf16": (c_bool, [c_void_p, c_uint32, c_int32, c_uint32, _P, _P, _ERR]),
    "ff_router_topk": (c_bool, [c_void_p, c_uint32, _P, c_uint32, c_uint32, _P, _P, _P, _P, _ERR]),
    "ff_moe_decode": (c_bool, [c_void_p, c_uint32, _P, _P, _P, _P, _P, _P, _ERR]),
    "ff_moe_verify": (c_bool, [c_void_p, c_uint32, _P, c_uint32, c_uint32, _P, _P, _P, _ERR]),
    "ff_moe_prefill": (c_bool, [c_void_p, c_uint32, _P, c_uint32, c_uint32, _P, _P, _P, _ERR]),
    "ff_moe_reduce": (c_bool, [c_void_p, _P, _P, _P, _P, c_uint32, _P, _ERR]),
    "ff_moe_reduce_indexed": (c_bool, [c_void_p, _P, _P, _P, _P, _P, c_uint32, _P, _ERR]),
    "ff_shared_ffn": (c_bool, [c_void_p, c_uint32, _P, c_uint32, c_uint32, _P, _P, _ERR]),
    "ff_shared_ffn_noalloc": (c_bool, [POINTER(FFProjection), POINTER(FFProjection),
                                       POINTER(FFProjection), _P, c_uint32, c_uint32, _P, c_uint32,
                                       _P, _ERR]),
    "ff_int4_gemv_rows": (c_bool, [c_void_p, POINTER(FFProjection), _P, c_uint32, c_uint32, _P,
                                   c_uint32, _P, _ERR]),
    "ff_rmsnorm": (c_bool, [c_void_p, _P, _P, c_float, c_uint32, _P, _P, _ERR]),
    "ff_moe_layer": (c_bool, [c_void_p, c_uint32, _P, c_uint32, _P, _P, _P, _P, _ERR]),
    "ff_moe_stack": (c_bool, [c_void_p, c_uint32, c_uint32, _P, c_uint32, c_float, _P, _P, _P, _ERR]),
    "ff_reset_device_error": (c_bool, [c_void_p, _ERR]),
    "ff_moe_layer_host": (c_bool, [c_void_p, c_uint32, _P, c_uint32, _P, _ERR]),
    "ff_make_token_expert_pairs": (c_uint64, [_P, _P, c_uint32, c_uint32, POINTER(FFTokenExpertPair)]),
    "ff_group_token_expert_pairs": (c_bool, [POINTER(FFTokenExpertPair), c_uint64, c_uint32, c_uint32,
                                             c_uint32, c_uint32, _P, POINTER(FFTokenExpertPair),
                                             POINTER(FFMoEGroup), POINTER(c_uint32),
                                             POINTER(FFMoETile), POINTER(c_uint32), _ERR]),
    "ff_last_prefill_routes": (c_bool, [c_void_p, POINTER(FFTokenExpertPair), _P, _ERR]),
    "ff_post_attn_setup": (c_bool, [c_void_p, _P, _P, _P, _P, _P, c_uint32, c_float, _P, _P, _P, _P, _ERR]),
    "ff_layer_tail": (c_bool, [c_void_p, _P, _P, _P, _P, _P, c_uint32, c_float, c_float, _P, _ERR]),
    "ff_sort_routes": (c_bool, [c_void_p, _P, c_uint32, c_uint32, _P, _P, _P, _ERR]),
    "ff_ep_create": (c_void_p, [POINTER(c_void_p), POINTER(c_void_p), c_uint32, c_uint32, _ERR]),
    "ff_ep_destroy": (None, [c_void_p]),
    "ff_ep_moe_layer": (c_bool, [c_void_p, c_uint32, POINTER(c_void_p), c_uint32, POINTER(c_void_p), _ERR]),
    "ff_ep_last_rows_sent": (c_uint64, [c_void_p]),
    "ff_ep_moe_stack": (c_bool, [c_void_p, c_uint32, c_uint32, POINTER(c_void_p), c_uint32, c_float,
                                 POINTER(c_void_p), _ERR]),
    "ff_ep_set_tracing": (None, [c_void_p, c_bool]),
    "ff_ep_get_phase_times": (c_uint32, [c_void_p, POINTER(ctypes.c_double), c_uint32]),
    "ff_ep_set_placement": (c_bool, [c_void_p, c_uint32, _P, _P, _ERR]),
}

_lib = None


def load() -> ctypes.CDLL:
    """The shared library with argument types set.  Raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FieldfareError(
            f"{LIB_PATH} is missing: build it with `python -m ane_fieldfare_b200.build` "
            "(nvcc, sm_100a).  There is no CPU fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def call(name: str, *args):
    """Calls a bool-returning entry point; raises FieldfareError with the library's message."""
    lib = load()
    err = c_char_p()
    ok = getattr(lib, name)(*args, ctypes.byref(err))
    if not ok:
        message = err.value.decode("utf-8", "replace") if err.value else "unknown error"
        raise FieldfareError(message)
    return True
