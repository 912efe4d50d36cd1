"""ctypes binding of libtq_b200.so (declared in include/tq_b200.h).

There is no CPU fallback: importing this module without the built library, or calling a
compute entry point without a CUDA device, raises.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtq_b200.so")

F32, F16, F64, BF16 = 0, 1, 2, 3
ROT_DENSE, ROT_WHT = 0, 1
FMT_TURBO2, FMT_TURBO3, FMT_TURBO4, FMT_Q8_0 = 2, 3, 4, 8
FMT_PROD2, FMT_PROD3, FMT_PROD4 = 18, 19, 20
DECODE_OVERLAP = 8  # tq_decode_attn_phases: TQ_DECODE_OVERLAP
DECODE_OVERLAP_Q = 8 | 64  # TQ_DECODE_OVERLAP_Q: the queries may be read early too
DECODE_OVERLAP_APPEND = 8 | 64 | 128  # TQ_DECODE_OVERLAP_APPEND: after the append of the step's token
DECODE_CHAIN_HEAD = 256  # TQ_DECODE_CHAIN_HEAD: calls with DECODE_OVERLAP_Q follow this one
DECODE_SPARSE_V = 16  # TQ_DECODE_SPARSE_V
DECODE_NO_DEQUANT = 32  # TQ_DECODE_NO_DEQUANT (measurement only)
FORMATS = {"turbo2": FMT_TURBO2, "turbo3": FMT_TURBO3, "turbo4": FMT_TURBO4, "q8_0": FMT_Q8_0,
           "prod2": FMT_PROD2, "prod3": FMT_PROD3, "prod4": FMT_PROD4}

ERR_INVALID = -1


class TQError(RuntimeError):
    """A libtq_b200 entry point returned a negative status."""


class QuantizerDesc(C.Structure):
    _fields_ = [("d", C.c_int32), ("bits", C.c_int32), ("rotation", C.c_int32),
                ("norm_correction", C.c_int32), ("rot", C.c_void_p), ("signs1", C.c_void_p),
                ("signs2", C.c_void_p), ("centroids", C.c_void_p), ("qjl", C.c_int32),
                ("qjl_s", C.c_void_p), ("qjl_signs1", C.c_void_p), ("qjl_signs2", C.c_void_p)]


class CacheLayout(C.Structure):
    _fields_ = [("d", C.c_int32), ("page_tokens", C.c_int32), ("num_kv_heads", C.c_int32),
                ("k_format", C.c_int32), ("v_format", C.c_int32), ("k_idx_bytes", C.c_int32),
                ("v_idx_bytes", C.c_int32), ("k_idx_off", C.c_int32), ("k_scale_off", C.c_int32),
                ("k_qjl_off", C.c_int32), ("k_rscale_off", C.c_int32), ("v_idx_off", C.c_int32),
                ("v_scale_off", C.c_int32), ("record_bytes", C.c_int32), ("head_stride", C.c_int64),
                ("page_stride", C.c_int64)]


_P, _I32, _I64, _F = C.c_void_p, C.c_int32, C.c_int64, C.c_float

# name -> (restype, argtypes); the list doubles as the table of symbols the header declares
SIGNATURES = {
    "tq_version": (C.c_char_p, []),
    "tq_error_string": (C.c_char_p, [C.c_int]),
    "tq_last_error": (C.c_char_p, []),
    "tq_quantizer_create": (C.c_int, [C.POINTER(QuantizerDesc), C.POINTER(_P)]),
    "tq_quantizer_destroy": (C.c_int, [_P]),
    "tq_quantize": (C.c_int, [_P, _P, _I32, _I64, _I64, _P, _P, _P, _P, _P, _P, _P]),
    "tq_dequantize": (C.c_int, [_P, _P, _P, _P, _P, _P, _F, _I64, _P, _I32, _P]),
    "tq_pack_indices": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "tq_unpack_indices": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "tq_pack_bits": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "tq_unpack_bits": (C.c_int, [_P, _I64, _I32, _P, _P]),
    "tq_sign_wht_f64": (C.c_int, [_P, _I64, _I32, _I32, _P, _P, _P, _P]),
    "tq_nearest_centroid_f64": (C.c_int, [_P, _I64, _P, _I32, _P, _P]),
    "tq_block_bytes": (C.c_int64, [_I32, _I32]),
    "tq_cache_export_blocks": (C.c_int, [_P, _P, _I32, _P, _I64, _I32, _P, _P]),
    "tq_cache_import_blocks": (C.c_int, [_P, _P, _I32, _P, _I64, _I32, _P, _P]),
    "tq_cache_requantize": (C.c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _I32, _I64, _P]),
    "tq_decode_attn_lse": (C.c_int, [_P, _P, _P, _P, _P, _I32, _P, _P, _I32, _I32, _I32, _F, _P, _I64, _P, _I32, _I32, _P, _P]),
    "tq_attn_merge": (C.c_int, [_P, _P, _P, _P, _I64, _I32, _P, _P, _P]),
    "tq_requantize": (C.c_int, [_P, _P, _P, _P, _I32, _I64, _P, _P, _P, _P]),
    "tq_quantize_residual": (C.c_int, [_P, _P, _I32, _I64, _I64, _P, _P, _P, _I64, _P]),
    "tq_dequantize_strided": (C.c_int, [_P, _P, _P, _I64, _P, _I64, _I32, _P]),
    "tq_qjl_quantize": (C.c_int, [_P, _P, _I32, _I64, _P, _P, _P]),
    "tq_qjl_dequantize": (C.c_int, [_P, _P, _P, _F, _I64, _P, _I32, _P]),
    "tq_cache_layout_init": (C.c_int, [C.POINTER(CacheLayout), _I32, _I32, _I32, _I32, _I32]),
    "tq_cache_append": (C.c_int, [_P, _P, C.POINTER(CacheLayout), _P, _P, _P, _I32, _I64, _P, _P]),
    "tq_cache_store": (C.c_int, [C.POINTER(CacheLayout), _P, _I32, _P, _P, _P, _P, _I64, _P, _P]),
    "tq_decode_workspace_bytes": (C.c_int64, [_I32, _I32, _I32, _I32]),
    "tq_decode_workspace_init": (C.c_int, [_P, _I64, _P]),
    "tq_decode_step_slots": (C.c_int, [_P, _I32, _P, _I32, _I32, _I32, _I64, _P, _P]),
    "tq_decode_status_sync": (C.c_int, [_P, _I64, C.POINTER(_I32)]),
    "tq_selftest_wait_gives_up": (C.c_int, [_P, _I64, _P]),
    "tq_decode_attn": (C.c_int, [_P, _P, C.POINTER(CacheLayout), _P, _P, _I32, _P, _P, _I32, _I32, _I32, _F,
                                 _P, _I64, _P, _I32, _P]),
    "tq_decode_attn_phases": (C.c_int, [_P, _P, C.POINTER(CacheLayout), _P, _P, _I32, _P, _P, _I32, _I32, _I32,
                                        _F, _P, _I64, _P, _I32, _I32, _P]),
    "tq_prefill_workspace_bytes": (C.c_int64, [_I32, _I32, _I32, _I32, _I32]),
    "tq_prefill_attn": (C.c_int, [_P, _P, C.POINTER(CacheLayout), _P, _P, _I32, _P, _P, _I32, _I32, _I32, _I32,
                                  _F, _P, _I64, _P, _I32, _P]),
    "tq_decode_attn_static": (C.c_int, [_P, _P, C.POINTER(CacheLayout), _P, _P, _I32, _P, _P, _I32, _I32, _I32,
                                        _F, _P, _I32, _P]),
    "tq_decode_static_status_sync": (C.c_int, [C.POINTER(_I32)]),
}

_lib = None


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: run `python -m turboquant_plus_b200.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc >= 0:
        return
    lib = load()
    msg = lib.tq_last_error().decode() or lib.tq_error_string(rc).decode()
    if rc == ERR_INVALID:
        raise ValueError(msg)
    raise TQError(f"{lib.tq_error_string(rc).decode()}: {msg}")


def call(name: str, *args):
    rc = getattr(load(), name)(*args)
    check(rc)
    return rc


def require_cuda():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("turboquant_plus_b200 needs a CUDA device (sm_100a); there is no CPU fallback")
    return torch


def stream_ptr():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t):
    """Device pointer of a torch tensor, or NULL for None."""
    return C.c_void_p(0 if t is None else t.data_ptr())


def torch_dtype_code(dt):
    import torch
    return {torch.float32: F32, torch.float16: F16, torch.float64: F64, torch.bfloat16: BF16}[dt]


def _dbl(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float64)


class Quantizer:
    """Owns one tq_quantizer handle on one device (constants uploaded at creation)."""

    def __init__(self, d, bits, rotation, norm_correction, centroids, rot=None, signs=None,
                 qjl_s=None, qjl_signs=None, device=None):
        torch = require_cuda()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        keep = [_dbl(centroids), _dbl(rot), _dbl(signs[0]) if signs else None, _dbl(signs[1]) if signs else None,
                _dbl(qjl_s), _dbl(qjl_signs[0]) if qjl_signs else None, _dbl(qjl_signs[1]) if qjl_signs else None]

        def hp(a):
            return C.c_void_p(0 if a is None else a.ctypes.data)

        desc = QuantizerDesc(d=d, bits=bits, rotation=rotation, norm_correction=int(bool(norm_correction)),
                             rot=hp(keep[1]), signs1=hp(keep[2]), signs2=hp(keep[3]), centroids=hp(keep[0]),
                             qjl=int(qjl_s is not None or qjl_signs is not None), qjl_s=hp(keep[4]),
                             qjl_signs1=hp(keep[5]), qjl_signs2=hp(keep[6]))
        h = _P()
        with torch.cuda.device(self.device):
            call("tq_quantizer_create", C.byref(desc), C.byref(h))
        self.handle = h
        self.d, self.bits, self.rotation = d, bits, rotation

    def __del__(self):
        h, self.handle = getattr(self, "handle", None), None
        if h and _lib is not None:
            try:
                _lib.tq_quantizer_destroy(h)
            except Exception:
                pass
