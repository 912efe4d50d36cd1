"""The C-ABI library loads and exports every symbol the header declares (no compute calls: CPU only)."""
import ctypes
import os
import re

from tests.conftest import ROOT


def test_library_exports_every_declared_symbol():
    from turboquant_plus_b200 import _native as nv
    from turboquant_plus_b200 import build
    build.build()
    lib = nv.load()
    header = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    body = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", body))
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in tq_b200.h but not exported"
    assert declared == set(nv.SIGNATURES), declared ^ set(nv.SIGNATURES)
    assert b"sm_100a" in lib.tq_version()
    assert lib.tq_error_string(-3) == b"misaligned pointer or stride"


def test_layout_arithmetic_and_argument_errors():
    from turboquant_plus_b200 import _native as nv
    lib = nv.load()
    L = nv.CacheLayout()
    assert lib.tq_cache_layout_init(ctypes.byref(L), 128, 128, 8, nv.FMT_TURBO3, nv.FMT_TURBO3) == 0
    assert L.record_bytes == 128 * 104 and L.k_idx_bytes == 48 and L.page_stride == 8 * 128 * 104
    assert lib.tq_cache_layout_init(ctypes.byref(L), 128, 128, 8, nv.FMT_PROD3, nv.FMT_TURBO3) == 0
    assert L.record_bytes == 128 * 108                       # 56 + 52 bytes per token
    assert lib.tq_cache_layout_init(ctypes.byref(L), 128, 128, 8, nv.FMT_Q8_0, nv.FMT_TURBO2) == 0
    assert L.record_bytes == 128 * (136 + 36)
    assert lib.tq_cache_layout_init(ctypes.byref(L), 64, 128, 8, 3, 3) == -2       # d != 128
    assert lib.tq_cache_layout_init(ctypes.byref(L), 128, 100, 8, 3, 3) == -1      # page size
    assert lib.tq_cache_layout_init(ctypes.byref(L), 128, 128, 8, 3, nv.FMT_PROD3) == -1   # QJL is K-only
    assert b"V format" in lib.tq_last_error()
    assert lib.tq_pack_indices(None, 10, 9, None, None) == -1
    assert b"bit_width must be 1-8" in lib.tq_last_error()
    assert lib.tq_quantize(None, None, 0, 128, 4, None, None, None, None, None, None, None) == -1
    assert lib.tq_decode_workspace_bytes(1, 32, 8, 256) > 0
    assert lib.tq_decode_workspace_bytes(0, 32, 8, 256) == -1
