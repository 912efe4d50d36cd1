"""turboquant_plus_b200: TurboQuant+ KV-cache compression on NVIDIA B200 (sm_100a).

Same public names as the reference package ``turboquant`` (TheTom/turboquant_plus):
PolarQuant, QJL, TurboQuant, TurboQuantMSE, CompressedVector, KVCacheCompressor (and
OutlierTurboQuant of ``turboquant/outlier.py``), with the
arithmetic in hand-written CUDA kernels behind the C ABI of ``include/tq_b200.h``.  New surface:
PagedKVCache (quantize-on-append and decode attention straight off the packed cache).
"""
from .polar_quant import PolarQuant
from .qjl import QJL
from .turboquant import TurboQuant, TurboQuantMSE, CompressedVector
from .kv_cache import KVCacheCompressor, CompressedKVCache
from .outlier import OutlierTurboQuant, OutlierCompressedVector
from .paged import PagedKVCache

__all__ = ["PolarQuant", "QJL", "TurboQuant", "TurboQuantMSE", "CompressedVector", "KVCacheCompressor",
           "CompressedKVCache", "PagedKVCache", "OutlierTurboQuant", "OutlierCompressedVector"]
