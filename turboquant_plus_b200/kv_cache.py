"""KV-cache compressor.  Drop-in for the reference's ``turboquant/kv_cache.py``: K through
TurboQuant (inner products), V through TurboQuantMSE, one pair of quantizers shared by all layers
and heads; (num_layers, num_heads, seq_len, head_dim) in, per-layer-per-head containers out.

Where the reference loops over layers and heads in Python, all layers x heads x positions go through
one kernel launch per tensor.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import _native as nv
from ._io import to_device
from .turboquant import CompressedVector, TurboQuant, TurboQuantMSE


@dataclass
class CompressedKVCache:
    """Fields as in turboquant/kv_cache.py:30-44."""
    k_compressed: list = field(default_factory=list)   # [layer][head] -> CompressedVector
    v_indices: list = field(default_factory=list)      # [layer][head] -> (seq_len, head_dim) indices
    v_norms: list = field(default_factory=list)        # [layer][head] -> (seq_len,) norms
    num_layers: int = 0
    num_heads: int = 0
    seq_len: int = 0
    head_dim: int = 0
    k_bit_width: int = 0
    v_bit_width: int = 0


class KVCacheCompressor:
    """compress / decompress / memory_stats as in turboquant/kv_cache.py:47-188, plus ``paged`` for the
    streaming cache the reference only sketches."""

    def __init__(self, head_dim: int, k_bits: int = 3, v_bits: int = 3, seed: int = 42,
                 norm_correction: bool = True, *, rotation: str = "dense", device=None):
        self.head_dim = head_dim
        self.k_bits = k_bits
        self.v_bits = v_bits
        self.seed = seed
        self.norm_correction = norm_correction
        self.rotation_kind = rotation
        self.device = device
        self.k_quantizer = TurboQuant(head_dim, bit_width=k_bits, seed=seed, norm_correction=norm_correction,
                                      rotation=rotation, device=device)
        self.v_quantizer = TurboQuantMSE(head_dim, bit_width=v_bits, seed=seed + 500,
                                         norm_correction=norm_correction, rotation=rotation, device=device)

    def compress(self, k_cache, v_cache) -> CompressedKVCache:
        """turboquant/kv_cache.py:98-141."""
        num_layers, num_heads, seq_len, head_dim = k_cache.shape
        assert head_dim == self.head_dim
        assert v_cache.shape == k_cache.shape
        result = CompressedKVCache(num_layers=num_layers, num_heads=num_heads, seq_len=seq_len, head_dim=head_dim,
                                   k_bit_width=self.k_bits, v_bit_width=self.v_bits)
        flat = num_layers * num_heads * seq_len
        kc = self.k_quantizer.quantize(k_cache.reshape(flat, head_dim))
        v_idx, v_nrm = self.v_quantizer.quantize(v_cache.reshape(flat, head_dim))

        def cut(a, layer, head):
            lo = (layer * num_heads + head) * seq_len
            return a[lo:lo + seq_len]

        for layer in range(num_layers):
            result.k_compressed.append([
                CompressedVector(mse_indices=cut(kc.mse_indices, layer, h), vector_norms=cut(kc.vector_norms, layer, h),
                                 qjl_signs=cut(kc.qjl_signs, layer, h), residual_norms=cut(kc.residual_norms, layer, h),
                                 bit_width=self.k_bits) for h in range(num_heads)])
            result.v_indices.append([cut(v_idx, layer, h) for h in range(num_heads)])
            result.v_norms.append([cut(v_nrm, layer, h) for h in range(num_heads)])
        return result

    def decompress(self, compressed: CompressedKVCache):
        """(k_cache, v_cache), both (num_layers, num_heads, seq_len, head_dim)
        (turboquant/kv_cache.py:143-165)."""
        torch = nv.require_cuda()
        L, H = compressed.num_layers, compressed.num_heads
        shape = (L, H, compressed.seq_len, compressed.head_dim)
        first = compressed.v_indices[0][0] if L and H else None
        on_device = isinstance(first, torch.Tensor)
        cat = torch.cat if on_device else np.concatenate
        pieces = [compressed.k_compressed[l][h] for l in range(L) for h in range(H)]
        merged = CompressedVector(mse_indices=cat([p.mse_indices for p in pieces]),
                                  vector_norms=cat([p.vector_norms for p in pieces]),
                                  qjl_signs=cat([p.qjl_signs for p in pieces]),
                                  residual_norms=cat([p.residual_norms for p in pieces]), bit_width=self.k_bits)
        k_hat = self.k_quantizer.dequantize(merged)
        v_hat = self.v_quantizer.dequantize(cat([compressed.v_indices[l][h] for l in range(L) for h in range(H)]),
                                            cat([compressed.v_norms[l][h] for l in range(L) for h in range(H)]))
        return k_hat.reshape(shape), v_hat.reshape(shape)

    def memory_stats(self, seq_len: int, num_layers: int, num_heads: int) -> dict:
        """Closed-form sizes, counted as the reference counts them: K with one 32-bit norm per vector,
        V without (turboquant/kv_cache.py:167-188)."""
        vectors = num_layers * num_heads * seq_len
        fp16_bytes = vectors * self.head_dim * 2
        k_total_bits = vectors * (self.head_dim * self.k_bits + 32)
        v_total_bits = vectors * self.head_dim * self.v_bits
        packed_bytes = (k_total_bits + v_total_bits) / 8
        return {
            "original_mb": fp16_bytes / 1024 / 1024,
            "compressed_mb": packed_bytes / 1024 / 1024,
            "compression_ratio": fp16_bytes / packed_bytes,
            "k_bits_per_value": self.k_bits,
            "v_bits_per_value": self.v_bits,
        }

    def paged(self, num_kv_heads: int, num_pages: int, page_tokens: int = 128, k_format=None, v_format=None):
        """One layer's paged cache sharing this compressor's quantizers where the formats match:
        K "prod<k_bits>" (this object's TurboQuant) and V "turbo<v_bits>" by default."""
        from .paged import PagedKVCache
        k_format = k_format or f"prod{self.k_bits}"
        v_format = v_format or f"turbo{self.v_bits}"
        kq = self.k_quantizer if k_format == f"prod{self.k_bits}" else None
        vq = self.v_quantizer.polar_quant if v_format == f"turbo{self.v_bits}" else None
        return PagedKVCache(self.head_dim, num_kv_heads, num_pages, page_tokens, k_format, v_format, seed=self.seed,
                            norm_correction=self.norm_correction, rotation=self.rotation_kind, device=self.device,
                            k_quantizer=kq, v_quantizer=vq)

    # ---- streaming interface (additive; the reference only has the bulk compress / decompress above) ----
    def init_cache(self, num_layers: int, num_kv_heads: int, num_pages: int, page_tokens: int = 128, formats=None):
        """Allocate paged caches for `num_layers` layers that share this compressor's quantizers.  `formats` is one
        (k_format, v_format) pair or a per-layer list; default K "prod<k_bits>", V "turbo<v_bits>"."""
        default = (f"prod{self.k_bits}", f"turbo{self.v_bits}")
        if formats is None:
            formats = [default] * num_layers
        elif isinstance(formats[0], str):
            formats = [tuple(formats)] * num_layers
        assert len(formats) == num_layers
        self._layers, shared = [], {}
        for kf, vf in formats:
            if (kf, vf) not in shared:
                shared[(kf, vf)] = self.paged(num_kv_heads, num_pages, page_tokens, kf, vf)
                self._layers.append(shared[(kf, vf)])
            else:
                from .paged import PagedKVCache
                donor = shared[(kf, vf)]
                self._layers.append(PagedKVCache(self.head_dim, num_kv_heads, num_pages, page_tokens, kf, vf,
                                                 seed=self.seed, norm_correction=self.norm_correction,
                                                 rotation=self.rotation_kind, device=self.device,
                                                 k_quantizer=donor.k_quantizer, v_quantizer=donor.v_quantizer))
        return self

    def _layer(self, layer: int):
        assert getattr(self, "_layers", None), "call init_cache() first"
        return self._layers[layer]

    def append(self, k, v, layer: int, slot_mapping):
        """Quantize-on-append: k, v (tokens, num_kv_heads, head_dim) CUDA tensors into the slots
        page * page_tokens + position of `slot_mapping` (negative slots are skipped)."""
        self._layer(layer).append(k, v, slot_mapping)

    def attend(self, q, layer: int, seq_lens, block_table, scale=None, **kw):
        """Decode attention of q (batch, num_q_heads, head_dim) over layer `layer`'s packed cache."""
        return self._layer(layer).attend(q, block_table, seq_lens, scale=scale, **kw)

    def prefill_attend(self, q_chunk, layer: int, kv_lens, block_table, scale=None, **kw):
        """Causal attention of a chunk of new queries (batch, chunk_tokens, num_q_heads, head_dim) whose K/V rows
        have already been appended."""
        return self._layer(layer).prefill_attend(q_chunk, block_table, kv_lens, scale=scale, **kw)
