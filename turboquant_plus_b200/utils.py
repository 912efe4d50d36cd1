"""Bit packing and footprint arithmetic (same functions as the reference's ``turboquant/utils.py``).

Packing runs on the GPU; NumPy in gives NumPy out, CUDA tensors stay on the device.
"""
from __future__ import annotations

import math

import numpy as np

from . import _native as nv
from ._io import ints_to_device


def _dev(x, dtype):
    torch = nv.require_cuda()
    was_numpy = not isinstance(x, torch.Tensor)
    dev = torch.device("cuda", torch.cuda.current_device()) if was_numpy or x.device.type != "cuda" else x.device
    return ints_to_device(x, dev, dtype), was_numpy


def pack_bits(signs):
    """{+1,-1} -> bits, +1 -> 1, eight per byte, most significant first, each row padded to whole
    bytes (turboquant/utils.py:20-49)."""
    torch = nv.require_cuda()
    t, was_numpy = _dev(signs, torch.int8)
    single = t.dim() == 1
    rows = t.reshape(1, -1) if single else t.reshape(-1, t.shape[-1])
    d = rows.shape[1]
    out = torch.empty((rows.shape[0], (d + 7) // 8), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        nv.call("tq_pack_bits", nv.ptr(rows), rows.shape[0], d, nv.ptr(out), nv.stream_ptr())
    out = out[0] if single else out
    return out.cpu().numpy() if was_numpy else out


def unpack_bits(packed, d: int):
    """Inverse of pack_bits, cropped to d (turboquant/utils.py:52-68)."""
    torch = nv.require_cuda()
    t, was_numpy = _dev(packed, torch.uint8)
    single = t.dim() == 1
    rows = t.reshape(1, -1) if single else t
    out = torch.empty((rows.shape[0], d), dtype=torch.int8, device=t.device)
    with torch.cuda.device(t.device):
        nv.call("tq_unpack_bits", nv.ptr(rows), rows.shape[0], d, nv.ptr(out), nv.stream_ptr())
    out = out[0] if single else out
    return out.cpu().numpy() if was_numpy else out


def pack_indices(indices, bit_width: int):
    """b-bit indices -> one flat MSB-first bit stream for b <= 4; b in 5..8 returns the indices
    as uint8 in their own shape (turboquant/utils.py:71-98)."""
    if bit_width <= 0 or bit_width > 8:
        raise ValueError(f"bit_width must be 1-8, got {bit_width}")
    torch = nv.require_cuda()
    t, was_numpy = _dev(indices, torch.uint8)
    n = t.numel()
    if bit_width > 4:
        out = t.clone()
    else:
        out = torch.empty(((n * bit_width + 7) // 8,), dtype=torch.uint8, device=t.device)
        with torch.cuda.device(t.device):
            nv.call("tq_pack_indices", nv.ptr(t), n, bit_width, nv.ptr(out), nv.stream_ptr())
    return out.cpu().numpy() if was_numpy else out


def unpack_indices(packed, bit_width: int, count: int):
    """Inverse of pack_indices (not in the reference; the read path needs it)."""
    if bit_width <= 0 or bit_width > 8:
        raise ValueError(f"bit_width must be 1-8, got {bit_width}")
    torch = nv.require_cuda()
    t, was_numpy = _dev(packed, torch.uint8)
    out = torch.empty((count,), dtype=torch.uint8, device=t.device)
    with torch.cuda.device(t.device):
        nv.call("tq_unpack_indices", nv.ptr(t), count, bit_width, nv.ptr(out), nv.stream_ptr())
    return out.cpu().numpy() if was_numpy else out


def memory_footprint_bytes(n_vectors: int, d: int, bit_width: int) -> dict:
    """Bytes of a TurboQuant-compressed cache: (b-1)-bit indices, 1-bit sketch, one fp32 norm
    (turboquant/utils.py:101-123)."""
    idx_bytes = int(math.ceil(n_vectors * d * (bit_width - 1) / 8))
    sketch_bytes = int(math.ceil(n_vectors * d * 1 / 8))
    norm_bytes = n_vectors * 4
    total = idx_bytes + sketch_bytes + norm_bytes
    fp16_bytes = n_vectors * d * 2
    return {
        "mse_indices_bytes": idx_bytes,
        "qjl_signs_bytes": sketch_bytes,
        "norms_bytes": norm_bytes,
        "total_bytes": total,
        "original_fp16_bytes": fp16_bytes,
        "compression_ratio": fp16_bytes / total if total > 0 else float("inf"),
    }
