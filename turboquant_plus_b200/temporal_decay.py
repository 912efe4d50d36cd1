"""Temporal decay: re-quantize stored codes of old tokens to a narrower codebook without leaving the
rotated domain (the reference's ``benchmarks/temporal_decay_prototype.py``: ``requantize_3to2``).

One kernel (``tq_requantize``) reads the packed index stream and the per-vector factor and writes the
narrower stream and its factor; nothing is rotated back.  Source and destination quantizers are
``PolarQuant(..., rotation="wht")`` objects built from the same seed.
"""
from __future__ import annotations

import numpy as np

from . import _native as nv
from ._io import floats_to_device, ints_to_device


def requantize_device(src_pq, dst_pq, packed, scale, *, scale_is_norm=False):
    """packed: (n, 16*src bits) uint8 CUDA tensor as ``quantize_device(packed=True)`` writes it; scale: (n,) fp32
    (``want_scale=True``), or the vector norms with ``scale_is_norm``.  Returns {'packed', 'norm', 'scale'} for the
    destination quantizer."""
    torch = nv.require_cuda()
    n, dev = packed.shape[0], packed.device
    out = {"packed": torch.empty((n, 16 * dst_pq.bit_width), dtype=torch.uint8, device=dev),
           "norm": torch.empty((n,), dtype=torch.float32, device=dev),
           "scale": torch.empty((n,), dtype=torch.float32, device=dev)}
    with torch.cuda.device(dev):
        nv.call("tq_requantize", src_pq._native(dev).handle, dst_pq._native(dev).handle, nv.ptr(packed), nv.ptr(scale),
                int(bool(scale_is_norm)), n, nv.ptr(out["packed"]), nv.ptr(out["norm"]), nv.ptr(out["scale"]),
                nv.stream_ptr())
    return out


def requantize(src_pq, dst_pq, indices, norms):
    """(indices of the destination codebook, corrected norm) from (indices, vector norm) of the source codebook:
    benchmarks/temporal_decay_prototype.py:93-125 with the two quantizers' codebooks in place of its constants.
    indices: (d,) or (batch, d); NumPy in, NumPy out."""
    torch = nv.require_cuda()
    dev = torch.device("cuda", torch.cuda.current_device()) if src_pq.device is None else torch.device(src_pq.device)
    it = ints_to_device(indices, dev, torch.uint8)
    single = it.dim() == 1
    it = it.reshape(1, -1) if single else it.reshape(-1, it.shape[-1])
    n, d = it.shape
    nt = floats_to_device(np.asarray(norms).reshape(-1), dev)
    packed = torch.empty((n, d * src_pq.bit_width // 8), dtype=torch.uint8, device=dev)
    idx2 = torch.empty((n, d), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        nv.call("tq_pack_indices", nv.ptr(it), n * d, src_pq.bit_width, nv.ptr(packed), nv.stream_ptr())
        out = requantize_device(src_pq, dst_pq, packed, nt, scale_is_norm=True)
        nv.call("tq_unpack_indices", nv.ptr(out["packed"]), n * d, dst_pq.bit_width, nv.ptr(idx2), nv.stream_ptr())
    idx2 = idx2.cpu().numpy()
    corrected = out["scale"].cpu().numpy().astype(np.float64)
    return (idx2[0], corrected[0]) if single else (idx2, corrected)
