"""TurboQuant (Algorithm 2) = (b-1)-bit PolarQuant + 1-bit QJL of the residual, and the MSE-only
variant (Algorithm 1).  Drop-in for the reference's ``turboquant/turboquant.py``.

One fused kernel launch (``tq_quantize`` with the QJL outputs) replaces the reference's three
matrix products per vector.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _native as nv
from ._io import floats_to_device, ints_to_device, to_device
from .polar_quant import PolarQuant
from .qjl import QJL
from .rotation import fast_rotation_matrix


@dataclass
class CompressedVector:
    """Fields as in turboquant/turboquant.py:33-40."""
    mse_indices: object    # (d,) or (batch, d): PolarQuant indices, (b-1)-bit integers
    vector_norms: object   # scalar or (batch,): ||x||_2
    qjl_signs: object      # (d,) or (batch, d): int8 in {+1, -1}
    residual_norms: object # scalar or (batch,): ||x - x_mse||_2
    bit_width: int         # total bits per coordinate


class TurboQuant:
    """Inner-product-oriented quantizer: PolarQuant(bit_width - 1, seed) followed by
    QJL(seed + 1000) on the residual (turboquant/turboquant.py:43-77)."""

    def __init__(self, d: int, bit_width: int, seed: int = 42, norm_correction: bool = True, *,
                 rotation: str = "dense", device=None):
        if bit_width < 2:
            raise ValueError("TurboQuant requires bit_width >= 2 (1 bit PolarQuant + 1 bit QJL). "
                             "For 1-bit, use QJL directly.")
        self.d = d
        self.bit_width = bit_width
        self.device = device
        self.rotation_kind = rotation
        self.polar_quant = PolarQuant(d, bit_width=bit_width - 1, seed=seed, norm_correction=norm_correction,
                                      rotation=rotation, device=device)
        self.qjl = QJL(d, seed=seed + 1000, kind=rotation, device=device)
        self._handles = {}
        self._uploaded = None

    def _native(self, device):
        pq, qj = self.polar_quant, self.qjl
        snap = (pq.rotation.tobytes(), pq.centroids.tobytes(), bool(pq.norm_correction), qj.S.tobytes())
        if snap != self._uploaded:
            self._handles.clear()
            self._uploaded = snap
        key = str(device)
        if key not in self._handles:
            wht = (self.rotation_kind == "wht" and pq.signs is not None and qj.signs is not None
                   and np.array_equal(pq.rotation, fast_rotation_matrix(*pq.signs))
                   and np.array_equal(qj.S, fast_rotation_matrix(*qj.signs)))
            if wht:
                self._handles[key] = nv.Quantizer(self.d, pq.bit_width, nv.ROT_WHT, pq.norm_correction, pq.centroids,
                                                  signs=pq.signs, qjl_signs=qj.signs, device=device)
            else:
                self._handles[key] = nv.Quantizer(self.d, pq.bit_width, nv.ROT_DENSE, pq.norm_correction, pq.centroids,
                                                  rot=pq.rotation, qjl_s=qj.S, device=device)
        return self._handles[key]

    # ---- device-level API ---------------------------------------------------------------
    def quantize_device(self, xt, *, packed=False, want_scale=False):
        """(n, d) CUDA tensor -> dict of CUDA tensors: 'idx' or 'packed', 'norm', 'qjl' (n, d/8) packed
        sign bits, 'rnorm', optionally 'scale'."""
        torch = nv.require_cuda()
        n = xt.shape[0]
        q = self._native(xt.device)
        bits = self.polar_quant.bit_width
        out = {"norm": torch.empty((n,), dtype=torch.float32, device=xt.device),
               "rnorm": torch.empty((n,), dtype=torch.float32, device=xt.device),
               "qjl": torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=xt.device)}
        if packed:
            out["packed"] = torch.empty((n, self.d * bits // 8), dtype=torch.uint8, device=xt.device)
        else:
            out["idx"] = torch.empty((n, self.d), dtype=torch.uint8, device=xt.device)
        if want_scale:
            out["scale"] = torch.empty((n,), dtype=torch.float32, device=xt.device)
        with torch.cuda.device(xt.device):
            nv.call("tq_quantize", q.handle, nv.ptr(xt), nv.torch_dtype_code(xt.dtype), xt.stride(0), n,
                    nv.ptr(out.get("packed")), nv.ptr(out.get("idx")), nv.ptr(out["norm"]), nv.ptr(out.get("scale")),
                    nv.ptr(out["qjl"]), nv.ptr(out["rnorm"]), nv.stream_ptr())
        return out

    # ---- reference-shaped API -----------------------------------------------------------------
    def quantize(self, x) -> CompressedVector:
        """turboquant/turboquant.py:79-100."""
        torch = nv.require_cuda()
        xt, was_numpy, src_dtype = to_device(x, self.device, allow_f64=self.rotation_kind != "wht")
        single = xt.dim() == 1
        xt = xt.reshape(1, -1) if single else xt.reshape(-1, xt.shape[-1])
        if xt.shape[1] != self.d:
            raise ValueError(f"expected vectors of dimension {self.d}, got {xt.shape[1]}")
        out = self.quantize_device(xt)
        n = xt.shape[0]
        signs = torch.empty((n, self.d), dtype=torch.int8, device=xt.device)
        with torch.cuda.device(xt.device):
            nv.call("tq_unpack_bits", nv.ptr(out["qjl"]), n, self.d, nv.ptr(signs), nv.stream_ptr())
        idx, nrm, rn = out["idx"], out["norm"], out["rnorm"]
        if was_numpy:
            idx = idx.cpu().numpy().astype(np.int64)
            nrm = nrm.cpu().numpy().astype(src_dtype if src_dtype is not None else np.float64)
            rn = rn.cpu().numpy().astype(np.float64)  # the reference's residual is fp64
            signs = signs.cpu().numpy()
        if single:
            idx, nrm, rn, signs = idx[0], nrm[0], rn[0], signs[0]
        return CompressedVector(mse_indices=idx, vector_norms=nrm, qjl_signs=signs, residual_norms=rn,
                                bit_width=self.bit_width)

    def dequantize(self, compressed: CompressedVector, shrinkage: float = 1.0):
        """PolarQuant reconstruction + shrinkage * QJL reconstruction (turboquant/turboquant.py:102-124)."""
        torch = nv.require_cuda()
        was_numpy = not isinstance(compressed.mse_indices, torch.Tensor)
        dev = (torch.device("cuda", torch.cuda.current_device()) if self.device is None else torch.device(self.device)) \
            if was_numpy or compressed.mse_indices.device.type != "cuda" else compressed.mse_indices.device
        it = ints_to_device(compressed.mse_indices, dev, torch.uint8)
        single = it.dim() == 1
        it = it.reshape(1, -1) if single else it.reshape(-1, it.shape[-1])
        st = ints_to_device(compressed.qjl_signs, dev, torch.int8).reshape(it.shape)
        as_flat = (lambda a: np.asarray(a).reshape(-1)) if was_numpy else (lambda a: a.reshape(-1))
        nt = floats_to_device(as_flat(compressed.vector_norms), dev)
        rt = floats_to_device(as_flat(compressed.residual_norms), dev)
        n = it.shape[0]
        q = self._native(dev)
        out_dtype = torch.float32 if q.rotation == nv.ROT_WHT else torch.float64
        bits = torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=dev)
        out = torch.empty((n, self.d), dtype=out_dtype, device=dev)
        with torch.cuda.device(dev):
            nv.call("tq_pack_bits", nv.ptr(st), n, self.d, nv.ptr(bits), nv.stream_ptr())
            nv.call("tq_dequantize", q.handle, None, nv.ptr(it), nv.ptr(nt), nv.ptr(bits), nv.ptr(rt),
                    float(shrinkage), n, nv.ptr(out), nv.torch_dtype_code(out_dtype), nv.stream_ptr())
        if was_numpy:
            out = out.cpu().numpy().astype(np.float64)
        return out[0] if single else out

    def compressed_size_bits(self, n_vectors: int) -> int:
        """b bits per coordinate plus one 32-bit norm per vector, as the reference counts it
        (turboquant/turboquant.py:126-136; the second stored norm is not counted there either)."""
        return n_vectors * (self.d * self.bit_width + 32)

    def compression_ratio(self, original_bits_per_value: int = 16) -> float:
        """turboquant/turboquant.py:138-149."""
        return (self.d * original_bits_per_value) / (self.d * self.bit_width + 32)


class TurboQuantMSE:
    """PolarQuant at the full bit width, no QJL stage: the "turbo2/3/4" cache types
    (turboquant/turboquant.py:152-171)."""

    def __init__(self, d: int, bit_width: int, seed: int = 42, norm_correction: bool = True, *,
                 rotation: str = "dense", device=None):
        self.d = d
        self.bit_width = bit_width
        self.polar_quant = PolarQuant(d, bit_width=bit_width, seed=seed, norm_correction=norm_correction,
                                      rotation=rotation, device=device)

    def quantize(self, x):
        return self.polar_quant.quantize(x)

    def dequantize(self, indices, norms):
        return self.polar_quant.dequantize(indices, norms)
