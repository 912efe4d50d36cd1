"""Fractional bit rates (2.5, 3.5 bits per channel) by splitting the channels of a vector into a
leading group quantized with one more bit and the rest.  Drop-in for the reference's
``turboquant/outlier.py``: same constructor, attributes, container and methods.

Three launches each way instead of the reference's seven matrix products and three
scatter/gather copies: the two sub-vector quantizers read column slices of the input in place and
write the two halves of one fp64 residual matrix (``tq_quantize_residual``), which the QJL kernel
sketches; dequantization writes the QJL reconstruction and adds the two sub-vector
reconstructions onto its column slices (``tq_dequantize_strided``).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import _native as nv
from ._io import floats_to_device, ints_to_device, to_device
from .polar_quant import PolarQuant
from .qjl import QJL


@dataclass
class OutlierCompressedVector:
    """Fields as in turboquant/outlier.py:33-42."""
    outlier_indices: object   # (n_outlier,) or (batch, n_outlier): indices of the leading channels
    outlier_norms: object     # scalar or (batch,)
    normal_indices: object    # (n_normal,) or (batch, n_normal)
    normal_norms: object      # scalar or (batch,)
    qjl_signs: object         # (d,) or (batch, d): int8 in {+1, -1}, sketch of the whole residual
    residual_norms: object    # scalar or (batch,)
    effective_bits: float


def _compute_channel_split(d: int, target_bits: float):
    """(n_outlier, outlier_bits, n_normal, normal_bits): round(d * frac) channels at floor + 1 bits
    (turboquant/outlier.py:45-66)."""
    low_bits = int(np.floor(target_bits))
    n_outlier = int(round(d * (target_bits - low_bits)))
    return n_outlier, low_bits + 1, d - n_outlier, low_bits


class OutlierTurboQuant:
    """TurboQuant with two channel groups (turboquant/outlier.py:69-108): PolarQuant(n_outlier,
    high_bits - 1, seed) on the first n_outlier channels, PolarQuant(n_normal, low_bits - 1, seed + 500)
    on the rest, QJL(d, seed + 1000) on the residual of the whole vector.

        oq = OutlierTurboQuant(d=128, target_bits=2.5, seed=42)
        compressed = oq.quantize(x)
        x_hat = oq.dequantize(compressed)
    """

    def __init__(self, d: int, target_bits: float, seed: int = 42, *, device=None):
        self.d = d
        self.target_bits = target_bits
        self.device = device
        self.n_outlier, self.high_bits, self.n_normal, self.low_bits = _compute_channel_split(d, target_bits)
        self.effective_bits = (self.n_outlier * self.high_bits + self.n_normal * self.low_bits) / d
        self.outlier_idx = np.arange(self.n_outlier)
        self.normal_idx = np.arange(self.n_outlier, d)
        self.pq_outlier = (PolarQuant(self.n_outlier, bit_width=self.high_bits - 1, seed=seed, device=device)
                           if self.n_outlier > 0 else None)
        self.pq_normal = (PolarQuant(self.n_normal, bit_width=self.low_bits - 1, seed=seed + 500, device=device)
                          if self.n_normal > 0 else None)
        self.qjl = QJL(d, seed=seed + 1000, device=device)

    # ---- device-level API (CUDA tensors in and out) ----------------------------------------
    def _groups(self):
        return ((self.pq_outlier, 0, self.n_outlier, "outlier"), (self.pq_normal, self.n_outlier, self.n_normal, "normal"))

    def quantize_device(self, xt):
        """xt: (n, d) CUDA tensor (fp64, fp32 or fp16).  Dict of CUDA tensors: '<group>_idx' (n, n_group) uint8 and
        '<group>_norm' (n,) fp32 for group in outlier / normal, 'qjl' (n, ceil(d/8)) packed sign bits, 'rnorm' (n,)."""
        torch = nv.require_cuda()
        n, dev = xt.shape[0], xt.device
        out = {}
        residual = torch.zeros((n, self.d), dtype=torch.float64, device=dev)
        with torch.cuda.device(dev):
            for pq, col, width, name in self._groups():
                if pq is None:
                    continue
                out[name + "_idx"] = torch.empty((n, width), dtype=torch.uint8, device=dev)
                out[name + "_norm"] = torch.empty((n,), dtype=torch.float32, device=dev)
                nv.call("tq_quantize_residual", pq._native(dev).handle, nv.ptr(xt[:, col:]),
                        nv.torch_dtype_code(xt.dtype), xt.stride(0), n, nv.ptr(out[name + "_idx"]),
                        nv.ptr(out[name + "_norm"]), nv.ptr(residual[:, col:]), self.d, nv.stream_ptr())
            out["qjl"] = torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=dev)
            out["rnorm"] = torch.empty((n,), dtype=torch.float32, device=dev)
            nv.call("tq_qjl_quantize", self.qjl._native(dev).handle, nv.ptr(residual), nv.F64, n, nv.ptr(out["qjl"]),
                    nv.ptr(out["rnorm"]), nv.stream_ptr())
        return out

    def dequantize_device(self, code):
        """Inverse of quantize_device: (n, d) fp64 CUDA tensor."""
        torch = nv.require_cuda()
        bits = code["qjl"]
        n, dev = bits.shape[0], bits.device
        out = torch.empty((n, self.d), dtype=torch.float64, device=dev)
        with torch.cuda.device(dev):
            nv.call("tq_qjl_dequantize", self.qjl._native(dev).handle, nv.ptr(bits), nv.ptr(code["rnorm"]), 1.0, n,
                    nv.ptr(out), nv.F64, nv.stream_ptr())
            for pq, col, width, name in self._groups():
                if pq is None:
                    continue
                nv.call("tq_dequantize_strided", pq._native(dev).handle, nv.ptr(code[name + "_idx"]),
                        nv.ptr(code[name + "_norm"]), n, nv.ptr(out[:, col:]), self.d, 1, nv.stream_ptr())
        return out

    # ---- reference-shaped API -----------------------------------------------------------------
    def quantize(self, x) -> OutlierCompressedVector:
        """turboquant/outlier.py:110-178."""
        torch = nv.require_cuda()
        xt, was_numpy, src_dtype = to_device(x, self.device, allow_f64=True)
        if xt.dtype == torch.bfloat16:
            xt = xt.float()
        single = xt.dim() == 1
        xt = xt.reshape(1, -1) if single else xt.reshape(-1, xt.shape[-1])
        if xt.shape[1] != self.d:
            raise ValueError(f"expected vectors of dimension {self.d}, got {xt.shape[1]}")
        n = xt.shape[0]
        code = self.quantize_device(xt)
        signs = torch.empty((n, self.d), dtype=torch.int8, device=xt.device)
        with torch.cuda.device(xt.device):
            nv.call("tq_unpack_bits", nv.ptr(code["qjl"]), n, self.d, nv.ptr(signs), nv.stream_ptr())
        norm_dtype = src_dtype if src_dtype is not None else np.float64

        def host(t, kind):
            if t is None:
                return np.array([])       # a group without channels, as the reference returns it
            if not was_numpy:
                return t[0] if single else t
            a = t.cpu().numpy()
            a = a.astype({"idx": np.int64, "norm": norm_dtype, "rnorm": np.float64, "signs": np.int8}[kind])
            return a[0] if single else a

        return OutlierCompressedVector(
            outlier_indices=host(code.get("outlier_idx"), "idx"), outlier_norms=host(code.get("outlier_norm"), "norm"),
            normal_indices=host(code.get("normal_idx"), "idx"), normal_norms=host(code.get("normal_norm"), "norm"),
            qjl_signs=host(signs, "signs"), residual_norms=host(code["rnorm"], "rnorm"),
            effective_bits=self.effective_bits)

    def dequantize(self, compressed: OutlierCompressedVector):
        """turboquant/outlier.py:180-208."""
        torch = nv.require_cuda()
        was_numpy = not isinstance(compressed.qjl_signs, torch.Tensor)
        if was_numpy or compressed.qjl_signs.device.type != "cuda":
            dev = torch.device("cuda", torch.cuda.current_device()) if self.device is None else torch.device(self.device)
        else:
            dev = compressed.qjl_signs.device
        st = ints_to_device(compressed.qjl_signs, dev, torch.int8)
        single = st.dim() == 1
        st = st.reshape(1, -1) if single else st.reshape(-1, st.shape[-1])
        n = st.shape[0]
        flat = (lambda a: np.asarray(a).reshape(-1)) if was_numpy else (lambda a: a.reshape(-1))
        code = {"qjl": torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=dev),
                "rnorm": floats_to_device(flat(compressed.residual_norms), dev)}
        with torch.cuda.device(dev):
            nv.call("tq_pack_bits", nv.ptr(st), n, self.d, nv.ptr(code["qjl"]), nv.stream_ptr())
        for pq, _, width, name in self._groups():
            if pq is None:
                continue
            idx = getattr(compressed, name + "_indices")
            code[name + "_idx"] = ints_to_device(idx, dev, torch.uint8).reshape(n, width)
            code[name + "_norm"] = floats_to_device(flat(getattr(compressed, name + "_norms")), dev)
        out = self.dequantize_device(code)
        if was_numpy:
            out = out.cpu().numpy()
        return out[0] if single else out

    def compression_ratio(self, original_bits: int = 16) -> float:
        """d * effective_bits plus three 32-bit norms per vector (turboquant/outlier.py:210-217)."""
        return self.d * original_bits / (self.d * self.effective_bits + 32 + 64)
