"""PolarQuant (Algorithm 1): rotate, then quantize each coordinate against a Lloyd-Max codebook.

Drop-in for the reference's ``turboquant/polar_quant.py`` -- same constructor, methods and shape
conventions -- with the arithmetic in CUDA kernels (``tq_quantize`` / ``tq_dequantize``).

``rotation="dense"`` (default) is the reference's QR rotation, computed on the GPU in fp64 like the
reference's fp64 GEMM, so indices agree with the reference's.  ``rotation="wht"`` is the
sign * Walsh-Hadamard rotation of ``turboquant/rotation.py:75-185`` computed in fp32 registers:
the production path ("turbo2/3/4"), d = 128 only.
"""
from __future__ import annotations

import numpy as np

from . import _native as nv
from ._io import floats_to_device, ints_to_device, to_device
from .codebook import optimal_centroids
from .rotation import fast_rotation_matrix, random_rotation_dense, random_rotation_fast


class PolarQuant:
    """MSE-oriented vector quantizer for vectors of any norm: the L2 norm is stored on the side
    and the unit vector is quantized (turboquant/polar_quant.py:33-54).

        pq = PolarQuant(d=128, bit_width=3, seed=42)
        indices, norms = pq.quantize(x)        # x: (d,) or (batch, d), NumPy or CUDA tensor
        x_hat = pq.dequantize(indices, norms)
    """

    def __init__(self, d: int, bit_width: int, seed: int = 42, norm_correction: bool = True, *,
                 rotation: str = "dense", device=None, rotation_matrix=None, signs=None, centroids=None):
        if rotation not in ("dense", "wht"):
            raise ValueError(f"rotation must be 'dense' or 'wht', got {rotation!r}")
        self.d = d
        self.bit_width = bit_width
        self.n_centroids = 1 << bit_width
        self.norm_correction = norm_correction
        self.rotation_kind = rotation
        self.device = device
        rng = np.random.default_rng(seed)
        if rotation == "dense":
            self.signs = None
            self.rotation = (np.asarray(rotation_matrix, dtype=np.float64) if rotation_matrix is not None
                             else random_rotation_dense(d, rng))
        else:
            if signs is None:
                s1, s2, padded = random_rotation_fast(d, rng)
                if padded != d:
                    raise ValueError(f"rotation='wht' needs d to be a power of two (kernels: d == 128), got {d}")
                signs = (s1, s2)
            self.signs = (np.asarray(signs[0], dtype=np.float64), np.asarray(signs[1], dtype=np.float64))
            self.rotation = fast_rotation_matrix(*self.signs)
        self.centroids = (np.asarray(centroids, dtype=np.float64) if centroids is not None
                          else optimal_centroids(bit_width, d))
        self._handles = {}
        self._uploaded = None

    # ---- native handle ------------------------------------------------------------------
    def _snapshot(self):
        return (self.rotation.tobytes(), self.centroids.tobytes(), bool(self.norm_correction))

    def _native(self, device):
        """The tq_quantizer for ``device``; rebuilt if rotation / centroids were reassigned."""
        snap = self._snapshot()
        if snap != self._uploaded:
            self._handles.clear()
            self._uploaded = snap
        key = str(device)
        if key not in self._handles:
            if self.rotation_kind == "wht" and self.signs is not None and np.array_equal(
                    self.rotation, fast_rotation_matrix(*self.signs)):
                self._handles[key] = nv.Quantizer(self.d, self.bit_width, nv.ROT_WHT, self.norm_correction,
                                                  self.centroids, signs=self.signs, device=device)
            else:
                self._handles[key] = nv.Quantizer(self.d, self.bit_width, nv.ROT_DENSE, self.norm_correction,
                                                  self.centroids, rot=self.rotation, device=device)
        return self._handles[key]

    @property
    def _is_wht(self):
        return self.rotation_kind == "wht"

    # ---- device-level API (CUDA tensors in and out) ----------------------------------------
    def quantize_device(self, xt, *, packed=False, want_scale=False):
        """xt: (n, d) CUDA tensor.  Returns dict with 'idx' (n, d) uint8 or 'packed'
        (n, d*bits/8) uint8, 'norm' (n,) fp32 and optionally 'scale' (n,) fp32."""
        torch = nv.require_cuda()
        n = xt.shape[0]
        q = self._native(xt.device)
        out = {"norm": torch.empty((n,), dtype=torch.float32, device=xt.device)}
        if packed:
            out["packed"] = torch.empty((n, self.d * self.bit_width // 8), dtype=torch.uint8, device=xt.device)
        else:
            out["idx"] = torch.empty((n, self.d), dtype=torch.uint8, device=xt.device)
        if want_scale:
            out["scale"] = torch.empty((n,), dtype=torch.float32, device=xt.device)
        with torch.cuda.device(xt.device):
            nv.call("tq_quantize", q.handle, nv.ptr(xt), nv.torch_dtype_code(xt.dtype), xt.stride(0), n,
                    nv.ptr(out.get("packed")), nv.ptr(out.get("idx")), nv.ptr(out["norm"]), nv.ptr(out.get("scale")),
                    None, None, nv.stream_ptr())
        return out

    def dequantize_device(self, norms, *, idx=None, packed=None, out_dtype=None):
        torch = nv.require_cuda()
        src = idx if idx is not None else packed
        n = src.shape[0]
        q = self._native(src.device)
        if out_dtype is None:
            out_dtype = torch.float32 if q.rotation == nv.ROT_WHT else torch.float64
        out = torch.empty((n, self.d), dtype=out_dtype, device=src.device)
        with torch.cuda.device(src.device):
            nv.call("tq_dequantize", q.handle, nv.ptr(packed), nv.ptr(idx), nv.ptr(norms), None, None, 1.0, n,
                    nv.ptr(out), nv.torch_dtype_code(out_dtype), nv.stream_ptr())
        return out

    # ---- reference-shaped API -----------------------------------------------------------------
    def quantize(self, x):
        """(indices, norms); a (d,) input gives (d,) indices and a scalar norm
        (turboquant/polar_quant.py:56-85)."""
        xt, was_numpy, src_dtype = to_device(x, self.device, allow_f64=not self._is_wht)
        single = xt.dim() == 1
        xt = xt.reshape(1, -1) if single else xt.reshape(-1, xt.shape[-1])
        if xt.shape[1] != self.d:
            raise ValueError(f"expected vectors of dimension {self.d}, got {xt.shape[1]}")
        out = self.quantize_device(xt)
        idx, nrm = out["idx"], out["norm"]
        if was_numpy:
            idx = idx.cpu().numpy().astype(np.int64)
            nrm = nrm.cpu().numpy().astype(src_dtype if src_dtype is not None else np.float64)
        return (idx[0], nrm[0]) if single else (idx, nrm)

    def dequantize(self, indices, norms):
        """Reconstruction (turboquant/polar_quant.py:87-119)."""
        torch = nv.require_cuda()
        was_numpy = not isinstance(indices, torch.Tensor)
        dev = (torch.device("cuda", torch.cuda.current_device()) if self.device is None else torch.device(self.device)) \
            if was_numpy or indices.device.type != "cuda" else indices.device
        it = ints_to_device(indices, dev, torch.uint8)
        single = it.dim() == 1
        it = it.reshape(1, -1) if single else it.reshape(-1, it.shape[-1])
        nt = floats_to_device(np.asarray(norms).reshape(-1) if was_numpy else norms.reshape(-1), dev)
        out = self.dequantize_device(nt, idx=it)
        if was_numpy:
            out = out.cpu().numpy().astype(np.float64)
        return out[0] if single else out

    def quantize_and_residual(self, x):
        """(indices, norms, x - dequantize(indices, norms)) (turboquant/polar_quant.py:121-132)."""
        torch = nv.require_cuda()
        if not self._is_wht:
            # dense mode: one launch, the residual taken against the fp64 norm as the reference does
            xt, was_numpy, src_dtype = to_device(x, self.device, allow_f64=True)
            if xt.dtype == torch.bfloat16:
                xt = xt.float()
            single = xt.dim() == 1
            xt = xt.reshape(1, -1) if single else xt.reshape(-1, xt.shape[-1])
            if xt.shape[1] != self.d:
                raise ValueError(f"expected vectors of dimension {self.d}, got {xt.shape[1]}")
            n = xt.shape[0]
            idx = torch.empty((n, self.d), dtype=torch.uint8, device=xt.device)
            nrm = torch.empty((n,), dtype=torch.float32, device=xt.device)
            res = torch.empty((n, self.d), dtype=torch.float64, device=xt.device)
            with torch.cuda.device(xt.device):
                nv.call("tq_quantize_residual", self._native(xt.device).handle, nv.ptr(xt), nv.torch_dtype_code(xt.dtype),
                        xt.stride(0), n, nv.ptr(idx), nv.ptr(nrm), nv.ptr(res), self.d, nv.stream_ptr())
            if was_numpy:
                idx = idx.cpu().numpy().astype(np.int64)
                nrm = nrm.cpu().numpy().astype(src_dtype if src_dtype is not None else np.float64)
                res = res.cpu().numpy()
            return (idx[0], nrm[0], res[0]) if single else (idx, nrm, res)
        indices, norms = self.quantize(x)
        x_hat = self.dequantize(indices, norms)
        if isinstance(x, torch.Tensor):
            return indices, norms, x.to(x_hat.dtype) - x_hat
        return indices, norms, np.asarray(x) - x_hat
