"""QJL: 1-bit quantized Johnson-Lindenstrauss sketch, z = sign(S r) with S orthogonal.

Drop-in for the reference's ``turboquant/qjl.py``; the projections run on the GPU in fp64
(``tq_qjl_quantize`` / ``tq_qjl_dequantize``).
"""
from __future__ import annotations

import numpy as np

from . import _native as nv
from ._io import floats_to_device, ints_to_device, to_device
from .rotation import fast_rotation_matrix, random_rotation_fast

QJL_CONST = np.sqrt(np.pi / 2)


class QJL:
    """sign(S r) as int8 +-1 plus ||r||; reconstruction sqrt(pi/2)/sqrt(d) * ||r|| * S^T z is
    unbiased for inner products (turboquant/qjl.py:35-70)."""

    _ORTHO_TOL = 1e-10

    def __init__(self, d: int, seed: int = 123, *, kind: str = "dense", device=None, matrix=None):
        self.d = d
        self.device = device
        rng = np.random.default_rng(seed)
        self.signs = None
        if matrix is not None:
            self.S = np.asarray(matrix, dtype=np.float64)
        elif kind == "dense":
            gauss = rng.standard_normal((d, d))
            q, r = np.linalg.qr(gauss)
            self.S = q * np.sign(np.diagonal(r))[np.newaxis, :]
        elif kind == "wht":
            s1, s2, padded = random_rotation_fast(d, rng)
            if padded != d:
                raise ValueError(f"kind='wht' needs d to be a power of two, got {d}")
            self.signs = (s1, s2)
            self.S = fast_rotation_matrix(s1, s2)
        else:
            raise ValueError(f"kind must be 'dense' or 'wht', got {kind!r}")
        defect = np.linalg.norm(self.S @ self.S.T - np.eye(d), "fro")
        assert defect < self._ORTHO_TOL, (
            f"QJL projection matrix not orthogonal: ||S S^T - I||_F = {defect:.2e} (tolerance {self._ORTHO_TOL:.0e})")
        self._handles = {}
        self._uploaded = None

    def _native(self, device):
        snap = self.S.tobytes()
        if snap != self._uploaded:
            self._handles.clear()
            self._uploaded = snap
        key = str(device)
        if key not in self._handles:
            self._handles[key] = nv.Quantizer(self.d, 1, nv.ROT_DENSE, True, np.array([-1.0, 1.0]), qjl_s=self.S,
                                              device=device)
        return self._handles[key]

    def quantize(self, r):
        """(signs int8 in {+1,-1}, ||r||); zeros of the projection count as +1 (turboquant/qjl.py:72-94)."""
        torch = nv.require_cuda()
        rt, was_numpy, src_dtype = to_device(r, self.device, allow_f64=True)
        single = rt.dim() == 1
        rt = rt.reshape(1, -1) if single else rt.reshape(-1, rt.shape[-1])
        if rt.dtype == torch.bfloat16:
            rt = rt.float()
        n = rt.shape[0]
        q = self._native(rt.device)
        bits = torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=rt.device)
        nrm = torch.empty((n,), dtype=torch.float32, device=rt.device)
        signs = torch.empty((n, self.d), dtype=torch.int8, device=rt.device)
        with torch.cuda.device(rt.device):
            nv.call("tq_qjl_quantize", q.handle, nv.ptr(rt), nv.torch_dtype_code(rt.dtype), n, nv.ptr(bits),
                    nv.ptr(nrm), nv.stream_ptr())
            nv.call("tq_unpack_bits", nv.ptr(bits), n, self.d, nv.ptr(signs), nv.stream_ptr())
        if was_numpy:
            signs = signs.cpu().numpy()
            nrm = nrm.cpu().numpy().astype(src_dtype if src_dtype is not None else np.float64)
        return (signs[0], nrm[0]) if single else (signs, nrm)

    def dequantize(self, signs, norms, shrinkage: float = 1.0):
        """shrinkage * sqrt(pi/2)/sqrt(d) * ||r|| * S^T z; shrinkage 1.0 is the unbiased estimator,
        2/pi the minimum-MSE one (turboquant/qjl.py:96-134)."""
        torch = nv.require_cuda()
        was_numpy = not isinstance(signs, torch.Tensor)
        dev = (torch.device("cuda", torch.cuda.current_device()) if self.device is None else torch.device(self.device)) \
            if was_numpy or signs.device.type != "cuda" else signs.device
        st = ints_to_device(signs, dev, torch.int8)
        single = st.dim() == 1
        st = st.reshape(1, -1) if single else st.reshape(-1, st.shape[-1])
        nt = floats_to_device(np.asarray(norms).reshape(-1) if was_numpy else norms.reshape(-1), dev)
        n = st.shape[0]
        q = self._native(dev)
        bits = torch.empty((n, (self.d + 7) // 8), dtype=torch.uint8, device=dev)
        out = torch.empty((n, self.d), dtype=torch.float64, device=dev)
        with torch.cuda.device(dev):
            nv.call("tq_pack_bits", nv.ptr(st), n, self.d, nv.ptr(bits), nv.stream_ptr())
            nv.call("tq_qjl_dequantize", q.handle, nv.ptr(bits), nv.ptr(nt), float(shrinkage), n, nv.ptr(out),
                    nv.F64, nv.stream_ptr())
        if was_numpy:
            out = out.cpu().numpy()
        return out[0] if single else out
