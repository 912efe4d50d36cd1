"""Rotations for PolarQuant: dense Haar matrices and the sign * Walsh-Hadamard fast rotation.

Same functions as the reference's ``turboquant/rotation.py``.  Constructors of constants run on
the host (they run once per quantizer); the transforms themselves run on the GPU in fp64 through
``tq_sign_wht_f64``.  Inputs may be NumPy arrays (NumPy comes back) or CUDA tensors.
"""
from __future__ import annotations

import numpy as np

from . import _native as nv


def random_rotation_dense(d: int, rng: np.random.Generator) -> np.ndarray:
    """Haar-distributed rotation with determinant +1 (reference: turboquant/rotation.py:25-50).

    Consumes ``rng`` exactly like the reference (one d x d standard-normal draw), so the same
    seed gives the same matrix.
    """
    if d < 1:
        raise ValueError(f"d must be >= 1, got {d}")
    gauss = rng.standard_normal((d, d))
    q, r = np.linalg.qr(gauss)
    diag_sign = np.sign(np.diagonal(r)).copy()
    diag_sign[diag_sign == 0] = 1.0
    q = q * diag_sign[np.newaxis, :]
    det_sign, _ = np.linalg.slogdet(q)
    if det_sign < 0:
        q[:, 0] *= -1.0
    return q


def _next_power_of_2(n: int) -> int:
    return 1 if n <= 1 else 1 << (int(n) - 1).bit_length()


def hadamard_matrix(n: int) -> np.ndarray:
    """Sylvester Hadamard matrix of +-1 entries (reference: turboquant/rotation.py:61-72)."""
    if n < 1 or (n & (n - 1)) != 0:
        raise ValueError(f"n must be a positive power of 2, got {n}")
    h = np.array([[1.0]])
    for _ in range(n.bit_length() - 1):
        h = np.kron(np.array([[1.0, 1.0], [1.0, -1.0]]), h)
    return h


def random_rotation_fast(d: int, rng: np.random.Generator):
    """Two +-1 sign vectors and the padded size (reference: turboquant/rotation.py:75-96)."""
    n = _next_power_of_2(d)
    first = rng.choice([-1.0, 1.0], size=n)
    second = rng.choice([-1.0, 1.0], size=n)
    return first, second, n


def _sign_wht(x, d, n, s1, s2):
    """rows of d values -> D2 (H/sqrt n) D1 rows, fp64, on the GPU."""
    torch = nv.require_cuda()
    as_numpy = not isinstance(x, torch.Tensor)
    xt = torch.as_tensor(np.ascontiguousarray(x, dtype=np.float64) if as_numpy else x).to("cuda", torch.float64)
    xt = xt.contiguous().reshape(-1, d)
    out = torch.empty_like(xt)
    s1t = None if s1 is None else torch.as_tensor(np.asarray(s1, dtype=np.float64)).to(xt.device)
    s2t = None if s2 is None else torch.as_tensor(np.asarray(s2, dtype=np.float64)).to(xt.device)
    with torch.cuda.device(xt.device):
        nv.call("tq_sign_wht_f64", nv.ptr(xt), xt.shape[0], d, n, nv.ptr(s1t), nv.ptr(s2t), nv.ptr(out),
                nv.stream_ptr())
    return out.cpu().numpy() if as_numpy else out


def fast_walsh_hadamard_transform(x):
    """Natural-order WHT scaled by 1/sqrt(n); returns a new array (turboquant/rotation.py:99-121)."""
    n = len(x)
    if n < 1 or (n & (n - 1)) != 0:
        raise ValueError(f"Input length must be a positive power of 2, got {n}")
    return _sign_wht(x, n, n, None, None).reshape(n)


def apply_fast_rotation(x, signs1, signs2, padded_d: int):
    """D2 H D1 x with zero padding to ``padded_d`` and cropping (turboquant/rotation.py:124-145)."""
    d = len(x)
    return _sign_wht(x, d, padded_d, signs1, signs2).reshape(d)


def apply_fast_rotation_transpose(y, signs1, signs2, padded_d: int):
    """The transpose D1 H D2 (turboquant/rotation.py:148-160)."""
    d = len(y)
    return _sign_wht(y, d, padded_d, signs2, signs1).reshape(d)


def apply_fast_rotation_batch(X, signs1, signs2, padded_d: int):
    """Rows of a (batch, d) array rotated at once (turboquant/rotation.py:163-185)."""
    batch, d = X.shape
    return _sign_wht(X, d, padded_d, signs1, signs2).reshape(batch, d)


def fast_rotation_matrix(signs1, signs2) -> np.ndarray:
    """Dense d x d form of D2 (H/sqrt d) D1 for d a power of two (host-side helper)."""
    n = len(signs1)
    return (np.asarray(signs2)[:, None] * hadamard_matrix(n) * np.asarray(signs1)[None, :]) / np.sqrt(n)
