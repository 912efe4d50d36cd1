"""Lloyd-Max codebooks for the post-rotation coordinate distribution N(0, 1/d).

Same functions as the reference's ``turboquant/codebook.py``.  Codebook construction is a
once-per-quantizer host computation (a few milliseconds); the nearest-centroid search runs on the
GPU (``tq_nearest_centroid_f64`` here, fused into the quantize kernels on the hot path).
"""
from __future__ import annotations

import numpy as np
from scipy import stats

from . import _native as nv


def _region_means(edges: np.ndarray, sigma: float) -> np.ndarray:
    """E[X | lo < X < hi] for consecutive edges of X ~ N(0, sigma^2), all regions at once.

    Arithmetic follows turboquant/codebook.py:88-118 term by term (tail regions use cdf / sf
    directly, interior ones a cdf difference) so that the centroids agree to the last bit.
    """
    lo, hi = edges[:-1], edges[1:]
    fin_lo, fin_hi = np.isfinite(lo), np.isfinite(hi)
    z_lo = np.where(fin_lo, lo / sigma, lo)
    z_hi = np.where(fin_hi, hi / sigma, hi)
    with np.errstate(invalid="ignore"):
        mass = np.where(~fin_lo, stats.norm.cdf(z_hi),
                        np.where(~fin_hi, stats.norm.sf(z_lo), stats.norm.cdf(z_hi) - stats.norm.cdf(z_lo)))
        dens = stats.norm.pdf(z_lo) - stats.norm.pdf(z_hi)
        mean = sigma * dens / np.where(mass < 1e-15, 1.0, mass)
        # vanishing mass: asymptotic values (codebook.py:106-115)
        tail = np.where(fin_lo & ~fin_hi, lo + sigma,
                        np.where(~fin_lo & fin_hi, hi - sigma, np.where(fin_lo & fin_hi, (lo + hi) / 2.0, 0.0)))
    return np.where(mass < 1e-15, tail, mean)


def _lloyds_gaussian(n_centroids: int, sigma: float, n_iter: int = 100) -> np.ndarray:
    """Lloyd iteration from uniform-quantile boundaries (turboquant/codebook.py:52-85)."""
    inner = stats.norm.ppf(np.linspace(0, 1, n_centroids + 1)[1:-1], scale=sigma)
    cent = _region_means(np.concatenate(([-np.inf], inner, [np.inf])), sigma)
    for _ in range(n_iter):
        inner = (cent[:-1] + cent[1:]) / 2.0
        cent = _region_means(np.concatenate(([-np.inf], inner, [np.inf])), sigma)
    return np.sort(cent)


def _gaussian_conditional_expectation(sigma: float, a: float, b: float) -> float:
    """E[X | a < X < b] for one interval (turboquant/codebook.py:88-118)."""
    return float(_region_means(np.array([a, b], dtype=np.float64), sigma)[0])


def optimal_centroids(bit_width: int, d: int) -> np.ndarray:
    """2**bit_width sorted centroids: closed form for 1 and 2 bits, Lloyd on N(0, 1/d) above
    (turboquant/codebook.py:29-49)."""
    if bit_width == 1:
        c = np.sqrt(2.0 / (np.pi * d))
        return np.array([-c, c])
    if bit_width == 2:
        return np.array([-1.51, -0.453, 0.453, 1.51]) / np.sqrt(d)
    return _lloyds_gaussian(1 << bit_width, sigma=1.0 / np.sqrt(d))


def nearest_centroid_indices(values, centroids):
    """Index of the nearest centroid = number of midpoints strictly below the value; a value on a
    midpoint takes the lower index (turboquant/codebook.py:121-134).  Runs on the GPU in fp64."""
    torch = nv.require_cuda()
    as_numpy = not isinstance(values, torch.Tensor)
    vt = torch.as_tensor(np.ascontiguousarray(values, dtype=np.float64) if as_numpy else values)
    vt = vt.to("cuda", torch.float64).contiguous()
    ct = torch.as_tensor(np.ascontiguousarray(centroids, dtype=np.float64)
                         if not isinstance(centroids, torch.Tensor) else centroids).to(vt.device, torch.float64)
    out = torch.empty(vt.shape, dtype=torch.int64, device=vt.device)
    with torch.cuda.device(vt.device):
        nv.call("tq_nearest_centroid_f64", nv.ptr(vt), vt.numel(), nv.ptr(ct), ct.numel(), nv.ptr(out),
                nv.stream_ptr())
    return out.cpu().numpy() if as_numpy else out
