"""CPU oracle for the TurboQuant+ KV-cache compression path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain NumPy, the algorithm of the reference project
(TheTom/turboquant_plus, package ``turboquant/``).  It exists to check the CUDA
path; the shipped package never imports it.  Only tests, the smoke check and the
CPU-baseline leg of the benchmark may call into it.

Parity status: PINNED.  Every function below is compared against outputs of the
reference itself (golden fixtures under tests/golden/, produced by
tests/golden/make_golden.py which imports the reference), and, when the
reference tree is importable, against the live reference classes.

Exceptions, marked "parity unpinned" where they are defined: the q8_0 block
format and multi-head / ragged attention, which the reference does not
implement (it only names q8_0 and only ever attends with one head).

Every function cites the reference file:line it follows.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

try:  # SciPy is only needed for Lloyd-Max codebooks with bit_width >= 3
    from scipy import stats as _stats
except Exception:  # pragma: no cover
    _stats = None


# --------------------------------------------------------------------------
# rotation.py
# --------------------------------------------------------------------------
def dense_rotation(d: int, rng: np.random.Generator) -> np.ndarray:
    """Haar rotation with det=+1.  Follows turboquant/rotation.py:25-50."""
    if d < 1:
        raise ValueError(f"d must be >= 1, got {d}")
    g = rng.standard_normal((d, d))
    q, r = np.linalg.qr(g)
    sg = np.sign(np.diag(r))
    sg[sg == 0] = 1.0
    q = q * sg[None, :]
    if np.linalg.slogdet(q)[0] < 0:
        q[:, 0] = -q[:, 0]
    return q


def next_pow2(n: int) -> int:
    """turboquant/rotation.py:53-58."""
    p = 1
    while p < n:
        p *= 2
    return p


def hadamard(n: int) -> np.ndarray:
    """Unnormalised Sylvester Hadamard matrix.  turboquant/rotation.py:61-72."""
    if n < 1 or n & (n - 1):
        raise ValueError(f"n must be a positive power of 2, got {n}")
    h = np.ones((1, 1))
    while h.shape[0] < n:
        h = np.block([[h, h], [h, -h]])
    return h


def wht_signs(d: int, rng: np.random.Generator):
    """Two +-1 vectors, signs1 drawn first.  turboquant/rotation.py:75-96."""
    pd = next_pow2(d)
    s1 = rng.choice([-1.0, 1.0], size=pd)
    s2 = rng.choice([-1.0, 1.0], size=pd)
    return s1, s2, pd


def fwht(x: np.ndarray) -> np.ndarray:
    """Natural-order WHT of one vector, scaled 1/sqrt(n), fp64.
    turboquant/rotation.py:99-121 (vectorised over the inner j loop)."""
    n = len(x)
    if n < 1 or n & (n - 1):
        raise ValueError(f"Input length must be a positive power of 2, got {n}")
    v = np.array(x, dtype=np.float64)
    h = 1
    while h < n:
        w = v.reshape(n // (2 * h), 2, h)
        a = w[:, 0, :].copy()
        b = w[:, 1, :].copy()
        w[:, 0, :] = a + b
        w[:, 1, :] = a - b
        h *= 2
    return v / np.sqrt(n)


def wht_rotate_batch(x: np.ndarray, s1: np.ndarray, s2: np.ndarray, pd: int) -> np.ndarray:
    """y = D2 (H/sqrt(n)) D1 x for a batch, pad/crop to d.
    turboquant/rotation.py:163-185 (and :124-145 for one vector)."""
    b, d = x.shape
    p = np.zeros((b, pd))
    p[:, :d] = x
    p *= s1[None, :]
    h = 1
    while h < pd:
        w = p.reshape(b, pd // (2 * h), 2, h)
        a = w[:, :, 0, :].copy()
        c = w[:, :, 1, :].copy()
        w[:, :, 0, :] = a + c
        w[:, :, 1, :] = a - c
        p = w.reshape(b, pd)
        h *= 2
    p /= np.sqrt(pd)
    p *= s2[None, :]
    return p[:, :d]


def wht_rotate_transpose_batch(y, s1, s2, pd):
    """Transpose = D1 H D2 (turboquant/rotation.py:148-160): swap the sign vectors."""
    return wht_rotate_batch(y, s2, s1, pd)


def wht_as_dense(s1: np.ndarray, s2: np.ndarray) -> np.ndarray:
    """The d x d matrix of D2 (H/sqrt(n)) D1 for n == d (power of two)."""
    n = len(s1)
    return (s2[:, None] * hadamard(n) * s1[None, :]) / np.sqrt(n)


# --------------------------------------------------------------------------
# codebook.py
# --------------------------------------------------------------------------
def _cond_mean(sigma: float, a: float, b: float) -> float:
    """E[X | a<X<b], X~N(0,sigma^2).  turboquant/codebook.py:88-118."""
    az = a / sigma if np.isfinite(a) else a
    bz = b / sigma if np.isfinite(b) else b
    if not np.isfinite(az):
        prob = _stats.norm.cdf(bz)
    elif not np.isfinite(bz):
        prob = _stats.norm.sf(az)
    else:
        prob = _stats.norm.cdf(bz) - _stats.norm.cdf(az)
    if prob < 1e-15:
        if np.isfinite(a) and not np.isfinite(b):
            return a + sigma
        if not np.isfinite(a) and np.isfinite(b):
            return b - sigma
        if np.isfinite(a) and np.isfinite(b):
            return (a + b) / 2.0
        return 0.0
    return sigma * (_stats.norm.pdf(az) - _stats.norm.pdf(bz)) / prob


def lloyd_gaussian(n_levels: int, sigma: float, n_iter: int = 100) -> np.ndarray:
    """turboquant/codebook.py:52-85."""
    bnd = _stats.norm.ppf(np.linspace(0, 1, n_levels + 1)[1:-1], scale=sigma)
    c = np.zeros(n_levels)

    def refresh(bnd):
        c[0] = _cond_mean(sigma, -np.inf, bnd[0])
        for i in range(1, n_levels - 1):
            c[i] = _cond_mean(sigma, bnd[i - 1], bnd[i])
        c[-1] = _cond_mean(sigma, bnd[-1], np.inf)

    refresh(bnd)
    for _ in range(n_iter):
        bnd = (c[:-1] + c[1:]) / 2.0
        refresh(bnd)
    return np.sort(c)


def centroids(bit_width: int, d: int) -> np.ndarray:
    """turboquant/codebook.py:29-49."""
    if bit_width == 1:
        c = np.sqrt(2.0 / (np.pi * d))
        return np.array([-c, c])
    if bit_width == 2:
        return np.array([-1.51, -0.453, 0.453, 1.51]) / np.sqrt(d)
    return lloyd_gaussian(1 << bit_width, sigma=1.0 / np.sqrt(d))


def boundaries(c: np.ndarray) -> np.ndarray:
    """fp64 midpoints.  turboquant/codebook.py:133."""
    return (c[:-1] + c[1:]) / 2.0


def nearest_index(values: np.ndarray, c: np.ndarray) -> np.ndarray:
    """#boundaries strictly below v (ties go to the lower index).
    turboquant/codebook.py:121-134."""
    return np.searchsorted(boundaries(c), values.ravel()).reshape(values.shape)


# --------------------------------------------------------------------------
# polar_quant.py
# --------------------------------------------------------------------------
def polar_quantize(x: np.ndarray, rot: np.ndarray, c: np.ndarray, return_rotated=False):
    """norm -> safe normalise -> rotate -> nearest centroid.
    turboquant/polar_quant.py:56-85.  x is (batch, d)."""
    nrm = np.linalg.norm(x, axis=1)
    safe = np.where(nrm > 0, nrm, 1.0)
    xn = x / safe[:, None]
    y = (rot @ xn.T).T
    idx = nearest_index(y, c)
    if return_rotated:
        return idx, nrm, y
    return idx, nrm


def polar_dequantize(idx: np.ndarray, nrm: np.ndarray, rot: np.ndarray, c: np.ndarray,
                     norm_correction: bool = True) -> np.ndarray:
    """lookup -> optional renormalise -> inverse rotate -> rescale.
    turboquant/polar_quant.py:87-119."""
    yh = c[idx]
    if norm_correction:
        n = np.linalg.norm(yh, axis=1, keepdims=True)
        n = np.where(n > 1e-10, n, 1.0)
        yh = yh / n
    xu = (rot.T @ yh.T).T
    return xu * np.asarray(nrm)[:, None]


def polar_residual(x, rot, c, norm_correction=True):
    """turboquant/polar_quant.py:121-132."""
    idx, nrm = polar_quantize(x, rot, c)
    return idx, nrm, x - polar_dequantize(idx, nrm, rot, c, norm_correction)


# --------------------------------------------------------------------------
# qjl.py
# --------------------------------------------------------------------------
QJL_CONST = math.sqrt(math.pi / 2.0)  # turboquant/qjl.py:32


def qjl_matrix(d: int, rng: np.random.Generator) -> np.ndarray:
    """Orthogonal projection (no determinant fix).  turboquant/qjl.py:56-62."""
    g = rng.standard_normal((d, d))
    q, r = np.linalg.qr(g)
    return q * np.sign(np.diag(r))[None, :]


def qjl_quantize(r: np.ndarray, s: np.ndarray):
    """sign(S r) as int8 with zeros mapped to +1, and ||r||.  turboquant/qjl.py:72-94."""
    nrm = np.linalg.norm(r, axis=1)
    z = np.sign((s @ r.T).T).astype(np.int8)
    z[z == 0] = 1
    return z, nrm


def qjl_dequantize(z: np.ndarray, nrm: np.ndarray, s: np.ndarray, shrinkage: float = 1.0):
    """sqrt(pi/2)/sqrt(d) * ||r|| * S^T z.  turboquant/qjl.py:96-134."""
    d = s.shape[0]
    rec = (s.T @ z.astype(np.float64).T).T
    return rec * ((QJL_CONST / np.sqrt(d) * np.asarray(nrm))[:, None] * shrinkage)


# --------------------------------------------------------------------------
# turboquant.py
# --------------------------------------------------------------------------
@dataclass
class ProdCode:
    """Mirror of CompressedVector (turboquant/turboquant.py:33-40)."""
    mse_indices: np.ndarray
    vector_norms: np.ndarray
    qjl_signs: np.ndarray
    residual_norms: np.ndarray
    bit_width: int


def prod_quantize(x, rot, c_bm1, s, bit_width, norm_correction=True) -> ProdCode:
    """(b-1)-bit PolarQuant then 1-bit QJL of the residual.  turboquant/turboquant.py:79-100."""
    idx, nrm, res = polar_residual(x, rot, c_bm1, norm_correction)
    z, rn = qjl_quantize(res, s)
    return ProdCode(idx, nrm, z, rn, bit_width)


def prod_dequantize(code: ProdCode, rot, c_bm1, s, norm_correction=True, shrinkage=1.0):
    """turboquant/turboquant.py:102-124."""
    return (polar_dequantize(code.mse_indices, code.vector_norms, rot, c_bm1, norm_correction)
            + qjl_dequantize(code.qjl_signs, code.residual_norms, s, shrinkage))


def prod_size_bits(d, bit_width, n):
    """turboquant/turboquant.py:126-136 (one 32-bit norm counted, as the reference does)."""
    return n * (d * bit_width + 32)


def prod_ratio(d, bit_width, original_bits=16):
    """turboquant/turboquant.py:138-149."""
    return (d * original_bits) / (d * bit_width + 32)


# --------------------------------------------------------------------------
# outlier.py
# --------------------------------------------------------------------------
def outlier_split(d: int, target_bits: float):
    """(n_outlier, high_bits, n_normal, low_bits): round(d * frac) leading channels get one more bit.
    turboquant/outlier.py:45-66."""
    low = int(np.floor(target_bits))
    n_out = int(round(d * (target_bits - low)))
    return n_out, low + 1, d - n_out, low


class OutlierOracle:
    """Fractional bit rates: the first n_outlier channels are their own PolarQuant sub-vector at
    (high_bits - 1) bits with the rotation drawn from ``seed``, the remaining channels another at
    (low_bits - 1) bits with ``seed + 500``; one QJL (``seed + 1000``) sketches the residual of the whole
    vector.  turboquant/outlier.py:69-108 (constructor), :110-178 (quantize), :180-208 (dequantize)."""

    def __init__(self, d: int, target_bits: float, seed: int = 42):
        self.d = d
        self.n_out, self.high_bits, self.n_norm, self.low_bits = outlier_split(d, target_bits)
        self.effective_bits = (self.n_out * self.high_bits + self.n_norm * self.low_bits) / d
        self.r_out = dense_rotation(self.n_out, np.random.default_rng(seed)) if self.n_out > 0 else None
        self.r_norm = dense_rotation(self.n_norm, np.random.default_rng(seed + 500)) if self.n_norm > 0 else None
        self.c_out = centroids(self.high_bits - 1, self.n_out) if self.n_out > 0 else None
        self.c_norm = centroids(self.low_bits - 1, self.n_norm) if self.n_norm > 0 else None
        self.s = qjl_matrix(d, np.random.default_rng(seed + 1000))

    def quantize(self, x: np.ndarray) -> dict:
        """x: (batch, d).  Keys follow OutlierCompressedVector (turboquant/outlier.py:33-42)."""
        res = np.zeros(x.shape, dtype=np.float64)
        code = {}
        if self.n_out > 0:
            code["outlier_indices"], code["outlier_norms"], res[:, :self.n_out] = polar_residual(
                x[:, np.arange(self.n_out)], self.r_out, self.c_out)   # fancy indexing as at outlier.py:119: the
            # copy it makes has its own memory order, which decides the summation order of the norm
        if self.n_norm > 0:
            code["normal_indices"], code["normal_norms"], res[:, self.n_out:] = polar_residual(
                x[:, np.arange(self.n_out, self.d)], self.r_norm, self.c_norm)
        code["qjl_signs"], code["residual_norms"] = qjl_quantize(res, self.s)
        return code

    def dequantize(self, code: dict) -> np.ndarray:
        out = qjl_dequantize(code["qjl_signs"], code["residual_norms"], self.s)
        if self.n_out > 0:
            out[:, :self.n_out] += polar_dequantize(code["outlier_indices"], code["outlier_norms"], self.r_out, self.c_out)
        if self.n_norm > 0:
            out[:, self.n_out:] += polar_dequantize(code["normal_indices"], code["normal_norms"], self.r_norm, self.c_norm)
        return out

    def compression_ratio(self, original_bits: int = 16) -> float:
        """Three 32-bit norms per vector.  turboquant/outlier.py:210-217."""
        return self.d * original_bits / (self.d * self.effective_bits + 96)


# --------------------------------------------------------------------------
# utils.py
# --------------------------------------------------------------------------
def pack_signs(z: np.ndarray) -> np.ndarray:
    """+1 -> bit 1, MSB first, padded to whole bytes per row.  turboquant/utils.py:20-49."""
    bits = (z > 0).astype(np.uint8)
    if bits.ndim == 1:
        return np.packbits(bits)
    return np.packbits(bits, axis=1)


def unpack_signs(p: np.ndarray, d: int) -> np.ndarray:
    """turboquant/utils.py:52-68."""
    if p.ndim == 1:
        return np.unpackbits(p)[:d].astype(np.int8) * 2 - 1
    return np.unpackbits(p, axis=1)[:, :d].astype(np.int8) * 2 - 1


def pack_idx(idx: np.ndarray, bit_width: int) -> np.ndarray:
    """MSB-first bitstream over the flattened array (b<=4); uint8 copy for 5..8.
    turboquant/utils.py:71-98."""
    if bit_width <= 0 or bit_width > 8:
        raise ValueError(f"bit_width must be 1-8, got {bit_width}")
    if bit_width > 4:
        return idx.astype(np.uint8)
    flat = idx.ravel().astype(np.uint8)
    shifts = np.arange(bit_width - 1, -1, -1, dtype=np.uint8)
    bits = (flat[:, None] >> shifts[None, :]) & 1
    return np.packbits(bits.ravel())


def unpack_idx(p: np.ndarray, bit_width: int, count: int) -> np.ndarray:
    """Inverse of pack_idx for b<=4 (the reference has no such function)."""
    bits = np.unpackbits(p)[: count * bit_width].reshape(count, bit_width)
    w = (1 << np.arange(bit_width - 1, -1, -1)).astype(np.int64)
    return (bits.astype(np.int64) * w[None, :]).sum(axis=1)


def footprint(n_vectors: int, d: int, bit_width: int) -> dict:
    """turboquant/utils.py:101-123."""
    mse = int(np.ceil(n_vectors * d * (bit_width - 1) / 8))
    qjl = int(np.ceil(n_vectors * d / 8))
    nb = n_vectors * 4
    tot = mse + qjl + nb
    orig = n_vectors * d * 2
    return {"mse_indices_bytes": mse, "qjl_signs_bytes": qjl, "norms_bytes": nb,
            "total_bytes": tot, "original_fp16_bytes": orig,
            "compression_ratio": orig / tot if tot > 0 else float("inf")}


# --------------------------------------------------------------------------
# kv_cache.py
# --------------------------------------------------------------------------
def kv_memory_stats(head_dim, k_bits, v_bits, seq_len, num_layers, num_heads) -> dict:
    """turboquant/kv_cache.py:167-188 (V counted without a norm, as the reference does)."""
    n = num_layers * num_heads * seq_len
    orig = n * head_dim * 2
    comp = (n * (head_dim * k_bits + 32) + n * head_dim * v_bits) / 8
    return {"original_mb": orig / 1024 / 1024, "compressed_mb": comp / 1024 / 1024,
            "compression_ratio": orig / comp, "k_bits_per_value": k_bits,
            "v_bits_per_value": v_bits}


class KVOracle:
    """K: prod quantizer (seed), V: MSE quantizer (seed+500), QJL (seed+1000); one set of
    constants shared by every layer and head.  turboquant/kv_cache.py:69-96,
    turboquant/turboquant.py:57-77, turboquant/polar_quant.py:46-54.

    ``mode='dense'`` builds the rotations exactly as the reference constructors do.
    ``mode='wht'`` replaces each rotation by the dense form of D2 (H/sqrt d) D1 and the QJL
    matrix by an independent sign-WHT drawn from the same seeds with
    turboquant/rotation.py:75-96; the reference's quantize/dequantize code is unchanged.
    ``k_kind='mse'`` stores K as b-bit PolarQuant only (the "turboN" cache types).
    """

    def __init__(self, head_dim, k_bits=3, v_bits=3, seed=42, norm_correction=True,
                 mode="dense", k_kind="prod", constants=None):
        self.d, self.k_bits, self.v_bits = head_dim, k_bits, v_bits
        self.nc, self.k_kind = norm_correction, k_kind
        if constants is not None:
            self.rk, self.rv, self.s = constants["rk"], constants["rv"], constants["s"]
        elif mode == "dense":
            self.rk = dense_rotation(head_dim, np.random.default_rng(seed))
            self.rv = dense_rotation(head_dim, np.random.default_rng(seed + 500))
            self.s = qjl_matrix(head_dim, np.random.default_rng(seed + 1000))
        else:
            a1, a2, _ = wht_signs(head_dim, np.random.default_rng(seed))
            b1, b2, _ = wht_signs(head_dim, np.random.default_rng(seed + 500))
            c1, c2, _ = wht_signs(head_dim, np.random.default_rng(seed + 1000))
            self.rk, self.rv, self.s = wht_as_dense(a1, a2), wht_as_dense(b1, b2), wht_as_dense(c1, c2)
        self.ck = centroids(k_bits - 1 if k_kind == "prod" else k_bits, head_dim)
        self.cv = centroids(v_bits, head_dim)

    def k_roundtrip(self, k):
        if self.k_kind == "prod":
            code = prod_quantize(k, self.rk, self.ck, self.s, self.k_bits, self.nc)
            return prod_dequantize(code, self.rk, self.ck, self.s, self.nc)
        i, n = polar_quantize(k, self.rk, self.ck)
        return polar_dequantize(i, n, self.rk, self.ck, self.nc)

    def v_roundtrip(self, v):
        i, n = polar_quantize(v, self.rv, self.cv)
        return polar_dequantize(i, n, self.rv, self.cv, self.nc)


def softmax_rows(x: np.ndarray) -> np.ndarray:
    """tests/test_kv_cache.py:128-131."""
    e = np.exp(x - np.max(x, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


def attend_one(q: np.ndarray, k_hat: np.ndarray, v_hat: np.ndarray, scale=None) -> np.ndarray:
    """softmax(q k^T * scale) v over a dequantized cache, no mask, scale 1/sqrt(d).
    tests/test_kv_cache.py:73-89.  q is (rows, d); k_hat, v_hat are (ctx, d)."""
    d = q.shape[-1]
    sc = (1.0 / np.sqrt(d)) if scale is None else scale
    return softmax_rows((q @ k_hat.T) * sc) @ v_hat


def attend_gqa(q, k_hat, v_hat, seq_lens=None, scale=None):
    """Dequantize-then-attend for a batch with grouped query heads.

    q (B, Hq, d); k_hat, v_hat (B, Hkv, ctx, d); query head h reads KV head h // (Hq//Hkv);
    sequence b uses its first seq_lens[b] positions.  Per (sequence, head) this is
    attend_one; the grouping and the ragged lengths are not in the reference
    (it only ever attends with one head) -- parity unpinned for those two aspects.
    """
    bsz, hq, d = q.shape
    hkv = k_hat.shape[1]
    g = hq // hkv
    out = np.zeros((bsz, hq, d))
    for b in range(bsz):
        n = k_hat.shape[2] if seq_lens is None else int(seq_lens[b])
        for h in range(hq):
            kh = h // g
            out[b, h] = attend_one(q[b, h][None].astype(np.float64),
                                   k_hat[b, kh, :n], v_hat[b, kh, :n], scale)[0]
    return out


def attend_chunk_gqa(q, k_hat, v_hat, kv_lens, scale=None):
    """Causal chunked prefill: q (B, Tq, Hq, d) holds the last Tq tokens of each sequence; query i of sequence b
    sits at position kv_lens[b] - Tq + i and attends to cached positions 0 .. that position (attend_one on the
    visible prefix).  The mask and the chunking are not in the reference -- parity unpinned for those aspects."""
    bsz, tq, hq, d = q.shape
    g = hq // k_hat.shape[1]
    out = np.zeros((bsz, tq, hq, d))
    for b in range(bsz):
        for i in range(tq):
            n = int(kv_lens[b]) - tq + i + 1
            if n <= 0:
                continue
            for h in range(hq):
                out[b, i, h] = attend_one(q[b, i, h][None].astype(np.float64), k_hat[b, h // g, :n],
                                          v_hat[b, h // g, :n], scale)[0]
    return out


# --------------------------------------------------------------------------
# q8_0 (not in the reference: parity unpinned)
# --------------------------------------------------------------------------
def q8_0_quantize(x: np.ndarray):
    """Blocks of 32 values: fp16 scale = max|x|/127, int8 = round-half-away(x/scale).

    The reference names this format (docs/decode-speed-hardware-analysis.md:354: 34 bytes
    per 32 values; README.md:42: 8.5 bits/value) but holds no implementation; the arithmetic
    lives in llama.cpp's ggml, which is not vendored and has no pinned version.  This restates
    ggml's published rule: d = amax/127 stored as fp16, q = round(x * (1/d)) computed with the
    unrounded fp32 d, zero block -> d = 0, q = 0.  Parity unpinned.
    """
    x = np.asarray(x, dtype=np.float32)
    n, d = x.shape
    blk = x.reshape(n, d // 32, 32)
    amax = np.abs(blk).max(axis=2)
    dd = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(dd > 0, np.float32(1.0) / np.where(dd > 0, dd, 1), 0).astype(np.float32)
    t = blk * inv[:, :, None]
    q = np.sign(t) * np.floor(np.abs(t) + np.float32(0.5))
    return q.astype(np.int8).reshape(n, d), dd.astype(np.float16)


def q8_0_dequantize(q: np.ndarray, scales: np.ndarray) -> np.ndarray:
    n, d = q.shape
    return (q.reshape(n, d // 32, 32).astype(np.float32)
            * scales.astype(np.float32)[:, :, None]).reshape(n, d)


# --------------------------------------------------------------------------
# Synthetic inputs standing in for real KV tensors (shapes and distributions of the
# benchmark configurations; no dataset is involved)
# --------------------------------------------------------------------------
def synth_keys(n: int, d: int = 128, seed: int = 0, dtype=np.float32):
    """N(0,1) per coordinate x lognormal(0, 0.5) per vector, 4 fixed outlier channels x10."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, d))
    x *= rng.lognormal(0.0, 0.5, size=(n, 1))
    ch = rng.choice(d, 4, replace=False)
    x[:, ch] *= 10.0
    return x.astype(dtype)


def rope_rotate(x: np.ndarray, positions: np.ndarray, base: float = 10000.0) -> np.ndarray:
    """Pairwise (2i, 2i+1) rotation by position * base^(-2i/d); only shapes the inputs."""
    d = x.shape[-1]
    inv = base ** (-np.arange(0, d, 2) / d)
    ang = positions[:, None] * inv[None, :]
    c, s = np.cos(ang), np.sin(ang)
    out = np.empty_like(x, dtype=np.float64)
    out[..., 0::2] = x[..., 0::2] * c - x[..., 1::2] * s
    out[..., 1::2] = x[..., 0::2] * s + x[..., 1::2] * c
    return out.astype(x.dtype)


# --------------------------------------------------------------------------
# benchmarks/temporal_decay_prototype.py
# --------------------------------------------------------------------------
def decay_requantize(idx_src: np.ndarray, norm_src, c_src: np.ndarray, c_dst: np.ndarray, mid_dst: np.ndarray):
    """One vector's codes re-quantized to a narrower codebook in the rotated domain: dequantize with the norm
    correction of the source codebook, renormalise, np.digitize against the destination midpoints (a tie goes to the
    upper cell), corrected norm for the destination codebook.  Returns (idx_dst uint8, corrected_norm).
    benchmarks/temporal_decay_prototype.py:71-80 (dequantize_3bit), :93-125 (requantize_3to2)."""
    cs = c_src[idx_src]
    rn = np.sqrt(np.sum(cs ** 2))
    values = cs * (norm_src / rn if rn > 1e-10 else norm_src)
    recon = np.linalg.norm(values)
    if recon > 1e-10:
        unit = values / recon
    else:
        unit, recon = values, 0.0
    idx_dst = np.digitize(unit, mid_dst).astype(np.uint8)
    cn = np.sqrt(np.sum(c_dst[idx_dst] ** 2))
    return idx_dst, (recon / cn if cn > 1e-10 else recon)


# --------------------------------------------------------------------------
# block formats of the reference's documents (no code in the reference tree: parity unpinned, the
# layouts restate docs/papers/block-size-experiment.md:25-37 and docs/papers/turbo4-resurrection.md:125-138,169,208)
# --------------------------------------------------------------------------
def block_bytes(bits: int, block_elems: int) -> int:
    if bits == 4:
        return 4 + block_elems // 2
    return 2 + block_elems // 4 + (block_elems // 8 if bits == 3 else 0)


def blocks_encode(idx: np.ndarray, scale: float, bits: int, block_elems: int) -> np.ndarray:
    """One 128-element vector's indices and corrected norm as 128 / block_elems storage blocks (uint8)."""
    out = []
    for b0 in range(0, len(idx), block_elems):
        blk = idx[b0:b0 + block_elems].astype(np.uint32)
        head = np.frombuffer(np.float16(scale).tobytes(), dtype=np.uint8)
        if bits == 4:
            qs = (blk[0::2] | (blk[1::2] << 4)).astype(np.uint8)
            out += [head, np.zeros(2, np.uint8), qs]
            continue
        low = blk & 3
        qs = (low[0::4] | (low[1::4] << 2) | (low[2::4] << 4) | (low[3::4] << 6)).astype(np.uint8)
        out += [head, qs]
        if bits == 3:
            hi = (blk >> 2) & 1
            out.append(sum(hi[j::8] << j for j in range(8)).astype(np.uint8))
    return np.concatenate(out)


def blocks_decode(raw: np.ndarray, bits: int, block_elems: int, d: int = 128):
    """Inverse, written with the documents' extraction expressions.  Returns (indices, norm of the first block)."""
    bb = block_bytes(bits, block_elems)
    idx = np.zeros(d, dtype=np.uint8)
    for b in range(d // block_elems):
        blk = raw[b * bb:(b + 1) * bb]
        if bits == 4:
            qs = blk[4:]
            for j in range(block_elems):
                idx[b * block_elems + j] = (qs[j // 2] >> ((j % 2) * 4)) & 0xF
            continue
        qs, signs = blk[2:2 + block_elems // 4], blk[2 + block_elems // 4:]
        for j in range(block_elems):
            m = (qs[j // 4] >> ((j % 4) * 2)) & 0x3
            if bits == 3 and signs[j // 8] & (1 << (j % 8)):
                m |= 4
            idx[b * block_elems + j] = m
    return idx, float(np.frombuffer(raw[:2].tobytes(), dtype=np.float16)[0])
