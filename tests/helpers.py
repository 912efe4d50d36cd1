"""Helpers shared by the GPU parity tests."""
import numpy as np

from oracle import tq_oracle as o

D = 128


def boundary_band(c):
    """Half-width of the band around a decision boundary inside which an index may differ from the
    fp64 reference: 1e-6 relative to the largest centroid magnitude."""
    return 1e-6 * np.abs(c).max()


def near_boundary(y, c):
    """Boolean mask: rotated coordinate within the band of some boundary."""
    b = o.boundaries(c)
    return (np.abs(y[..., None] - b).min(axis=-1) <= boundary_band(c))


def check_indices(idx_gpu, idx_ref, y_ref, c):
    """Indices equal except inside the boundary band; returns (mismatches, coordinates in band)."""
    diff = idx_gpu != idx_ref
    band = near_boundary(y_ref, c)
    assert not (diff & ~band).any(), f"{int((diff & ~band).sum())} index mismatches outside the boundary band"
    assert (np.abs(idx_gpu.astype(np.int64) - idx_ref.astype(np.int64))[diff] <= 1).all()
    return int(diff.sum()), int(band.sum())


def max_rel(out, ref):
    """Max-relative error per row: max|out-ref| / max|ref|, worst row."""
    out = np.asarray(out, dtype=np.float64).reshape(-1, out.shape[-1])
    ref = np.asarray(ref, dtype=np.float64).reshape(-1, ref.shape[-1])
    return float((np.abs(out - ref).max(axis=1) / np.abs(ref).max(axis=1)).max())


def wht_dense(c, seed):
    return o.wht_as_dense(c[f"wht_s1_{seed}"], c[f"wht_s2_{seed}"])


def fill_cache(cache, k, v, seq_lens, rng, page_tokens=128):
    """Append per-sequence K/V (lists of (len, Hkv, d) arrays) into randomly chosen pages; returns
    the block table."""
    import torch
    n_pages = [(int(n) + page_tokens - 1) // page_tokens for n in seq_lens]
    perm = rng.permutation(cache.num_pages)[: sum(n_pages)]
    max_pages = max(n_pages)
    bt = np.zeros((len(seq_lens), max_pages), dtype=np.int32)
    pos = 0
    for b, n in enumerate(seq_lens):
        pages = perm[pos:pos + n_pages[b]]
        pos += n_pages[b]
        bt[b, : n_pages[b]] = pages
        t = np.arange(int(n))
        slots = pages[t // page_tokens].astype(np.int64) * page_tokens + t % page_tokens
        cache.append(torch.as_tensor(k[b]).to(cache.device), torch.as_tensor(v[b]).to(cache.device),
                     torch.as_tensor(slots))
    return torch.as_tensor(bt)
