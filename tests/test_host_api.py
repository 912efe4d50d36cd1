"""Host-side logic that needs no GPU: constants, size formulae, error behaviour, no CPU fallback."""
import numpy as np
import pytest

import turboquant_plus_b200 as tq
from turboquant_plus_b200 import codebook, rotation, utils


def test_constants_equal_reference_exports(g_const):
    p = tq.PolarQuant(128, 3, seed=42)
    assert np.array_equal(p.rotation, g_const["rot_42"]) and np.array_equal(p.centroids, g_const["centroids_b3"])
    assert p.n_centroids == 8 and p.norm_correction is True and p.d == 128 and p.bit_width == 3
    w = tq.PolarQuant(128, 2, seed=542, rotation="wht")
    assert np.array_equal(w.signs[0], g_const["wht_s1_542"]) and np.array_equal(w.signs[1], g_const["wht_s2_542"])
    t = tq.TurboQuant(128, 3, seed=42)
    assert t.polar_quant.bit_width == 2 and np.array_equal(t.qjl.S, g_const["qjl_1042"])
    assert np.array_equal(tq.QJL(128).S, g_const["qjl_123"])
    kv = tq.KVCacheCompressor(128, 3, 3, seed=42)
    assert np.array_equal(kv.v_quantizer.polar_quant.rotation, g_const["rot_542"])
    assert np.array_equal(rotation.random_rotation_dense(64, np.random.default_rng(42)), g_const["rot_d64_42"])
    for b in (1, 2, 3, 4):
        assert np.array_equal(codebook.optimal_centroids(b, 128), g_const[f"centroids_b{b}"])


def test_known_answers():
    # closed forms (reference: tests/test_codebook.py:12-31)
    c1 = codebook.optimal_centroids(1, 128)
    assert np.allclose(c1, [-np.sqrt(2 / (np.pi * 128)), np.sqrt(2 / (np.pi * 128))], atol=1e-10)
    assert np.allclose(codebook.optimal_centroids(2, 64) * 8, [-1.51, -0.453, 0.453, 1.51])
    assert abs(codebook._gaussian_conditional_expectation(1.0, 0, np.inf) - np.sqrt(2 / np.pi)) < 1e-12
    h = rotation.hadamard_matrix(16)
    assert np.array_equal(h @ h.T, 16 * np.eye(16))
    r = rotation.random_rotation_dense(32, np.random.default_rng(0))
    assert np.abs(r @ r.T - np.eye(32)).max() < 1e-10 and abs(np.linalg.det(r) - 1) < 1e-10
    s1, s2, n = rotation.random_rotation_fast(100, np.random.default_rng(0))
    assert n == 128 and set(np.unique(s1)) <= {-1.0, 1.0}
    m = rotation.fast_rotation_matrix(*rotation.random_rotation_fast(64, np.random.default_rng(3))[:2])
    assert np.abs(m @ m.T - np.eye(64)).max() < 1e-12


def test_errors_and_sizes(g_prim, g_kv):
    with pytest.raises(ValueError):
        rotation.random_rotation_dense(0, np.random.default_rng(0))
    with pytest.raises(ValueError):
        rotation.hadamard_matrix(12)
    with pytest.raises(ValueError):
        tq.TurboQuant(128, 1)
    with pytest.raises(ValueError):
        tq.PolarQuant(128, 3, rotation="fft")
    t = tq.TurboQuant(128, 3)
    assert t.compressed_size_bits(100) == 100 * (128 * 3 + 32)
    assert t.compression_ratio() == 128 * 16 / (128 * 3 + 32)
    fp = utils.memory_footprint_bytes(1000, 128, 3)
    assert [fp[k] for k in sorted(fp)] == list(g_prim["footprint_vals"])
    st = tq.KVCacheCompressor(128).memory_stats(1024, 32, 32)
    assert [st[k] for k in sorted(st)] == list(g_kv["stats_vals"])
    assert st["compression_ratio"] > 2.0


def test_no_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        tq.PolarQuant(128, 3).quantize(np.zeros((2, 128), np.float32))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        utils.pack_bits(np.ones(8, np.int8))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        tq.PagedKVCache(128, 8, 4)
