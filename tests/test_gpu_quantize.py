"""CUDA quantize / dequantize against the golden fixtures and the NumPy oracle (through the C ABI)."""
import numpy as np
import pytest

from oracle import tq_oracle as o
from tests.helpers import D, boundary_band, check_indices, wht_dense

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tq():
    import turboquant_plus_b200 as pkg
    return pkg


def _rot(g_const, mode, seed):
    return g_const[f"rot_{seed}"] if mode == "dense" else wht_dense(g_const, seed)


@pytest.mark.parametrize("mode", ["dense", "wht"])
@pytest.mark.parametrize("b", [2, 3, 4])
def test_polar_golden(tq, g_const, g_polar, mode, b):
    x = g_polar["x"]
    q = tq.TurboQuantMSE(D, b, seed=42, rotation=mode)
    assert np.array_equal(q.polar_quant.rotation, _rot(g_const, mode, 42))
    assert np.array_equal(q.polar_quant.centroids, g_const[f"centroids_b{b}"])
    idx, nrm = q.quantize(x)
    tag = f"{mode}_b{b}"
    ref_idx, ref_nrm = g_polar[f"{tag}_idx"], g_polar[f"{tag}_norms"]
    assert idx.dtype == np.int64 and nrm.dtype == np.float32
    _, _, y = o.polar_quantize(x, q.polar_quant.rotation, q.polar_quant.centroids, return_rotated=True)
    mism, band = check_indices(idx, ref_idx, y, q.polar_quant.centroids)
    print(f"{tag}: {mism} index mismatches, {band} coordinates inside the boundary band, of {idx.size}")
    # norms within 1e-6 relative; row 6 has squares in the fp32 subnormal range, where the reference's own
    # fp32 sum of squares is only good to ~1e-3
    ok = np.ones(len(x), bool)
    ok[6] = False
    assert np.allclose(nrm[ok], ref_nrm[ok], rtol=1e-6, atol=0)
    assert np.allclose(nrm[6], ref_nrm[6], rtol=2e-2)
    assert nrm[5] == 0.0
    # packed stream = the reference's pack_indices of the same indices
    import torch
    out = q.polar_quant.quantize_device(torch.as_tensor(x).cuda(), packed=True, want_scale=True)
    assert np.array_equal(out["packed"].cpu().numpy().ravel(), o.pack_idx(idx, b))
    if mism == 0:
        assert np.array_equal(out["packed"].cpu().numpy().ravel(), g_polar[f"{tag}_packed"])
    cn = np.linalg.norm(q.polar_quant.centroids[idx], axis=1)
    assert np.allclose(out["scale"].cpu().numpy()[ok], (nrm / np.where(cn > 1e-10, cn, 1))[ok], rtol=2e-6)
    # dequantize (from the reference's indices, so that near-boundary flips do not enter)
    deq = q.dequantize(ref_idx.astype(np.int64), ref_nrm)
    ref = g_polar[f"{tag}_deq"]
    tol = 1e-12 if mode == "dense" else 2e-6
    scale = np.maximum(np.abs(ref).max(axis=1, keepdims=True), 1e-300)
    assert (np.abs(deq - ref) / scale).max() < tol
    qn = tq.TurboQuantMSE(D, b, seed=42, rotation=mode, norm_correction=False)
    deq = qn.dequantize(ref_idx.astype(np.int64), ref_nrm)
    assert (np.abs(deq - g_polar[f"{tag}_deq_nonc"]) / scale).max() < tol
    # packed dequantize path
    dq = q.polar_quant.dequantize_device(out["norm"], packed=out["packed"]).cpu().numpy()
    assert (np.abs(dq - q.dequantize(idx, nrm)) / scale).max() < 1e-6


def test_single_vector_convention(tq, g_polar):
    q = tq.PolarQuant(D, 3, seed=42)
    i1, n1 = q.quantize(g_polar["x"][0])
    assert i1.shape == (D,) and np.shape(n1) == ()
    assert np.array_equal(i1, g_polar["single_idx"]) and n1 == g_polar["single_norm"]
    x1 = q.dequantize(i1, n1)
    assert x1.shape == (D,) and np.abs(x1 - g_polar["single_deq"]).max() < 1e-12 * np.abs(x1).max()


@pytest.mark.parametrize("mode", ["dense", "wht"])
@pytest.mark.parametrize("b", [2, 3, 4])
def test_prod_golden(tq, g_const, g_prod, mode, b):
    x = g_prod["x"]
    t = tq.TurboQuant(D, b, seed=42, rotation=mode)
    assert np.array_equal(t.qjl.S, g_const["qjl_1042"] if mode == "dense" else wht_dense(g_const, 1042))
    c = t.quantize(x)
    tag = f"{mode}_b{b}"
    cb = t.polar_quant.centroids
    _, _, y = o.polar_quantize(x, t.polar_quant.rotation, cb, return_rotated=True)
    mism, _ = check_indices(c.mse_indices, g_prod[f"{tag}_idx"], y, cb)
    assert c.qjl_signs.dtype == np.int8 and set(np.unique(c.qjl_signs)) <= {-1, 1}
    ref_signs = o.unpack_signs(g_prod[f"{tag}_signs"], D)
    rows_ok = (c.mse_indices == g_prod[f"{tag}_idx"]).all(axis=1)
    rows_ok[6] = False            # subnormal squares, see test_polar_golden
    flips = (c.qjl_signs != ref_signs)[rows_ok]
    # a sign may differ only where the projected residual is within rounding of zero
    _, _, res = o.polar_residual(x, t.polar_quant.rotation, cb)
    proj = (t.qjl.S @ res.T).T
    rel = np.abs(proj) / np.maximum(np.linalg.norm(res, axis=1, keepdims=True), 1e-300)
    assert (rel[rows_ok][flips] < 1e-5).all()
    print(f"{tag}: {mism} index mismatches, {int(flips.sum())} sign flips near zero of {flips.size}")
    if mode == "dense":
        assert flips.sum() == 0
    assert (c.qjl_signs[5] == 1).all() and c.residual_norms[5] == 0.0
    assert np.allclose(c.residual_norms[rows_ok], g_prod[f"{tag}_rnorms"][rows_ok], rtol=1e-5 if mode == "wht" else 1e-6)
    ref_code = o.ProdCode(g_prod[f"{tag}_idx"].astype(np.int64), g_prod[f"{tag}_norms"], ref_signs,
                          g_prod[f"{tag}_rnorms"], b)
    import dataclasses
    cv = tq.CompressedVector(**dataclasses.asdict(ref_code))
    ref = g_prod[f"{tag}_deq"]
    scale = np.maximum(np.abs(ref).max(axis=1, keepdims=True), 1e-300)
    tol = 1e-7 if mode == "dense" else 3e-6      # norms travel as fp32
    assert (np.abs(t.dequantize(cv) - ref) / scale).max() < tol
    assert (np.abs(t.dequantize(cv, shrinkage=2 / np.pi) - g_prod[f"{tag}_deq_shrink"]) / scale).max() < tol
    assert t.compressed_size_bits(100) == 100 * (128 * b + 32)


@pytest.mark.parametrize("target_bits", [2.5, 3.5, 3.25])
def test_outlier_golden(tq, g_outlier, target_bits):
    """OutlierTurboQuant (turboquant/outlier.py) against the fixture made by running the reference: same split, the
    indices of both channel groups (equal outside the boundary band), norms to 1e-6, sign sketch of the whole residual
    (a sign may differ only where the projection is within rounding of zero), reconstruction from the reference's own
    code and from ours."""
    g, tag = g_outlier, f"t{int(round(target_bits * 100))}"
    x = g["x"]
    oq = tq.OutlierTurboQuant(D, target_bits, seed=42)
    orc = o.OutlierOracle(D, target_bits, seed=42)
    assert [oq.n_outlier, oq.high_bits, oq.n_normal, oq.low_bits] == g[f"{tag}_split"].tolist()
    assert oq.effective_bits == float(g[f"{tag}_effective_bits"]) and oq.compression_ratio() == float(g[f"{tag}_ratio"])
    c = oq.quantize(x)
    assert c.effective_bits == oq.effective_bits
    rows_ok = np.ones(len(x), dtype=bool)
    for name, sl, rot, cb in (("outlier", slice(0, oq.n_outlier), orc.r_out, orc.c_out),
                              ("normal", slice(oq.n_outlier, D), orc.r_norm, orc.c_norm)):
        idx, nrm = getattr(c, name + "_indices"), getattr(c, name + "_norms")
        _, _, y = o.polar_quantize(np.ascontiguousarray(x[:, sl]), rot, cb, return_rotated=True)
        mism, _ = check_indices(idx, g[f"{tag}_{name}_idx"], y, cb)
        assert idx.dtype == np.int64 and nrm.dtype == np.float64
        assert np.allclose(nrm, g[f"{tag}_{name}_norms"], rtol=1e-6, atol=0)
        rows_ok &= (idx == g[f"{tag}_{name}_idx"]).all(axis=1)
        assert np.array_equal(pq_rotation(oq, name), rot)
    ref_signs = o.unpack_signs(g[f"{tag}_signs"], D)
    assert c.qjl_signs.dtype == np.int8 and set(np.unique(c.qjl_signs)) <= {-1, 1}
    flips = (c.qjl_signs != ref_signs)[rows_ok]
    assert flips.sum() == 0, f"{int(flips.sum())} sign flips"
    assert (c.qjl_signs[7] == 1).all() and c.residual_norms[7] == 0.0          # the zero vector
    assert np.allclose(c.residual_norms[rows_ok], g[f"{tag}_rnorms"][rows_ok], rtol=1e-6)
    ref = g[f"{tag}_deq"]
    scale = np.maximum(np.abs(ref).max(axis=1, keepdims=True), 1e-300)
    ref_code = tq.OutlierCompressedVector(
        outlier_indices=g[f"{tag}_outlier_idx"].astype(np.int64), outlier_norms=g[f"{tag}_outlier_norms"],
        normal_indices=g[f"{tag}_normal_idx"].astype(np.int64), normal_norms=g[f"{tag}_normal_norms"],
        qjl_signs=ref_signs, residual_norms=g[f"{tag}_rnorms"], effective_bits=oq.effective_bits)
    assert (np.abs(oq.dequantize(ref_code) - ref) / scale).max() < 1e-7        # norms travel as fp32
    assert (np.abs(oq.dequantize(c) - ref)[rows_ok] / scale[rows_ok]).max() < 1e-6
    # single-vector convention (turboquant/outlier.py:152-165) and batch == single (tests/test_outlier.py:82-97)
    c1 = oq.quantize(x[3])
    assert c1.qjl_signs.shape == (D,) and np.shape(c1.residual_norms) == () and c1.outlier_indices.shape == (oq.n_outlier,)
    x1 = oq.dequantize(c1)
    assert x1.shape == (D,) and np.abs(x1 - g[f"{tag}_single_deq"]).max() < 1e-6 * np.abs(x1).max()
    assert np.abs(x1 - oq.dequantize(c)[3]).max() < 1e-10 * np.abs(x1).max()


def pq_rotation(oq, name):
    return getattr(oq, "pq_" + name).rotation


def test_outlier_quality_and_device_path(tq):
    """Round-trip quality as the reference tests it (tests/test_outlier.py:30-48: 3.5 bits on unit vectors, mean MSE
    below twice the 3-bit bound), an integer rate (no outlier group) and CUDA tensors in and out, fp32 input."""
    import torch
    rng = np.random.default_rng(99)
    x = rng.standard_normal((200, D))
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    oq = tq.OutlierTurboQuant(D, 3.5, seed=42)
    mse = np.mean((x - oq.dequantize(oq.quantize(x))) ** 2)
    assert mse < 0.03 * 2.0
    orc = o.OutlierOracle(D, 3.5, seed=42)
    assert abs(mse - np.mean((x - orc.dequantize(orc.quantize(x))) ** 2)) < 1e-9
    whole = tq.OutlierTurboQuant(D, 3.0, seed=42)
    assert whole.n_outlier == 0 and whole.pq_outlier is None
    cw = whole.quantize(x)
    assert cw.outlier_indices.size == 0
    ow = o.OutlierOracle(D, 3.0, seed=42)
    assert np.abs(whole.dequantize(cw) - ow.dequantize(ow.quantize(x))).max() < 1e-6
    xt = torch.as_tensor(x, dtype=torch.float32).cuda()
    ct = oq.quantize(xt)
    assert ct.qjl_signs.is_cuda and ct.outlier_indices.dtype == torch.uint8
    back = oq.dequantize(ct)
    assert back.is_cuda and back.dtype == torch.float64
    ref32 = orc.dequantize(orc.quantize(x.astype(np.float32).astype(np.float64)))
    rows = (ct.outlier_indices.cpu().numpy() == orc.quantize(x.astype(np.float32).astype(np.float64))["outlier_indices"]).all(axis=1)
    assert rows.mean() > 0.9 and np.abs(back.cpu().numpy() - ref32)[rows].max() < 1e-5


def test_polar_residual_fused(tq, g_polar):
    """PolarQuant.quantize_and_residual (turboquant/polar_quant.py:121-132), dense mode, in one launch."""
    x = g_polar["x"].astype(np.float64)
    q = tq.PolarQuant(D, 3, seed=42)
    idx, nrm, res = q.quantize_and_residual(x)
    ri, rn, rr = o.polar_residual(x, q.rotation, q.centroids)
    rows = (idx == ri).all(axis=1)
    assert rows.mean() > 0.9 and np.allclose(nrm, rn, rtol=1e-6)
    # norms are carried in fp32 (6e-8 relative): against the reference's residual, taken with its fp64 norm, that
    # much of x_hat remains; against x - dequantize(indices, returned norms), the reference's definition, nothing
    assert np.abs(res - rr)[rows].max() < 2e-7 * np.abs(x).max()
    assert np.abs(res - (x - q.dequantize(idx, nrm))).max() < 1e-12 * np.abs(x).max()
    i1, n1, r1 = q.quantize_and_residual(x[2])
    assert i1.shape == (D,) and np.shape(n1) == () and np.abs(r1 - rr[2]).max() < 2e-7 * np.abs(x).max()


def test_temporal_decay_golden(tq, g_decay):
    """tq_requantize against the fixture made by running requantize_3to2 of the reference's
    benchmarks/temporal_decay_prototype.py (its constants as the two codebooks): 2-bit indices equal except where the
    renormalised value is within the boundary band of a midpoint, corrected norms to 1e-6; then the device path
    (packed stream and scale straight from quantize_device) against the same restatement, and the argument checks."""
    import torch
    from turboquant_plus_b200 import temporal_decay as td
    g = g_decay
    src = tq.PolarQuant(D, 3, seed=42, rotation="wht", centroids=g["c3"])
    dst = tq.PolarQuant(D, 2, seed=42, rotation="wht", centroids=g["c2"])
    idx2, corrected = td.requantize(src, dst, g["idx3"], g["norms"])
    unit = g["c3"][g["idx3"]] / np.linalg.norm(g["c3"][g["idx3"]], axis=1, keepdims=True)
    unit[9] = 0.0
    mism, _ = check_indices(idx2, g["idx2"], unit, g["c2"])
    rows = (idx2 == g["idx2"]).all(axis=1)
    assert rows.mean() > 0.9 and np.allclose(corrected[rows], g["corrected"][rows], rtol=1e-6, atol=0)
    assert corrected[9] == 0.0
    i1, c1 = td.requantize(src, dst, g["idx3"][5], g["norms"][5])
    assert i1.shape == (D,) and np.array_equal(i1, idx2[5]) and c1 == corrected[5]
    # device path with the Lloyd-Max codebooks, 4 -> 3, 4 -> 2, 3 -> 2, 3 -> 1 bits
    x = torch.as_tensor(o.synth_keys(4099, seed=3)).cuda().half()
    for bs, bd in ((4, 3), (4, 2), (3, 2), (3, 1), (2, 2)):
        a = tq.PolarQuant(D, bs, seed=42, rotation="wht")
        b = tq.PolarQuant(D, bd, seed=42, rotation="wht")
        code = a.quantize_device(x, packed=True, want_scale=True)
        out = td.requantize_device(a, b, code["packed"], code["scale"])
        ia = o.unpack_idx(code["packed"].cpu().numpy().reshape(-1), bs, len(x) * D).reshape(-1, D)
        ib = o.unpack_idx(out["packed"].cpu().numpy().reshape(-1), bd, len(x) * D).reshape(-1, D)
        sc, new_scale, new_norm = code["scale"].cpu().numpy(), out["scale"].cpu().numpy(), out["norm"].cpu().numpy()
        mid = o.boundaries(b.centroids)
        bad = 0
        for r in range(0, len(ia), 41):
            nrm = sc[r] * np.linalg.norm(a.centroids[ia[r]])
            want_idx, want_scale = o.decay_requantize(ia[r], nrm, a.centroids, b.centroids, mid)
            u = a.centroids[ia[r]] / np.linalg.norm(a.centroids[ia[r]])
            near = np.abs(u[:, None] - mid).min(axis=1) <= boundary_band(b.centroids)
            assert (ib[r] == want_idx)[~near].all()
            if (ib[r] == want_idx).all():
                assert abs(new_scale[r] - want_scale) <= 2e-6 * want_scale and abs(new_norm[r] - nrm) <= 2e-6 * nrm
            else:
                bad += 1
        assert bad <= 2
        # the narrower code still points the same way: cosine with the source reconstruction
        ya, yb = a.centroids[ia] * sc[:, None], b.centroids[ib] * new_scale[:, None]
        cos = (ya * yb).sum(1) / np.maximum(np.linalg.norm(ya, axis=1) * np.linalg.norm(yb, axis=1), 1e-30)
        print(f"{bs} -> {bd} bits: mean cosine {cos.mean():.4f}")
        assert cos.mean() > {1: 0.78, 2: 0.93, 3: 0.98}[bd]
    other = tq.PolarQuant(D, 2, seed=43, rotation="wht")
    with pytest.raises(ValueError):
        td.requantize_device(a, other, code["packed"], code["scale"])
    with pytest.raises(ValueError):
        td.requantize_device(b, tq.PolarQuant(D, 3, seed=42, rotation="wht"), out["packed"], out["scale"])


def test_qjl_golden(tq, g_const, g_qjl):
    qj = tq.QJL(D, seed=123)
    assert np.array_equal(qj.S, g_const["qjl_123"])
    z, n = qj.quantize(g_qjl["r"])
    assert np.array_equal(o.pack_signs(z), g_qjl["signs"])
    assert np.allclose(n, g_qjl["norms"], rtol=1e-7) and n[4] == 0 and (z[4] == 1).all()
    assert np.abs(qj.dequantize(z, g_qjl["norms"]) - g_qjl["deq"]).max() < 1e-7 * np.abs(g_qjl["deq"]).max()
    assert np.abs(qj.dequantize(z, g_qjl["norms"], shrinkage=0.5) - g_qjl["deq_shrink"]).max() < 1e-7
    z1, n1 = qj.quantize(g_qjl["r"][0])
    assert z1.shape == (D,) and np.shape(n1) == ()


def test_primitives_golden(tq, g_prim, g_const):
    from turboquant_plus_b200 import codebook, rotation, utils
    p = g_prim
    assert np.array_equal(rotation.fast_walsh_hadamard_transform(p["fwht_in"]), p["fwht_out"])
    s1, s2 = p["fast_s1"], p["fast_s2"]
    assert np.array_equal(rotation.apply_fast_rotation(p["fast_x"], s1, s2, 128), p["fast_y"])
    assert np.array_equal(rotation.apply_fast_rotation_transpose(p["fast_x"], s1, s2, 128), p["fast_yT"])
    assert np.array_equal(rotation.apply_fast_rotation_batch(p["fast_xb"], s1, s2, 128), p["fast_yb"])
    with pytest.raises(ValueError):
        rotation.fast_walsh_hadamard_transform(np.ones(12))
    assert np.array_equal(codebook.nearest_centroid_indices(p["nci_vals"], g_const["centroids_b3"]).astype(np.uint8),
                          p["nci_idx"])
    c2 = g_const["centroids_b2"]
    assert list(codebook.nearest_centroid_indices(o.boundaries(c2), c2)) == [0, 1, 2]      # ties go down
    assert np.array_equal(utils.pack_bits(p["bits_in"]), p["bits_packed"])
    assert np.array_equal(utils.pack_bits(p["bits_in1"]), p["bits_packed1"])
    assert np.array_equal(utils.unpack_bits(p["bits_packed"], 21), p["bits_unpacked"])
    for b in (1, 2, 3, 4, 6):
        idx = p["idx_in"] % (1 << b)
        packed = utils.pack_indices(idx, b)
        assert np.array_equal(packed, p[f"idx_packed_b{b}"])
        if b <= 4:
            assert np.array_equal(utils.unpack_indices(packed, b, idx.size), idx.ravel())
    with pytest.raises(ValueError):
        utils.pack_indices(p["idx_in"], 9)
    assert utils.pack_indices(np.zeros((0, 128), np.uint8), 3).size == 0      # empty input


@pytest.mark.parametrize("mode", ["wht", "dense"])
def test_config0_full_size(tq, mode):
    """65,536 synthetic key vectors (N(0,1) x lognormal scale, 4 outlier channels x10, seed 0), b = 2, 3, 4:
    indices against the oracle, MSE and inner-product distortion against 4,096 N(0,1) queries."""
    x = o.synth_keys(65536, seed=0)
    qv = np.random.default_rng(1).standard_normal((4096, D))
    for b in (2, 3, 4):
        q = tq.TurboQuantMSE(D, b, seed=42, rotation=mode)
        rot, cb = q.polar_quant.rotation, q.polar_quant.centroids
        ref_idx, ref_nrm, y = o.polar_quantize(x, rot, cb, return_rotated=True)
        idx, nrm = q.quantize(x)
        mism, band = check_indices(idx, ref_idx, y, cb)
        assert np.allclose(nrm, ref_nrm, rtol=1e-6, atol=0)
        xh = q.dequantize(idx, nrm)
        xr = o.polar_dequantize(ref_idx, ref_nrm, rot, cb)
        mse, mse_ref = np.mean((x - xh) ** 2), np.mean((x - xr) ** 2)
        ip = np.mean((qv @ (x[:4096] - xh[:4096]).T) ** 2)
        ip_ref = np.mean((qv @ (x[:4096] - xr[:4096]).T) ** 2)
        print(f"{mode} turbo{b}: {mism} index mismatches / {band} in band of {idx.size}; "
              f"MSE {mse:.6f} (oracle {mse_ref:.6f}); IP distortion {ip:.5f} (oracle {ip_ref:.5f})")
        assert abs(mse / mse_ref - 1) < 1e-4 and abs(ip / ip_ref - 1) < 1e-3
    # prod, 3 bits, on a slice (the oracle needs three fp64 GEMMs per vector)
    xs = x[:16384]
    t = tq.TurboQuant(D, 3, seed=42, rotation=mode)
    c = t.quantize(xs)
    ref = o.prod_quantize(xs, t.polar_quant.rotation, t.polar_quant.centroids, t.qjl.S, 3)
    rows = (c.mse_indices == ref.mse_indices).all(axis=1)
    flips = int((c.qjl_signs != ref.qjl_signs)[rows].sum())
    print(f"{mode} prod3: {int((~rows).sum())} rows with an index mismatch, {flips} sign flips of {rows.sum() * D}")
    assert (~rows).sum() <= 8 and flips <= 32
    assert np.allclose(c.residual_norms[rows], ref.residual_norms[rows], rtol=2e-5)


def test_reference_style_behaviour(tq):
    """Cases the reference's own tests pin (tests/test_polar_quant.py, test_turbo4.py, test_turboquant.py):
    batch equals single, determinism, zero vector, odd head dimensions, MSE bound, bad bit width."""
    rng = np.random.default_rng(7)
    for d in (64, 96, 128, 200):
        q = tq.PolarQuant(d, 3, seed=42)
        xb = rng.standard_normal((6, d))
        ib, nb = q.quantize(xb)
        for r in range(6):
            i1, n1 = q.quantize(xb[r])
            assert np.array_equal(i1, ib[r]) and n1 == nb[r]
        assert np.array_equal(q.quantize(xb)[0], ib)
        i0, n0 = q.quantize(np.zeros(d))
        assert n0 == 0.0 and np.abs(q.dequantize(i0, n0)).max() == 0.0
        u = xb / np.linalg.norm(xb, axis=1, keepdims=True)
        uh = q.dequantize(*q.quantize(u))
        assert np.mean(np.sum((u - uh) ** 2, axis=1)) < 3 * 0.03       # paper bound for 3 bits, 3x slack
    with pytest.raises(ValueError):
        tq.TurboQuant(128, 1)
    t = tq.TurboQuant(64, 3, seed=1)
    xb = rng.standard_normal((5, 64))
    c = t.quantize(xb)
    assert c.mse_indices.shape == (5, 64) and c.mse_indices.max() < 4 and c.bit_width == 3
    c1 = t.quantize(xb[2])
    assert np.array_equal(c1.mse_indices, c.mse_indices[2]) and np.array_equal(c1.qjl_signs, c.qjl_signs[2])
    assert np.allclose(t.dequantize(c1), t.dequantize(c)[2])


def test_kv_compressor_matches_reference(tq, g_kv):
    comp = tq.KVCacheCompressor(D, k_bits=3, v_bits=3, seed=42)
    cc = comp.compress(g_kv["k"], g_kv["v"])
    assert (cc.num_layers, cc.num_heads, cc.seq_len, cc.head_dim, cc.k_bit_width, cc.v_bit_width) == (1, 2, 200, D, 3, 3)
    assert len(cc.k_compressed) == 1 and len(cc.k_compressed[0]) == 2 and cc.v_indices[0][1].shape == (200, D)
    kh, vh = comp.decompress(cc)
    assert kh.shape == g_kv["k"].shape
    assert np.abs(kh - g_kv["dense_prod_k_hat"]).max() < 2e-5 * np.abs(kh).max()
    assert np.abs(vh - g_kv["dense_prod_v_hat"]).max() < 2e-5 * np.abs(vh).max()
    st = comp.memory_stats(1024, 32, 32)
    assert [st[k] for k in sorted(st)] == list(g_kv["stats_vals"])
    with pytest.raises(AssertionError):
        comp.compress(np.zeros((1, 1, 4, 64)), np.zeros((1, 1, 4, 64)))


@pytest.mark.parametrize("b", [3, 4])
def test_prod_packed_path_matches_unpacked(tq, b):
    """PROD quantization with packed output (the tensor-core kernel with its QJL stage, what a cache append runs)
    against the same call with unpacked output (the butterfly kernel, which the golden vectors pin): indices, norms,
    residual norms and sketch bits, for fp32, fp16 and bf16 rows, a zero vector among them."""
    import torch
    from turboquant_plus_b200 import utils
    x = o.synth_keys(8192, seed=11).astype(np.float32)
    x[5] = 0.0
    t = tq.TurboQuant(D, b, seed=42, rotation="wht")
    for dt in (torch.float32, torch.float16, torch.bfloat16):
        xt = torch.as_tensor(x).cuda().to(dt)
        fast = t.quantize_device(xt, packed=True, want_scale=True)
        ref = t.quantize_device(xt.float(), packed=False, want_scale=True)
        ref_packed = utils.pack_indices(ref["idx"].cpu().numpy(), b - 1)
        rows = (fast["packed"].cpu().numpy() == ref_packed.reshape(len(x), -1)).all(axis=1)
        flips = int(np.unpackbits(fast["qjl"].cpu().numpy()[rows] ^ ref["qjl"].cpu().numpy()[rows]).sum())
        print(f"prod{b} {dt}: {int((~rows).sum())} rows with an index mismatch, {flips} sketch bits differ of {rows.sum() * D}")
        assert (~rows).sum() <= 4 and flips <= 16
        for key, tol in (("norm", 1e-6), ("scale", 2e-6), ("rnorm", 2e-5)):
            torch.testing.assert_close(fast[key][torch.as_tensor(rows).cuda()], ref[key][torch.as_tensor(rows).cuda()],
                                       rtol=tol, atol=0)
        assert rows[5] and (fast["qjl"][5] == 0xFF).all() and float(fast["rnorm"][5]) == 0.0


def test_input_dtypes_and_errors(tq):
    import torch
    x = o.synth_keys(1000, seed=5)
    q = tq.PolarQuant(D, 3, seed=42, rotation="wht")
    a = q.quantize_device(torch.as_tensor(x).cuda(), packed=True)
    h = q.quantize_device(torch.as_tensor(x).cuda().half().float(), packed=True)
    h16 = q.quantize_device(torch.as_tensor(x).cuda().half(), packed=True)
    b16 = q.quantize_device(torch.as_tensor(x).cuda().bfloat16(), packed=True)
    b32 = q.quantize_device(torch.as_tensor(x).cuda().bfloat16().float(), packed=True)
    # 16-bit rows go through the tensor-core Hadamard as they are, fp32 rows as three exact bf16 terms: the same
    # values up to fp32 rounding, so indices may differ only for coordinates that sit on a decision boundary
    for lo, hi in ((h, h16), (b32, b16)):
        differ = (lo["packed"] != hi["packed"]).any(dim=1).sum().item()
        assert differ <= 2, differ
        torch.testing.assert_close(lo["norm"], hi["norm"], rtol=1e-6, atol=0)
    assert a["packed"].shape == (1000, 48)
    with pytest.raises(ValueError):
        q.quantize(np.zeros((3, 64)))
    with pytest.raises(ValueError):
        tq.PolarQuant(96, 3, rotation="wht")
    # n not a multiple of the 4 vectors a warp handles
    for n in (1, 2, 3, 5, 33):
        r = q.quantize_device(torch.as_tensor(x[:n]).cuda(), packed=True)
        assert torch.equal(r["packed"], a["packed"][:n]) and torch.equal(r["norm"], a["norm"][:n])
