"""Generate the golden fixtures in this folder by RUNNING the reference.

Usage (only where the reference tree is present):

    python tests/golden/make_golden.py [/path/to/reference]

It imports the reference package ``turboquant`` unmodified, feeds it small seeded inputs
and stores inputs, exported constants (rotation matrices, sign vectors, QJL matrix,
codebooks) and outputs as ``.npz`` files.  The tests compare both the NumPy oracle and the
CUDA path with these files; nothing at test time needs the reference tree.

WHT-mode fixtures use the reference classes with their ``rotation`` (and ``S``) attribute
overwritten by the dense form of D2 (H/sqrt d) D1 built from the reference's own
``random_rotation_fast`` and ``hadamard_matrix``; the quantize/dequantize code that runs is
still the reference's.
"""
import os
import sys

import numpy as np

# path of the reference checkout: argument, $TQ_REFERENCE, or a directory `reference` beside the repository
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get(
    "TQ_REFERENCE", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))), "reference"))
sys.path.insert(0, REF)

from turboquant import KVCacheCompressor, PolarQuant, QJL, TurboQuant, TurboQuantMSE  # noqa: E402
from turboquant.codebook import nearest_centroid_indices, optimal_centroids  # noqa: E402
from turboquant.rotation import (apply_fast_rotation, apply_fast_rotation_batch,  # noqa: E402
                                 apply_fast_rotation_transpose, fast_walsh_hadamard_transform,
                                 hadamard_matrix, random_rotation_dense, random_rotation_fast)
from turboquant.utils import memory_footprint_bytes, pack_bits, pack_indices, unpack_bits  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
D = 128


def keys(n, seed):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((n, D))
    x *= rng.lognormal(0.0, 0.5, size=(n, 1))
    ch = rng.choice(D, 4, replace=False)
    x[:, ch] *= 10.0
    return x.astype(np.float32)


def wht_dense(seed):
    s1, s2, pd = random_rotation_fast(D, np.random.default_rng(seed))
    m = (s2[:, None] * hadamard_matrix(pd) * s1[None, :]) / np.sqrt(pd)
    probe = np.random.default_rng(1).standard_normal((5, D))
    assert np.abs(apply_fast_rotation_batch(probe, s1, s2, pd) - probe @ m.T).max() < 1e-12
    return s1, s2, m


def main():
    out = {}
    # ---------------- constants ----------------
    const = {}
    for seed in (42, 542):
        const[f"rot_{seed}"] = PolarQuant(D, 3, seed=seed).rotation
    const["qjl_1042"] = TurboQuant(D, 3, seed=42).qjl.S
    const["qjl_123"] = QJL(D).S
    for seed in (42, 542, 1042):
        s1, s2, m = wht_dense(seed)
        const[f"wht_s1_{seed}"], const[f"wht_s2_{seed}"] = s1, s2
    for b in (1, 2, 3, 4):
        const[f"centroids_b{b}"] = optimal_centroids(b, D)
    for d in (64, 96):
        const[f"centroids_b3_d{d}"] = optimal_centroids(3, d)
    const["rot_d64_42"] = random_rotation_dense(64, np.random.default_rng(42))
    np.savez_compressed(os.path.join(HERE, "constants_d128.npz"), **const)

    # ---------------- PolarQuant / TurboQuantMSE ----------------
    x = keys(64, 7)
    x[5] = 0.0                    # zero vector
    x[6] *= 1e-20                 # tiny norm
    x[7] *= 1e12                  # huge norm
    pol = {"x": x}
    for mode in ("dense", "wht"):
        for b in (2, 3, 4):
            for nc in (True, False):
                q = TurboQuantMSE(D, b, seed=42, norm_correction=nc)
                if mode == "wht":
                    q.polar_quant.rotation = wht_dense(42)[2]
                idx, nrm = q.quantize(x)
                tag = f"{mode}_b{b}"
                if nc:
                    pol[f"{tag}_idx"] = idx.astype(np.uint8)
                    pol[f"{tag}_norms"] = nrm
                    pol[f"{tag}_packed"] = pack_indices(idx, b)
                    pol[f"{tag}_deq"] = q.dequantize(idx, nrm)
                else:
                    pol[f"{tag}_deq_nonc"] = q.dequantize(idx, nrm)
    # single-vector convention
    q = PolarQuant(D, 3, seed=42)
    i1, n1 = q.quantize(x[0])
    pol["single_idx"], pol["single_norm"] = i1.astype(np.uint8), np.asarray(n1)
    pol["single_deq"] = q.dequantize(i1, n1)
    np.savez_compressed(os.path.join(HERE, "polar_d128.npz"), **pol)

    # ---------------- TurboQuant (prod) ----------------
    prod = {"x": x}
    for mode in ("dense", "wht"):
        for b in (2, 3, 4):
            t = TurboQuant(D, b, seed=42)
            if mode == "wht":
                t.polar_quant.rotation = wht_dense(42)[2]
                t.qjl.S = wht_dense(1042)[2]
            c = t.quantize(x)
            tag = f"{mode}_b{b}"
            prod[f"{tag}_idx"] = c.mse_indices.astype(np.uint8)
            prod[f"{tag}_norms"] = c.vector_norms
            prod[f"{tag}_signs"] = pack_bits(c.qjl_signs)
            prod[f"{tag}_rnorms"] = c.residual_norms
            prod[f"{tag}_deq"] = t.dequantize(c)
            prod[f"{tag}_deq_shrink"] = t.dequantize(c, shrinkage=2 / np.pi)
            if b > 1:
                prod[f"{tag}_idx_packed"] = pack_indices(c.mse_indices, b - 1)
    prod["size_bits_100_b3"] = np.asarray(TurboQuant(D, 3).compressed_size_bits(100))
    prod["ratio_b3"] = np.asarray(TurboQuant(D, 3).compression_ratio())
    np.savez_compressed(os.path.join(HERE, "prod_d128.npz"), **prod)

    # ---------------- QJL alone ----------------
    r = np.random.default_rng(3).standard_normal((32, D))
    r[4] = 0.0
    qj = QJL(D, seed=123)
    z, g = qj.quantize(r)
    np.savez_compressed(os.path.join(HERE, "qjl_d128.npz"), r=r, signs=pack_bits(z), norms=g,
                        deq=qj.dequantize(z, g), deq_shrink=qj.dequantize(z, g, shrinkage=0.5))

    # ---------------- primitives ----------------
    rng = np.random.default_rng(11)
    v = rng.standard_normal(256)
    s1, s2, pd = random_rotation_fast(96, np.random.default_rng(5))   # padded case 96 -> 128
    xv = rng.standard_normal(96)
    xb = rng.standard_normal((9, 96))
    vals = rng.standard_normal(500) * 0.1
    sg = rng.choice([-1, 1], size=(6, 21)).astype(np.int8)
    ii = rng.integers(0, 8, size=(5, 128))
    prim = dict(
        fwht_in=v, fwht_out=fast_walsh_hadamard_transform(v),
        hadamard8=hadamard_matrix(8),
        fast_s1=s1, fast_s2=s2, fast_x=xv, fast_y=apply_fast_rotation(xv, s1, s2, pd),
        fast_yT=apply_fast_rotation_transpose(xv, s1, s2, pd),
        fast_xb=xb, fast_yb=apply_fast_rotation_batch(xb, s1, s2, pd),
        nci_vals=vals, nci_idx=nearest_centroid_indices(vals, optimal_centroids(3, D)).astype(np.uint8),
        bits_in=sg, bits_packed=pack_bits(sg), bits_unpacked=unpack_bits(pack_bits(sg), 21),
        bits_in1=sg[0], bits_packed1=pack_bits(sg[0]),
        idx_in=ii.astype(np.uint8),
    )
    for b in (1, 2, 3, 4, 6):
        prim[f"idx_packed_b{b}"] = pack_indices(ii % (1 << b), b)
    fp = memory_footprint_bytes(1000, D, 3)
    prim["footprint_keys"] = np.array(sorted(fp))
    prim["footprint_vals"] = np.array([fp[k] for k in sorted(fp)], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "primitives.npz"), **prim)

    # ---------------- KV cache + dequantize-then-attend ----------------
    def softmax(x):
        e = np.exp(x - np.max(x, axis=-1, keepdims=True))
        return e / np.sum(e, axis=-1, keepdims=True)

    rng = np.random.default_rng(21)
    L, H, S = 1, 2, 200
    G = 4
    kc = np.stack([keys(S, 100 + h) for h in range(H)])[None].astype(np.float32)
    vc = rng.standard_normal((L, H, S, D)).astype(np.float32)
    qh = rng.standard_normal((H * G, D)).astype(np.float16)
    kv = {"k": kc, "v": vc, "q": qh}
    for mode in ("dense", "wht"):
        for kk in ("prod", "mse"):
            comp = KVCacheCompressor(D, k_bits=3, v_bits=3, seed=42)
            if kk == "mse":          # "turbo3" cache type: K is 3-bit PolarQuant only
                comp.k_quantizer = TurboQuantMSE(D, 3, seed=42)
            if mode == "wht":
                comp.k_quantizer.polar_quant.rotation = wht_dense(42)[2]
                comp.v_quantizer.polar_quant.rotation = wht_dense(542)[2]
                if kk == "prod":
                    comp.k_quantizer.qjl.S = wht_dense(1042)[2]
            if kk == "prod":
                cc = comp.compress(kc, vc)
                k_hat, v_hat = comp.decompress(cc)
            else:
                k_hat = np.zeros(kc.shape)
                v_hat = np.zeros(vc.shape)
                for h in range(H):
                    k_hat[0, h] = comp.k_quantizer.dequantize(*comp.k_quantizer.quantize(kc[0, h]))
                    v_hat[0, h] = comp.v_quantizer.dequantize(*comp.v_quantizer.quantize(vc[0, h]))
            o = np.zeros((H * G, D))
            for h in range(H * G):
                sc = qh[h:h + 1].astype(np.float64) @ k_hat[0, h // G].T / np.sqrt(D)
                o[h] = (softmax(sc) @ v_hat[0, h // G])[0]
            if mode == "dense" and kk == "prod":
                kv["dense_prod_k_hat"] = k_hat.astype(np.float32)
                kv["dense_prod_v_hat"] = v_hat.astype(np.float32)
            kv[f"{mode}_{kk}_out"] = o
    st = KVCacheCompressor(D, 3, 3).memory_stats(1024, 32, 32)
    kv["stats_keys"] = np.array(sorted(st))
    kv["stats_vals"] = np.array([st[k] for k in sorted(st)], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "kv_attention.npz"), **kv)
    # ---------------- OutlierTurboQuant (fractional bit rates) ----------------
    from turboquant.outlier import OutlierTurboQuant
    xo = keys(48, 23).astype(np.float64)
    xo[7] = 0.0
    outl = {"x": xo}
    for tb in (2.5, 3.5, 3.25):
        oq = OutlierTurboQuant(D, tb, seed=42)
        c = oq.quantize(xo)
        tag = f"t{int(round(tb * 100))}"
        outl[f"{tag}_split"] = np.array([oq.n_outlier, oq.high_bits, oq.n_normal, oq.low_bits])
        outl[f"{tag}_outlier_idx"] = c.outlier_indices.astype(np.uint8)
        outl[f"{tag}_outlier_norms"] = c.outlier_norms
        outl[f"{tag}_normal_idx"] = c.normal_indices.astype(np.uint8)
        outl[f"{tag}_normal_norms"] = c.normal_norms
        outl[f"{tag}_signs"] = pack_bits(c.qjl_signs)
        outl[f"{tag}_rnorms"] = c.residual_norms
        outl[f"{tag}_deq"] = oq.dequantize(c)
        outl[f"{tag}_ratio"] = np.asarray(oq.compression_ratio())
        outl[f"{tag}_effective_bits"] = np.asarray(oq.effective_bits)
        c1 = oq.quantize(xo[3])
        outl[f"{tag}_single_deq"] = oq.dequantize(c1)
    np.savez_compressed(os.path.join(HERE, "outlier_d128.npz"), **outl)

    # ---------------- temporal decay prototype (3 -> 2 bits in the rotated domain) ----------------
    sys.path.insert(0, os.path.join(REF, "benchmarks"))
    import temporal_decay_prototype as tdp
    s1, s2, pd = random_rotation_fast(D, np.random.default_rng(42))
    xd = keys(64, 31)
    xd[9] = 0.0
    dec = {"x": xd, "c3": tdp.CENTROIDS_3BIT, "c2": tdp.CENTROIDS_2BIT, "mid3": tdp.MIDPOINTS_3BIT,
           "mid2": tdp.MIDPOINTS_2BIT, "idx3": np.zeros((64, D), np.uint8), "norms": np.zeros(64, np.float32),
           "idx2": np.zeros((64, D), np.uint8), "corrected": np.zeros(64), "deq3": np.zeros((64, D))}
    for i in range(64):
        nrm = np.linalg.norm(xd[i])
        rot = apply_fast_rotation(xd[i] / nrm if nrm > 0 else xd[i], s1, s2, pd)
        dec["idx3"][i] = tdp.quantize_3bit(rot)
        dec["norms"][i] = nrm
        dec["deq3"][i] = tdp.dequantize_3bit(dec["idx3"][i], nrm)
        dec["idx2"][i], dec["corrected"][i] = tdp.requantize_3to2(dec["idx3"][i], nrm)
    np.savez_compressed(os.path.join(HERE, "temporal_decay.npz"), **dec)

    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KB")


if __name__ == "__main__":
    main()
