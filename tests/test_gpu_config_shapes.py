"""Parity at the shapes the benchmark runs: decode attention of configurations 2 and 4, chunked prefill of
configuration 3 (128-query chunks x 64 query / 8 KV heads over 16,384 and 131,072 tokens), bf16 inputs, and values of
large norm.  The caches are filled at full size on the GPU; the oracle (dequantize, then attention in fp64) is run
on sampled sequences, heads and query rows so that the CPU side stays at seconds.

Tolerance as everywhere: max |out - ref| over a row / max |ref| of that row <= 2e-3 against the reference's
dequantize-then-attend (tests/test_kv_cache.py:73-89 of the reference).
"""
import numpy as np
import pytest

from oracle import tq_oracle as o
from tests.helpers import D, max_rel
from tests.test_gpu_attention import oracle_roundtrip

pytestmark = pytest.mark.gpu
TOL = 2e-3
PT = 128


@pytest.fixture(scope="module")
def tq():
    import turboquant_plus_b200 as pkg
    return pkg


def _keys(rng, n, hkv):
    """Keys of the benchmark's distribution: N(0,1) x lognormal(0, 0.5) per vector, 4 outlier channels x10, RoPE."""
    k = rng.standard_normal((n, hkv, D)).astype(np.float32)
    k *= np.exp(0.5 * rng.standard_normal((n, hkv, 1))).astype(np.float32)
    k[:, :, rng.permutation(D)[:4]] *= 10.0
    return np.stack([o.rope_rotate(k[:, h], np.arange(n)) for h in range(hkv)], axis=1).astype(np.float32)


def _fill(cache, bt_row, k, v):
    """Append one sequence's (n, hkv, d) rows at the pages of its block-table row."""
    import torch
    n = k.shape[0]
    t = np.arange(n)
    slots = bt_row[t // PT].astype(np.int64) * PT + t % PT
    cache.append(torch.as_tensor(k).to(cache.device), torch.as_tensor(v).to(cache.device), torch.as_tensor(slots))


def _ref_rows(cache, k, v, q_rows, heads, group, n_visible=None):
    """Oracle output for query heads `heads` (indices into the query-head axis) of one sequence.
    q_rows: (len(heads), d) fp64; attends over the first n_visible tokens (all when None)."""
    out = np.zeros((len(heads), D))
    cache_kv = {}
    for j, hq in enumerate(heads):
        h = hq // group
        if h not in cache_kv:
            cache_kv[h] = (oracle_roundtrip(cache, k[:, h], "k"), oracle_roundtrip(cache, v[:, h], "v"))
        kh, vh = cache_kv[h]
        n = kh.shape[0] if n_visible is None else n_visible
        out[j] = o.attend_one(q_rows[j][None], kh[:n], vh[:n])[0]
    return out


def test_config2_shape_layered_q8_0_turbo2(tq):
    """Configuration 2: batch 16 x context 8,192, 32 query / 8 KV heads, K q8_0; one boundary layer (V q8_0) and one
    inner layer (V turbo2) of a per-layer format table.  All heads of two sequences against the oracle."""
    import torch
    from turboquant_plus_b200.layered import LayeredKVCache, boundary_format_table
    rng = np.random.default_rng(202)
    batch, ctx, hkv, hq = 16, 8192, 8, 32
    formats = boundary_format_table(4, ("q8_0", "turbo2"), ("q8_0", "q8_0"), keep=1)
    assert formats[0] == ("q8_0", "q8_0") and formats[1] == ("q8_0", "turbo2")
    pages_per_seq = ctx // PT
    cache = LayeredKVCache(4, D, hkv, batch * pages_per_seq, PT, formats, seed=42)
    bt = rng.permutation(batch * pages_per_seq).astype(np.int32).reshape(batch, pages_per_seq)
    sampled = (3, 15)
    kept = {}
    for b in range(batch):
        k, v = _keys(rng, ctx, hkv), rng.standard_normal((ctx, hkv, D)).astype(np.float32)
        for layer in (0, 1):
            _fill(cache.layers[layer], bt[b], k, v)
        if b in sampled:
            kept[b] = (k, v)
    q = rng.standard_normal((batch, hq, D)).astype(np.float16)
    sl = torch.full((batch,), ctx, dtype=torch.int32)
    worst = 0.0
    for layer in (0, 1):
        lc = cache.layers[layer]
        out = lc.attend(torch.as_tensor(q).cuda().float(), torch.as_tensor(bt), sl).cpu().numpy()
        assert lc.kernel_status() == 0
        for b in sampled:
            ref = _ref_rows(lc, kept[b][0], kept[b][1], q[b].astype(np.float64), list(range(hq)), hq // hkv)
            err = max_rel(out[b], ref)
            print(f"config 2, layer {layer} ({lc.k_format}/{lc.v_format}), sequence {b}: max-rel {err:.2e}")
            worst = max(worst, err)
    assert worst < TOL


def test_config4_shape_ragged_prod3_turbo3(tq):
    """Configuration 4: batch 256, contexts uniform in [1,024, 32,768] (the benchmark's seeded lengths), K prod3
    (2-bit PolarQuant + QJL sketch), V turbo3, shuffled block table: the split plan takes its 32-page-chunk branch.
    Eight sequences (the shortest and the longest among them), two KV heads each, against the oracle."""
    import torch
    rng = np.random.default_rng(404)
    hkv, hq = 8, 32
    lens = np.random.default_rng(4).integers(1024, 32769, size=256).tolist()
    n_pages = [(n + PT - 1) // PT for n in lens]
    cache = tq.PagedKVCache(D, hkv, sum(n_pages), PT, "prod3", "turbo3", seed=42)
    perm = rng.permutation(sum(n_pages)).astype(np.int32)
    bt = np.zeros((256, max(n_pages)), dtype=np.int32)
    off = 0
    for b, npg in enumerate(n_pages):
        bt[b, :npg] = perm[off:off + npg]
        off += npg
    order = np.argsort(lens)
    sampled = [int(order[0]), int(order[-1])] + [int(x) for x in rng.choice(order[1:-1], 6, replace=False)]
    kept = {}
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    for b, n in enumerate(lens):
        if b in sampled:
            k, v = _keys(rng, n, hkv), rng.standard_normal((n, hkv, D)).astype(np.float32)
            kept[b] = (k, v)
            _fill(cache, bt[b], k, v)
        else:       # not compared: generated on the device
            k = torch.randn((n, hkv, D), generator=gen, device="cuda")
            k *= torch.exp(0.5 * torch.randn((n, hkv, 1), generator=gen, device="cuda"))
            v = torch.randn((n, hkv, D), generator=gen, device="cuda")
            t = np.arange(n)
            cache.append(k, v, torch.as_tensor(bt[b][t // PT].astype(np.int64) * PT + t % PT))
    q = rng.standard_normal((256, hq, D)).astype(np.float16)
    out = cache.attend(torch.as_tensor(q).cuda().float(), torch.as_tensor(bt), torch.tensor(lens)).cpu().numpy()
    assert cache.kernel_status() == 0 and np.isfinite(out).all()
    worst = 0.0
    for b in sampled:
        heads = [0, 1, 2, 3, 28, 29, 30, 31]        # KV heads 0 and 7
        ref = _ref_rows(cache, kept[b][0], kept[b][1], q[b, heads].astype(np.float64), heads, hq // hkv)
        err = max_rel(out[b, heads], ref)
        print(f"config 4, sequence {b} ({lens[b]} tokens): max-rel {err:.2e}")
        worst = max(worst, err)
    assert worst < TOL


@pytest.mark.parametrize("ctx", [16384, 131072])
def test_config3_shape_prefill_chunk(tq, ctx):
    """Configuration 3 / the benchmark's prefill probe: one 128-query chunk x 64 query / 8 KV heads (eight row blocks
    per KV head, the wave-aware split plan) over a turbo3 cache of 16,384 and of 131,072 tokens.  First, middle and
    last query of the chunk, all eight query heads of two KV heads, against the oracle over the visible prefix."""
    import torch
    rng = np.random.default_rng(303 + ctx)
    hkv, hq, chunk = 8, 64, 128
    cache = tq.PagedKVCache(D, hkv, ctx // PT, PT, "turbo3", "turbo3", seed=42)
    bt = rng.permutation(ctx // PT).astype(np.int32)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(ctx)
    check_heads = (1, 6)
    kept_k = np.zeros((ctx, hkv, D), dtype=np.float32)   # only the checked heads are kept on the host
    kept_v = np.zeros((ctx, hkv, D), dtype=np.float32)
    for lo in range(0, ctx, 16384):
        k = torch.randn((16384, hkv, D), generator=gen, device="cuda")
        k *= torch.exp(0.5 * torch.randn((16384, hkv, 1), generator=gen, device="cuda"))
        v = torch.randn((16384, hkv, D), generator=gen, device="cuda")
        t = np.arange(lo, lo + 16384)
        cache.append(k, v, torch.as_tensor(bt[t // PT].astype(np.int64) * PT + t % PT))
        for h in check_heads:
            kept_k[lo:lo + 16384, h] = k[:, h].cpu().numpy()
            kept_v[lo:lo + 16384, h] = v[:, h].cpu().numpy()
    q = rng.standard_normal((1, chunk, hq, D)).astype(np.float16)
    out = cache.prefill_attend(torch.as_tensor(q).cuda().float(), torch.as_tensor(bt[None]), torch.tensor([ctx]))
    out = out.cpu().numpy()
    assert cache.kernel_status() == 0 and np.isfinite(out).all()
    worst = 0.0
    g = hq // hkv
    for qi in (0, chunk // 2 - 1, chunk - 1):
        heads = [h * g + j for h in check_heads for j in range(g)]
        ref = _ref_rows(cache, kept_k, kept_v, q[0, qi, heads].astype(np.float64), heads, g, n_visible=ctx - chunk + qi + 1)
        err = max_rel(out[0, qi, heads], ref)
        print(f"prefill, ctx {ctx}, query {qi} of the chunk: max-rel {err:.2e}")
        worst = max(worst, err)
    assert worst < TOL
    # the chunk's last query sees the whole cache: decode attention must agree with it
    dec = cache.attend(torch.as_tensor(q[:, -1]).cuda().float(), torch.as_tensor(bt[None]), torch.tensor([ctx])).cpu().numpy()
    assert max_rel(out[:, -1].reshape(-1, D), dec.reshape(-1, D)) < TOL


def test_bf16_inputs_against_the_oracle(tq):
    """bf16 K / V / queries are defined as "upcast to fp32, then the reference path": append, quantize entry point and
    decode attention fed bf16 tensors against the oracle run on the upcast values."""
    import torch
    from tests.helpers import check_indices
    rng = np.random.default_rng(77)
    hkv, hq, n = 2, 8, 700
    k16 = torch.as_tensor(_keys(rng, n, hkv)).bfloat16()
    v16 = torch.as_tensor(rng.standard_normal((n, hkv, D)).astype(np.float32)).bfloat16()
    q16 = torch.as_tensor(rng.standard_normal((1, hq, D)).astype(np.float32)).bfloat16()
    k32, v32, q32 = k16.float().numpy(), v16.float().numpy(), q16.float().numpy()
    cache = tq.PagedKVCache(D, hkv, 8, PT, "turbo3", "turbo3", seed=42)
    bt = rng.permutation(8).astype(np.int32)
    t = np.arange(n)
    cache.append(k16.cuda(), v16.cuda(), torch.as_tensor(bt[t // PT].astype(np.int64) * PT + t % PT))
    out = cache.attend(q16.cuda(), torch.as_tensor(bt[None]), torch.tensor([n]))
    assert out.dtype == torch.bfloat16 and cache.kernel_status() == 0
    ref = _ref_rows(cache, k32, v32, q32[0].astype(np.float64), list(range(hq)), hq // hkv)
    err = max_rel(out[0].float().cpu().numpy(), ref)
    print(f"bf16 K/V/q, decode attention vs oracle on the upcast values: max-rel {err:.2e}")
    assert err < TOL + 4e-3          # the bf16 rounding of the output itself is 2^-9 = 2e-3 relative, worst element 4e-3
    out32 = cache.attend(q16.cuda().float(), torch.as_tensor(bt[None]), torch.tensor([n]))
    assert max_rel(out32[0].cpu().numpy(), ref) < TOL
    # the quantize entry point on bf16 rows: indices equal to the oracle's outside the boundary band, norms to 1e-6
    kq = cache.k_quantizer
    rows = k16.reshape(-1, D)
    got = kq.quantize_device(rows.cuda(), packed=False, want_scale=False)
    idx_ref, norm_ref, y = o.polar_quantize(rows.float().numpy(), kq.rotation, kq.centroids, return_rotated=True)
    mism, band = check_indices(got["idx"].cpu().numpy(), idx_ref, y, kq.centroids)
    print(f"bf16 quantize: {mism} index differences, all inside the band ({band} coordinates in the band)")
    assert np.allclose(got["norm"].cpu().numpy(), norm_ref, rtol=1e-6, atol=0)


def test_large_norm_values(tq):
    """Values whose norm is ~1e4 (the reference pins extreme norms for its quantizers: tests/test_turbo4.py:8,
    tests/test_polar_quant.py:45-68): the V scale meets the softmax weight in fp32 before the fp16 product, so the
    kernels must neither overflow nor lose the tolerance.  Decode (specialised and generic kernel) and prefill."""
    import torch
    rng = np.random.default_rng(88)
    hkv, n = 2, 1500
    k = _keys(rng, n, hkv)
    v = (rng.standard_normal((n, hkv, D)) * (1e4 / np.sqrt(D))).astype(np.float32)     # ||v|| ~ 1e4
    v[::7] *= 3.0
    for hq, kf in ((8, "turbo3"), (16, "turbo3"), (8, "prod3")):
        cache = tq.PagedKVCache(D, hkv, 12, PT, kf, "turbo3", seed=42)
        bt = rng.permutation(12).astype(np.int32)
        _fill(cache, bt, k, v)
        q = rng.standard_normal((1, hq, D)).astype(np.float32)
        out = cache.attend(torch.as_tensor(q).cuda(), torch.as_tensor(bt[None]), torch.tensor([n])).cpu().numpy()
        assert cache.kernel_status() == 0 and np.isfinite(out).all()
        ref = _ref_rows(cache, k, v, q[0].astype(np.float64), list(range(hq)), hq // hkv)
        err = max_rel(out[0], ref)
        print(f"||v|| ~ 1e4, {hq // hkv} query heads per KV head, K {kf}: max-rel {err:.2e}")
        assert err < TOL
        if kf == "turbo3":
            qc = rng.standard_normal((1, 16, hq, D)).astype(np.float32)
            pre = cache.prefill_attend(torch.as_tensor(qc).cuda(), torch.as_tensor(bt[None]), torch.tensor([n])).cpu().numpy()
            assert np.isfinite(pre).all()
            refp = _ref_rows(cache, k, v, qc[0, -1].astype(np.float64), list(range(hq)), hq // hkv)
            assert max_rel(pre[0, -1], refp) < TOL
