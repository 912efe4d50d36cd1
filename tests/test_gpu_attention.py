"""Decode attention off the packed paged cache against dequantize-then-attend (golden + oracle).

Tolerance: outputs within 2e-3 max-relative (max |out - ref| over a row / max |ref| of that row) of the
reference's dequantize-then-fp32/fp64 attention.
"""
import numpy as np
import pytest

from oracle import tq_oracle as o
from tests.helpers import D, fill_cache, max_rel, wht_dense

pytestmark = pytest.mark.gpu
TOL = 2e-3


@pytest.fixture(scope="module")
def tq():
    import turboquant_plus_b200 as pkg
    return pkg


def oracle_roundtrip(cache, x, which):
    """Reference quantize -> dequantize of (n, d) rows with the cache's own constants."""
    quant = cache.k_quantizer if which == "k" else cache.v_quantizer
    fmt = cache.k_format if which == "k" else cache.v_format
    x32 = np.asarray(x, dtype=np.float32)
    if fmt == "q8_0":
        return o.q8_0_dequantize(*o.q8_0_quantize(x32)).astype(np.float64)
    if fmt.startswith("prod"):
        pq = quant.polar_quant
        code = o.prod_quantize(x32, pq.rotation, pq.centroids, quant.qjl.S, quant.bit_width, pq.norm_correction)
        return o.prod_dequantize(code, pq.rotation, pq.centroids, quant.qjl.S, pq.norm_correction)
    i, n = o.polar_quantize(x32, quant.rotation, quant.centroids)
    return o.polar_dequantize(i, n, quant.rotation, quant.centroids, quant.norm_correction)


def oracle_attention(cache, ks, vs, q, seq_lens):
    bsz, hq = q.shape[0], q.shape[1]
    hkv = cache.num_kv_heads
    ctx = max(int(n) for n in seq_lens)
    kh = np.zeros((bsz, hkv, ctx, D))
    vh = np.zeros((bsz, hkv, ctx, D))
    for b in range(bsz):
        n = int(seq_lens[b])
        for h in range(hkv):
            kh[b, h, :n] = oracle_roundtrip(cache, ks[b][:, h], "k")
            vh[b, h, :n] = oracle_roundtrip(cache, vs[b][:, h], "v")
    return o.attend_gqa(np.asarray(q, dtype=np.float64), kh, vh, seq_lens)


@pytest.mark.parametrize("mode", ["wht", "dense"])
@pytest.mark.parametrize("kk", ["mse", "prod"])
def test_attention_golden(tq, g_kv, mode, kk):
    """Fixture produced by the reference: compress -> decompress -> softmax(q k^T / sqrt d) v.
    kk = "prod": K through TurboQuant (2-bit PolarQuant + QJL), exactly KVCacheCompressor(k_bits=3)."""
    import torch
    k, v, q = g_kv["k"], g_kv["v"], g_kv["q"]          # (1, 2, 200, 128) x2, (8, 128) fp16
    cache = tq.PagedKVCache(D, 2, num_pages=7, k_format="turbo3" if kk == "mse" else "prod3", v_format="turbo3",
                            seed=42, rotation=mode)
    ks = [np.ascontiguousarray(k[0].transpose(1, 0, 2))]
    vs = [np.ascontiguousarray(v[0].transpose(1, 0, 2))]
    bt = fill_cache(cache, ks, vs, [200], np.random.default_rng(0))
    out = cache.attend(torch.as_tensor(q[None]).cuda(), bt, torch.tensor([200]))
    assert cache.kernel_status() == 0
    err = max_rel(out[0].float().cpu().numpy(), g_kv[f"{mode}_{kk}_out"])
    print(f"{mode} {cache.k_format}/turbo3 vs reference fixture: max-rel {err:.2e}")
    assert err < TOL + 1e-3          # fp16 output rounding of the fixture comparison (4.9e-4) included
    out32 = cache.attend(torch.as_tensor(q[None]).cuda().float(), bt, torch.tensor([200]))
    err = max_rel(out32[0].cpu().numpy(), g_kv[f"{mode}_{kk}_out"])
    print(f"   fp32 output: max-rel {err:.2e}")
    assert err < TOL


@pytest.mark.parametrize("kf,vf", [("turbo3", "turbo3"), ("turbo2", "turbo2"), ("turbo4", "turbo4"),
                                   ("turbo4", "turbo2"), ("turbo2", "turbo3"), ("turbo3", "turbo4"),
                                   ("q8_0", "turbo2"), ("q8_0", "q8_0"), ("q8_0", "turbo4"),
                                   ("prod3", "turbo3"), ("prod2", "turbo2"), ("prod4", "turbo4"), ("prod3", "turbo2")])
def test_ragged_paged_batch(tq, kf, vf):
    """Ragged lengths (1, page edges, several pages), shuffled pages, 4 query heads per KV head."""
    import torch
    rng = np.random.default_rng(3)
    hkv, g = 2, 4
    seq_lens = [1, 17, 127, 128, 129, 300, 1000, 640]
    cache = tq.PagedKVCache(D, hkv, num_pages=40, k_format=kf, v_format=vf, seed=42)
    ks = [np.stack([o.rope_rotate(o.synth_keys(n, seed=50 + 7 * b + h), np.arange(n)) for h in range(hkv)], axis=1)
          for b, n in enumerate(seq_lens)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in seq_lens]
    bt = fill_cache(cache, ks, vs, seq_lens, rng)
    q = rng.standard_normal((len(seq_lens), hkv * g, D)).astype(np.float16)
    out = cache.attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor(seq_lens)).cpu().numpy()
    assert cache.kernel_status() == 0
    ref = oracle_attention(cache, ks, vs, q, seq_lens)
    err = max_rel(out, ref)
    print(f"{kf}/{vf}: max-rel {err:.2e}")
    assert err < TOL
    # run to run the bits are identical (fixed split order, no atomics on the data path)
    out2 = cache.attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor(seq_lens)).cpu().numpy()
    assert np.array_equal(out, out2)
    # an empty sequence yields zeros and leaves the others alone
    sl0 = list(seq_lens)
    sl0[2] = 0
    out0 = cache.attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor(sl0)).cpu().numpy()
    assert np.abs(out0[2]).max() == 0 and np.array_equal(out0[3], out[3])


@pytest.mark.parametrize("g", [1, 2, 8])
def test_group_sizes_and_fp16_io(tq, g):
    import torch
    rng = np.random.default_rng(11)
    hkv = 3
    seq_lens = [333, 64]
    cache = tq.PagedKVCache(D, hkv, num_pages=8, seed=42)
    ks = [rng.standard_normal((n, hkv, D)).astype(np.float16) for n in seq_lens]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16) for n in seq_lens]
    bt = fill_cache(cache, ks, vs, seq_lens, rng)
    q = rng.standard_normal((2, hkv * g, D)).astype(np.float16)
    out = cache.attend(torch.as_tensor(q).cuda(), bt, torch.tensor(seq_lens))
    assert out.dtype == torch.float16
    ref = oracle_attention(cache, ks, vs, q, seq_lens)
    assert max_rel(out.float().cpu().numpy(), ref) < TOL + 1e-3
    with pytest.raises(Exception):
        cache.attend(torch.zeros((2, hkv * 9, D), device="cuda"), bt, torch.tensor(seq_lens))


def test_config1_full_size(tq):
    """32 query / 8 KV heads, batch 1, context 32,768, turbo3 K and V, fp16 queries: against the oracle."""
    import torch
    rng = np.random.default_rng(0)
    hkv, g, n = 8, 4, 32768
    cache = tq.PagedKVCache(D, hkv, num_pages=n // 128, seed=42)
    pos = np.arange(n)
    ks = [np.stack([o.rope_rotate(o.synth_keys(n, seed=h), pos) for h in range(hkv)], axis=1).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(cache, ks, vs, [n], rng)
    q = rng.standard_normal((1, hkv * g, D)).astype(np.float16)
    out = cache.attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor([n])).cpu().numpy()
    assert cache.kernel_status() == 0
    ref = oracle_attention(cache, ks, vs, q, [n])
    err = max_rel(out, ref)
    print(f"config 1 (ctx 32768, 32/8 heads, turbo3/turbo3): max-rel {err:.2e}")
    assert err < TOL


def test_append_matches_bulk_quantize(tq):
    """Records written by quantize-on-append hold exactly the bytes of the bulk quantize entry point."""
    import torch
    rng = np.random.default_rng(5)
    hkv, n = 2, 300
    cache = tq.PagedKVCache(D, hkv, num_pages=4, seed=42)
    k = torch.as_tensor(o.synth_keys(n * hkv, seed=2).reshape(n, hkv, D)).cuda()
    v = torch.as_tensor(rng.standard_normal((n, hkv, D)).astype(np.float32)).cuda()
    slots = torch.as_tensor(rng.permutation(4 * 128)[:n].astype(np.int64))
    slots[7] = -1                                                 # skipped token
    cache.append(k, v, slots)
    L = cache.layout
    pool = cache.pool.cpu().numpy()
    kq = cache.k_quantizer.quantize_device(k.reshape(-1, D), packed=True, want_scale=True)
    vq = cache.v_quantizer.quantize_device(v.reshape(-1, D), packed=True, want_scale=True)
    for t in range(n):
        s = int(slots[t])
        if s < 0:
            continue
        page, within = divmod(s, 128)
        for h in range(hkv):
            rec = pool[page, h]
            row = t * hkv + h
            assert np.array_equal(rec[L.k_idx_off + within * 48: L.k_idx_off + within * 48 + 48],
                                  kq["packed"][row].cpu().numpy())
            assert np.array_equal(rec[L.v_idx_off + within * 48: L.v_idx_off + within * 48 + 48],
                                  vq["packed"][row].cpu().numpy())
            assert rec[L.k_scale_off + within * 4: L.k_scale_off + within * 4 + 4].view(np.float32)[0] == \
                kq["scale"][row].item()
            assert rec[L.v_scale_off + within * 4: L.v_scale_off + within * 4 + 4].view(np.float32)[0] == \
                vq["scale"][row].item()
    assert cache.bytes_per_token == 104


def test_q8_0_and_prod_records_match_oracle(tq):
    """Bytes written by quantize-on-append for q8_0 (against the restated block rule) and PROD (sign sketch and
    residual scale against the oracle)."""
    import torch
    rng = np.random.default_rng(9)
    hkv, n = 2, 200
    cache = tq.PagedKVCache(D, hkv, num_pages=2, k_format="q8_0", v_format="q8_0")
    k = o.synth_keys(n * hkv, seed=4).reshape(n, hkv, D)
    k[3] = 0
    v = rng.standard_normal((n, hkv, D)).astype(np.float32)
    slots = torch.arange(n, dtype=torch.int64)
    cache.append(torch.as_tensor(k).cuda(), torch.as_tensor(v).cuda(), slots)
    pool, L = cache.pool.cpu().numpy(), cache.layout
    for name, x, io, so in (("k", k, L.k_idx_off, L.k_scale_off), ("v", v, L.v_idx_off, L.v_scale_off)):
        q_ref, s_ref = o.q8_0_quantize(x.reshape(-1, D))
        for t in (0, 3, 127, 128, 199):
            page, w = divmod(t, 128)
            for h in range(hkv):
                rec = pool[page, h]
                assert np.array_equal(rec[io + w * 128: io + w * 128 + 128].view(np.int8), q_ref[t * hkv + h]), name
                assert np.array_equal(rec[so + w * 8: so + w * 8 + 8].view(np.float16), s_ref[t * hkv + h]), name
    assert cache.bytes_per_token == 272
    cache = tq.PagedKVCache(D, hkv, num_pages=2, k_format="prod3", v_format="turbo3", seed=42)
    cache.append(torch.as_tensor(k).cuda(), torch.as_tensor(v).cuda(), slots)
    pool, L = cache.pool.cpu().numpy(), cache.layout
    kq = cache.k_quantizer
    code = o.prod_quantize(k.reshape(-1, D), kq.polar_quant.rotation, kq.polar_quant.centroids, kq.qjl.S, 3)
    bits_ref = o.pack_signs(code.qjl_signs)
    flips = 0
    for t in range(n):
        page, w = divmod(t, 128)
        for h in range(hkv):
            rec, row = pool[page, h], t * hkv + h
            got_idx = rec[L.k_idx_off + w * 32: L.k_idx_off + w * 32 + 32]
            if not np.array_equal(got_idx, o.pack_idx(code.mse_indices[row], 2)):
                continue                                   # a near-boundary index moves the residual
            flips += int(np.unpackbits(rec[L.k_qjl_off + w * 16: L.k_qjl_off + w * 16 + 16] ^ bits_ref[row]).sum())
            rs = rec[L.k_rscale_off + w * 4: L.k_rscale_off + w * 4 + 4].view(np.float32)[0]
            assert abs(rs - code.residual_norms[row] * o.QJL_CONST / np.sqrt(D)) <= 2e-5 * abs(rs) + 1e-30
    assert flips <= 4
    assert cache.bytes_per_token == 108


@pytest.mark.parametrize("kf,vf,mode", [("turbo3", "turbo3", "wht"), ("turbo4", "turbo2", "wht"), ("turbo2", "turbo2", "wht"),
                                        ("turbo3", "turbo3", "dense")])
def test_prefill_chunk_tcgen05(tq, kf, vf, mode):
    """Causal chunked prefill (tcgen05 kernel) against dequantize-then-attend on the visible prefix: ragged
    lengths, a chunk that starts the sequence, a chunk that crosses page edges, 8 query heads per KV head."""
    import torch
    rng = np.random.default_rng(23)
    hkv, g, tq_len = 2, 8, 24
    kv_lens = [24, 128, 129, 400, 1000]          # first: the chunk is the whole sequence
    cache = tq.PagedKVCache(D, hkv, num_pages=24, k_format=kf, v_format=vf, seed=42, rotation=mode)
    ks = [np.stack([o.rope_rotate(o.synth_keys(n, seed=9 * b + h), np.arange(n)) for h in range(hkv)], axis=1)
          for b, n in enumerate(kv_lens)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in kv_lens]
    bt = fill_cache(cache, ks, vs, kv_lens, rng)
    q = rng.standard_normal((len(kv_lens), tq_len, hkv * g, D)).astype(np.float16)
    out = cache.prefill_attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor(kv_lens)).cpu().numpy()
    assert cache.kernel_status() == 0
    ctx = max(kv_lens)
    kh = np.zeros((len(kv_lens), hkv, ctx, D))
    vh = np.zeros((len(kv_lens), hkv, ctx, D))
    for b, n in enumerate(kv_lens):
        for h in range(hkv):
            kh[b, h, :n] = oracle_roundtrip(cache, ks[b][:, h], "k")
            vh[b, h, :n] = oracle_roundtrip(cache, vs[b][:, h], "v")
    ref = o.attend_chunk_gqa(q.astype(np.float64), kh, vh, kv_lens)
    err = max_rel(out.reshape(-1, D), ref.reshape(-1, D))
    print(f"prefill {kf}/{vf} {mode}: max-rel {err:.2e}")
    assert err < TOL
    # the last query of a chunk sees the whole cache: same answer as decode attention for that token
    dec = cache.attend(torch.as_tensor(q[:, -1]).cuda().float(), bt, torch.tensor(kv_lens)).cpu().numpy()
    assert max_rel(out[:, -1], dec) < TOL
    out2 = cache.prefill_attend(torch.as_tensor(q).cuda().float(), bt, torch.tensor(kv_lens)).cpu().numpy()
    assert np.array_equal(out, out2)


def test_prefill_split_pages(tq):
    """Long contexts: the page range of a row block is split over several CTAs and folded by the last one."""
    import torch
    rng = np.random.default_rng(29)
    hkv, g, tq_len = 2, 8, 40
    kv_lens = [4096, 3000]
    cache = tq.PagedKVCache(D, hkv, num_pages=64, seed=42)
    ks = [np.stack([o.rope_rotate(o.synth_keys(n, seed=11 * b + h), np.arange(n)) for h in range(hkv)], axis=1)
          for b, n in enumerate(kv_lens)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in kv_lens]
    bt = fill_cache(cache, ks, vs, kv_lens, rng)
    from turboquant_plus_b200 import _native as nv
    assert nv.load().tq_prefill_workspace_bytes(2, tq_len, hkv * g, hkv, bt.shape[1]) > 4 * 128 * 130 * 4
    q = rng.standard_normal((2, tq_len, hkv * g, D)).astype(np.float16)
    out = cache.prefill_attend(torch.as_tensor(q).cuda(), bt, torch.tensor(kv_lens))
    assert cache.kernel_status() == 0 and out.dtype == torch.float16
    kh = np.zeros((2, hkv, 4096, D))
    vh = np.zeros((2, hkv, 4096, D))
    for b, n in enumerate(kv_lens):
        for h in range(hkv):
            kh[b, h, :n] = oracle_roundtrip(cache, ks[b][:, h], "k")
            vh[b, h, :n] = oracle_roundtrip(cache, vs[b][:, h], "v")
    ref = o.attend_chunk_gqa(q.astype(np.float64), kh, vh, kv_lens)
    err = max_rel(out.float().cpu().numpy().reshape(-1, D), ref.reshape(-1, D))
    print(f"prefill with split pages: max-rel {err:.2e}")
    assert err < TOL + 1e-3          # fp16 output rounding included
    out2 = cache.prefill_attend(torch.as_tensor(q).cuda(), bt, torch.tensor(kv_lens))
    assert torch.equal(out, out2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_prefill_16bit_rows_equal_the_fp32_call(tq, dtype):
    """Queries and outputs of a chunk in fp16 / bf16: the kernel widens the queries exactly and rounds the outputs to
    nearest, so the call gives the bits of the fp32 call on the widened queries, rounded by torch.  A ragged last row
    block (40 queries x 8 heads = 2.5 row blocks) and a split page range are part of the case."""
    import torch
    dt = getattr(torch, dtype)
    rng = np.random.default_rng(31)
    hkv, g, tq_len = 2, 8, 40
    kv_lens = [2500, 700]
    cache = tq.PagedKVCache(D, hkv, num_pages=32, seed=42)
    ks = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in kv_lens]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in kv_lens]
    bt = fill_cache(cache, ks, vs, kv_lens, rng)
    q = torch.as_tensor(rng.standard_normal((2, tq_len, hkv * g, D)).astype(np.float32)).cuda().to(dt)
    out16 = cache.prefill_attend(q, bt, torch.tensor(kv_lens))
    out32 = cache.prefill_attend(q.float(), bt, torch.tensor(kv_lens))
    assert cache.kernel_status() == 0 and out16.dtype == dt and out32.dtype == torch.float32
    assert torch.isfinite(out32).all() and float(out32.abs().max()) > 0
    assert torch.equal(out16, out32.to(dt))


@pytest.mark.gpu
def test_bounded_wait_gives_up_and_reports(tq):
    """The give-up path of the kernels' bounded waits, run where it is harmless (tq_selftest_wait_gives_up: a wait that
    nothing satisfies, limited to 2^20 clocks): the status word of the workspace reads 1 once, then 0 again, and the
    same workspace serves the next attention call with the same bytes as before."""
    import torch
    from turboquant_plus_b200 import _native as nv
    rng = np.random.default_rng(5)
    hkv, hq, n = 2, 8, 700
    c = tq.PagedKVCache(D, hkv, num_pages=6, seed=42)
    ks = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(c, ks, vs, [n], rng).cuda()
    sl = torch.tensor([n], dtype=torch.int32, device="cuda")
    q = torch.as_tensor(rng.standard_normal((1, hq, D)).astype(np.float16)).cuda()
    ws = c.workspace(1, hq, 6)
    before = c.attend(q, bt, sl, workspace=ws).clone()
    assert c.kernel_status(ws) == 0
    nv.call("tq_selftest_wait_gives_up", nv.ptr(ws), ws.numel(), nv.stream_ptr())
    torch.cuda.synchronize()
    assert c.kernel_status(ws) == 1       # a wait gave up since the last read ...
    assert c.kernel_status(ws) == 0       # ... and reading it cleared it
    after = c.attend(q, bt, sl, workspace=ws)
    assert torch.equal(after, before) and c.kernel_status(ws) == 0


@pytest.mark.parametrize("fmt", [("turbo3", "turbo3"), ("prod3", "turbo3"), ("q8_0", "turbo2")])
def test_attend_right_after_append(tq, fmt):
    """overlap="append": the attention call that follows the append of the step's token streams every page but the
    last of each sequence while the append is still running, and fetches that page afterwards.  Eight decode steps
    back to back (append one token per sequence, attend) against the same steps in stream order on a second cache:
    every step's output must see its new token."""
    import torch
    rng = np.random.default_rng(31)
    hkv, hq, B, steps = 4, 16, 24, 8
    lens = [int(x) for x in rng.integers(100, 900, size=B)]
    lens[0], lens[1] = 127, 128          # the new token opens a page / is the last of one
    ks = [rng.standard_normal((n + steps, hkv, D)).astype(np.float16) for n in lens]
    vs = [rng.standard_normal((n + steps, hkv, D)).astype(np.float16) for n in lens]
    outs = {}
    for mode in ("append", False):
        c = tq.PagedKVCache(D, hkv, num_pages=8 * B, k_format=fmt[0], v_format=fmt[1], seed=42)
        # pages for the steps to come too; only the first n tokens of a sequence are in the cache before the steps
        perm, bt = np.random.default_rng(7).permutation(c.num_pages), np.zeros((B, 8), dtype=np.int32)
        for b, n in enumerate(lens):
            bt[b] = perm[8 * b: 8 * b + 8]
            tpos = np.arange(n)
            c.append(torch.as_tensor(ks[b][:n]).cuda(), torch.as_tensor(vs[b][:n]).cuda(),
                     torch.as_tensor(bt[b][tpos // 128].astype(np.int64) * 128 + tpos % 128))
        bt = torch.as_tensor(bt).cuda()
        ws = c.workspace(B, hq, bt.shape[1])
        res = []
        for s in range(steps):
            pos = torch.tensor([n + s for n in lens])
            slots = bt.cpu()[torch.arange(B), pos // 128].long() * 128 + pos % 128
            kn = torch.as_tensor(np.stack([k[n + s] for k, n in zip(ks, lens)])).cuda()
            vn = torch.as_tensor(np.stack([v[n + s] for v, n in zip(vs, lens)])).cuda()
            q = torch.as_tensor(rng.standard_normal((B, hq, D)).astype(np.float16)).cuda() if mode == "append" else outs["q"][s]
            sl = (pos + 1).to(torch.int32).cuda()
            slots = slots.cuda()
            torch.cuda.synchronize()
            c.append(kn, vn, slots)
            res.append(c.attend(q, bt, sl, workspace=ws, overlap=mode).clone())
            if mode == "append":
                outs.setdefault("q", []).append(q)
        torch.cuda.synchronize()
        assert c.kernel_status(ws) == 0
        outs[mode] = res
    for a, b in zip(outs["append"], outs[False]):
        # the four-warp form sums its tiles in another order than the eight-warp form: fp32 rounding apart
        assert float((a.float() - b.float()).abs().max()) <= 2e-3 * float(b.float().abs().max())
    # and the last step against the oracle, per sequence.  With 24 sequences of up to 900 tokens a handful of
    # coordinates sit within rounding of a decision boundary and take the neighbouring index in the oracle (the band
    # rule of the quantizer tests); where such a token carries weight its sequence shows it, so the bound holds for
    # the typical sequence and a looser one for every sequence.
    ref = oracle_attention(c, ks, vs, outs["q"][-1].float().cpu().numpy(), [n + steps for n in lens])
    got = outs["append"][-1].float().cpu().numpy()
    per_seq = np.array([max_rel(got[b], ref[b]) for b in range(B)])
    print("per-sequence max-rel:", " ".join(f"{e:.1e}" for e in per_seq))
    assert np.median(per_seq) < 1e-3 and (per_seq < TOL).sum() >= B - 6 and per_seq.max() < 5e-2


@pytest.mark.parametrize("hq", [16, 32])
def test_overlap_launch_and_compressor_streaming_api(tq, hq):
    """(1) TQ_DECODE_OVERLAP (programmatic dependent launch) changes when the kernel starts, never what it computes:
    a chain of overlapped calls, eager and replayed from a CUDA graph, returns the bytes of the plain calls.  With
    eight query heads per KV head (hq = 32) the chain mode "q" deals a group to two CTAs of the specialised kernel,
    the plain calls run the general kernel.
    (2) KVCacheCompressor.init_cache / append / attend / prefill_attend give what the paged cache gives."""
    import torch
    rng = np.random.default_rng(21)
    hkv, n = 4, 1500
    caches = []
    for i in range(3):
        c = tq.PagedKVCache(D, hkv, num_pages=12, seed=42)
        ks = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
        vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
        bt = fill_cache(c, ks, vs, [n], rng)
        caches.append((c, bt.cuda()))
    sl = torch.tensor([n], dtype=torch.int32, device="cuda")
    q = torch.as_tensor(rng.standard_normal((1, hq, D)).astype(np.float16)).cuda()
    ws = caches[0][0].workspace(1, hq, 12)
    plain = [c.attend(q, bt, sl, workspace=ws).clone() for c, bt in caches]
    outs = [torch.empty_like(q) for _ in caches]

    for mode in (True, "q"):      # "q": the queries may be read before the preceding call has completed, too
        def chain():
            for (c, bt), o_ in zip(caches, outs):
                c.attend(q, bt, sl, out=o_, workspace=ws, overlap=mode)

        def same(a, b):
            # plain overlap runs the very same kernel; "q" runs four-warp CTAs, whose warps add their tiles in another
            # order: equal to fp32 rounding (the fp16 outputs differ by at most an ulp), and bit-stable run to run
            if mode is True:
                return torch.equal(a, b)
            return float((a.float() - b.float()).abs().max()) <= 2e-3 * float(b.float().abs().max())

        for o_ in outs:
            o_.zero_()
        for _ in range(4):        # back to back: a call's page loop runs under the tail of the call before
            chain()
        torch.cuda.synchronize()
        eager = [o_.clone() for o_ in outs]
        for a, b in zip(plain, outs):
            assert same(b, a)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            chain()
        for o_ in outs:
            o_.zero_()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        for a, b, e in zip(plain, outs, eager):
            assert same(b, a) and torch.equal(b, e)
        # the sparse-V option has both forms too; on this flat softmax no tile is skipped: the dense bytes
        for (c, bt), o_, e in zip(caches, outs, eager):
            c.attend(q, bt, sl, out=o_, workspace=ws, overlap=mode, sparse_v=True)
        torch.cuda.synchronize()
        for o_, e in zip(outs, eager):
            assert torch.equal(o_, e)
        assert caches[0][0].kernel_status(ws) == 0

    comp = tq.KVCacheCompressor(D, k_bits=3, v_bits=3, seed=42, rotation="wht").init_cache(2, hkv, 12)
    ks = [rng.standard_normal((300, hkv, D)).astype(np.float16)]
    vs = [rng.standard_normal((300, hkv, D)).astype(np.float16)]
    slots = torch.arange(300)
    bt = torch.arange(12, dtype=torch.int32)[None]
    for layer in range(2):
        comp.append(torch.as_tensor(ks[0]).cuda(), torch.as_tensor(vs[0]).cuda(), layer, slots)
    out = comp.attend(q.float(), 1, torch.tensor([300]), bt).cpu().numpy()
    ref = oracle_attention(comp._layers[1], ks, vs, q.float().cpu().numpy(), [300])
    assert comp._layers[1].k_format == "prod3" and max_rel(out, ref) < TOL
    # prefill over PROD keys (the reference's default K quantizer, turboquant/kv_cache.py:89-96): the chunk's queries
    # go through the decode kernel, each with its causal length
    qc = rng.standard_normal((1, 8, hq, D)).astype(np.float32)
    pre = comp.prefill_attend(torch.as_tensor(qc).cuda(), 1, torch.tensor([300]), bt).cpu().numpy()
    for i in (0, 3, 7):
        ks_i, vs_i = [ks[0][:300 - 8 + i + 1]], [vs[0][:300 - 8 + i + 1]]
        ref_i = oracle_attention(comp._layers[1], ks_i, vs_i, qc[:, i], [300 - 8 + i + 1])
        assert max_rel(pre[:, i], ref_i) < TOL


@pytest.mark.gpu
def test_many_splits_long_context(tq):
    """One sequence, one KV head, 70,000 tokens: the split plan cuts it into ~270 two-page splits, so the merge by
    the last split folds more than 64 partials (several rounds) -- and the two groups of a CTA serve different
    splits of the same head.  Checked against the oracle over the dequantized cache."""
    import torch
    rng = np.random.default_rng(33)
    n, hkv, hq = 70000, 1, 4
    cache = tq.PagedKVCache(D, hkv, num_pages=(n + 127) // 128, seed=42)
    ks = [(rng.standard_normal((n, hkv, D)) * np.exp(0.3 * rng.standard_normal((n, hkv, 1)))).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(cache, ks, vs, [n], rng)
    q = rng.standard_normal((1, hq, D)).astype(np.float32)
    out = cache.attend(torch.as_tensor(q).cuda(), bt, torch.tensor([n])).cpu().numpy()
    assert cache.kernel_status() == 0
    ref = oracle_attention(cache, ks, vs, q, [n])
    err = max_rel(out, ref)
    print(f"70,000 tokens, 1 KV head: max-rel {err:.2e}")
    assert err < TOL
    out2 = cache.attend(torch.as_tensor(q).cuda(), bt, torch.tensor([n]), overlap=True).cpu().numpy()
    assert np.array_equal(out, out2)


@pytest.mark.gpu
@pytest.mark.parametrize("group", [4, 8])
def test_sparse_v_option(tq, group):
    """TQ_DECODE_SPARSE_V skips the V work of 16-token tiles whose weights are all below 1e-6 of the running maximum
    (the reference's sparse V, docs/papers/sparse-v-dequant.md:64-84).  With keys of very different norms most tiles
    qualify; the output must stay within the attention tolerance of the dense oracle and within 1e-4 of the dense
    kernel, and on flat weights (nothing below the threshold) it must equal the dense kernel bit for bit."""
    import torch
    rng = np.random.default_rng(41 + group)
    n, hkv = 6000, 2
    hq = hkv * group
    cache = tq.PagedKVCache(D, hkv, num_pages=(n + 127) // 128, seed=42)
    scale = np.exp(1.2 * rng.standard_normal((n, hkv, 1)))          # a few tokens dominate the softmax
    ks = [(rng.standard_normal((n, hkv, D)) * scale).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(cache, ks, vs, [n], rng)
    q = (3.0 * rng.standard_normal((1, hq, D))).astype(np.float32)
    qd = torch.as_tensor(q).cuda()
    dense = cache.attend(qd, bt, torch.tensor([n])).cpu().numpy()
    sparse = cache.attend(qd, bt, torch.tensor([n]), sparse_v=True).cpu().numpy()
    ref = oracle_attention(cache, ks, vs, q, [n])
    print(f"group {group}: sparse vs oracle {max_rel(sparse, ref):.2e}, sparse vs dense kernel {max_rel(sparse, dense):.2e}")
    assert max_rel(sparse, ref) < TOL and max_rel(sparse, dense) < 1e-4
    flat = cache.attend(torch.zeros_like(qd), bt, torch.tensor([n]))
    flat_s = cache.attend(torch.zeros_like(qd), bt, torch.tensor([n]), sparse_v=True)
    assert torch.equal(flat, flat_s)


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,block", [("turbo3", 32), ("turbo3", 128), ("turbo3", 64), ("turbo2", 32), ("turbo2", 128),
                                       ("turbo4", 128)])
def test_block_codec_and_state_dict(tq, fmt, block):
    """Wire formats (the block layouts of the reference's documents: turbo3 14 B / 32 or 50 B / 128, turbo4 68 B / 128):
    exported bytes equal the NumPy restatement of the documents' extraction expressions, import into a second cache
    restores the index arrays bit for bit and the scales to fp16, attention over the imported cache stays inside the
    tolerance; state_dict / load_state_dict reproduce the pool and the attention output exactly."""
    import torch
    rng = np.random.default_rng(17)
    n, hkv, hq, bits = 300, 2, 8, int(fmt[-1])
    cache = tq.PagedKVCache(D, hkv, num_pages=4, k_format=fmt, v_format=fmt, seed=42)
    ks = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(cache, ks, vs, [n], rng)
    t = np.arange(n)
    slots = torch.as_tensor(bt[0].numpy()[t // 128].astype(np.int64) * 128 + t % 128)
    assert cache.block_bytes("k", block) == o.block_bytes(bits, block) == {(3, 32): 14, (3, 64): 26, (3, 128): 50,
                                                                        (2, 32): 10, (2, 128): 34, (4, 128): 68}[(bits, block)]
    L, pool = cache.layout, cache.pool.cpu().numpy()
    other = tq.PagedKVCache(D, hkv, num_pages=4, k_format=fmt, v_format=fmt, seed=42)
    for which, idx_off, scale_off in (("k", L.k_idx_off, L.k_scale_off), ("v", L.v_idx_off, L.v_scale_off)):
        blocks = cache.export_blocks(which, slots, block)
        assert tuple(blocks.shape) == (n, hkv, D // block, o.block_bytes(bits, block))
        raw = blocks.cpu().numpy()
        for tok in (0, 1, 127, 128, 299):
            page, off = int(slots[tok]) // 128, int(slots[tok]) % 128
            for h in range(hkv):
                rec = pool[page, h]
                idx = o.unpack_idx(rec[idx_off + off * 16 * bits: idx_off + (off + 1) * 16 * bits], bits, D)
                scale = rec[scale_off + 4 * off: scale_off + 4 * off + 4].view(np.float32)[0]
                assert np.array_equal(raw[tok, h].reshape(-1), o.blocks_encode(idx, scale, bits, block))
                back, nrm = o.blocks_decode(raw[tok, h].reshape(-1), bits, block)
                assert np.array_equal(back, idx) and nrm == float(np.float16(scale))
        other.import_blocks(which, blocks, slots, block)
    p2 = other.pool.cpu().numpy()
    pages = np.unique(bt[0].numpy())
    for page in pages:
        for h in range(hkv):
            a, b = pool[page, h], p2[page, h]
            valid = min(128, n - 128 * int(np.where(bt[0].numpy() == page)[0][0]))
            for off_i, off_s in ((L.k_idx_off, L.k_scale_off), (L.v_idx_off, L.v_scale_off)):
                assert np.array_equal(a[off_i: off_i + valid * 16 * bits], b[off_i: off_i + valid * 16 * bits])
                sa = a[off_s: off_s + 4 * valid].view(np.float32)
                sb = b[off_s: off_s + 4 * valid].view(np.float32)
                assert np.array_equal(sa.astype(np.float16).astype(np.float32), sb)
    q = torch.as_tensor(rng.standard_normal((1, hq, D)).astype(np.float32)).cuda()
    ref = cache.attend(q, bt, torch.tensor([n])).cpu().numpy()
    got = other.attend(q, bt, torch.tensor([n])).cpu().numpy()
    assert max_rel(got, ref) < TOL
    clone = tq.PagedKVCache(D, hkv, num_pages=4, k_format=fmt, v_format=fmt, seed=42)
    clone.load_state_dict(cache.state_dict())
    assert torch.equal(clone.pool, cache.pool)
    assert np.array_equal(clone.attend(q, bt, torch.tensor([n])).cpu().numpy(), ref)
    with pytest.raises(ValueError):
        tq.PagedKVCache(D, hkv, num_pages=5, k_format=fmt, v_format=fmt).load_state_dict(cache.state_dict())
    if bits == 4:
        with pytest.raises(ValueError):
            cache.block_bytes("k", 32)


@pytest.mark.gpu
def test_model_hooks_and_cache_adapter(tq):
    """Caller-side adapters.  (1) patch_model_attention (the reference's benchmarks/benchmark_norm_correction.py:45-96):
    the keys a layer's k_proj produces come back quantize -> dequantized per KV head with seed = head index; checked
    against the oracle's dense PolarQuant round trip on a stand-in model with the attribute layout the hook walks.
    (2) TurboQuantCache: update() of a prompt then of single positions, attend() for a chunk (prefill kernel) and for
    one position (decode kernel) against dequantize-then-attend."""
    import torch
    from turboquant_plus_b200 import integration as integ
    torch.manual_seed(0)
    hidden, heads, hkv = 512, 4, 2           # head_dim 128

    class Attn(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.k_proj = torch.nn.Linear(hidden, hkv * D, bias=False)

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.self_attn = Attn()

    class Inner(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList([Layer(), Layer()])

    class Model(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.model = Inner()
            self.config = type("Cfg", (), {"hidden_size": hidden, "num_attention_heads": heads,
                                           "num_key_value_heads": hkv})()

    model = Model().cuda()
    x = torch.randn(2, 9, hidden, device="cuda")
    plain = [layer.self_attn.k_proj(x) for layer in model.model.layers]
    hooks = integ.patch_model_attention(model, lambda d, seed: tq.TurboQuantMSE(d, 3, seed=seed))
    patched = [layer.self_attn.k_proj(x) for layer in model.model.layers]
    integ.unpatch_model(hooks)
    assert all(isinstance(layer.self_attn.k_proj, torch.nn.Linear) for layer in model.model.layers)
    for k0, k1 in zip(plain, patched):
        assert k1.shape == k0.shape and k1.dtype == k0.dtype
        k0n = k0.detach().cpu().numpy().astype(np.float64).reshape(2 * 9, hkv, D)
        for h in range(hkv):
            rot = o.dense_rotation(D, np.random.default_rng(h))
            c = o.centroids(3, D)
            i, nrm = o.polar_quantize(k0n[:, h], rot, c)
            want = o.polar_dequantize(i, nrm, rot, c)
            got = k1.detach().cpu().numpy().reshape(2 * 9, hkv, D)[:, h]
            assert max_rel(got, want) < 1e-5

    rng = np.random.default_rng(3)
    B, hq, prompt, extra = 2, 8, 150, 3
    cache = integ.TurboQuantCache(num_layers=2, head_dim=D, num_kv_heads=hkv, max_batch=B, max_seq_len=300)
    k = rng.standard_normal((B, hkv, prompt + extra, D)).astype(np.float16)
    v = rng.standard_normal((B, hkv, prompt + extra, D)).astype(np.float16)
    q = rng.standard_normal((B, hq, prompt + extra, D)).astype(np.float16)
    kt, vt, qt = (torch.as_tensor(a).cuda() for a in (k, v, q))
    layer = 1
    pq = cache.store.layers[layer]
    kh = np.stack([[oracle_roundtrip(pq, k[b, h].astype(np.float32), "k") for h in range(hkv)] for b in range(B)])
    vh = np.stack([[oracle_roundtrip(pq, v[b, h].astype(np.float32), "v") for h in range(hkv)] for b in range(B)])
    assert cache.update(kt[:, :, :prompt], vt[:, :, :prompt], layer) == prompt and cache.get_seq_length(layer) == prompt
    chunk = 16
    out = cache.attend(qt[:, :, prompt - chunk:prompt], layer)
    assert tuple(out.shape) == (B, hq, chunk, D)
    ref = o.attend_chunk_gqa(q[:, :, prompt - chunk:prompt].transpose(0, 2, 1, 3).astype(np.float64),
                             kh[:, :, :prompt], vh[:, :, :prompt], [prompt] * B)
    assert max_rel(out.permute(0, 2, 1, 3).float().cpu().numpy().reshape(-1, D), ref.reshape(-1, D)) < TOL
    for step in range(extra):
        n = prompt + step
        cache.update(kt[:, :, n:n + 1], vt[:, :, n:n + 1], layer)
        out1 = cache.attend(qt[:, :, n:n + 1], layer)
        assert tuple(out1.shape) == (B, hq, 1, D)
        ref1 = o.attend_gqa(q[:, :, n].astype(np.float64), kh[:, :, :n + 1], vh[:, :, :n + 1], [n + 1] * B)
        assert max_rel(out1[:, :, 0].float().cpu().numpy(), ref1) < TOL
    assert cache.get_seq_length(0) == 0
    with pytest.raises(ValueError):
        cache.update(kt[:, :, :200], vt[:, :, :200], layer)


@pytest.mark.gpu
def test_layered_decode_step_from_host_buffers(tq):
    """LayeredKVCache.decode_step: pinned host buffers in, one captured graph (slot computation, quantize-on-append of
    every layer on its own branch, attention per layer), host buffer out.  Three layers with a per-layer format table,
    two sequences of different lengths, four steps; every step's output is checked against dequantize-then-attend over
    everything appended so far."""
    import torch
    from turboquant_plus_b200.layered import LayeredKVCache
    rng = np.random.default_rng(29)
    L, hkv, hq, B, steps = 3, 2, 8, 2, 4
    lens = [130, 40]
    formats = [("turbo4", "turbo4"), ("turbo3", "turbo3"), ("turbo3", "turbo2")]
    cache = LayeredKVCache(L, D, hkv, num_pages=6, formats=formats, seed=42)
    bt = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    ks = [[rng.standard_normal((n + steps, hkv, D)).astype(np.float16) for n in lens] for _ in range(L)]
    vs = [[rng.standard_normal((n + steps, hkv, D)).astype(np.float16) for n in lens] for _ in range(L)]
    for i in range(L):
        for b, n in enumerate(lens):
            t = np.arange(n)
            slots = torch.as_tensor(bt[b].numpy()[t // 128].astype(np.int64) * 128 + t % 128)
            cache.append(i, torch.as_tensor(ks[i][b][:n]).cuda(), torch.as_tensor(vs[i][b][:n]).cuda(), slots)
    cache.prepare_decode(B, hq, bt, torch.tensor(lens))
    qh = torch.empty((L, B, hq, D), dtype=torch.float16).pin_memory()
    kh = torch.empty((L, B, hkv, D), dtype=torch.float16).pin_memory()
    vh = torch.empty((L, B, hkv, D), dtype=torch.float16).pin_memory()
    oh = torch.empty((L, B, hq, D), dtype=torch.float16).pin_memory()
    for s in range(steps):
        if s == 2:          # the cache's own staging buffers: q, k, v adjacent, one copy per step, a new graph
            qh, kh, vh, oh = cache.host_buffers()
            assert kh.data_ptr() == qh.data_ptr() + qh.numel() * 2 and qh.is_pinned() and vh.is_pinned()
        q = rng.standard_normal((L, B, hq, D)).astype(np.float16)
        qh.copy_(torch.as_tensor(q))
        for i in range(L):
            for b, n in enumerate(lens):
                kh[i, b] = torch.as_tensor(ks[i][b][n + s])
                vh[i, b] = torch.as_tensor(vs[i][b][n + s])
        out = cache.decode_step(qh, kh, vh, oh).float().numpy().copy()
        now = [n + s + 1 for n in lens]
        for i in range(L):
            ref = oracle_attention(cache.layers[i], [ks[i][b][:now[b]] for b in range(B)],
                                   [vs[i][b][:now[b]] for b in range(B)], q[i].astype(np.float32), now)
            err = max_rel(out[i], ref)
            assert err < TOL, f"step {s} layer {i}: {err:.2e}"
    assert cache._step["len"].cpu().tolist() == [n + steps for n in lens]
    assert cache.layers[0].kernel_status(cache.layers[0]._ws) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("group", [4, 8])
def test_decayed_pages_and_merged_attention(tq, group):
    """Temporal decay at cache level: the first three pages of a 600-token turbo3 sequence are re-quantized into a
    turbo2 cache (tq_cache_requantize), attention runs over the old part (turbo2 cache) and the recent part (turbo3
    cache) separately and the two are joined from their log-sum-exps.  Oracle: old tokens dequantized from the
    restated requantize_3to2 of the reference's prototype, recent tokens from the 3-bit code, one softmax over all.
    Also: lse of a plain call equals the oracle's log-sum-exp, merging with an empty part changes nothing."""
    import torch
    from turboquant_plus_b200.paged import merge_attention
    rng = np.random.default_rng(31 + group)
    n, old, hkv = 600, 384, 2
    hq = hkv * group
    hot = tq.PagedKVCache(D, hkv, num_pages=5, k_format="turbo3", v_format="turbo3", seed=42)
    cold = tq.PagedKVCache(D, hkv, num_pages=3, k_format="turbo2", v_format="turbo2", seed=42)
    ks = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float16)]
    bt = fill_cache(hot, ks, vs, [n], rng)
    q = rng.standard_normal((1, hq, D)).astype(np.float32)
    qd = torch.as_tensor(q).cuda()
    # plain call: lse against the oracle
    out_all, lse_all = hot.attend(qd, bt, torch.tensor([n]), return_lse=True)
    kh = np.stack([oracle_roundtrip(hot, ks[0][:, h], "k") for h in range(hkv)])          # (hkv, n, D)
    vh = np.stack([oracle_roundtrip(hot, vs[0][:, h], "v") for h in range(hkv)])
    logits = np.stack([kh[h // group] @ q[0, h].astype(np.float64) / np.sqrt(D) for h in range(hq)])   # (hq, n)
    want_lse = np.log(np.exp(logits - logits.max(1, keepdims=True)).sum(1)) + logits.max(1)
    assert np.abs(lse_all.cpu().numpy()[0] - want_lse).max() < 2e-3
    # decay the first three pages
    t = np.arange(old)
    src_slots = torch.as_tensor(bt[0].numpy()[t // 128].astype(np.int64) * 128 + t % 128)
    dst_slots = torch.as_tensor(t.astype(np.int64))
    hot.decay_into(cold, src_slots, dst_slots)
    bt_cold = torch.tensor([[0, 1, 2]], dtype=torch.int32)
    bt_hot = bt[:, old // 128:].contiguous()
    oa, la = cold.attend(qd, bt_cold, torch.tensor([old]), return_lse=True)
    ob, lb = hot.attend(qd, bt_hot, torch.tensor([n - old]), return_lse=True)
    got, lse = merge_attention(oa, la, ob, lb)
    # oracle for the old part: 3-bit code -> requantize_3to2 restatement -> rotate back
    for which, quant3, quant2, xs, hat in (("k", hot.k_quantizer, cold.k_quantizer, ks[0], kh),
                                           ("v", hot.v_quantizer, cold.v_quantizer, vs[0], vh)):
        for h in range(hkv):
            x32 = xs[:old, h].astype(np.float32)
            i3, nrm = o.polar_quantize(x32, quant3.rotation, quant3.centroids)
            y = np.zeros((old, D))
            for r in range(old):
                i2, corrected = o.decay_requantize(i3[r], nrm[r], quant3.centroids, quant2.centroids,
                                                   o.boundaries(quant2.centroids))
                y[r] = quant2.centroids[i2] * corrected
            hat[h, :old] = y @ quant3.rotation          # x = R^T y, row-wise
    ref = o.attend_gqa(q.astype(np.float64), kh[None], vh[None], [n])
    err = max_rel(got.cpu().numpy(), ref)
    print(f"group {group}: decayed + recent, merged: max-rel {err:.2e}")
    assert err < TOL
    logits2 = np.stack([kh[h // group] @ q[0, h].astype(np.float64) / np.sqrt(D) for h in range(hq)])
    want2 = np.log(np.exp(logits2 - logits2.max(1, keepdims=True)).sum(1)) + logits2.max(1)
    assert np.abs(lse.cpu().numpy()[0] - want2).max() < 2e-3
    # an empty part: lse = -inf, the merge returns the other part
    oe, le = cold.attend(qd, bt_cold, torch.tensor([0]), return_lse=True)
    assert torch.isinf(le).all() and (le < 0).all() and (oe == 0).all()
    same, ls = merge_attention(oe, le, ob, lb)
    assert torch.equal(same, ob) and torch.allclose(ls, lb)
    with pytest.raises(ValueError):
        cold.decay_into(hot, dst_slots, src_slots)         # wider destination


@pytest.mark.gpu
def test_side_entry_points_edge_cases(tq):
    """Skipped tokens (negative slots), empty calls and argument errors of the block codec, the cache-level
    re-quantization and the merge."""
    import torch
    from turboquant_plus_b200.paged import merge_attention
    rng = np.random.default_rng(5)
    n, hkv = 40, 2
    cache = tq.PagedKVCache(D, hkv, num_pages=2, k_format="turbo3", v_format="turbo3", seed=42)
    x = torch.as_tensor(rng.standard_normal((n, hkv, D)).astype(np.float16)).cuda()
    cache.append(x, x, torch.arange(n))
    slots = torch.arange(n)
    slots[3] = -1
    slots[17] = -5
    blocks = cache.export_blocks("k", slots, 32)
    assert (blocks[3] == 0).all() and (blocks[17] == 0).all() and (blocks[4] != 0).any()
    full = cache.export_blocks("k", torch.arange(n), 32)
    keep = [i for i in range(n) if i not in (3, 17)]
    assert torch.equal(blocks[keep], full[keep])
    other = tq.PagedKVCache(D, hkv, num_pages=2, k_format="turbo3", v_format="turbo3", seed=42)
    other.import_blocks("k", blocks, slots, 32)
    L = cache.layout
    a, b = cache.pool.cpu().numpy()[0, 0], other.pool.cpu().numpy()[0, 0]
    assert np.array_equal(a[L.k_idx_off + 4 * 48: L.k_idx_off + 5 * 48], b[L.k_idx_off + 4 * 48: L.k_idx_off + 5 * 48])
    assert not b[L.k_idx_off + 3 * 48: L.k_idx_off + 4 * 48].any()        # skipped on import: record untouched
    assert tuple(cache.export_blocks("v", torch.zeros(0, dtype=torch.int64), 128).shape) == (0, hkv, 1, 50)
    with pytest.raises(ValueError):
        cache.export_blocks("k", slots, 48)
    with pytest.raises(ValueError):
        other.import_blocks("k", blocks[:5], slots, 32)
    q8 = tq.PagedKVCache(D, hkv, num_pages=2, k_format="q8_0", v_format="turbo3", seed=42)
    with pytest.raises(ValueError):
        q8.block_bytes("k", 32)
    # cache-level re-quantization: skipped tokens leave the destination untouched
    cold = tq.PagedKVCache(D, hkv, num_pages=2, k_format="turbo2", v_format="turbo2", seed=42)
    cache.decay_into(cold, slots, torch.arange(n))
    c = cold.pool.cpu().numpy()[0, 0]
    Lc = cold.layout
    assert not c[Lc.k_idx_off + 3 * 32: Lc.k_idx_off + 4 * 32].any() and c[Lc.k_idx_off + 4 * 32: Lc.k_idx_off + 5 * 32].any()
    cache.decay_into(cold, torch.zeros(0, dtype=torch.int64), torch.zeros(0, dtype=torch.int64))
    with pytest.raises(ValueError):
        cache.decay_into(cold, slots, torch.arange(n - 1))
    wrong_seed = tq.PagedKVCache(D, hkv, num_pages=2, k_format="turbo2", v_format="turbo2", seed=43)
    with pytest.raises(ValueError):
        cache.decay_into(wrong_seed, slots, torch.arange(n))
    with pytest.raises(tq._native.TQError):
        q8.decay_into(cold, slots, torch.arange(n))
    # merge: equal log-sum-exps average, fp16 and fp32, in place
    for dt in (torch.float16, torch.float32, torch.bfloat16):
        oa = torch.randn((3, 4, D), device="cuda").to(dt)
        ob = torch.randn((3, 4, D), device="cuda").to(dt)
        la = torch.tensor([[0.0, 1.0, -2.0, 5.0]] * 3, device="cuda")
        lb = torch.tensor([[0.0, -1.0, 2.0, float("-inf")]] * 3, device="cuda")
        got, lse = merge_attention(oa, la, ob, lb)
        wa = torch.exp(la - torch.logaddexp(la, lb))[..., None]
        want = oa.float() * wa + ob.float() * (1 - wa)
        assert (got.float() - want).abs().max() < (1e-5 if dt == torch.float32 else 2e-2)
        assert torch.allclose(lse, torch.logaddexp(la, lb), atol=1e-5)
        inplace, _ = merge_attention(oa, la, ob, lb, out=oa)
        assert inplace.data_ptr() == oa.data_ptr() and torch.equal(inplace, got)
