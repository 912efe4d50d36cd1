"""tq_decode_attn_static: decode attention for callers that cannot allocate device memory.

Such callers (a plugin inside a server whose pool owns all of HBM, a loop that cannot take
cudaMalloc's device-wide synchronisation, a foreign-language host with pointers but no allocator)
pass only inputs and outputs; the scratch is an 8 MiB array compiled into the library.  The test
calls the entry point through the C ABI twice in a row -- the second call with other queries and
lengths, so that it runs over whatever the first left in the shared array -- and compares each
result with the regular entry point fed a caller-owned workspace.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import tq_oracle as o
from tests.helpers import D, fill_cache, max_rel

pytestmark = pytest.mark.gpu


def _decode(cache, name, q, bt, sl, out, ws=None):
    import torch
    from turboquant_plus_b200 import _native as nv
    lib = nv.load()
    head = [cache._handle(cache.k_quantizer), cache._handle(cache.v_quantizer), C.byref(cache.layout),
            nv.ptr(cache.pool), nv.ptr(bt), bt.shape[1], nv.ptr(sl), nv.ptr(q), nv.torch_dtype_code(q.dtype),
            q.shape[0], q.shape[1], 0.0]
    tail = [nv.ptr(out), nv.torch_dtype_code(out.dtype), nv.stream_ptr()]
    mid = [] if ws is None else [nv.ptr(ws), ws.numel()]
    rc = getattr(lib, name)(*head, *mid, *tail)
    torch.cuda.synchronize()
    return rc


def test_static_scratch_matches_workspace_entry_point_twice():
    import torch
    import turboquant_plus_b200 as tq
    from turboquant_plus_b200 import _native as nv
    rng = np.random.default_rng(17)
    hkv, g = 2, 4
    seq_lens = [700, 129, 1, 380]
    cache = tq.PagedKVCache(D, hkv, num_pages=16, seed=42)
    ks = [np.stack([o.synth_keys(n, seed=3 * b + h) for h in range(hkv)], axis=1) for b, n in enumerate(seq_lens)]
    vs = [rng.standard_normal((n, hkv, D)).astype(np.float32) for n in seq_lens]
    bt = fill_cache(cache, ks, vs, seq_lens, rng).cuda()
    ws = cache.workspace(len(seq_lens), hkv * g, bt.shape[1])
    for call, lens in enumerate((seq_lens, [64, 129, 1, 0])):          # second call: other lengths, one empty
        q = torch.as_tensor(rng.standard_normal((len(lens), hkv * g, D)).astype(np.float32)).cuda()
        sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        ref = torch.full_like(q, float("nan"))
        got = torch.full_like(q, float("nan"))
        assert _decode(cache, "tq_decode_attn", q, bt, sl, ref, ws) == 0
        assert _decode(cache, "tq_decode_attn_static", q, bt, sl, got) == 0, nv.load().tq_last_error()
        live = [i for i, n in enumerate(lens) if n > 0]
        err = max_rel(got[live].cpu().numpy(), ref[live].cpu().numpy())
        print(f"call {call}: max-rel difference to tq_decode_attn {err:.1e}")
        assert err < 2e-3                      # the tolerance of the attention tests ...
        assert torch.equal(got, ref)           # ... and in fact the same bits: same kernels, same split order
        assert torch.isfinite(got).all()
        # the shared array has a status word of its own: no bounded wait gave up in either call
        st = C.c_int32(-1)
        assert nv.load().tq_decode_static_status_sync(C.byref(st)) == 0 and st.value == 0


def test_static_scratch_refuses_shapes_beyond_its_size():
    import torch
    import turboquant_plus_b200 as tq
    from turboquant_plus_b200 import _native as nv
    cache = tq.PagedKVCache(D, 8, num_pages=2, seed=42)
    batch, hq, pages = 256, 32, 256                        # needs ~34 MB of scratch
    assert nv.load().tq_decode_workspace_bytes(batch, hq, 8, pages) > 8 * 1024 * 1024
    q = torch.zeros((batch, hq, D), device="cuda")
    out = torch.empty_like(q)
    bt = torch.zeros((batch, pages), dtype=torch.int32, device="cuda")
    sl = torch.zeros((batch,), dtype=torch.int32, device="cuda")
    assert _decode(cache, "tq_decode_attn_static", q, bt, sl, out) == -5          # TQ_ERR_TOO_LARGE
    msg = nv.load().tq_last_error().decode()
    assert "8388608" in msg and "tq_decode_attn" in msg
