"""Paged compressed KV cache: quantize-on-append and decode attention straight off the packed pages.

New surface (the reference's KVCacheCompressor only has bulk compress / decompress; the streaming
``compress_token`` its docstring names, turboquant/kv_cache.py:65-66, is never defined).  One object is
one layer's cache; K and V formats are chosen per layer:

    "turbo2" | "turbo3" | "turbo4"   b-bit PolarQuant, MSE-only (TurboQuantMSE), fp32 scale per vector
    "prod2"  | "prod3"  | "prod4"    (b-1)-bit PolarQuant + 1-bit QJL sketch (TurboQuant), K only
    "q8_0"                            int8 with an fp16 scale per 32 values

The attention computed is the reference tests' dequantize-then-attend
(tests/test_kv_cache.py:73-89): softmax(q k_hat^T / sqrt(d)) v_hat, per sequence and query head.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np

from . import _native as nv
from .polar_quant import PolarQuant
from .turboquant import TurboQuant


def _fmt_bits(fmt: str) -> int:
    return int(fmt[-1])


class PagedKVCache:
    def __init__(self, head_dim: int, num_kv_heads: int, num_pages: int, page_tokens: int = 128,
                 k_format: str = "turbo3", v_format: str = "turbo3", seed: int = 42,
                 norm_correction: bool = True, rotation: str = "wht", device=None,
                 k_quantizer=None, v_quantizer=None, pool=None):
        torch = nv.require_cuda()
        if k_format not in nv.FORMATS or v_format not in nv.FORMATS:
            raise ValueError(f"unknown cache format {k_format!r} / {v_format!r}")
        if v_format.startswith("prod"):
            raise ValueError("V is stored MSE-only (turboN) or q8_0; the QJL sketch is a K format")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.head_dim, self.num_kv_heads, self.num_pages, self.page_tokens = head_dim, num_kv_heads, num_pages, page_tokens
        self.k_format, self.v_format = k_format, v_format
        self.layout = nv.CacheLayout()
        nv.call("tq_cache_layout_init", C.byref(self.layout), head_dim, page_tokens, num_kv_heads,
                nv.FORMATS[k_format], nv.FORMATS[v_format])
        # K uses the compressor's seed, V seed + 500, QJL seed + 1000 (turboquant/kv_cache.py:89-96,
        # turboquant/turboquant.py:77)
        if k_quantizer is None and k_format != "q8_0":
            if k_format.startswith("prod"):
                k_quantizer = TurboQuant(head_dim, _fmt_bits(k_format), seed=seed, norm_correction=norm_correction,
                                         rotation=rotation, device=self.device)
            else:
                k_quantizer = PolarQuant(head_dim, _fmt_bits(k_format), seed=seed, norm_correction=norm_correction,
                                         rotation=rotation, device=self.device)
        if v_quantizer is None and v_format != "q8_0":
            v_quantizer = PolarQuant(head_dim, _fmt_bits(v_format), seed=seed + 500, norm_correction=norm_correction,
                                     rotation=rotation, device=self.device)
        self.k_quantizer, self.v_quantizer = k_quantizer, v_quantizer
        if pool is None:
            pool = torch.zeros((num_pages, num_kv_heads, self.layout.record_bytes), dtype=torch.uint8, device=self.device)
        elif tuple(pool.shape) != (num_pages, num_kv_heads, self.layout.record_bytes) or not pool.is_contiguous():
            raise ValueError("pool must be a contiguous uint8 tensor of shape (num_pages, num_kv_heads, record bytes)")
        self.pool = pool        # may be a slice of a larger tensor that several caches share (LayeredKVCache)
        self._ws = None
        self._dummy = None

    # bytes one cached token of one KV head occupies (K + V), the figure roofline arithmetic uses
    @property
    def bytes_per_token(self) -> int:
        L = self.layout
        def tensor(fmt, idx_bytes):
            if fmt == "q8_0":
                return idx_bytes + (self.head_dim // 32) * 2
            return idx_bytes + 4 + ((self.head_dim // 8 + 4) if fmt.startswith("prod") else 0)
        return tensor(self.k_format, L.k_idx_bytes) + tensor(self.v_format, L.v_idx_bytes)

    def _handle(self, quantizer):
        if quantizer is None:
            return self._placeholder().handle
        return quantizer._native(self.device).handle

    def _placeholder(self):
        """q8_0 tensors need no codebook; the attention entry point still takes the rotation, which for
        q8_0 is the identity."""
        if self._dummy is None:
            self._dummy = nv.Quantizer(self.head_dim, 1, nv.ROT_DENSE, False, np.array([-1.0, 1.0]),
                                       rot=np.eye(self.head_dim), device=self.device)
        return self._dummy

    def append(self, k, v, slot_mapping):
        """k, v: (n_tokens, num_kv_heads, head_dim) CUDA tensors (fp16, bf16 or fp32);
        slot_mapping: (n_tokens,) int64, page * page_tokens + offset, negative = skip."""
        torch = nv.require_cuda()
        k, v = k.contiguous(), v.contiguous()
        n = k.shape[0]
        assert k.shape == v.shape == (n, self.num_kv_heads, self.head_dim)
        assert k.dtype == v.dtype
        slots = slot_mapping.to(device=self.device, dtype=torch.int64).contiguous()
        wht_ok = all(q is None or q._native(self.device).rotation == nv.ROT_WHT
                     for q in (self.k_quantizer, self.v_quantizer))
        with torch.cuda.device(self.device):
            if wht_ok:
                nv.call("tq_cache_append", self._handle(self.k_quantizer) if self.k_quantizer else None,
                        self._handle(self.v_quantizer) if self.v_quantizer else None, C.byref(self.layout),
                        nv.ptr(self.pool), nv.ptr(k), nv.ptr(v), nv.torch_dtype_code(k.dtype), n, nv.ptr(slots),
                        nv.stream_ptr())
                return
            # dense-rotation quantizers: quantize into rows, then scatter the rows into the pages
            for which, (x, quant, fmt) in enumerate(((k, self.k_quantizer, self.k_format),
                                                     (v, self.v_quantizer, self.v_format))):
                rows = x.reshape(n * self.num_kv_heads, self.head_dim)
                if fmt == "q8_0":
                    raise nv.TQError("mixing q8_0 with dense-rotation quantizers in one cache is not built")
                if rows.dtype == torch.bfloat16:
                    rows = rows.float()
                out = quant.quantize_device(rows, packed=True, want_scale=True)
                qjl = rscale = None
                if fmt.startswith("prod"):
                    qjl = out["qjl"]
                    rscale = out["rnorm"] * (math.sqrt(math.pi / 2) / math.sqrt(self.head_dim))
                nv.call("tq_cache_store", C.byref(self.layout), nv.ptr(self.pool), which, nv.ptr(out["packed"]),
                        nv.ptr(out["scale"]), nv.ptr(qjl), nv.ptr(rscale), n, nv.ptr(slots), nv.stream_ptr())

    def workspace(self, batch: int, num_q_heads: int, max_pages: int):
        torch = nv.require_cuda()
        need = nv.load().tq_decode_workspace_bytes(batch, num_q_heads, self.num_kv_heads, max_pages)
        nv.check(int(need))
        if self._ws is None or self._ws.numel() < need:
            # zero-filled: the ticket counters at the end of a workspace must start at zero
            self._ws = torch.zeros((int(need),), dtype=torch.uint8, device=self.device)
        return self._ws

    def attend(self, q, block_table, seq_lens, scale=None, out=None, workspace=None, phases=7, overlap=False,
               sparse_v=False, return_lse=False, chain_head=False):
        """q: (batch, num_q_heads, head_dim) CUDA tensor; block_table: (batch, max_pages) int32 page
        numbers; seq_lens: (batch,) int32.  Returns (batch, num_q_heads, head_dim) in q's dtype.

        overlap=True lets the kernel start while the preceding kernel of the stream is still running; until
        that kernel has completed it only reads cache pages, the block table and the sequence lengths.  Use it
        only when the preceding kernel writes none of those (another layer's attention call); after an append
        into this cache launch in stream order (overlap=False).  overlap="q" says in addition that the preceding
        kernel does not write ``q`` either (a chain of calls whose queries all exist beforehand): the kernel then
        waits for its predecessor only before it writes.  overlap="append" is for the call that follows the append
        of the step's new token into this cache: of what the call reads, the preceding kernel writes only the last
        position of each sequence; every other page is streamed while it runs.  chain_head=True is a hint for a call
        in stream order that is followed by calls with overlap="q" (the first layer of a step).

        return_lse=True returns (out, lse) with lse (batch, num_q_heads) fp32, the natural log of the softmax
        denominator: what merge_attention needs to join calls over disjoint parts of a sequence."""
        if overlap:   # "q": the preceding kernel does not write the queries either (they are read early too)
            phases = int(phases) | (nv.DECODE_OVERLAP_Q if overlap == "q" else
                                    nv.DECODE_OVERLAP_APPEND if overlap == "append" else nv.DECODE_OVERLAP)
        if chain_head:
            phases = int(phases) | nv.DECODE_CHAIN_HEAD
        if sparse_v:  # skip V work where every weight of a 16-token tile is below 1e-6 (the reference's sparse V)
            phases = int(phases) | nv.DECODE_SPARSE_V
        torch = nv.require_cuda()
        q = q.contiguous()
        bsz, hq, d = q.shape
        assert d == self.head_dim
        bt = block_table.to(device=self.device, dtype=torch.int32).contiguous()
        sl = seq_lens.to(device=self.device, dtype=torch.int32).contiguous()
        ws = self.workspace(bsz, hq, bt.shape[1]) if workspace is None else workspace
        if out is None:
            out = torch.empty_like(q)
        with torch.cuda.device(self.device):
            if return_lse:
                lse = torch.empty((bsz, hq), dtype=torch.float32, device=self.device)
                nv.call("tq_decode_attn_lse", self._handle(self.k_quantizer), self._handle(self.v_quantizer),
                        C.byref(self.layout), nv.ptr(self.pool), nv.ptr(bt), bt.shape[1], nv.ptr(sl), nv.ptr(q),
                        nv.torch_dtype_code(q.dtype), bsz, hq, float(scale) if scale else 0.0, nv.ptr(ws), ws.numel(),
                        nv.ptr(out), nv.torch_dtype_code(out.dtype), int(phases), nv.ptr(lse), nv.stream_ptr())
                return out, lse
            nv.call("tq_decode_attn_phases", self._handle(self.k_quantizer), self._handle(self.v_quantizer),
                    C.byref(self.layout), nv.ptr(self.pool), nv.ptr(bt), bt.shape[1], nv.ptr(sl), nv.ptr(q),
                    nv.torch_dtype_code(q.dtype), bsz, hq, float(scale) if scale else 0.0, nv.ptr(ws), ws.numel(),
                    nv.ptr(out), nv.torch_dtype_code(out.dtype), int(phases), nv.stream_ptr())
        return out

    def decay_into(self, dst: "PagedKVCache", src_slots, dst_slots):
        """Temporal decay at cache level (benchmarks/temporal_decay_prototype.py:93-125): the K and V codes of the
        tokens at ``src_slots`` of this cache are re-quantized, in the rotated domain, into the records at
        ``dst_slots`` of ``dst``, a cache with narrower turboN formats built from the same seed.  The caller then
        frees the source pages and attends over both caches with ``attend(..., return_lse=True)`` +
        ``merge_attention``."""
        torch = nv.require_cuda()
        ss = src_slots.to(device=self.device, dtype=torch.int64).contiguous()
        ds = dst_slots.to(device=self.device, dtype=torch.int64).contiguous()
        if ss.numel() != ds.numel():
            raise ValueError("src_slots and dst_slots must name the same number of tokens")
        with torch.cuda.device(self.device):
            for which, (a, b) in enumerate(((self.k_quantizer, dst.k_quantizer), (self.v_quantizer, dst.v_quantizer))):
                if a is None or b is None:
                    raise nv.TQError("decay_into converts turboN tensors; q8_0 tensors have no narrower codebook")
                nv.call("tq_cache_requantize", self._handle(a), dst._handle(b), C.byref(self.layout), nv.ptr(self.pool),
                        nv.ptr(ss), C.byref(dst.layout), nv.ptr(dst.pool), nv.ptr(ds), which, ss.numel(), nv.stream_ptr())

    def prefill_attend(self, q, block_table, kv_lens, scale=None, out=None, workspace=None):
        """Chunked prefill on the tcgen05 tensor cores.  q: (batch, chunk_tokens, num_q_heads, head_dim) CUDA
        tensor of a chunk whose K/V rows are already in the cache; kv_lens: (batch,) cached tokens including
        the chunk.  Query i of a sequence sees cached positions 0 .. kv_len - chunk_tokens + i.  turbo2/3/4 K and V
        take the tcgen05 kernel; PROD or q8_0 tensors run the chunk's queries through the decode kernel."""
        torch = nv.require_cuda()
        q = q.contiguous()
        bsz, tq, hq, d = q.shape
        assert d == self.head_dim
        bt = block_table.to(device=self.device, dtype=torch.int32).contiguous()
        kl = kv_lens.to(device=self.device, dtype=torch.int32).contiguous()
        if not (self.k_format.startswith("turbo") and self.v_format.startswith("turbo")):
            # PROD and q8_0 tensors have no tensor-memory pipeline: every query of the chunk runs as a row of the decode
            # kernel with its own causal length (the cache is read once per query; the pages of a sequence stay in L2)
            lens = (kl[:, None] - tq + 1 + torch.arange(tq, device=self.device, dtype=torch.int32)[None, :]).clamp_(min=0)
            res = self.attend(q.reshape(bsz * tq, hq, d), bt.repeat_interleave(tq, dim=0), lens.reshape(-1), scale=scale)
            res = res.reshape(bsz, tq, hq, d)
            if out is not None:
                out.copy_(res)
                return out
            return res
        if workspace is None:
            need = int(nv.load().tq_prefill_workspace_bytes(bsz, tq, hq, self.num_kv_heads, bt.shape[1]))
            nv.check(need)
            if self._ws is None or self._ws.numel() < need:
                self._ws = torch.zeros((need,), dtype=torch.uint8, device=self.device)
            ws = self._ws
        else:
            ws = workspace
        if out is None:
            out = torch.empty_like(q)
        with torch.cuda.device(self.device):
            nv.call("tq_prefill_attn", self._handle(self.k_quantizer), self._handle(self.v_quantizer),
                    C.byref(self.layout), nv.ptr(self.pool), nv.ptr(bt), bt.shape[1], nv.ptr(kl), nv.ptr(q),
                    nv.torch_dtype_code(q.dtype), bsz, tq, hq, float(scale) if scale else 0.0, nv.ptr(ws), ws.numel(),
                    nv.ptr(out), nv.torch_dtype_code(out.dtype), nv.stream_ptr())
        return out

    # ---- wire / on-disk forms ---------------------------------------------------------------------------
    def block_bytes(self, which: str, block_elems: int = 128) -> int:
        fmt = self.k_format if which == "k" else self.v_format
        n = int(nv.load().tq_block_bytes(nv.FORMATS[fmt], block_elems))
        if n < 0:
            raise ValueError(f"no block format for {fmt} with {block_elems} elements per block")
        return n

    def export_blocks(self, which: str, slot_mapping, block_elems: int = 128):
        """The K ("k") or V ("v") codes of the tokens at ``slot_mapping`` in the block format the reference's
        documents describe for its llama.cpp fork (turbo3: fp16 norm, 2-bit plane, high-bit plane; turbo2; turbo4
        nibbles): uint8 CUDA tensor (n_tokens, num_kv_heads, 128 // block_elems, block bytes)."""
        torch = nv.require_cuda()
        bb = self.block_bytes(which, block_elems)
        slots = slot_mapping.to(device=self.device, dtype=torch.int64).contiguous()
        out = torch.empty((slots.numel(), self.num_kv_heads, self.head_dim // block_elems, bb), dtype=torch.uint8,
                          device=self.device)        # the kernel writes every byte (zeros for skipped tokens)
        with torch.cuda.device(self.device):
            nv.call("tq_cache_export_blocks", C.byref(self.layout), nv.ptr(self.pool), 0 if which == "k" else 1,
                    nv.ptr(slots), slots.numel(), block_elems, nv.ptr(out), nv.stream_ptr())
        return out

    def import_blocks(self, which: str, blocks, slot_mapping, block_elems: int = 128):
        """Inverse of export_blocks: writes the codes into the records of the tokens at ``slot_mapping``."""
        torch = nv.require_cuda()
        bb = self.block_bytes(which, block_elems)
        slots = slot_mapping.to(device=self.device, dtype=torch.int64).contiguous()
        blocks = blocks.to(device=self.device, dtype=torch.uint8).contiguous()
        if blocks.numel() != slots.numel() * self.num_kv_heads * (self.head_dim // block_elems) * bb:
            raise ValueError("block buffer does not match (n_tokens, num_kv_heads, 128 // block_elems, block bytes)")
        with torch.cuda.device(self.device):
            nv.call("tq_cache_import_blocks", C.byref(self.layout), nv.ptr(self.pool), 0 if which == "k" else 1,
                    nv.ptr(slots), slots.numel(), block_elems, nv.ptr(blocks), nv.stream_ptr())

    def state_dict(self) -> dict:
        """Everything needed to rebuild the cache contents elsewhere: geometry, formats and the pool bytes (host
        tensor).  Quantizer constants are not stored; they follow from the seed the cache is built with."""
        return {"head_dim": self.head_dim, "num_kv_heads": self.num_kv_heads, "num_pages": self.num_pages,
                "page_tokens": self.page_tokens, "k_format": self.k_format, "v_format": self.v_format,
                "record_bytes": int(self.layout.record_bytes), "pool": self.pool.cpu()}

    def load_state_dict(self, state: dict) -> None:
        for key in ("head_dim", "num_kv_heads", "num_pages", "page_tokens", "k_format", "v_format"):
            if state[key] != getattr(self, key):
                raise ValueError(f"cache state mismatch: {key} is {state[key]!r}, this cache has {getattr(self, key)!r}")
        if int(state["record_bytes"]) != int(self.layout.record_bytes):
            raise ValueError("cache state mismatch: record size")
        self.pool.copy_(state["pool"].to(self.device))

    def kernel_status(self, workspace=None) -> int:
        """0 after a clean decode; 1 if a bounded wait inside the kernel gave up (synchronises)."""
        ws = self._ws if workspace is None else workspace
        if ws is None:
            return 0
        st = C.c_int32(0)
        nv.call("tq_decode_status_sync", nv.ptr(ws), ws.numel(), C.byref(st))
        return st.value


def merge_attention(out_a, lse_a, out_b, lse_b, out=None):
    """Joins the attention outputs of two disjoint parts of a sequence from their log-sum-exps:
    (e^la a + e^lb b) / (e^la + e^lb).  Returns (out, lse); out may be one of the inputs."""
    torch = nv.require_cuda()
    out_a, out_b = out_a.contiguous(), out_b.contiguous()
    assert out_a.shape == out_b.shape and out_a.dtype == out_b.dtype and out_a.shape[-1] == 128
    rows = out_a.numel() // 128
    if out is None:
        out = torch.empty_like(out_a)
    lse = torch.empty((rows,), dtype=torch.float32, device=out_a.device)
    with torch.cuda.device(out_a.device):
        nv.call("tq_attn_merge", nv.ptr(out_a), nv.ptr(lse_a.contiguous()), nv.ptr(out_b), nv.ptr(lse_b.contiguous()), rows,
                nv.torch_dtype_code(out_a.dtype), nv.ptr(out), nv.ptr(lse), nv.stream_ptr())
    return out, lse.reshape(lse_a.shape)
