"""Caller-side adapters: what a model's attention code touches.

* ``quant_dequant_keys`` / ``patch_model_attention`` / ``unpatch_model``: the reference's real-model validation
  hook (benchmarks/benchmark_norm_correction.py:45-96): every layer's ``k_proj`` is wrapped so that the keys it
  produces go through quantize -> dequantize, one quantizer per KV head (seed = head index).  Here the tensors
  never leave the GPU and a head's quantizer is built once, not once per call.
* ``TurboQuantCache``: a cache object shaped like the ``update`` / ``get_seq_length`` protocol of transformer
  libraries, backed by the paged compressed cache: ``update`` quantizes the new K/V rows into pages, ``attend``
  runs decode (one query position) or chunked-prefill attention straight off the packed pages, so the
  dequantized cache is never materialised.
"""
from __future__ import annotations

from . import _native as nv
from .layered import LayeredKVCache


def quant_dequant_keys(key_states, quantizer_factory, _cache=None):
    """key_states: (B, H, S, D) CUDA tensor.  Head h goes through ``quantizer_factory(D, seed=h)`` -- any object with
    the PolarQuant / TurboQuantMSE ``quantize`` / ``dequantize`` pair -- and comes back in the input's dtype
    (benchmarks/benchmark_norm_correction.py:45-58)."""
    torch = nv.require_cuda()
    B, H, S, D = key_states.shape
    out = torch.empty_like(key_states)
    for h in range(H):
        if _cache is not None and h in _cache:
            q = _cache[h]
        else:
            q = quantizer_factory(D, seed=h)
            if _cache is not None:
                _cache[h] = q
        rows = key_states[:, h].reshape(B * S, D).float()
        indices, norms = q.quantize(rows)
        out[:, h] = q.dequantize(indices, norms).reshape(B, S, D).to(key_states.dtype)
    return out


def patch_model_attention(model, quant_factory):
    """Wraps ``layer.self_attn.k_proj`` of every decoder layer (benchmarks/benchmark_norm_correction.py:62-91).
    Returns the hooks ``unpatch_model`` needs."""
    torch = nv.require_cuda()
    head_dim = model.config.hidden_size // model.config.num_attention_heads
    num_kv_heads = model.config.num_key_value_heads

    class QuantizedKProj(torch.nn.Module):
        def __init__(self, orig):
            super().__init__()
            self.orig = orig
            self.quantizers = {}

        def forward(self, x):
            k = self.orig(x)
            B, S, _ = k.shape
            k4 = k.view(B, S, num_kv_heads, head_dim).permute(0, 2, 1, 3)
            k4 = quant_dequant_keys(k4, quant_factory, self.quantizers)
            return k4.permute(0, 2, 1, 3).reshape(B, S, -1)

    hooks = []
    for layer in model.model.layers:
        attn = layer.self_attn
        original = attn.k_proj
        attn.k_proj = QuantizedKProj(original)
        hooks.append((attn, original))
    return hooks


def unpatch_model(hooks):
    """benchmarks/benchmark_norm_correction.py:94-96."""
    for attn, orig in hooks:
        attn.k_proj = orig


class TurboQuantCache:
    """Compressed KV cache behind the (key_states, value_states, layer_idx) protocol.  Every sequence of the batch
    owns ``ceil(max_seq_len / page_tokens)`` pages; all sequences advance together (same number of new tokens per
    ``update``), as in a padded batch.

        cache = TurboQuantCache(num_layers, head_dim, num_kv_heads, max_batch=2, max_seq_len=4096)
        cache.update(k, v, layer_idx)          # k, v: (B, Hkv, S_new, D)
        out = cache.attend(q, layer_idx)       # q: (B, Hq, S_new, D) -> (B, Hq, S_new, D), causal within the chunk
    """

    def __init__(self, num_layers: int, head_dim: int, num_kv_heads: int, max_batch: int, max_seq_len: int,
                 formats=("turbo3", "turbo3"), page_tokens: int = 128, seed: int = 42, device=None):
        torch = nv.require_cuda()
        self.page_tokens = page_tokens
        self.pages_per_seq = (max_seq_len + page_tokens - 1) // page_tokens
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.store = LayeredKVCache(num_layers, head_dim, num_kv_heads, max_batch * self.pages_per_seq, page_tokens,
                                    formats=formats, seed=seed, device=device)
        self.device = self.store.device
        self.block_table = torch.arange(max_batch * self.pages_per_seq, dtype=torch.int32,
                                        device=self.device).reshape(max_batch, self.pages_per_seq)
        self._seen = [0] * num_layers

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen[layer_idx]

    def update(self, key_states, value_states, layer_idx: int):
        """Appends S_new positions per sequence to layer ``layer_idx``.  Returns the new sequence length."""
        torch = nv.require_cuda()
        B, H, S, D = key_states.shape
        start = self._seen[layer_idx]
        if B > self.max_batch or start + S > self.max_seq_len:
            raise ValueError(f"cache holds {self.max_batch} sequences of {self.max_seq_len} positions; "
                             f"got batch {B}, positions {start}..{start + S}")
        pos = torch.arange(start, start + S, device=self.device, dtype=torch.int64)
        page = self.block_table[:B].to(torch.int64)[:, pos // self.page_tokens]          # (B, S)
        slots = (page * self.page_tokens + pos % self.page_tokens).reshape(-1)
        k = key_states.permute(0, 2, 1, 3).reshape(B * S, H, D)
        v = value_states.permute(0, 2, 1, 3).reshape(B * S, H, D)
        self.store.append(layer_idx, k, v, slots)
        self._seen[layer_idx] = start + S
        return self._seen[layer_idx]

    def attend(self, query_states, layer_idx: int, scale=None):
        """query_states: (B, Hq, S_q, D), the queries of the last S_q cached positions.  One position: the decode
        kernel; more: the chunked-prefill kernel (query i sees positions 0 .. len - S_q + i)."""
        torch = nv.require_cuda()
        B, Hq, S, D = query_states.shape
        n = self._seen[layer_idx]
        lens = torch.full((B,), n, dtype=torch.int32, device=self.device)
        bt = self.block_table[:B]
        layer = self.store.layers[layer_idx]
        if S == 1:
            out = layer.attend(query_states[:, :, 0], bt, lens, scale=scale)
            return out.unsqueeze(2)
        q = query_states.permute(0, 2, 1, 3).contiguous()                                # (B, S, Hq, D)
        return layer.prefill_attend(q, bt, lens, scale=scale).permute(0, 2, 1, 3)
