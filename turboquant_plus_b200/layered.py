"""A stack of per-layer paged caches with a per-layer (K format, V format) table, and a decode step
that takes host buffers: copy in, quantize-on-append + attention for every layer (one CUDA graph),
copy out.  Covers asymmetric K/V formats and boundary layers kept at higher precision
(the reference's layer-aware policy: docs/papers/layer-aware-v-compression.md:25-28).
"""
from __future__ import annotations

from . import _native as nv
from .paged import PagedKVCache


def boundary_format_table(num_layers: int, inner=("q8_0", "turbo2"), boundary=("q8_0", "q8_0"), keep: int = 2):
    """First and last ``keep`` layers use ``boundary``, the rest ``inner``."""
    return [boundary if (i < keep or i >= num_layers - keep) else inner for i in range(num_layers)]


class LayeredKVCache:
    def __init__(self, num_layers: int, head_dim: int, num_kv_heads: int, num_pages: int, page_tokens: int = 128,
                 formats=("turbo3", "turbo3"), seed: int = 42, norm_correction: bool = True,
                 rotation: str = "wht", device=None):
        if isinstance(formats[0], str):
            formats = [tuple(formats)] * num_layers
        assert len(formats) == num_layers
        self.formats = [tuple(f) for f in formats]
        # Layers of one (K format, V format) pair share the quantizers and one pool tensor: layer j of the group owns
        # pages [j * num_pages, (j + 1) * num_pages) of it.  `groups` holds, per pair, a cache object over the whole
        # tensor, through which one launch appends a token to every layer of the group.
        self.layers = [None] * num_layers
        self.groups = []
        by_format = {}
        for i, fmt in enumerate(self.formats):
            by_format.setdefault(fmt, []).append(i)
        for (kf, vf), members in by_format.items():
            whole = PagedKVCache(head_dim, num_kv_heads, num_pages * len(members), page_tokens, kf, vf, seed=seed,
                                 norm_correction=norm_correction, rotation=rotation, device=device)
            for j, i in enumerate(members):
                self.layers[i] = PagedKVCache(head_dim, num_kv_heads, num_pages, page_tokens, kf, vf, seed=seed,
                                              norm_correction=norm_correction, rotation=rotation, device=device,
                                              k_quantizer=whole.k_quantizer, v_quantizer=whole.v_quantizer,
                                              pool=whole.pool[j * num_pages:(j + 1) * num_pages])
            self.groups.append((whole, members))
        self.num_pages = num_pages
        self.device = self.layers[0].device
        self.num_layers, self.head_dim, self.num_kv_heads = num_layers, head_dim, num_kv_heads
        self.page_tokens = page_tokens
        self._step = None

    def bytes_per_token_all_layers(self) -> int:
        return sum(layer.bytes_per_token for layer in self.layers)

    def append(self, layer: int, k, v, slot_mapping):
        self.layers[layer].append(k, v, slot_mapping)

    def attend(self, layer: int, q, block_table, seq_lens, **kw):
        return self.layers[layer].attend(q, block_table, seq_lens, **kw)

    # ------------------------------------------------------------------------------------------
    def prepare_decode(self, batch: int, num_q_heads: int, block_table, seq_lens, dtype=None):
        """Allocates the static device buffers of a decode step and captures the per-layer launches
        (append one token per sequence, attend) into one CUDA graph.  ``block_table`` must already hold
        a page for position seq_lens[b] of every sequence."""
        torch = nv.require_cuda()
        dtype = dtype or torch.float16
        dev, L, d = self.device, self.num_layers, self.head_dim
        # q, k and v of a step are three views of one buffer, so that host buffers laid out the same way
        # (host_buffers()) arrive with a single copy
        nq, nk = L * batch * num_q_heads * d, L * batch * self.num_kv_heads * d
        qkv = torch.zeros((nq + 2 * nk,), dtype=dtype, device=dev)
        st = {
            "qkv": qkv,
            "q": qkv[:nq].view(L, batch, num_q_heads, d),
            "k": qkv[nq:nq + nk].view(L, batch, self.num_kv_heads, d),
            "v": qkv[nq + nk:].view(L, batch, self.num_kv_heads, d),
            "out": torch.zeros((L, batch, num_q_heads, d), dtype=dtype, device=dev),
            "bt": block_table.to(device=dev, dtype=torch.int32).contiguous(),
            "len": seq_lens.to(device=dev, dtype=torch.int32).clone(),
            # slots of the step's new tokens, once per layer of the largest format group: layer l of a group has its
            # pages at l * num_pages in the group's pool
            "slots": torch.zeros((max(len(m) for _, m in self.groups), batch), dtype=torch.int64, device=dev),
        }
        ws = self.layers[0].workspace(batch, num_q_heads, st["bt"].shape[1])

        # per format group: which layers, and where each layer's pages start inside the group's pool
        plans = []
        for whole, members in self.groups:
            idx = None if members == list(range(L)) else torch.tensor(members, device=dev)
            plans.append((whole, idx, len(members)))

        def append_part():
            # slots of the new tokens and the lengths' increment: one launch
            with torch.cuda.device(dev):
                nv.call("tq_decode_step_slots", nv.ptr(st["bt"]), st["bt"].shape[1], nv.ptr(st["len"]), self.page_tokens,
                        batch, st["slots"].shape[0], self.num_pages * self.page_tokens, nv.ptr(st["slots"]),
                        nv.stream_ptr())
            # one quantize-on-append launch per format group: the new token of every layer of the group at once
            for whole, idx, n in plans:
                k = st["k"] if idx is None else st["k"].index_select(0, idx)
                v = st["v"] if idx is None else st["v"].index_select(0, idx)
                whole.append(k.reshape(n * batch, self.num_kv_heads, d), v.reshape(n * batch, self.num_kv_heads, d),
                             st["slots"][:n].reshape(-1))

        def attend_part(lo, hi):
            for i in range(lo, hi):
                layer = self.layers[i]
                # An attention call that follows another layer's attention call may start early: that kernel writes
                # nothing this one reads before its dependency wait, and the queries of every layer are in place
                # before the first launch of the step (they arrive with the step's host-to-device copy).  The first
                # call follows the append, which writes the cache slot of the new token: it runs in stream order, in
                # the form of the calls that follow it.
                layer.attend(st["q"][i], st["bt"], st["len"], out=st["out"][i], workspace=ws,
                             overlap="q" if i > 0 else False, chain_head=(i == 0))

        def body():
            append_part()
            attend_part(0, L)

        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):      # warm-up outside capture (sets kernel attributes, fills caches)
            saved = st["len"].clone()
            body()
            st["len"].copy_(saved)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            body()
        st["len"].copy_(saved)
        st["graph"] = graph
        st["body"] = body
        st["parts"] = (append_part, attend_part)
        st["io_stream"] = side
        self._step = st
        return st

    def host_buffers(self):
        """Pinned host tensors (q, k, v, out) for decode_step, q/k/v carved from one allocation in the order of the
        device buffers: a step then needs one host-to-device copy instead of three."""
        torch = nv.require_cuda()
        st = self._step
        flat = torch.zeros(st["qkv"].shape, dtype=st["qkv"].dtype).pin_memory()
        nq, nk = st["q"].numel(), st["k"].numel()
        out = torch.zeros(st["out"].shape, dtype=st["out"].dtype).pin_memory()
        return (flat[:nq].view(st["q"].shape), flat[nq:nq + nk].view(st["k"].shape), flat[nq + nk:].view(st["v"].shape), out)

    def _copy_in(self, q_host, k_host, v_host):
        st = self._step
        esz = q_host.element_size()
        if (q_host.is_contiguous() and k_host.is_contiguous() and v_host.is_contiguous()
                and k_host.data_ptr() == q_host.data_ptr() + q_host.numel() * esz
                and v_host.data_ptr() == k_host.data_ptr() + k_host.numel() * esz
                and q_host.dtype == st["qkv"].dtype and q_host.numel() == st["q"].numel()):
            flat = q_host.reshape(-1).as_strided((st["qkv"].numel(),), (1,))     # the three views as one extent
            st["qkv"].copy_(flat, non_blocking=True)
        else:
            st["q"].copy_(q_host, non_blocking=True)
            st["k"].copy_(k_host, non_blocking=True)
            st["v"].copy_(v_host, non_blocking=True)

    def decode_step(self, q_host, k_host, v_host, out_host):
        """One decode step from host buffers (tensors shaped like the static device buffers): H2D of the step's
        queries and new K/V rows, the captured launches, D2H of the outputs.  With pinned buffers the copies are
        nodes of the same graph as the kernels, captured the first time a set of buffers is seen, so that a step
        is one graph launch and one synchronisation; pass the same buffers every step."""
        torch = nv.require_cuda()
        st = self._step
        hosts = (q_host, k_host, v_host, out_host)
        key = (q_host.data_ptr(), k_host.data_ptr(), v_host.data_ptr(), out_host.data_ptr())
        # (buffers seen before are known to be pinned: the query of that attribute costs microseconds per tensor)
        if st.get("io_key") == key or all(t.is_pinned() for t in hosts):
            if st.get("io_key") != key:
                graph = torch.cuda.CUDAGraph()
                append_part, attend_part = st["parts"]
                side, half = st["io_stream"], self.num_layers // 2
                with torch.cuda.graph(graph):
                    # The copies are branches of the graph.  In: the new K/V rows first, then the queries on a side
                    # branch under the append, which needs only the rows.  Out: the outputs of the lower half of the
                    # layers leave while the upper half is still computing.
                    main = torch.cuda.current_stream(self.device)
                    nq, nk = st["q"].numel(), st["k"].numel()
                    if (k_host.is_contiguous() and v_host.is_contiguous() and k_host.dtype == st["qkv"].dtype
                            and k_host.numel() == nk and v_host.numel() == nk
                            and v_host.data_ptr() == k_host.data_ptr() + nk * k_host.element_size()):
                        # rows of K and V adjacent on the host (host_buffers()): one copy
                        st["qkv"][nq:].copy_(k_host.reshape(-1).as_strided((2 * nk,), (1,)), non_blocking=True)
                    else:
                        st["k"].copy_(k_host, non_blocking=True)
                        st["v"].copy_(v_host, non_blocking=True)
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        st["q"].copy_(q_host, non_blocking=True)
                    append_part()
                    main.wait_stream(side)
                    attend_part(0, half)
                    side.wait_stream(main)
                    with torch.cuda.stream(side):
                        out_host[:half].copy_(st["out"][:half], non_blocking=True)
                    attend_part(half, self.num_layers)
                    out_host[half:].copy_(st["out"][half:], non_blocking=True)
                    main.wait_stream(side)
                st["io_graph"], st["io_key"], st["io_refs"] = graph, key, hosts   # the graph holds raw host pointers
            st["io_graph"].replay()
        else:
            self._copy_in(q_host, k_host, v_host)
            st["graph"].replay()
            out_host.copy_(st["out"], non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return out_host
