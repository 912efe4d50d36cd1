"""Benchmark of the TurboQuant+ hot path on B200: decode attention over a turbo3-compressed KV cache.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (N = 1): single-layer decode attention, Llama-3-8B shaped -- 32 query / 8 KV heads, d = 128,
batch 1, context 32,768, K and V stored as turbo3 (3-bit PolarQuant, fp32 scale: 52 B per vector), fp16
queries.  One cache is 27.3 MB and would sit in the 126 MB L2, so a step is one decode-attention pass over
each of LAYERS distinct layer caches of that shape (1.09 GB of packed cache per step, larger than L2).
Synthetic data: keys N(0,1) x lognormal(0, 0.5) per vector with 4 outlier channels x10 and a RoPE-style
rotation by position, values N(0,1), generated on the device from a fixed seed and written through the
quantize-on-append kernel.

value  = KV-tokens/s (one KV-token = one cached position of one KV head, its K and its V vector), whole job,
         cache resident in HBM, launches replayed from a CUDA graph, timed with CUDA events.
e2e    = the same metric through LayeredKVCache.decode_step with host buffers: every step copies the
         queries and the new token's K/V rows from pinned host memory, appends (quantizes) them, attends,
         and copies the outputs back.
With N > 1 ranks each rank owns its own sequence (batch sharding, no collective on the data path): weak scaling.

--impl reference times the reference's algorithm for this path on the host cores: dequantize the whole
compressed cache, then NumPy softmax attention (the reference's dequantize-then-attend), through the NumPy
port under oracle/ (the reference itself is a Python package that is not present on the GPU box).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D, HQ, HKV, CTX, PT = 128, 32, 8, 32768, 128
LAYERS = 40
BYTES_PER_KV_TOKEN = 104          # turbo3 K (48 + 4) + turbo3 V (48 + 4)
METRIC = "turbo3_decode_attn_kv_tokens_per_s"
UNIT = "KV-tokens/s"


_STDOUT_FD = None


def emit(record):
    """Writes one JSON line to the process's original stdout."""
    data = (json.dumps(record) + "\n").encode()
    if _STDOUT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_STDOUT_FD, data)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["bf16_tflops"]), "measured cuBLAS bf16 burst"
    return 1590.0, "fallback"


def head_start(torch):
    """Keeps the idle GPU busy for ~0.1 ms (a spin kernel: no memory traffic, the caches stay as they are) so that
    the host has enqueued the timed launches before the first event completes: the events then bracket the kernels
    and not the host's way to the first launch."""
    torch.cuda._sleep(200_000)


def prefill_probe(torch, tq, dev, gen):
    """Chunked prefill (tcgen05 kernel), Llama-3-70B head shape: one 128-query chunk x 64 query heads / 8 KV heads
    over a 16,384-token turbo3 cache of one layer.  FLOPs counted: the two contractions over the visible prefix."""
    hq, hkv, tq_len, n = 64, 8, 128, 16384
    cache = tq.PagedKVCache(D, hkv, n // PT, PT, "turbo3", "turbo3", seed=42, device=dev)
    k, v = synth_layer(torch, gen, dev, n, 0)
    cache.append(k, v, torch.arange(n, device=dev))
    bt = torch.arange(n // PT, device=dev, dtype=torch.int32)[None]
    kv_len = torch.tensor([n], dtype=torch.int32, device=dev)
    q = torch.randn((1, tq_len, hq, D), generator=gen, device=dev).half()
    out = torch.empty_like(q)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    flush = torch.empty((512 << 20,), dtype=torch.uint8, device=dev)   # four times the L2
    times = []
    for _ in range(8):
        torch.cuda.synchronize(dev)
        # The 13.6 MB cache would stay in L2 from one call to the next: a write of 512 MB in front of every timed
        # call evicts it, and while it runs the host enqueues the call, so that the events bracket the kernel and
        # not the host's way to the launch.
        flush.fill_(1)
        ev[0].record()
        cache.prefill_attend(q, bt, kv_len, out=out)
        ev[1].record()
        torch.cuda.synchronize(dev)
        times.append(ev[0].elapsed_time(ev[1]))
    del flush
    assert cache.kernel_status() == 0 and torch.isfinite(out.float()).all()
    ms = statistics.median(times[3:])
    visible = sum(n - tq_len + i + 1 for i in range(tq_len))       # cached positions seen by the chunk's queries
    flops = 2 * 2 * hq * D * visible
    peak, src = tensor_peak()
    return {"bound": "tensor", "kernel": "k_prefill_attn2<3,3> (tcgen05)", "achieved": flops / (ms * 1e-3) / 1e12,
            "peak": peak, "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / peak, "peak_source": src,
            "ms": ms, "row_blocks": (tq_len * hq // hkv // 128) * hkv, "l2": "flushed before every timed call",
            "workload": f"{tq_len}-query chunk, {hq}q/{hkv}kv heads, ctx {n}, turbo3 K+V, one layer"}


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(index), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples is "under load"
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's algorithm (dequantize the cache, then softmax attention) in NumPy
# ----------------------------------------------------------------------------------------------
def cpu_reference_run(steps: int, warmup: int, heads: int = HKV):
    """One step = one layer of the workload: for each of `heads` KV heads, dequantize 32,768 K and V vectors
    (3-bit PolarQuant, WHT-equivalent dense rotation, fp64 as in the reference) and attend with 4 query heads."""
    from oracle import tq_oracle as o
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        cores = os.cpu_count() or 1
    rng = np.random.default_rng(0)
    a1, a2, _ = o.wht_signs(D, np.random.default_rng(42))
    b1, b2, _ = o.wht_signs(D, np.random.default_rng(542))
    rk, rv, c = o.wht_as_dense(a1, a2), o.wht_as_dense(b1, b2), o.centroids(3, D)
    k = o.rope_rotate(o.synth_keys(CTX, seed=0), np.arange(CTX)).astype(np.float32)
    v = rng.standard_normal((CTX, D)).astype(np.float32)
    ki, kn = o.polar_quantize(k, rk, c)
    vi, vn = o.polar_quantize(v, rv, c)
    q = rng.standard_normal((HQ // HKV, D)).astype(np.float16).astype(np.float64)

    def step():
        for _ in range(heads):
            kh = o.polar_dequantize(ki, kn, rk, c)
            vh = o.polar_dequantize(vi, vn, rv, c)
            o.attend_one(q, kh, vh)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"value": CTX * heads / dt, "ms_per_step": dt * 1e3, "cores": int(cores),
            "sample": f"{heads} KV heads x {CTX} tokens of one layer per step (dequantize K and V, then attend "
                      f"with {HQ // HKV} query heads each), {steps} steps"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # one step is ~0.6 s of NumPy on the host cores: W warm-up steps and K timed steps as asked (K capped at 40 so that
    # the arm ends within a few minutes)
    steps = max(1, min(args.steps, 40))
    r = cpu_reference_run(steps, args.warmup)
    line = {"metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic", "impl": "reference",
            "config": {"workload": "decode attention, 32q/8kv heads, d=128, batch 1, ctx 32768, turbo3 K+V "
                                   "(reference algorithm: dequantize the cache, then NumPy attention; the quantization "
                                   "of the step's new token, which the GPU arm's e2e includes, is not in this arm)"},
            "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


# ----------------------------------------------------------------------------------------------
def synth_layer(torch, gen, dev, n, seed_shift):
    """(n, HKV, D) fp16 keys and values on the device, distributions as in the module docstring."""
    k = torch.randn((n, HKV, D), generator=gen, device=dev)
    k *= torch.exp(0.5 * torch.randn((n, HKV, 1), generator=gen, device=dev))
    ch = torch.randperm(D, generator=gen, device=dev)[:4]
    k[:, :, ch] *= 10.0
    pos = torch.arange(n, device=dev, dtype=torch.float32)[:, None]
    inv = 10000.0 ** (-torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D)
    ang = pos * inv[None, :]
    cs, sn = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    ke, ko = k[..., 0::2].clone(), k[..., 1::2].clone()
    k[..., 0::2] = ke * cs - ko * sn
    k[..., 1::2] = ke * sn + ko * cs
    v = torch.randn((n, HKV, D), generator=gen, device=dev)
    return k.half(), v.half()


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import turboquant_plus_b200 as tq
    from turboquant_plus_b200.layered import LayeredKVCache

    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    pages_per_seq = CTX // PT + 1                      # one spare page for the tokens appended by the e2e leg
    cache = LayeredKVCache(LAYERS, D, HKV, pages_per_seq, PT, ("turbo3", "turbo3"), seed=42, device=dev)
    bt = torch.randperm(pages_per_seq, generator=gen, device=dev).to(torch.int32)[None, :]
    pos = torch.arange(CTX, device=dev)
    slots = bt[0, pos // PT].to(torch.int64) * PT + pos % PT

    # ---- fill the caches through quantize-on-append, timing it (quantize vectors/s) ----
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    q_ms = []
    for layer in range(LAYERS):
        k, v = synth_layer(torch, gen, dev, CTX, layer)
        torch.cuda.synchronize(dev)
        ev[0].record()
        cache.append(layer, k, v, slots)
        ev[1].record()
        torch.cuda.synchronize(dev)
        q_ms.append(ev[0].elapsed_time(ev[1]))
        del k, v
    append_layer_ms = statistics.median(q_ms[3:])      # two launches from Python per layer, launch gaps included
    # quantize kernel alone: 2^22 fp16 vectors (1 GiB in, larger than L2) into a paged cache, one launch per pass
    nq = 1 << 22
    qcache = tq.PagedKVCache(D, 1, nq // PT, PT, "turbo3", "turbo3", seed=42, device=dev)
    xq = torch.randn((nq, 1, D), generator=gen, device=dev).half()
    qslots = torch.randperm(nq // PT, generator=gen, device=dev).repeat_interleave(PT) * PT + \
        torch.arange(nq, device=dev) % PT
    qt = []
    for _ in range(6):
        torch.cuda.synchronize(dev)
        head_start(torch)
        ev[0].record()
        qcache.append(xq, xq, qslots)                  # K and V launches: 2 * nq vectors
        ev[1].record()
        torch.cuda.synchronize(dev)
        qt.append(ev[0].elapsed_time(ev[1]))
    append_ms = statistics.median(qt[2:])
    vec_per_s = 2 * nq / (append_ms * 1e-3)
    append_bytes = 2 * nq * (D * 2 + 52)               # fp16 in, 52 B out per vector
    # the same with fp32 rows (the dtype of the reference's own round-trip configuration): 2^21 vectors, 1 GiB in
    nq32 = nq // 2
    x32 = xq[:nq32].float()
    qt = []
    for _ in range(6):
        torch.cuda.synchronize(dev)
        head_start(torch)
        ev[0].record()
        qcache.append(x32, x32, qslots[:nq32])
        ev[1].record()
        torch.cuda.synchronize(dev)
        qt.append(ev[0].elapsed_time(ev[1]))
    append32_ms = statistics.median(qt[2:])
    append32_bytes = 2 * nq32 * (D * 4 + 52)
    del qcache, x32
    # keys through the reference's default K quantizer (TurboQuant = PolarQuant + 1-bit QJL sketch of the residual,
    # turboquant/kv_cache.py:89-96), 3 bits in all: 2^21 fp16 vectors as prod3 K beside turbo3 V
    pcache = tq.PagedKVCache(D, 1, nq32 // PT, PT, "prod3", "turbo3", seed=42, device=dev)
    xp, pslots = xq[:nq32], torch.arange(nq32, device=dev)
    qt = []
    for _ in range(6):
        torch.cuda.synchronize(dev)
        head_start(torch)
        ev[0].record()
        pcache.append(xp, xp, pslots)
        ev[1].record()
        torch.cuda.synchronize(dev)
        qt.append(ev[0].elapsed_time(ev[1]))
    appendp_ms = statistics.median(qt[2:])
    appendp_bytes = nq32 * (D * 2 + 56) + nq32 * (D * 2 + 52)   # prod3 K: 32 B indices, 16 B sketch, two scales
    del pcache, xq, xp, qslots, pslots
    seq_lens = torch.full((1,), CTX, dtype=torch.int32, device=dev)
    q = torch.randn((LAYERS, 1, HQ, D), generator=gen, device=dev).half()
    out = torch.empty_like(q)
    ws = cache.layers[0].workspace(1, HQ, pages_per_seq)

    def one_step(phases=7, sparse_v=False):
        for i, layer in enumerate(cache.layers):
            # the queries of all layers exist before the step starts: the calls of a step may overlap completely
            layer.attend(q[i], bt, seq_lens, out=out[i], workspace=ws, phases=phases, overlap="q", sparse_v=sparse_v)

    one_step()
    torch.cuda.synchronize(dev)
    assert cache.layers[-1].kernel_status(ws) == 0, "a bounded wait in the decode kernel gave up"
    graphs = {}
    for ph in (7, 2):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            one_step(ph)
        graphs[ph] = g
    # the reference's sparse-V option (skip V work where all weights of a tile are below 1e-6): reported beside the
    # headline, never as the headline -- the headline does all the work
    dense_out = out.clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one_step(7, sparse_v=True)
    graphs["sparse_v"] = g
    g.replay()
    torch.cuda.synchronize(dev)
    sparse_dev = float((out.float() - dense_out.float()).abs().max() / dense_out.float().abs().max())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def timed_once(graph, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            graph.replay()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def timed(graph, steps, warmup):
        """Exactly `steps` steps per timed region; the region is repeated (every rank the same number of
        times) until ~0.4 s have been spent so that the clock sampler sees the GPU under load; median region."""
        for _ in range(warmup):
            graph.replay()
        first = timed_once(graph, steps)
        rounds = max(1, min(40, int(400.0 / max(first * steps, 1e-3))))
        return statistics.median([first] + [timed_once(graph, steps) for _ in range(rounds - 1)])

    sampler = ClockSampler(local) if rank == 0 else None
    ms_step = timed(graphs[7], args.steps, args.warmup)
    ms_kernel_step = timed(graphs[2], args.steps, args.warmup)
    ms_sparse_step = timed(graphs["sparse_v"], args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None

    # ---- end to end: host buffers in, host buffers out, one graph replay per step ----
    st = cache.prepare_decode(1, HQ, bt, seq_lens)
    qh, kh, vh, oh = cache.host_buffers()               # pinned; q, k, v adjacent so that a step copies them in one go
    qh.copy_(torch.randn((LAYERS, 1, HQ, D)).half())
    kh.copy_(torch.randn((LAYERS, 1, HKV, D)).half())
    vh.copy_(torch.randn((LAYERS, 1, HKV, D)).half())
    e2e_steps = min(args.steps, PT - 8 - args.warmup)
    len0 = st["len"].clone()

    def e2e_region():
        """Warm-up steps, then exactly e2e_steps timed steps from the same starting length (the tokens of a region
        land in the slots of the region before: the same work every time)."""
        st["len"].copy_(len0)
        for _ in range(args.warmup):
            cache.decode_step(qh, kh, vh, oh)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(e2e_steps):
            cache.decode_step(qh, kh, vh, oh)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / e2e_steps

    # like the headline, the region is repeated (every rank the same number of times) and the median taken: a single
    # region of a few milliseconds right after the graph capture catches the GPU on its way back from idle
    e2e_ms = statistics.median([e2e_region() for _ in range(9)])
    assert torch.isfinite(oh.float()).all()

    # The order of a model's own decode loop, on the device: per layer, append the layer's new token, then attend.
    # Every attention call then follows an append into its cache; reported for the call in stream order and with
    # overlap="append" (all pages but the last of the sequence stream while the append runs).
    loop = {}
    if rank == 0:
        kn = torch.randn((LAYERS, 1, HKV, D), generator=gen, device=dev).half()
        slot1 = (bt[0, CTX // PT].to(torch.int64) * PT)[None]
        len1 = torch.full((1,), CTX + 1, dtype=torch.int32, device=dev)
        for mode in (False, "append"):
            def loop_step():
                for i, layer in enumerate(cache.layers):
                    layer.append(kn[i], kn[i], slot1)
                    layer.attend(q[i], bt, len1, out=out[i], workspace=ws, overlap=mode)
            loop_step()
            torch.cuda.synchronize(dev)
            lg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(lg):
                loop_step()
            for _ in range(3):
                lg.replay()
            torch.cuda.synchronize(dev)
            le = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            le[0].record()
            for _ in range(10):
                lg.replay()
            le[1].record()
            torch.cuda.synchronize(dev)
            loop["overlap_append" if mode else "stream_order"] = le[0].elapsed_time(le[1]) / 10 * 1e3 / LAYERS
        assert cache.layers[0].kernel_status(ws) == 0

    pre = prefill_probe(torch, tq, dev, gen) if rank == 0 else None
    # the other configurations of the benchmark family, a few steps each, so that every record carries them; with more
    # than one rank they run sharded (KV heads / token-balanced batch) and check the shards against one GPU
    others = {}
    if not args.headline_only:
        del cache, graphs, g, st
        torch.cuda.empty_cache()
        k_other = max(1, min(args.steps, 5))
        for name in ("config2", "config4"):
            others[name] = measure_decode_config(name, k_other, 3)
            torch.cuda.empty_cache()
        others["config3"] = measure_config3(k_other, 3)
    if rank == 0:
        peak, peak_src = peaks()
        tokens_step = LAYERS * CTX * HKV * world
        value = tokens_step / (ms_step * 1e-3)
        kernel_s = ms_kernel_step * 1e-3 / LAYERS
        achieved = CTX * HKV * BYTES_PER_KV_TOKEN / kernel_s / 1e9
        cpu = cpu_reference_run(10, 1) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 tensor-core products, f32 accumulate and softmax", "data": "synthetic",
            "config": {"workload": f"decode attention, 32q/8kv heads, d=128, batch 1 per GPU, ctx {CTX}, turbo3 K+V, "
                                   f"fp16 queries; step = {LAYERS} distinct layer caches (1.09 GB packed > L2)",
                       "l2": "inputs larger than L2", "page_tokens": PT, "layers_per_step": LAYERS,
                       "parallelism": f"batch-sharded x{world}, no collective"},
            "kv_tokens_per_s_per_gpu": value / world,
            "hbm_gbs_algorithmic": value / world * BYTES_PER_KV_TOKEN / 1e9,
            "frac_of_8tbs": value / world * BYTES_PER_KV_TOKEN / 8e12,
            "quantize_vectors_per_s": vec_per_s,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": f"{peak_src} copy bandwidth",
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch in an ncu capture of this
                         # workload: a constant taken from that profile, not something this run measures
                         "traffic": 27343104, "traffic_source": "ncu capture of this workload, not measured in this run",
                         "kernel": "k_decode_attn_g4<3,3,dense V>", "us_per_launch": kernel_s * 1e6,
                         "bytes_per_launch": CTX * HKV * BYTES_PER_KV_TOKEN},
            "sparse_v_option": {"ms_per_step": ms_sparse_step, "kv_tokens_per_s": tokens_step / (ms_sparse_step * 1e-3),
                                "max_rel_deviation_from_dense": sparse_dev,
                                "note": "TQ_DECODE_SPARSE_V: V work of a 16-token tile skipped when all its weights "
                                        "are below 1e-6 of the running maximum; an option, not the headline"},
            "roofline_quantize": {"bound": "hbm", "kernel": "k_quantize_mma<half,3>, 2 launches of 2^22 vectors into pages",
                                  "append_one_layer_ms": append_layer_ms,
                                  "achieved": append_bytes / (append_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                  "frac": append_bytes / (append_ms * 1e-3) / 1e9 / peak,
                                  "bytes_per_vector": D * 2 + 52},
            "roofline_quantize_f32": {"bound": "hbm", "kernel": "k_quantize_mma<float,3>, 2 launches of 2^21 fp32 vectors into pages",
                                      "vectors_per_s": 2 * nq32 / (append32_ms * 1e-3),
                                      "achieved": append32_bytes / (append32_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                      "frac": append32_bytes / (append32_ms * 1e-3) / 1e9 / peak,
                                      "bytes_per_vector": D * 4 + 52},
            "decode_loop_us_per_layer": {"stream_order": loop.get("stream_order"), "overlap_append": loop.get("overlap_append"),
                                         "note": "per layer: quantize-on-append of one token, then decode attention over "
                                                 "ctx + 1 tokens; 40 layers, one graph, no host copies"},
            "roofline_quantize_prod": {"bound": "hbm", "kernel": "k_quantize_mma<half,2,QJL stage> for the K rows + k_quantize_mma<half,3> for the V rows, 2^21 vectors each",
                                       "vectors_per_s": 2 * nq32 / (appendp_ms * 1e-3),
                                       "achieved": appendp_bytes / (appendp_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                       "frac": appendp_bytes / (appendp_ms * 1e-3) / 1e9 / peak,
                                       "bytes_per_vector": "K 312, V 308"},
            "e2e": {"value": LAYERS * CTX * HKV * world / (e2e_ms * 1e-3), "unit": UNIT,
                    "ms_per_step": e2e_ms, "steps": e2e_steps, "regions": 9,
                    "h2d_bytes_per_step": int(qh.numel() + kh.numel() + vh.numel()) * 2,
                    "d2h_bytes_per_step": int(oh.numel()) * 2},
            "roofline_prefill": pre,
            "other_configs": others,
            "gpu_launches": LAYERS,
            "clocks": clocks,
        }
        if cpu:
            line["cpu_baseline"] = {"value": cpu["value"], "unit": UNIT, "cores": cpu["cores"], "kind": "port",
                                    "sample": cpu["sample"]}
        emit(line)


# ----------------------------------------------------------------------------------------------
# Other decode workloads of the benchmark family (not the headline line): --workload config2 | config4
# ----------------------------------------------------------------------------------------------
OTHER_WORKLOADS = {
    "config2": "config2: 32 layers, 32q/8kv heads, d128, batch 16, ctx 8192, K q8_0 + V turbo2, layers 0,1,30,31 q8_0/q8_0",
    "config4": "config4: 2 layers, 32q/8kv heads, d128, batch 256, ragged ctx uniform in [1024, 32768], K prod3 + V turbo3, "
               "shuffled block table",
}


def _dist_ctx():
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    return world, rank, torch.device("cuda", local)


def _kv_rows(torch, gen, dev, n, hkv, heads=None):
    """(n, hkv, D) fp16 keys (N(0,1) x lognormal(0, 0.5)) and values on the device; `heads` keeps a head slice."""
    k = torch.randn((n, hkv, D), generator=gen, device=dev)
    k *= torch.exp(0.5 * torch.randn((n, hkv, 1), generator=gen, device=dev))
    v = torch.randn((n, hkv, D), generator=gen, device=dev)
    if heads is not None:
        k, v = k[:, heads.start:heads.stop], v[:, heads.start:heads.stop]
    return k.half().contiguous(), v.half().contiguous()


def measure_decode_config(name, steps, warmup):
    """config2: 32 layers, batch 16, ctx 8,192, K q8_0, V turbo2 (layers 0,1,30,31 q8_0/q8_0), sharded by KV head.
    config4: batch 256, ragged contexts uniform in [1,024, 32,768], K prod3 (2-bit PolarQuant + QJL), V turbo3,
    2 layers, sequences sharded over the ranks balanced by cached tokens.
    Strong scaling: the job is fixed, every rank holds its shard.  With more than one rank, layer 0 is filled from
    seeds shared by all ranks, rank 0 also builds that layer unsharded, and the all-gathered outputs of the shards are
    compared with the unsharded result (shard_check)."""
    import torch
    import torch.distributed as dist
    world, rank, dev = _dist_ctx()
    from turboquant_plus_b200.layered import LayeredKVCache, boundary_format_table
    from turboquant_plus_b200 import sharding
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + rank)
    common = torch.Generator(device=dev)      # layer 0: the same stream on every rank
    if name == "config2":
        layers, batch = 32, 16
        heads = sharding.shard_kv_heads(HKV, world, rank)
        hkv, hq = len(heads), len(heads) * (HQ // HKV)
        all_lens = [8192] * batch
        mine = list(range(batch))
        formats = boundary_format_table(layers, ("q8_0", "turbo2"), ("q8_0", "q8_0"), keep=2)
        par = f"KV heads sharded x{world}"
    else:
        layers, hkv, hq, heads = 2, HKV, HQ, None
        all_lens = np.random.default_rng(4).integers(1024, 32769, size=256).tolist()
        parts = sharding.shard_batch_by_tokens(all_lens, world)
        mine = parts[rank]
        formats = [("prod3", "turbo3")] * layers
        par = f"sequences sharded x{world}, balanced by tokens"
    lens = [all_lens[i] for i in mine]

    def tables(seq_lens, g):
        n_pages = [(n + PT - 1) // PT for n in seq_lens]
        bt = torch.zeros((len(seq_lens), max(n_pages)), dtype=torch.int32, device=dev)
        perm = torch.randperm(sum(n_pages), generator=g, device=dev).to(torch.int32)
        off = 0
        for b, npg in enumerate(n_pages):
            bt[b, :npg] = perm[off:off + npg]
            off += npg
        return bt, sum(n_pages)

    def fill_layer0(cache_layer, bt, seq_ids, head_slice):
        for b, s in enumerate(seq_ids):
            common.manual_seed(5000 + s)
            k, v = _kv_rows(torch, common, dev, all_lens[s], HKV, head_slice)
            pos = torch.arange(all_lens[s], device=dev)
            cache_layer.append(k, v, bt[b, pos // PT].to(torch.int64) * PT + pos % PT)

    bt, total_pages = tables(lens, gen)
    cache = LayeredKVCache(layers, D, hkv, total_pages, PT, formats, seed=42, device=dev)
    fill_layer0(cache.layers[0], bt, mine, heads)
    for layer in range(1, layers):
        for b, n in enumerate(lens):
            k, v = _kv_rows(torch, gen, dev, n, hkv)
            pos = torch.arange(n, device=dev)
            cache.append(layer, k, v, bt[b, pos // PT].to(torch.int64) * PT + pos % PT)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
    common.manual_seed(77)
    q_all = torch.randn((len(all_lens), HQ, D), generator=common, device=dev).half()     # layer-0 queries, every rank alike
    q = torch.randn((layers, len(lens), hq, D), generator=gen, device=dev).half()
    q0 = q_all[torch.as_tensor(mine, device=dev)]
    q[0] = q0 if heads is None else q0[:, heads.start * (HQ // HKV):heads.stop * (HQ // HKV)]
    out = torch.empty_like(q)
    ws = cache.layers[0].workspace(len(lens), hq, bt.shape[1])

    def one_step():
        for i, layer in enumerate(cache.layers):
            layer.attend(q[i], bt, seq_lens, out=out[i], workspace=ws, overlap="q")

    one_step()
    torch.cuda.synchronize(dev)
    assert cache.layers[0].kernel_status(ws) == 0 and torch.isfinite(out.float()).all()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one_step()
    for _ in range(warmup):
        g.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / steps
    tokens = float(sum(lens)) * hkv * layers
    nbytes = float(sum(lens)) * hkv * sum(layer.bytes_per_token for layer in cache.layers)
    if world > 1:
        t = torch.tensor([ms, tokens, nbytes], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, tokens, nbytes = float(tmax[0]), float(t[1]), float(t[2])
    check = None
    if world > 1:
        # the shards' layer-0 outputs, gathered, against the same layer held by one GPU
        if name == "config2":
            got = sharding.all_gather_heads(out[0])
        else:
            got = sharding.all_gather_batch(out[0], [len(p) for p in parts], parts)
        if rank == 0:
            del cache
            torch.cuda.empty_cache()
            every = list(range(len(all_lens)))
            fbt, fpages = tables(all_lens, gen)
            full = LayeredKVCache(1, D, HKV, fpages, PT, [formats[0]], seed=42, device=dev)
            fill_layer0(full.layers[0], fbt, every, None)
            ref = full.layers[0].attend(q_all, fbt, torch.tensor(all_lens, dtype=torch.int32, device=dev))
            torch.cuda.synchronize(dev)
            diff = float((got.float() - ref.float()).abs().max())
            ref_max = float(ref.float().abs().max())
            assert diff <= 2e-3 * ref_max, f"sharded outputs differ from the unsharded layer by {diff} (of {ref_max})"
            check = {"layer": 0, "max_abs_diff": diff, "max_abs_ref": ref_max,
                     "bit_equal": bool(torch.equal(got, ref)), "tolerance": "2e-3 of max_abs_ref, asserted",
                     "note": "all-gathered shard outputs vs the unsharded layer on one GPU; the split plan depends on "
                             "the number of (sequence, KV head) pairs a GPU holds, so sharding can change the order in "
                             "which split partials are summed (fp32 rounding: an fp16 ulp or two in the output)"}
    peak, src = peaks()
    return {"metric": "decode_attn_kv_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "scaling": "strong",
            "workload": OTHER_WORKLOADS[name], "parallelism": par,
            "hbm_gbs_algorithmic": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peak / world,
            "frac_of": f"{src} HBM copy bandwidth x {world} GPUs", "gpu_launches": layers, "shard_check": check}


def run_other_workload(args):
    r = measure_decode_config(args.workload, args.steps, args.warmup)
    if int(os.environ.get("RANK", "0")) == 0:
        r.update({"higher_is_better": True, "vs_baseline": None, "data": "synthetic",
                  "dtype": "f16 tensor-core products, f32 accumulate and softmax",
                  "config": {"workload": r["workload"], "parallelism": r["parallelism"], "l2": "inputs larger than L2"}})
        emit(r)


def measure_config3(steps, warmup):
    """config3: Llama-3-70B shape, one layer: 131,072 tokens of fp16 K/V (8 KV heads, sharded over the ranks) are
    quantize-on-appended as turbo3 into 128-token pages in 8,192-token chunks, then one 128-query chunk x 64 query
    heads runs chunked-prefill attention (tcgen05) over the whole prefix.  Append vectors/s against the HBM roofline,
    prefill TFLOP/s against the tensor roofline; with more than one rank the gathered prefill outputs are compared
    with the unsharded layer on rank 0."""
    import torch
    import torch.distributed as dist
    world, rank, dev = _dist_ctx()
    import turboquant_plus_b200 as tq
    from turboquant_plus_b200 import sharding
    n, hq_all, hkv_all, chunk, tq_len = 131072, 64, 8, 8192, 128
    heads = sharding.shard_kv_heads(hkv_all, world, rank)
    hkv, hq, grp = len(heads), len(heads) * (hq_all // hkv_all), hq_all // hkv_all
    common = torch.Generator(device=dev)
    common.manual_seed(7)
    cache = tq.PagedKVCache(D, hkv, n // PT, PT, "turbo3", "turbo3", seed=42, device=dev)
    k_all = torch.randn((n, hkv_all, D), generator=common, device=dev).half()
    v_all = torch.randn((n, hkv_all, D), generator=common, device=dev).half()
    q_all = torch.randn((1, tq_len, hq_all, D), generator=common, device=dev).half()
    k = k_all[:, heads.start:heads.stop].contiguous()
    v = v_all[:, heads.start:heads.stop].contiguous()
    q = q_all[:, :, heads.start * grp:heads.stop * grp].contiguous()
    if not (world > 1 and rank == 0):
        del k_all, v_all
    slots = torch.arange(n, device=dev)

    def append_all(c=cache, kk=k, vv=v):
        for lo in range(0, n, chunk):
            c.append(kk[lo:lo + chunk], vv[lo:lo + chunk], slots[lo:lo + chunk])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    append_all()
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()      # the launches of one pass, replayed without host overhead
    with torch.cuda.graph(graph):
        append_all()
    for _ in range(max(warmup, 3)):
        graph.replay()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    sync()
    append_ms = e0.elapsed_time(e1) / steps
    bt = torch.arange(n // PT, device=dev, dtype=torch.int32)[None]
    kv_len = torch.tensor([n], dtype=torch.int32, device=dev)
    out = torch.empty_like(q)
    for _ in range(3):
        cache.prefill_attend(q, bt, kv_len, out=out)
    sync()
    e0.record()
    for _ in range(steps):
        cache.prefill_attend(q, bt, kv_len, out=out)
    e1.record()
    sync()
    prefill_ms = e0.elapsed_time(e1) / steps
    assert cache.kernel_status() == 0 and torch.isfinite(out.float()).all()
    check = None
    if world > 1:
        t = torch.tensor([append_ms, prefill_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        append_ms, prefill_ms = float(t[0]), float(t[1])
        parts = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(parts, out)
        if rank == 0:
            got = torch.cat(parts, dim=2)
            del cache
            torch.cuda.empty_cache()
            full = tq.PagedKVCache(D, hkv_all, n // PT, PT, "turbo3", "turbo3", seed=42, device=dev)
            append_all(full, k_all, v_all)
            ref = full.prefill_attend(q_all, bt, kv_len)
            torch.cuda.synchronize(dev)
            diff, ref_max = float((got.float() - ref.float()).abs().max()), float(ref.float().abs().max())
            assert diff <= 2e-3 * ref_max, f"sharded prefill outputs differ from the unsharded layer by {diff} (of {ref_max})"
            check = {"max_abs_diff": diff, "max_abs_ref": ref_max, "bit_equal": bool(torch.equal(got, ref)),
                     "tolerance": "2e-3 of max_abs_ref, asserted",
                     "note": "gathered prefill outputs of the head shards vs the unsharded layer on one GPU (the page "
                             "split of a row block depends on how many row blocks a GPU holds)"}
    vectors = 2.0 * n * hkv_all
    visible = sum(n - tq_len + i + 1 for i in range(tq_len))
    flops = 2.0 * 2 * hq_all * D * visible
    hbm, src = peaks()
    tpeak, tsrc = tensor_peak()
    return {"metric": "quantize_append_vectors_per_s", "value": vectors / (append_ms * 1e-3), "unit": "vectors/s",
            "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": append_ms, "scaling": "strong",
            "workload": "config3: one layer, 64q/8kv heads, d128, 131072 tokens appended as turbo3 K+V in "
                        "8192-token chunks, then a 128-query chunk of prefill attention over the prefix",
            "parallelism": f"KV heads sharded x{world}",
            "roofline": {"bound": "hbm", "achieved": vectors * 308 / (append_ms * 1e-3) / 1e9 / world, "peak": hbm,
                         "unit": "GB/s", "frac": vectors * 308 / (append_ms * 1e-3) / 1e9 / world / hbm,
                         "peak_source": src, "kernel": "k_quantize_mma<half,3>", "bytes_per_vector": 308},
            "prefill": {"ms": prefill_ms, "tflops": flops / (prefill_ms * 1e-3) / 1e12,
                        "frac_of_tensor_peak": flops / (prefill_ms * 1e-3) / 1e12 / world / tpeak, "peak": tpeak,
                        "peak_source": tsrc, "kernel": "k_prefill_attn2<3,3> (tcgen05)"},
            "gpu_launches": 2 * (n // chunk), "shard_check": check}


def run_config3(args):
    r = measure_config3(args.steps, args.warmup)
    if int(os.environ.get("RANK", "0")) == 0:
        r.update({"higher_is_better": True, "vs_baseline": None, "data": "synthetic",
                  "dtype": "f16 in, exact +-1 tensor-core products, f32 accumulate",
                  "config": {"workload": r["workload"], "parallelism": r["parallelism"], "l2": "inputs larger than L2"}})
        emit(r)


def run_side_kernels(args):
    """--workload side: the kernels next to the hot path (temporal-decay re-quantization, block-format export and
    import, OutlierTurboQuant), each timed alone with CUDA events on inputs larger than L2 and set against the HBM
    peak by its algorithmic bytes.  Not the headline line: one JSON line with a list of kernels."""
    import torch
    import turboquant_plus_b200 as tq
    from turboquant_plus_b200 import temporal_decay as td
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_src = peaks()
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / args.steps

    rows = []

    def row(name, ms, nbytes, units, unit_name):
        rows.append({"kernel": name, "ms": ms, unit_name + "_per_s": units / (ms * 1e-3),
                     "hbm_gbs_algorithmic": nbytes / (ms * 1e-3) / 1e9,
                     "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / peak})

    n = 1 << 22                                   # 4 Mi vectors: 218 MB of 3-bit codes in, 168 MB of 2-bit codes out
    x = torch.randn((n, D), generator=gen, device=dev).half()
    a = tq.PolarQuant(D, 3, seed=42, rotation="wht", device=dev)
    b = tq.PolarQuant(D, 2, seed=42, rotation="wht", device=dev)
    code = a.quantize_device(x, packed=True, want_scale=True)
    del x
    row("k_requantize 3->2 bits", timed(lambda: td.requantize_device(a, b, code["packed"], code["scale"])),
        n * (48 + 4 + 32 + 8), n, "vectors")
    del code

    hkv, pages = 8, 2048                          # 262,144 tokens x 8 heads: 218 MB of records
    cache = tq.PagedKVCache(D, hkv, pages, k_format="turbo3", v_format="turbo3", seed=42, device=dev)
    for lo in range(0, pages * PT, 32768):
        k = torch.randn((32768, hkv, D), generator=gen, device=dev).half()
        cache.append(k, k, torch.arange(lo, lo + 32768, device=dev))
    slots = torch.arange(pages * PT, device=dev)
    nvec = pages * PT * hkv
    for block in (32, 128):
        bb = cache.block_bytes("k", block) * (D // block)
        blocks = cache.export_blocks("k", slots, block)
        row(f"k_cache_blocks export turbo3 K, {block}-element blocks", timed(lambda: cache.export_blocks("k", slots, block)),
            nvec * (52 + bb), nvec, "vectors")
        row(f"k_cache_blocks import turbo3 K, {block}-element blocks",
            timed(lambda: cache.import_blocks("k", blocks, slots, block)), nvec * (52 + bb), nvec, "vectors")
        del blocks
    del cache

    m = 1 << 16                                   # fp64 reference-parity path (dense rotations): compute bound
    xo = torch.randn((m, D), generator=gen, device=dev, dtype=torch.float64)
    oq = tq.OutlierTurboQuant(D, 3.5, seed=42, device=dev)
    c = oq.quantize_device(xo)
    row("OutlierTurboQuant.quantize 3.5 bits (fp64, 3 launches)", timed(lambda: oq.quantize_device(xo)),
        m * (D * 8 + D + 8 + 16 + 4), m, "vectors")
    row("OutlierTurboQuant.dequantize 3.5 bits (fp64, 3 launches)", timed(lambda: oq.dequantize_device(c)),
        m * (D * 8 + D + 8 + 16 + 4), m, "vectors")
    print(json.dumps({"metric": "side_kernels", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "data": "synthetic", "hbm_peak_gbs": peak, "hbm_peak_source": peak_src, "kernels": rows}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config1", choices=["config1", "config2", "config3", "config4", "side"],
                    help="config1 is the headline workload; the others print a line of the same shape")
    ap.add_argument("--headline-only", action="store_true", help="config1 without the other_configs block")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        # The one line on stdout is the JSON line.  NCCL writes its version banner to stdout when the first communicator
        # is made (whatever set NCCL_DEBUG, the environment or a configuration file): from here on file descriptor 1
        # leads to stderr, and emit() writes the JSON line to the descriptor that was stdout.
        global _STDOUT_FD
        sys.stdout.flush()
        _STDOUT_FD = os.dup(1)
        os.dup2(2, 1)
        import torch
        import torch.distributed as dist
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if args.workload == "config3":
        run_config3(args)
    elif args.workload == "side":
        run_side_kernels(args)
    elif args.workload != "config1":
        run_other_workload(args)
    else:
        run_ours(args)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
