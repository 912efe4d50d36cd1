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
    times = []
    for _ in range(6):
        torch.cuda.synchronize(dev)
        ev[0].record()
        cache.prefill_attend(q, bt, kv_len, out=out)
        ev[1].record()
        torch.cuda.synchronize(dev)
        times.append(ev[0].elapsed_time(ev[1]))
    assert cache.kernel_status() == 0 and torch.isfinite(out.float()).all()
    ms = statistics.median(times[2:])
    visible = sum(n - tq_len + i + 1 for i in range(tq_len))       # cached positions seen by the chunk's queries
    flops = 2 * 2 * hq * D * visible
    peak, src = tensor_peak()
    return {"bound": "tensor", "kernel": "k_prefill_attn2<3,3> (tcgen05)", "achieved": flops / (ms * 1e-3) / 1e12,
            "peak": peak, "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / peak, "peak_source": src,
            "ms": ms, "ctas": (tq_len * hq // hkv // 128) * hkv,
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
    r = cpu_reference_run(max(1, min(args.steps, 20)), 1)
    line = {"metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64", "data": "synthetic", "impl": "reference",
            "config": {"workload": "decode attention, 32q/8kv heads, d=128, batch 1, ctx 32768, turbo3 K+V "
                                   "(reference algorithm: dequantize the cache, then NumPy attention)"},
            "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                             "sample": r["sample"]},
            "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
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
        ev[0].record()
        qcache.append(xq, xq, qslots)                  # K and V launches: 2 * nq vectors
        ev[1].record()
        torch.cuda.synchronize(dev)
        qt.append(ev[0].elapsed_time(ev[1]))
    append_ms = statistics.median(qt[2:])
    vec_per_s = 2 * nq / (append_ms * 1e-3)
    append_bytes = 2 * nq * (D * 2 + 52)               # fp16 in, 52 B out per vector
    del qcache, xq, qslots
    seq_lens = torch.full((1,), CTX, dtype=torch.int32, device=dev)
    q = torch.randn((LAYERS, 1, HQ, D), generator=gen, device=dev).half()
    out = torch.empty_like(q)
    ws = cache.layers[0].workspace(1, HQ, pages_per_seq)

    def one_step(phases=7, sparse_v=False):
        for i, layer in enumerate(cache.layers):
            layer.attend(q[i], bt, seq_lens, out=out[i], workspace=ws, phases=phases, overlap=True, sparse_v=sparse_v)

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
    for _ in range(args.warmup):
        cache.decode_step(qh, kh, vh, oh)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        cache.decode_step(qh, kh, vh, oh)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= e2e_steps
    assert torch.isfinite(oh.float()).all()

    pre = prefill_probe(torch, tq, dev, gen) if rank == 0 else None
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
                         # dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture summarised in
                         # profiles/k_decode_attn_turbo3_ctx32768.md
                         "traffic": 27338240,
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
            "e2e": {"value": LAYERS * CTX * HKV * world / (e2e_ms * 1e-3), "unit": UNIT,
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(qh.numel() + kh.numel() + vh.numel()) * 2,
                    "d2h_bytes_per_step": int(oh.numel()) * 2},
            "roofline_prefill": pre,
            "gpu_launches": LAYERS,
            "clocks": clocks,
        }
        if cpu:
            line["cpu_baseline"] = {"value": cpu["value"], "unit": UNIT, "cores": cpu["cores"], "kind": "port",
                                    "sample": cpu["sample"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()



# ----------------------------------------------------------------------------------------------
# Other decode workloads of the benchmark family (not the headline line): --workload config2 | config4
# ----------------------------------------------------------------------------------------------
OTHER_WORKLOADS = {
    "config2": "config2: 32 layers, 32q/8kv heads, d128, batch 16, ctx 8192, K q8_0 + V turbo2, layers 0,1,30,31 q8_0/q8_0",
    "config4": "config4: 2 layers, 32q/8kv heads, d128, batch 256, ragged ctx uniform in [1024, 32768], K prod3 + V turbo3, "
               "shuffled block table",
}


def run_other_workload(args):
    """config2: 32 layers, batch 16, ctx 8,192, K q8_0, V turbo2 (layers 0,1,30,31 q8_0/q8_0), sharded by KV head.
    config4: batch 256, ragged contexts uniform in [1,024, 32,768], K prod3 (2-bit PolarQuant + QJL), V turbo3,
    2 layers, sequences sharded over the ranks balanced by cached tokens."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from turboquant_plus_b200.layered import LayeredKVCache, boundary_format_table
    from turboquant_plus_b200 import sharding
    gen = torch.Generator(device=dev)
    gen.manual_seed(99 + rank)
    if args.workload == "config2":
        layers, hkv, hq = 32, HKV // world, HQ // world
        lens = [8192] * 16
        formats = boundary_format_table(layers, ("q8_0", "turbo2"), ("q8_0", "q8_0"), keep=2)
        par = f"KV heads sharded x{world}"
    else:
        layers, hkv, hq = 2, HKV, HQ
        all_lens = np.random.default_rng(4).integers(1024, 32769, size=256).tolist()
        lens = [all_lens[i] for i in sharding.shard_batch_by_tokens(all_lens, world)[rank]]
        formats = [("prod3", "turbo3")] * layers
        par = f"sequences sharded x{world}, balanced by tokens"
    n_pages = [(n + PT - 1) // PT for n in lens]
    cache = LayeredKVCache(layers, D, hkv, sum(n_pages), PT, formats, seed=42, device=dev)
    bt = torch.zeros((len(lens), max(n_pages)), dtype=torch.int32, device=dev)
    perm = torch.randperm(sum(n_pages), generator=gen, device=dev).to(torch.int32)
    off = 0
    for b, npg in enumerate(n_pages):
        bt[b, :npg] = perm[off:off + npg]
        off += npg
    for layer in range(layers):
        for b, n in enumerate(lens):
            k = torch.randn((n, hkv, D), generator=gen, device=dev)
            k *= torch.exp(0.5 * torch.randn((n, hkv, 1), generator=gen, device=dev))
            v = torch.randn((n, hkv, D), generator=gen, device=dev)
            pos = torch.arange(n, device=dev)
            cache.append(layer, k.half(), v.half(), bt[b, pos // PT].to(torch.int64) * PT + pos % PT)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
    q = torch.randn((layers, len(lens), hq, D), generator=gen, device=dev).half()
    out = torch.empty_like(q)
    ws = cache.layers[0].workspace(len(lens), hq, bt.shape[1])

    def one_step():
        for i, layer in enumerate(cache.layers):
            layer.attend(q[i], bt, seq_lens, out=out[i], workspace=ws, overlap=True)

    one_step()
    torch.cuda.synchronize(dev)
    assert cache.layers[0].kernel_status(ws) == 0 and torch.isfinite(out.float()).all()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        one_step()
    for _ in range(args.warmup):
        g.replay()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        g.replay()
    e1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    tokens = float(sum(lens)) * hkv * layers
    nbytes = float(sum(lens)) * hkv * sum(layer.bytes_per_token for layer in cache.layers)
    if world > 1:
        t = torch.tensor([ms, tokens, nbytes], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ms, tokens, nbytes = float(tmax[0]), float(t[1]), float(t[2])
    if rank == 0:
        peak, src = peaks()
        print(json.dumps({
            "metric": "decode_attn_kv_tokens_per_s", "value": tokens / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 tensor-core products, f32 accumulate and softmax",
            "data": "synthetic",
            "config": {"workload": OTHER_WORKLOADS[args.workload],
                       "parallelism": par, "l2": "inputs larger than L2"},
            "hbm_gbs_algorithmic": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peak / world,
            "peak_source": src, "gpu_launches": layers}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_config3(args):
    """config3: Llama-3-70B shape, one layer: 131,072 tokens of fp16 K/V (8 KV heads, sharded over the ranks) are
    quantize-on-appended as turbo3 into 128-token pages in 8,192-token chunks, then one 128-query chunk x 64 query
    heads runs chunked-prefill attention (tcgen05) over the whole prefix.  Prints append vectors/s (HBM roofline)
    and prefill TFLOP/s (tensor roofline)."""
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    import turboquant_plus_b200 as tq
    n, hq_all, hkv_all, chunk, tq_len = 131072, 64, 8, 8192, 128
    hkv, hq = hkv_all // world, hq_all // world
    gen = torch.Generator(device=dev)
    gen.manual_seed(7 + rank)
    cache = tq.PagedKVCache(D, hkv, n // PT, PT, "turbo3", "turbo3", seed=42, device=dev)
    k = torch.randn((n, hkv, D), generator=gen, device=dev).half()
    v = torch.randn((n, hkv, D), generator=gen, device=dev).half()
    slots = torch.arange(n, device=dev)

    def append_all():
        for lo in range(0, n, chunk):
            cache.append(k[lo:lo + chunk], v[lo:lo + chunk], slots[lo:lo + chunk])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    append_all()
    torch.cuda.synchronize(dev)
    graph = torch.cuda.CUDAGraph()      # the 32 launches of one pass, replayed without host overhead
    with torch.cuda.graph(graph):
        append_all()
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        graph.replay()
    e1.record()
    sync()
    append_ms = e0.elapsed_time(e1) / args.steps
    bt = torch.arange(n // PT, device=dev, dtype=torch.int32)[None]
    kv_len = torch.tensor([n], dtype=torch.int32, device=dev)
    q = torch.randn((1, tq_len, hq, D), generator=gen, device=dev).half()
    out = torch.empty_like(q)
    for _ in range(3):
        cache.prefill_attend(q, bt, kv_len, out=out)
    sync()
    e0.record()
    for _ in range(args.steps):
        cache.prefill_attend(q, bt, kv_len, out=out)
    e1.record()
    sync()
    prefill_ms = e0.elapsed_time(e1) / args.steps
    assert cache.kernel_status() == 0 and torch.isfinite(out.float()).all()
    if world > 1:
        t = torch.tensor([append_ms, prefill_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        append_ms, prefill_ms = float(t[0]), float(t[1])
    if rank == 0:
        vectors = 2.0 * n * hkv_all
        visible = sum(n - tq_len + i + 1 for i in range(tq_len))
        flops = 2.0 * 2 * hq_all * D * visible
        hbm, src = peaks()
        tpeak, tsrc = tensor_peak()
        print(json.dumps({
            "metric": "quantize_append_vectors_per_s", "value": vectors / (append_ms * 1e-3), "unit": "vectors/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": append_ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 in, exact +-1 tensor-core products, f32 accumulate", "data": "synthetic",
            "config": {"workload": "config3: one layer, 64q/8kv heads, d128, 131072 tokens appended as turbo3 K+V in "
                                   "8192-token chunks, then a 128-query chunk of prefill attention over the prefix",
                       "parallelism": f"KV heads sharded x{world}", "l2": "inputs larger than L2"},
            "roofline": {"bound": "hbm", "achieved": vectors * 308 / (append_ms * 1e-3) / 1e9 / world, "peak": hbm,
                         "unit": "GB/s", "frac": vectors * 308 / (append_ms * 1e-3) / 1e9 / world / hbm,
                         "peak_source": src, "kernel": "k_quantize_mma<half,3>", "bytes_per_vector": 308},
            "prefill": {"ms": prefill_ms, "tflops": flops / (prefill_ms * 1e-3) / 1e12,
                        "frac_of_tensor_peak": flops / (prefill_ms * 1e-3) / 1e12 / world / tpeak, "peak": tpeak,
                        "peak_source": tsrc, "kernel": "k_prefill_attn2<3,3> (tcgen05)"},
            "gpu_launches": 2 * (n // chunk)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "config3":
        run_config3(args)
    elif args.workload == "side":
        run_side_kernels(args)
    elif args.workload != "config1":
        run_other_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
