"""Multi-rank plumbing on CPU: world_size-2 gloo ranks shard a job by KV head and by sequence, compute their
slice with the oracle, all-gather the slices and must reproduce the single-rank result exactly."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tq_oracle as o
from turboquant_plus_b200 import sharding


def test_partition_helpers():
    assert list(sharding.shard_kv_heads(8, 4, 1)) == [2, 3]
    assert list(sharding.query_heads_of(range(2, 4), 4)) == list(range(8, 16))
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(8, 3, 0)
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(8, 2, 2)
    lens = [100, 3000, 50, 2900, 10, 10]
    parts = sharding.shard_batch_by_tokens(lens, 2)
    assert sorted(i for p in parts for i in p) == list(range(6))
    loads = [sum(lens[i] for i in p) for p in parts]
    assert abs(loads[0] - loads[1]) <= 200
    assert sharding.shard_batch_by_tokens(lens, 2) == parts          # deterministic
    assert sharding.shard_batch_by_tokens([], 3) == [[], [], []]


def _job():
    rng = np.random.default_rng(0)
    d, hkv, g = 128, 4, 2
    lens = [40, 7, 33, 20]
    kv = o.KVOracle(d, 3, 3, seed=42, mode="wht", k_kind="mse")
    k = rng.standard_normal((len(lens), hkv, 40, d)).astype(np.float32)
    v = rng.standard_normal((len(lens), hkv, 40, d)).astype(np.float32)
    q = rng.standard_normal((len(lens), hkv * g, d)).astype(np.float16).astype(np.float64)
    return kv, k, v, q, lens, g


def _attend(kv, k, v, q, lens):
    kh = np.stack([np.stack([kv.k_roundtrip(k[b, h]) for h in range(k.shape[1])]) for b in range(k.shape[0])])
    vh = np.stack([np.stack([kv.v_roundtrip(v[b, h]) for h in range(k.shape[1])]) for b in range(k.shape[0])])
    return o.attend_gqa(q, kh, vh, lens)


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    kv, k, v, q, lens, g = _job()
    full = _attend(kv, k, v, q, lens)
    # by KV head
    heads = sharding.shard_kv_heads(k.shape[1], world, rank)
    qh = sharding.query_heads_of(heads, g)
    local = _attend(kv, k[:, heads.start:heads.stop], v[:, heads.start:heads.stop], q[:, qh.start:qh.stop], lens)
    got = sharding.all_gather_heads(torch.as_tensor(local)).numpy()
    ok_heads = np.array_equal(got, full)
    # by sequence, balanced by tokens
    parts = sharding.shard_batch_by_tokens(lens, world)
    mine = parts[rank]
    local = _attend(kv, k[mine], v[mine], q[mine], [lens[i] for i in mine])
    got = sharding.all_gather_batch(torch.as_tensor(local), [len(p) for p in parts], parts).numpy()
    ok_batch = np.array_equal(got, full)
    ret[rank] = (ok_heads, ok_batch)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_single_rank():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, True), 1: (True, True)}
