"""The N > 1 paths on CPU: two gloo ranks shard the hot path by batch and by KV head, run the oracle on
their shard, and the reassembled output equals the unsharded run bit for bit.  Also the failure behaviour
of the host-side partitioning (uneven heads, an empty rank)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kvmix_b200 import sharding
from oracle.glue import RefLayerCache
from util import make_kv, make_q


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _state():
    B, hkv, nh, T = 4, 4, 8, 300
    k, v = make_kv(77, B, hkv, T)
    q = make_q(77, B, nh)
    return B, hkv, nh, T, k, v, q


def _attend(k, v, q):
    c = RefLayerCache(4, 2, 32, residual_length=128)
    c.prefill(k, v)
    return c.attend(q, ref_rounding=7)


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, hkv, nh, T, k, v, q = _state()
        if mode == "batch":
            lo, hi = sharding.shard_batch(B, world, rank)
            out = torch.from_numpy(_attend(k[lo:hi], v[lo:hi], q[lo:hi]))
            parts = [torch.empty_like(out) for _ in range(world)]
            dist.all_gather(parts, out)                     # only to check; the data path itself has no collective
            full = torch.cat(parts, 0)
        else:
            (klo, khi), (qlo, qhi) = sharding.shard_kv_heads(nh, hkv, world, rank)
            out = torch.from_numpy(_attend(k[:, klo:khi], v[:, klo:khi], q[:, qlo:qhi]))
            full = sharding.all_gather_heads(out)
        slow = sharding.max_over_ranks(1.0 + rank, torch.device("cpu"))
        if rank == 0:
            ret["full"] = full.numpy()
            ret["slow"] = slow
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["batch", "kv_head"])
def test_two_ranks_reassemble_to_the_unsharded_result(mode):
    B, hkv, nh, T, k, v, q = _state()
    want = _attend(k, v, q)
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, _free_port(), mode, ret), nprocs=2, join=True)
        got, slow = ret["full"], ret["slow"]
    assert got.shape == want.shape
    assert (got.view(np.uint16) == want.view(np.uint16)).all()
    assert slow == 2.0                                   # max over ranks, not rank 0's own time


def test_partition_rules():
    assert [sharding.shard_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sharding.shard_batch(64, 8, 7) == (56, 64)
    assert sharding.shard_kv_heads(32, 8, 4, 1) == ((2, 4), (8, 16))
    with pytest.raises(ValueError, match="evenly"):
        sharding.shard_kv_heads(32, 8, 3, 0)
    with pytest.raises(ValueError, match="no sequence"):
        sharding.shard_batch(1, 2, 1)
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)
