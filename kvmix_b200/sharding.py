"""Partitioning of the decode hot path across the GPUs of one node (one process per GPU).

(batch, kv-head) rows of the cache never interact, so there are exactly two ways to split:

* ``batch``   -- each rank keeps whole sequences (benchmark configurations 2-4).  No collective on the data
                 path; ranks only meet at the timing barrier.
* ``kv_head`` -- each rank keeps some KV heads of every sequence together with their query heads
                 (configuration 5, one 131k-token sequence).  The per-layer attention output
                 [B, nh_local * D] is all-gathered (NCCL over NVLink on GPUs, gloo in the CPU tests) before
                 the output projection.  That all-gather is the only exchange step of the path.

Upstream is single-GPU (every script pins ``device_map="cuda:0"``); this module has no counterpart there.
"""
import torch
import torch.distributed as dist


def shard_range(n, world, rank):
    """Contiguous, balanced slice [lo, hi) of n units for `rank`; the first n % world ranks get one extra."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("bad world/rank")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_batch(global_batch, world, rank):
    lo, hi = shard_range(global_batch, world, rank)
    if hi == lo:
        raise ValueError(f"rank {rank} of {world} gets no sequence out of {global_batch}")
    return lo, hi


def shard_kv_heads(n_heads, n_kv_heads, world, rank):
    """KV heads [lo, hi) of this rank and the query heads that read them."""
    if n_kv_heads % world != 0:
        raise ValueError("kv heads must divide evenly across ranks (the all-gather uses equal blocks)")
    lo, hi = shard_range(n_kv_heads, world, rank)
    rep = n_heads // n_kv_heads
    return (lo, hi), (lo * rep, hi * rep)


def all_gather_heads(out_local, group=None):
    """[B, nh_local, 1, D] on every rank -> [B, nh, 1, D], heads in rank order."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return out_local
    B, nhl, one, D = out_local.shape
    flat = out_local.transpose(0, 1).contiguous()                 # [nh_local, B, 1, D]: gather along dim 0
    full = torch.empty((world * nhl, B, one, D), dtype=out_local.dtype, device=out_local.device)
    dist.all_gather_into_tensor(full, flat, group=group)
    return full.transpose(0, 1).contiguous()


def max_over_ranks(value, device, group=None):
    """The slowest rank's time: what a multi-GPU step costs."""
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
