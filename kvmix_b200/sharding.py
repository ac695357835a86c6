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
    """[B, nh_local, 1, D] on every rank -> [B, nh, 1, D], heads in rank order (allocates; see HeadGather)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return out_local
    return HeadGather(out_local.shape[0], out_local.shape[1], out_local.shape[3], out_local.dtype, out_local.device,
                      group)(out_local)


class HeadGather:
    """The per-layer exchange of the kv-head-sharded decode step with everything preallocated: one
    ``all_gather_into_tensor`` per call into a buffer made once.  With one sequence per rank (the long-context
    configuration) the rank-major gather layout [world, 1, nh_local, 1, D] already *is* [1, nh, 1, D], so the result is
    a view; with B > 1 one strided copy reorders it."""

    def __init__(self, batch, nh_local, head_dim, dtype, device, group=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.B, self.nhl, self.D = batch, nh_local, head_dim
        self.full = torch.empty((self.world, batch, nh_local, 1, head_dim), dtype=dtype, device=device)
        self.out = self.full.view(1, self.world * nh_local, 1, head_dim) if batch == 1 else \
            torch.empty((batch, self.world * nh_local, 1, head_dim), dtype=dtype, device=device)

    def __call__(self, out_local):
        if self.world == 1:
            return out_local
        if not out_local.is_contiguous():
            out_local = out_local.contiguous()
        dist.all_gather_into_tensor(self.full.view(self.world * self.B, self.nhl, 1, self.D), out_local, group=self.group)
        if self.B == 1:
            return self.out
        self.out.view(self.B, self.world, self.nhl, 1, self.D).copy_(self.full.permute(1, 0, 2, 3, 4))
        return self.out


def max_over_ranks(value, device, group=None):
    """The slowest rank's time: what a multi-GPU step costs."""
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
