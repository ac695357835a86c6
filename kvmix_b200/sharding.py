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


class PeerGather:
    """The same exchange without a collective launch: every rank's attention kernel stores the rows it finishes
    straight into all ranks' gather buffers (plain peer stores over NVLink, ``kvq_attn_args.peer_out``) and raises their
    arrival counters; the consumer waits on its own counter with a bounded device-side poll (``kvq_peer_wait``).

    ``depth`` gather buffers are used round-robin, one per layer: a rank that is ``depth`` layers ahead has already
    seen every rank arrive ``depth - 1`` layers back, so nobody still reads the buffer it is about to overwrite.
    Buffers and counters live in symmetric memory (``torch.distributed._symmetric_memory``); ``available()`` says
    whether this process can use it.  ``peers`` may be given instead for tests: a list of (buffer, counters) tensors,
    one pair per emulated rank, all on this GPU."""

    MAX_POLLS = 2_000_000          # ~2 s of polling before a wait gives up and reports it

    def __init__(self, batch, nh_local, head_dim, device, group=None, depth=2, peers=None, rank=None):
        import ctypes as C
        from . import _lib
        self._C, self._lib = C, _lib.lib()
        self.B, self.nhl, self.D, self.depth = batch, nh_local, head_dim, depth
        if peers is None:
            import torch.distributed._symmetric_memory as symm
            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
            nh = self.world * nh_local
            self.buf = symm.empty((depth, batch, nh, 1, head_dim), dtype=torch.float16, device=device)
            self.cnt = symm.empty((depth * 32,), dtype=torch.int32, device=device)
            self.buf.zero_()
            self.cnt.zero_()
            g = group if group is not None else dist.group.WORLD
            hb, hc = symm.rendezvous(self.buf, g), symm.rendezvous(self.cnt, g)
            self.buf_ptrs, self.cnt_ptrs = list(hb.buffer_ptrs), list(hc.buffer_ptrs)
            torch.cuda.synchronize()
            dist.barrier(group)
        else:
            self.world, self.rank = len(peers), rank or 0
            self.buf, self.cnt = peers[self.rank]
            self.buf_ptrs = [b.data_ptr() for b, _ in peers]
            self.cnt_ptrs = [c.data_ptr() for _, c in peers]
        if self.world > 8:
            raise ValueError("at most 8 ranks")
        self.status = torch.zeros(2, dtype=torch.int32, device=device)
        self.gen = torch.zeros(depth * 32, dtype=torch.int32, device=device)   # uses of each counter so far (device side)
        self.layer = 0
        self._slot_bytes = batch * self.world * nh_local * head_dim * 2

    @staticmethod
    def available():
        try:
            import torch.distributed._symmetric_memory as symm  # noqa: F401
            return dist.is_initialized() and dist.get_backend() == "nccl"
        except Exception:
            return False

    def fill(self, a):
        """Point the exchange fields of a kvq_attn_args block at the next layer's gather buffer."""
        slot = self.layer % self.depth
        a.n_peers, a.peer_head0 = self.world, self.rank * self.nhl
        for p in range(self.world):
            a.peer_out[p] = self.buf_ptrs[p] + slot * self._slot_bytes
            a.peer_flag[p] = self.cnt_ptrs[p] + slot * 128
        a.peer_sB, a.peer_sH = self.world * self.nhl * self.D, self.D

    def wait(self):
        """Enqueue the bounded wait for the layer just launched; returns the gathered [B, nh, 1, D] view."""
        slot = self.layer % self.depth
        from . import _lib
        # the target (uses so far x arrivals per use) lives on the device, so this launch replays from a CUDA graph
        _lib.check(self._lib.kvq_peer_wait_next(self._C.c_void_p(self.cnt.data_ptr() + slot * 128),
                                                self.B * self.world * self.nhl,
                                                self._C.c_void_p(self.gen.data_ptr() + slot * 128), self.MAX_POLLS,
                                                self._C.c_void_p(self.status.data_ptr()),
                                                self._C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        self.layer += 1
        return self.buf[slot]

    def check(self):
        """Host-side check after a step (synchronises): raises if a wait gave up."""
        st = self.status.tolist()
        if st[0]:
            raise RuntimeError(f"head-sharded exchange: a rank's attention output did not arrive (counter at {st[1] & 0xFFFFFFFF})")


def max_over_ranks(value, device, group=None):
    """The slowest rank's time: what a multi-GPU step costs."""
    t = torch.tensor([float(value)], device=device, dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
