"""The head-sharded exchange on ONE GPU: ranks are emulated as separate caches, gather buffers and arrival counters
on the same device, and both ranks' attention kernels are launched before anybody waits (on one GPU a waiting kernel
and the kernel it waits for are never in flight together).  The gathered buffer of every rank must equal the
unsharded output, layer after layer through the round-robin buffers; a counter that nothing raises makes the bounded
wait give up and report it, with the context still usable afterwards."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kb,vb,G,nh,hkv", [(2, 2, 32, 4, 4), (4, 2, 64, 16, 4), (3, 2, 128, 8, 2)])
def test_emulated_two_rank_exchange(cuda, kb, vb, G, nh, hkv):
    import kvmix_b200 as kv
    from kvmix_b200 import configs, sharding
    B, T, world, layers = 2, 3000, 2, 5
    k, v = configs.synth_kv(B, hkv, T, 128, cuda, seed=9)
    full = kv.KVmixLayerCache(B, hkv, 128, T + 16, kb, vb, G, residual_length=128, device=cuda)
    full.prefill(k, v)
    nhl, hkl = nh // world, hkv // world
    shards = []
    for r in range(world):
        c = kv.KVmixLayerCache(B, hkl, 128, T + 16, kb, vb, G, residual_length=128, device=cuda)
        c.prefill(k[:, r * hkl:(r + 1) * hkl], v[:, r * hkl:(r + 1) * hkl])
        shards.append(c)
    peers = [(torch.zeros((2, B, nh, 1, 128), dtype=torch.float16, device=cuda),
              torch.zeros(2 * 32, dtype=torch.int32, device=cuda)) for _ in range(world)]
    gathers = [sharding.PeerGather(B, nhl, 128, cuda, peers=peers, rank=r) for r in range(world)]
    g = torch.Generator(device=cuda).manual_seed(4)
    for layer in range(layers):                                  # "layers" reuse the same caches: decode steps
        q = torch.randn((B, nh, 1, 128), generator=g, device=cuda, dtype=torch.float16)
        kn = torch.randn((B, hkv, 1, 128), generator=g, device=cuda, dtype=torch.float16)
        vn = torch.randn((B, hkv, 1, 128), generator=g, device=cuda, dtype=torch.float16)
        want = full.decode_step(q, kn, vn)
        for r in range(world):                                   # every rank's attention first ...
            shards[r].decode_step(q[:, r * nhl:(r + 1) * nhl].contiguous(), kn[:, r * hkl:(r + 1) * hkl].contiguous(),
                                  vn[:, r * hkl:(r + 1) * hkl].contiguous(), peers=gathers[r])
        for r in range(world):                                   # ... then the waits, which find everything arrived
            got = gathers[r].wait()
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"layer {layer}, rank {r}"
            gathers[r].check()
    assert [int(x) for x in peers[0][1][[0, 32]].tolist()] == [3 * B * nh, 2 * B * nh]   # layers 0,2,4 / 1,3


def test_wait_gives_up_and_reports(cuda):
    from kvmix_b200 import _lib
    L = _lib.lib()
    cnt = torch.zeros(4, dtype=torch.int32, device=cuda)          # nothing ever raises this counter
    status = torch.zeros(2, dtype=torch.int32, device=cuda)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.kvq_peer_wait(C.c_void_p(cnt.data_ptr()), 5, 2000, C.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()                                     # returns after ~2 ms of polling
    assert status.tolist() == [1, 0]
    cnt[0] = 7
    status.zero_()
    assert L.kvq_peer_wait(C.c_void_p(cnt.data_ptr()), 5, 2000, C.c_void_p(status.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert status.tolist() == [0, 0]                             # already there: no report, and the context still works
    assert L.kvq_peer_wait(None, 5, 2000, C.c_void_p(status.data_ptr()), stream) == -10
    assert L.kvq_peer_wait(C.c_void_p(cnt.data_ptr()), 5, 0, C.c_void_p(status.data_ptr()), stream) == -7


def test_generation_wait(cuda):
    """kvq_peer_wait_next keeps the target on the device: use g of a counter waits for g * per_use arrivals."""
    from kvmix_b200 import _lib
    L = _lib.lib()
    cnt = torch.zeros(1, dtype=torch.int32, device=cuda)
    gen = torch.zeros(1, dtype=torch.int32, device=cuda)
    status = torch.zeros(2, dtype=torch.int32, device=cuda)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    cnt.fill_(8)                                                 # two uses' worth of arrivals are already there
    for use in (1, 2):
        assert L.kvq_peer_wait_next(p(cnt), 4, p(gen), 2000, p(status), stream) == 0
        torch.cuda.synchronize()
        assert gen.item() == use and status.tolist() == [0, 0]
    assert L.kvq_peer_wait_next(p(cnt), 4, p(gen), 2000, p(status), stream) == 0      # the third use never arrives
    torch.cuda.synchronize()
    assert gen.item() == 3 and status.tolist() == [1, 8]
    assert L.kvq_peer_wait_next(None, 4, p(gen), 2000, p(status), stream) == -10
    assert L.kvq_peer_wait_next(p(cnt), 0, p(gen), 2000, p(status), stream) == -7
