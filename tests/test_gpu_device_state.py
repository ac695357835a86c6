"""Device-resident cache state: fused decode steps that read the lengths and ring starts from device memory, apply the
window policy on the device and advance the state themselves -- driven eagerly, with a frozen argument block, and from
a captured CUDA graph replayed many times -- against the host-driven path step by step: identical packed codes, scales,
tails and state, attention within the split-plan tolerance (the replayed grid is laid out for a longer context, so a
head may be cut differently: two split plans differ by the fp16 rounding of p * scale, see test_gpu_configs.py)."""
import numpy as np
import pytest
import torch

from util import make_kv, make_q, row_rel

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


CASES = [(2, 2, 32, 4, 4, dict(residual_length=128), 600), (3, 2, 32, 2, 2, dict(residual_length=128), 1200),
         (4, 4, 64, 8, 2, dict(residual_length=128), 5000), (2, 2, 32, 4, 4, dict(k_residual_ratio=0.2, v_residual_ratio=0.2), 400)]


@pytest.mark.parametrize("kb,vb,G,nh,hkv,policy,L", CASES)
def test_device_driven_steps_match_host_driven(cuda, kb, vb, G, nh, hkv, policy, L):
    import kvmix_b200 as kv
    B, warm, steps = 2, 40, 90
    k, v = make_kv(77, B, hkv, L + warm + steps)
    kt, vt = _t(k, cuda), _t(v, cuda)
    host = kv.KVmixLayerCache(B, hkv, 128, L + warm + steps + 8, kb, vb, G, device=cuda, **policy)
    dev = kv.KVmixLayerCache(B, hkv, 128, L + warm + steps + 8, kb, vb, G, device=cuda, device_state=True, **policy)
    host.prefill(kt[:, :, :L], vt[:, :, :L])
    dev.prefill(kt[:, :, :L], vt[:, :, :L])
    for i in range(warm):                                        # reach steady state (the ratio policy shrinks the tail first)
        t = L + i
        q = _t(make_q(t, B, nh), cuda)
        a = host.decode_step(q, kt[:, :, t:t + 1], vt[:, :, t:t + 1])
        b = dev.decode_step(q, kt[:, :, t:t + 1], vt[:, :, t:t + 1])
        assert torch.equal(a, b)
    assert dev.steady() and dev._fused is True
    assert dev.state.tolist()[:6] == [dev.kv_seq_len, dev.tkq, dev.tvq, dev.k_start, dev.v_start, 0]

    # a decode step captured once, laid out for every length it will be replayed at
    qs = torch.zeros((B, nh, 1, 128), device=cuda, dtype=torch.float16)
    ks = torch.zeros((B, hkv, 1, 128), device=cuda, dtype=torch.float16)
    vs = torch.zeros((B, hkv, 1, 128), device=cuda, dtype=torch.float16)
    outs = torch.zeros_like(qs)
    plan_tokens = L + warm + steps
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    snapshot = dev.state.clone()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            dev.decode_step(qs, ks, vs, out=outs, plan_tokens=plan_tokens)
    torch.cuda.current_stream().wait_stream(side)
    # capturing launched nothing: the device state is untouched; the host mirror took the step, put it back
    assert torch.equal(dev.state, snapshot)
    dev.kv_seq_len, dev.tkq, dev.tvq, dev.k_start, dev.v_start = snapshot.tolist()[:5]
    dev.k_len, dev.v_len = dev.kv_seq_len - dev.tkq, dev.kv_seq_len - dev.tvq

    worst = 0.0
    for i in range(steps):
        t = L + warm + i
        q = _t(make_q(t, B, nh), cuda)
        want = host.decode_step(q, kt[:, :, t:t + 1], vt[:, :, t:t + 1])
        qs.copy_(q); ks.copy_(kt[:, :, t:t + 1]); vs.copy_(vt[:, :, t:t + 1])
        graph.replay()
        dev.advance_mirror(1)
        torch.cuda.synchronize()
        assert dev.state.tolist()[:6] == [host.kv_seq_len, host.tkq, host.tvq, host.k_start, host.v_start, 0], f"step {i}"
        assert torch.isfinite(outs.float()).all()
        worst = max(worst, float(row_rel(outs.cpu().numpy(), want.cpu().numpy()).max()))
    assert worst <= 1e-3, worst
    assert (dev.kv_seq_len, dev.tkq, dev.tvq, dev.k_start, dev.v_start) == (host.kv_seq_len, host.tkq, host.tvq, host.k_start, host.v_start)
    for x, y in zip(dev.as_tuple()[:8], host.as_tuple()[:8]):
        assert torch.equal(x, y)                                 # codes, scales, minima and tails bit for bit


@pytest.mark.parametrize("kinds,nh,hkv,G,with_exchange", [([(4, 4), (3, 2), (2, 2)], 4, 4, 32, False),
                                                          ([(4, 4), (3, 2), (3, 2), (2, 2)], 8, 2, 128, True)])
def test_whole_step_captured_once(cuda, kinds, nh, hkv, G, with_exchange):
    """A stack of layers (different bit settings) as ONE captured graph, replayed 40 times, against the same stack
    driven from the host layer by layer; with_exchange adds the head-sharded exchange of a one-rank "world" (peer
    stores into this GPU's own gather buffer and the device-side generation wait) inside the graph."""
    import kvmix_b200 as kv
    from kvmix_b200 import sharding
    B, L0, steps = 2, 900, 40
    layers = len(kinds)
    k, v = make_kv(5, B, hkv, L0 + steps + 2)
    kt, vt = _t(k, cuda), _t(v, cuda)
    mk = lambda kb, vb, ds: kv.KVmixLayerCache(B, hkv, 128, L0 + steps + 16, kb, vb, G, residual_length=128, device=cuda,
                                               device_state=ds)
    host = [mk(kb, vb, False) for kb, vb in kinds]
    devc = [mk(kb, vb, True) for kb, vb in kinds]
    for c in host + devc:
        c.prefill(kt[:, :, :L0], vt[:, :, :L0])
    peers = None
    if with_exchange:
        pair = [(torch.zeros((2, B, nh, 1, 128), dtype=torch.float16, device=cuda), torch.zeros(64, dtype=torch.int32, device=cuda))]
        peers = sharding.PeerGather(B, nh, 128, cuda, peers=pair, rank=0)
    qs = [torch.zeros((B, nh, 1, 128), device=cuda, dtype=torch.float16) for _ in range(layers)]
    ks = [torch.zeros((B, hkv, 1, 128), device=cuda, dtype=torch.float16) for _ in range(layers)]
    vs = [torch.zeros((B, hkv, 1, 128), device=cuda, dtype=torch.float16) for _ in range(layers)]
    outs = [torch.zeros((B, nh, 1, 128), device=cuda, dtype=torch.float16) for _ in range(layers)]
    # one eager step first: the fused path is taken and the workspaces exist
    for l in range(layers):
        q = _t(make_q(1000 + l, B, nh), cuda)
        a = host[l].decode_step(q, kt[:, :, L0:L0 + 1], vt[:, :, L0:L0 + 1])
        b = devc[l].decode_step(q, kt[:, :, L0:L0 + 1], vt[:, :, L0:L0 + 1], peers=peers)
        if peers is not None:
            assert torch.equal(peers.wait(), a)
        assert torch.equal(a, b)
    step = kv.CapturedDecodeStep(devc, qs, ks, vs, outs, max_replays=steps, peers=peers)
    assert [c.kv_seq_len for c in devc] == [L0 + 1] * layers          # capturing moved nothing
    worst = 0.0
    for i in range(steps):
        t = L0 + 1 + i
        want = []
        for l in range(layers):
            q = _t(make_q(2000 + 7 * i + l, B, nh), cuda)
            qs[l].copy_(q); ks[l].copy_(kt[:, :, t:t + 1]); vs[l].copy_(vt[:, :, t:t + 1])
            want.append(host[l].decode_step(q, kt[:, :, t:t + 1], vt[:, :, t:t + 1]))
        step.replay()
        torch.cuda.synchronize()
        for l in range(layers):
            worst = max(worst, float(row_rel(outs[l].cpu().numpy(), want[l].cpu().numpy()).max()))
            if peers is not None and l >= layers - peers.depth:  # the round-robin gather buffers still hold the last layers
                assert torch.equal(step.gathered[l], outs[l])
    assert worst <= 1e-3, worst
    if peers is not None:
        peers.check()
    for h, d in zip(host, devc):
        assert (h.kv_seq_len, h.tkq, h.tvq, h.k_start, h.v_start) == (d.kv_seq_len, d.tkq, d.tvq, d.k_start, d.v_start)
        assert d.state.tolist()[:5] == [h.kv_seq_len, h.tkq, h.tvq, h.k_start, h.v_start]
        for x, y in zip(d.as_tuple()[:8], h.as_tuple()[:8]):
            assert torch.equal(x, y)
    with pytest.raises(RuntimeError, match="beyond the context"):
        step.replay()
