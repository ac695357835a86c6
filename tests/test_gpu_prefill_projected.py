"""Prefill straight from the projections (kvq_prefill): rotary embedding + split + both quantizers + tail copies in the
library, against the same thing made of framework ops (RoPE as upstream's model files apply it, on fp16 tensors) followed
by the oracle's quantizer -- packed codes, scales, minima and the fp16 tails bit for bit -- and against the library's own
prefill() on pre-rotated [B, Hkv, L, D] tensors."""
import numpy as np
import pytest
import torch

from oracle.glue import RefLayerCache

pytestmark = pytest.mark.gpu


def rotate_half(x):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def rope_tables(L, D, dev, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D))
    freqs = torch.arange(L, dtype=torch.float32, device=dev)[:, None] * inv[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(torch.float16), emb.sin().to(torch.float16)


@pytest.mark.parametrize("kb,vb,G,policy", [(2, 2, 32, dict(residual_length=128)), (4, 4, 64, dict(residual_length=128)),
                                            (3, 2, 32, dict(k_residual_ratio=0.2, v_residual_ratio=0.2)),
                                            (1, 4, 128, dict(residual_length=256)), (4, 2, 32, dict(residual_length=700))])
def test_prefill_from_projections_matches_framework_rope_plus_oracle(cuda, kb, vb, G, policy):
    import kvmix_b200 as kv
    B, Hkv, L, D = 2, 4, 1000 if "residual_length" in policy else 777, 128
    g = torch.Generator(device=cuda).manual_seed(kb * 10 + vb)
    k_proj = torch.randn((B, L, Hkv * D), generator=g, device=cuda, dtype=torch.float16)
    v_proj = torch.randn((B, L, Hkv * D), generator=g, device=cuda, dtype=torch.float16)
    k_proj[..., 5] *= 8.0
    cos, sin = rope_tables(L, D, cuda)
    # what upstream's forward does on fp16 tensors: view, transpose, rotate
    k4 = k_proj.view(B, L, Hkv, D).transpose(1, 2)
    v4 = v_proj.view(B, L, Hkv, D).transpose(1, 2)
    k_rot = (k4 * cos[None, None]) + (rotate_half(k4) * sin[None, None])
    ref = RefLayerCache(kb, vb, G, **policy)
    ref.prefill(k_rot.cpu().numpy(), v4.contiguous().cpu().numpy())

    c = kv.KVmixLayerCache(B, Hkv, D, L + 8, kb, vb, G, device=cuda, **policy)
    n0 = kv.ops.LAUNCHES[0]
    c.prefill_projected(k_proj, v_proj, cos, sin)
    assert kv.ops.LAUNCHES[0] - n0 <= 3
    assert (c.tkq, c.tvq, c.k_len, c.v_len, c.kv_seq_len) == (ref.tkq, ref.tvq, ref.kfull.shape[2], ref.vfull.shape[2], L)
    tup = c.as_tuple()
    for got, want in zip(tup[:8], [ref.kcode, ref.kfull, ref.kscale, ref.kmn, ref.vcode, ref.vfull, ref.vscale, ref.vmn]):
        if want is None:
            assert got is None
            continue
        gn = got.cpu().numpy()
        assert gn.shape == want.shape
        assert np.array_equal(gn.view(np.uint16) if gn.dtype == np.float16 else gn,
                              want.view(np.uint16) if want.dtype == np.float16 else want)
    # same state as the library's prefill() on pre-rotated tensors, and a decode step on top agrees
    c2 = kv.KVmixLayerCache(B, Hkv, D, L + 8, kb, vb, G, device=cuda, **policy)
    c2.prefill(k_rot, v4)
    q = torch.randn((B, Hkv, 1, D), generator=g, device=cuda, dtype=torch.float16)
    kn = torch.randn((B, Hkv, 1, D), generator=g, device=cuda, dtype=torch.float16)
    assert torch.equal(c.decode_step(q, kn, kn), c2.decode_step(q, kn, kn))
    # keys that arrive rotated: no tables
    c3 = kv.KVmixLayerCache(B, Hkv, D, L + 8, kb, vb, G, device=cuda, **policy)
    c3.prefill_projected(k_rot.transpose(1, 2).contiguous().view(B, L, Hkv * D), v_proj)
    for x, y in zip(c3.as_tuple()[:8], tup[:8]):
        assert (x is None and y is None) or torch.equal(x, y)
