"""The benchmark configurations at their FULL attention shapes, one layer each, on the GPU.

What the oracle can finish in seconds (one sequence) is compared directly: packed codes bit-exact, fp16
scale/min bit-exact, attention within the two-part 2e-3 statement.  The rest of the batch is covered by
size-independent properties: a sequence's result does not depend on its neighbours in the batch, and
sharding KV heads into halves reproduces the unsharded output (what the head-sharded 2-GPU run of the
long-context configuration relies on).  Those comparisons allow 1e-3 relative per row rather than bit
equality: the number of token splits is chosen from the number of heads in the launch, every split scales
its probabilities by its own maximum, and p*scale is rounded to fp16 once per token -- so two split plans
are two independent draws of that rounding noise (measured 4.0e-4 .. 4.9e-4 between them over 24 seeds,
against 3.7e-4 .. 4.6e-4 between either and the oracle).
"""
import numpy as np
import pytest
import torch

import oracle
from oracle.glue import RefLayerCache
from util import assert_attn_parity, row_rel

pytestmark = pytest.mark.gpu


def _layer(cuda, B, hkv, T, kb, vb, G, window, extra=8):
    import kvmix_b200 as kv
    from kvmix_b200 import configs
    c = kv.KVmixLayerCache(B, hkv, 128, T + extra, kb, vb, G, residual_length=window, device=cuda)
    k, v = configs.synth_kv(B, hkv, T, 128, cuda, seed=kb * 10 + vb)
    c.prefill(k, v)
    return c, k, v


def _query(cuda, B, nh, seed):
    g = torch.Generator(device=cuda).manual_seed(seed)
    return torch.randn((B, nh, 1, 128), generator=g, device=cuda, dtype=torch.float16)


def _ref_for_sequence(k, v, b, kb, vb, G, window):
    ref = RefLayerCache(kb, vb, G, residual_length=window)
    ref.prefill(k[b:b + 1].cpu().numpy(), v[b:b + 1].cpu().numpy())
    return ref


def _check_one_sequence(cuda, c, k, v, q, b, kb, vb, G, window):
    import kvmix_b200 as kv
    ref = _ref_for_sequence(k, v, b, kb, vb, G, window)
    tup = c.as_tuple()
    assert ref.tkq == c.tkq and ref.tvq == c.tvq
    for got, want in [(tup[0], ref.kcode), (tup[2], ref.kscale), (tup[3], ref.kmn), (tup[4], ref.vcode),
                      (tup[6], ref.vscale), (tup[7], ref.vmn)]:
        g = got[b:b + 1].cpu().numpy()
        assert g.shape == want.shape
        assert (g.view(np.uint16) == want.view(np.uint16)).all() if g.dtype == np.float16 else (g == want).all()
    qn = q[b:b + 1].cpu().numpy()

    def kernel(rs):
        return c.attend(q, round_scores=rs)[b:b + 1].cpu().numpy()
    assert_attn_parity(kernel, ref, qn)


@pytest.mark.parametrize("kb,vb", [(4, 4), (2, 2)])
def test_config2_layer_full_batch_other_bit_settings(cuda, kb, vb):
    """The other two bit settings of the Llama-2-7B map at the full batch: K4V4 and K2V2, group 32, window 128."""
    B, H, T = 64, 32, 4096
    c, k, v = _layer(cuda, B, H, T, kb, vb, 32, 128)
    q = _query(cuda, B, H, 112 + kb)
    _check_one_sequence(cuda, c, k, v, q, 41, kb, vb, 32, 128)


def test_config2_layer_full_batch(cuda):
    """Llama-2-7B geometry: batch 64, 32 heads (MHA), context 4096, K3V2 (group 11 / 32), window 128."""
    B, H, T = 64, 32, 4096
    c, k, v = _layer(cuda, B, H, T, 3, 2, 32, 128)
    q = _query(cuda, B, H, 102)
    _check_one_sequence(cuda, c, k, v, q, 5, 3, 2, 32, 128)
    # a sequence's output does not depend on the rest of the batch
    full = c.attend(q)
    import kvmix_b200 as kv
    solo = kv.KVmixLayerCache(1, H, 128, T + 8, 3, 2, 32, residual_length=128, device=cuda)
    solo.prefill(k[17:18], v[17:18])
    assert row_rel(solo.attend(q[17:18]).cpu().numpy(), full[17:18].cpu().numpy()).max() <= 1e-3


@pytest.mark.parametrize("kb,vb", [(4, 4), (3, 4), (2, 2), (2, 1)])
def test_config3_layer_gqa_long_context(cuda, kb, vb):
    """Mistral-7B geometry: batch 8, 32 query / 8 KV heads, context 32768, group 64 (11 for 3-bit keys), window 128:
    every bit setting of its layer map that upstream's format can hold."""
    B, nh, hkv, T = 8, 32, 8, 32768
    c, k, v = _layer(cuda, B, hkv, T, kb, vb, 64, 128)
    q = _query(cuda, B, nh, 103)
    _check_one_sequence(cuda, c, k, v, q, 3, kb, vb, 64, 128)


def test_config5_layer_131k_tokens_and_head_sharding(cuda):
    """Llama-3-8B geometry: one sequence of 131072 tokens, 32 query / 8 KV heads, K3V2, group 128, window 256."""
    import kvmix_b200 as kv
    from kvmix_b200 import sharding
    B, nh, hkv, T = 1, 32, 8, 131072
    c, k, v = _layer(cuda, B, hkv, T, 3, 2, 128, 256)
    q = _query(cuda, B, nh, 105)
    _check_one_sequence(cuda, c, k, v, q, 0, 3, 2, 128, 256)
    full = c.attend(q)
    parts = []
    for rank in range(2):                                   # what each of two head-sharded ranks would compute
        (klo, khi), (qlo, qhi) = sharding.shard_kv_heads(nh, hkv, 2, rank)
        shard = kv.KVmixLayerCache(B, khi - klo, 128, T + 8, 3, 2, 128, residual_length=256, device=cuda)
        shard.prefill(k[:, klo:khi], v[:, klo:khi])
        parts.append(shard.attend(q[:, qlo:qhi].contiguous()))
    assert row_rel(torch.cat(parts, 1).cpu().numpy(), full.cpu().numpy()).max() <= 1e-3


def test_config4_quantizer_cells(cuda):
    """Quantize-on-append sweep cells: [16,32,8192,128] keys and values, Student-t outlier channels; a slice is
    compared with the oracle bit for bit, the whole tensor through idempotence: re-quantizing the dequantized
    tensor with the same grouping reproduces the same codes."""
    import kvmix_b200 as kv
    g = torch.Generator(device=cuda).manual_seed(3)
    x = torch.randn((16, 32, 8192, 128), generator=g, device=cuda, dtype=torch.float16)
    chi = torch.randn((16, 32, 8192, 4, 3), generator=g, device=cuda).pow(2).sum(-1).div(3.0).sqrt()
    x[..., :4] = (x[..., :4].float() / chi).to(torch.float16)
    for bits, G, style in [(4, 128, "k"), (1, 32, "k"), (2, 128, "v"), (3, 11, "k")]:
        src = x[:, :, :8184].transpose(2, 3) if bits == 3 else (x.transpose(2, 3) if style == "k" else x)
        code, sc, mn = kv.quantize_pack_last_dim_cuda(src, G, bits)
        sl = src[7:8, 3:5].contiguous().cpu().numpy()
        cw, sw, mw = oracle.quantize_pack_last_dim(sl, G, bits)
        assert (code[7:8, 3:5].cpu().numpy() == cw).all()
        assert (sc[7:8, 3:5].cpu().numpy().view(np.uint16) == sw.view(np.uint16)).all()
        assert (mn[7:8, 3:5].cpu().numpy().view(np.uint16) == mw.view(np.uint16)).all()
        if bits != 3:        # idempotence needs every code level reachable; the 3-bit word saturates its 11th field
            f = 32 // bits
            w = code.to(torch.int64) & 0xFFFFFFFF
            fields = torch.stack([(w >> (bits * i)) & (2 ** bits - 1) for i in range(f)], -1).reshape(src.shape)
            deq = (fields.float() * sc.float().repeat_interleave(G, -1) + mn.float().repeat_interleave(G, -1))
            lo = deq.reshape(*deq.shape[:-1], -1, G).amin(-1)
            hi = deq.reshape(*deq.shape[:-1], -1, G).amax(-1)
            assert (lo.to(torch.float16) == mn).all()            # the group's min survives dequantization exactly
            assert (hi >= lo).all() and (fields.reshape(*deq.shape[:-1], -1, G).amin(-1) == 0).all()
            del w, fields, deq, lo, hi
