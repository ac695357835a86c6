"""The fused decode step (cache update inside the attention launch) against the same step made of separate launches
(ring append, group quantizers, attention) and against the oracle: after every step the two caches hold identical
packed codes, scales, minima and fp16 tails, and return bit-identical attention outputs -- across several group
boundaries, for multi-head and grouped-query layouts, both window policies, with and without a padding mask."""
import numpy as np
import pytest
import torch

from oracle.glue import RefLayerCache
from util import assert_close_to_upstream, make_kv, make_q

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


CASES = [  # kb, vb, G, nh, hkv, policy, prompt, steps, fused expected
    (2, 2, 32, 4, 4, dict(residual_length=128), 700, 70, True),
    (4, 4, 32, 4, 4, dict(k_residual_ratio=0.3, v_residual_ratio=0.3), 500, 70, True),
    (3, 2, 32, 2, 2, dict(residual_length=128), 1000, 40, True),
    (4, 2, 128, 4, 4, dict(residual_length=256), 5000, 140, True),
    (2, 2, 64, 8, 2, dict(residual_length=128), 4200, 70, True),                  # grouped queries 4:1
    (3, 4, 64, 8, 2, dict(k_residual_ratio=0.2, v_residual_ratio=0.3), 900, 70, True),
    (4, 4, 128, 4, 2, dict(residual_length=256), 2300, 140, True),                 # grouped queries 2:1
    (2, 2, 32, 8, 2, dict(residual_length=128), 700, 40, False),                  # 2-bit keys in groups of 32: per-head CTAs share a kv head
    (2, 2, 64, 16, 2, dict(residual_length=128), 700, 40, False),                 # 8 query heads per kv head: two CTAs per kv head
]


@pytest.mark.parametrize("kb,vb,G,nh,hkv,policy,L,steps,fused", CASES)
def test_fused_step_equals_separate_launches(cuda, kb, vb, G, nh, hkv, policy, L, steps, fused):
    import kvmix_b200 as kv
    B = 2
    k, v = make_kv(300 + kb * 10 + vb, B, hkv, L + steps)
    kt, vt = _t(k, cuda), _t(v, cuda)
    ref = RefLayerCache(kb, vb, G, **policy)
    ref.prefill(k[:, :, :L], v[:, :, :L])
    a = kv.KVmixLayerCache(B, hkv, 128, L + steps + 8, kb, vb, G, device=cuda, **policy)      # decode_step (fused if possible)
    b = kv.KVmixLayerCache(B, hkv, 128, L + steps + 8, kb, vb, G, device=cuda, **policy)      # append + attend
    a.prefill(kt[:, :, :L], vt[:, :, :L])
    b.prefill(kt[:, :, :L], vt[:, :, :L])
    mask = None
    launches = []
    for i in range(steps):
        t = L + i
        q = _t(make_q(5000 + t, B, nh), cuda)
        if i % 7 == 3:                                           # a left-padding mask now and then
            mask = torch.zeros((B, 1, 1, t + 1), device=cuda, dtype=torch.float32)
            mask[1, 0, 0, :t // 3] = torch.finfo(torch.float32).min
        else:
            mask = None
        n0 = kv.ops.LAUNCHES[0]
        got = a.decode_step(q, kt[:, :, t:t + 1], vt[:, :, t:t + 1], attention_mask=mask)
        launches.append(kv.ops.LAUNCHES[0] - n0)
        b.append(kt[:, :, t:t + 1], vt[:, :, t:t + 1])
        want = b.attend(q, attention_mask=mask)
        assert (a.tkq, a.tvq, a.k_len, a.v_len, a.k_start, a.v_start, a.kv_seq_len) == \
               (b.tkq, b.tvq, b.k_len, b.v_len, b.k_start, b.v_start, b.kv_seq_len)
        assert torch.equal(got, want), f"step {i}: fused and separate launches differ by {(got.float() - want.float()).abs().max().item():.3e}"
        if i in (0, steps // 2, steps - 1):                      # and both agree with the oracle
            ref_now = ref
            while ref_now.kv_seq_len < t + 1:
                s = ref_now.kv_seq_len
                ref_now.append(k[:, :, s:s + 1], v[:, :, s:s + 1])
            qn = q.cpu().numpy()
            mn = None if mask is None else mask.cpu().numpy()
            assert_close_to_upstream(got.cpu().numpy(), ref_now.attend(qn, ref_rounding=7, attention_mask=mn),
                                     ref_now.attend(qn, ref_rounding=0, attention_mask=mn), dominated_rows=1)
    assert a._fused is fused
    if fused:
        # one launch per step; upstream's ratio policy first shrinks the prompt's fp16 tail geometrically, several groups
        # per step, and those steps run unfused (the fused launch takes at most one group per step)
        assert set(launches[-30:]) == {1} and ("residual_length" not in policy or set(launches) == {1})
    else:
        assert min(launches) >= 2
    assert a.tkq > (L // 2) and a.tkq == ref.tkq and a.tvq == ref.tvq
    for x, y, w in zip(a.as_tuple()[:8], b.as_tuple()[:8],
                       [ref.kcode, ref.kfull, ref.kscale, ref.kmn, ref.vcode, ref.vfull, ref.vscale, ref.vmn]):
        assert torch.equal(x, y)
        xn = x.cpu().numpy()
        assert np.array_equal(xn.view(np.uint16) if xn.dtype == np.float16 else xn, w.view(np.uint16) if w.dtype == np.float16 else w)


def test_fused_step_argument_errors(cuda):
    """The C ABI refuses inconsistent fused-step requests before launching anything."""
    import ctypes as C
    import kvmix_b200 as kv
    from kvmix_b200 import _lib
    c = kv.KVmixLayerCache(1, 2, 128, 600, 2, 2, 32, residual_length=128, device=cuda)
    k, v = make_kv(1, 1, 2, 400)
    c.prefill(_t(k, cuda), _t(v, cuda))
    q = _t(make_q(1, 1, 2), cuda)
    out = torch.empty_like(q)
    kn, vn = _t(k[:, :, :1], cuda), _t(v[:, :, :1], cuda)
    c.decode_step(q, kn, vn, out=out)                           # fills c._att for this geometry
    a = c._att
    L = _lib.lib()
    a.k_new, a.v_new = kn.data_ptr(), 0
    assert L.kvq_decode_attn(C.byref(a), None) == -10           # one of the two rows missing
    a.v_new = vn.data_ptr()
    a.kn_sB, a.kn_sH, a.vn_sB, a.vn_sH = kn.stride(0), kn.stride(1), vn.stride(0), vn.stride(1)
    a.k_quant = 17
    assert L.kvq_decode_attn(C.byref(a), None) == -9            # not a whole group
    a.k_quant, a.k_quant_slot = 32, c.k_cap - 8
    assert L.kvq_decode_attn(C.byref(a), None) == -7            # the group would run past the ring
    a.k_quant, a.k_quant_slot, a.nh = 0, 0, 16
    q16 = torch.zeros((1, 16, 1, 128), device=cuda, dtype=torch.float16)
    a.q, a.q_sB, a.q_sH = q16.data_ptr(), q16.stride(0), q16.stride(1)
    assert L.kvq_decode_attn(C.byref(a), None) == -11           # 8 query heads per kv head: not fused
