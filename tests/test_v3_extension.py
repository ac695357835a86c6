"""3-bit VALUES at head_dim 128: an extension upstream does not have (its 3-bit rule needs head_dim % 11 == 0,
quant_cuda/csrc/quantization_cuda.cu:433-434,649), so nothing upstream-produced can pin it -- "parity unpinned".

What is checked instead:
  * the restatement of the extension equals upstream's (pinned) 3-bit rule wherever that rule applies: on rows whose
    length is a multiple of 11 it is word-for-word the pinned quantizer, and on a 128-channel row its first 11 words
    are the pinned quantizer of the first 121 channels; the short last group is checked against a closed form;
  * the library's quantizer reproduces the restatement bit-exactly (codes, fp16 scale and min);
  * decode attention over a K?/V3 cache is within 2e-3 per row of the restatement, MHA and GQA, with a mask, over
    appended steps, and through prefill_projected.
"""
import numpy as np
import pytest

import oracle
from oracle.glue import RefLayerCache
from util import REL_TOL, make_kv, make_q, row_rel


def _closed_form_group(x):
    """One group of <= 10 elements by the 3-bit rule, fp32: codes, scale, min."""
    x = x.astype(np.float32)
    lo, hi = x.min(), x.max()
    sc = np.float32(hi - lo) / np.float32(7.0)
    with np.errstate(invalid="ignore", divide="ignore"):
        n = (x - lo) / sc
    q = np.where(np.isnan(n), 0, np.floor(n + np.float32(0.5))).astype(np.int64)       # n >= 0: roundf == floor(n + .5)
    return np.clip(q, 0, 7), np.float16(np.float32(hi - lo) * np.float32(1.0 / 7.0)), np.float16(lo)


def test_restatement_equals_pinned_rule_on_full_groups():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 3, 17, 121)).astype(np.float16)
    c0, s0, m0 = oracle.quantize_pack_last_dim(x, 11, 3)
    c1, s1, m1 = oracle.quantize_ragged3(x)
    assert (c0 == c1).all() and (s0.view(np.uint16) == s1.view(np.uint16)).all() and (m0.view(np.uint16) == m1.view(np.uint16)).all()


def test_restatement_on_128_channels():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((1, 2, 33, 128)).astype(np.float16)
    x[0, 0, 5, 121:] = 0.25                                       # a constant short group: scale 0, all codes 0
    c, s, m = oracle.quantize_ragged3(x)
    assert c.shape == (1, 2, 33, 12) and s.shape == (1, 2, 33, 12) and m.shape == (1, 2, 33, 12)
    c0, s0, m0 = oracle.quantize_pack_last_dim(np.ascontiguousarray(x[..., :121]), 11, 3)
    assert (c[..., :11] == c0).all() and (s[..., :11].view(np.uint16) == s0.view(np.uint16)).all()
    assert (m[..., :11].view(np.uint16) == m0.view(np.uint16)).all()
    for h in range(2):
        for t in range(33):
            q, sc, lo = _closed_form_group(x[0, h, t, 121:])
            word = sum(int(q[i]) << (3 * i) for i in range(7))
            assert (int(c[0, h, t, 11]) & 0xFFFFFFFF) == word
            assert np.float16(s[0, h, t, 11]).view(np.uint16) == sc.view(np.uint16)
            assert np.float16(m[0, h, t, 11]).view(np.uint16) == lo.view(np.uint16)
    assert c[0, 0, 5, 11] == 0 and s[0, 0, 5, 11] == 0


def test_reference_cache_holds_v3():
    k, v = make_kv(7, 1, 2, 300)
    ref = RefLayerCache(2, 3, 32, residual_length=64)
    ref.prefill(k, v)
    assert ref.vcode.shape == (1, 2, ref.tvq, 12) and ref.vscale.shape == (1, 2, ref.tvq, 12)
    q = make_q(8, 1, 4)
    a = ref.attend(q, ref_rounding=0).astype(np.float32)
    # dequantize by hand and attend in float64
    vq = np.zeros((1, 2, ref.tvq, 132), np.float64)
    for j in range(12):
        w = ref.vcode[..., j].astype(np.int64) & 0xFFFFFFFF
        for i in range(11):
            f = (w >> (3 * i)) & (7 if i < 10 else 3)
            vq[..., 11 * j + i] = f * ref.vscale[..., j].astype(np.float64) + ref.vmn[..., j].astype(np.float64)
    vall = np.concatenate([vq[..., :128], ref.vfull.astype(np.float64)], axis=2).astype(np.float16)
    # the output is linear in V: the same keys over the hand-dequantized values held as an fp16 tail must agree (up to
    # the fp16 rounding of those values)
    out = oracle.decode_attention(q, ref.kcode, ref.kscale, ref.kmn, ref.kfull, None, None, None, vall, 2, 32, 4, 32,
                                  ref_rounding=0).astype(np.float32)
    assert vall.shape[2] == 300
    assert row_rel(a.reshape(4, 128), out.reshape(4, 128)).max() < 1.5e-3


# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(1, 2, 40, 128), (2, 3, 129, 128), (1, 1, 7, 40), (1, 2, 64, 121)])
def test_library_quantizer_bit_exact(cuda, shape):
    import torch
    from kvmix_b200 import ops
    rng = np.random.default_rng(sum(shape))
    x = (rng.standard_normal(shape) * rng.choice([0.1, 1.0, 30.0], size=shape[:3] + (1,))).astype(np.float16)
    x[0, 0, 1, -5:] = x[0, 0, 1, -5]                             # constant tail
    B, H, A, S = shape
    nw = -(-S // 11)
    xt = torch.from_numpy(x).to(cuda)
    for by_div in (False, True):
        code = torch.full((B, H, A, nw), -1, dtype=torch.int32, device=cuda)
        scale = torch.empty((B, H, A, nw), dtype=torch.float16, device=cuda)
        mn = torch.empty_like(scale)
        ops.quantize_into(xt, 11, 3, code, scale, mn, scale_by_division=by_div, ragged_tail=True)
        c, s, m = oracle.quantize_ragged3(x, scale_by_division=by_div)
        assert (code.cpu().numpy() == c).all()
        assert (scale.cpu().numpy().view(np.uint16) == s.view(np.uint16)).all()
        assert (mn.cpu().numpy().view(np.uint16) == m.view(np.uint16)).all()


@pytest.mark.gpu
def test_upstream_rules_unchanged_without_the_flag(cuda):
    import torch
    from kvmix_b200 import ops
    x = torch.zeros((1, 1, 4, 128), dtype=torch.float16, device=cuda)
    with pytest.raises(RuntimeError, match="divisible by 11"):
        ops.quantize_pack_last_dim_cuda(x, 11, 3)


@pytest.mark.gpu
@pytest.mark.parametrize("kb,nh,hkv,G,T,mask", [(4, 4, 4, 32, 700, False), (2, 8, 2, 64, 1500, True), (3, 8, 2, 64, 2300, False)])
def test_attention_over_v3_cache(cuda, kb, nh, hkv, G, T, mask):
    import torch
    import kvmix_b200 as kv
    B, steps = 2, 70
    k, v = make_kv(100 + kb, B, hkv, T + steps)
    ref = RefLayerCache(kb, 3, G, residual_length=128)
    ref.prefill(k[:, :, :T], v[:, :, :T])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    c = kv.KVmixLayerCache(B, hkv, 128, T + steps + 8, kb, 3, G, residual_length=128, device=cuda)
    c.prefill(t(k[:, :, :T]), t(v[:, :, :T]))
    worst = 0.0
    for s in range(steps):
        q = make_q(500 + s, B, nh)
        m = None
        if mask:
            m = np.zeros((B, 1, 1, T + s + 1), np.float32)
            m[1, 0, 0, :37] = np.finfo(np.float32).min
        kn, vn = k[:, :, T + s:T + s + 1], v[:, :, T + s:T + s + 1]
        got = c.decode_step(t(q), t(kn), t(vn), attention_mask=None if m is None else t(m)).cpu().numpy()
        ref.append(kn, vn)
        if s % 23 == 0 or s == steps - 1:
            want = ref.attend(q, ref_rounding=7, attention_mask=m)
            worst = max(worst, row_rel(got.reshape(B * nh, 128), want.reshape(B * nh, 128)).max())
    tup = c.as_tuple()
    assert c.tvq == ref.tvq and tup[4].shape[3] == 12
    assert (tup[4].cpu().numpy() == ref.vcode).all()
    assert (tup[6].cpu().numpy().view(np.uint16) == ref.vscale.view(np.uint16)).all()
    assert (tup[7].cpu().numpy().view(np.uint16) == ref.vmn.view(np.uint16)).all()
    assert (tup[0].cpu().numpy() == ref.kcode).all()
    assert worst <= REL_TOL, f"attention over 3-bit values: {worst:.3e} from the restatement"


@pytest.mark.gpu
def test_prefill_projected_v3(cuda):
    import torch
    import kvmix_b200 as kv
    B, hkv, L = 1, 2, 512
    k, v = make_kv(77, B, hkv, L)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    a = kv.KVmixLayerCache(B, hkv, 128, L + 8, 2, 3, 32, residual_length=128, device=cuda)
    a.prefill(t(k), t(v))
    b = kv.KVmixLayerCache(B, hkv, 128, L + 8, 2, 3, 32, residual_length=128, device=cuda)
    to_proj = lambda x: t(x).transpose(1, 2).reshape(B, L, hkv * 128).contiguous()
    b.prefill_projected(to_proj(k), to_proj(v))
    for x, y in zip(a.as_tuple()[:8], b.as_tuple()[:8]):
        assert torch.equal(x, y)
