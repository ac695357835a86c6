"""CPU checks of the oracle itself: the C restatement against independent numpy closed forms,
upstream's argument rules, and the cache-update glue.  No GPU, no product code."""
import numpy as np
import pytest

import oracle
from oracle.glue import RefLayerCache, split_point
from util import assert_attn_close, make_kv, make_q


def np_quant(x, G, bits):
    """Closed form of the quantizer in numpy fp32 (independent of the C code)."""
    S = x.shape[-1]
    fpi = oracle.features_per_int(bits)
    xf = x.astype(np.float32).reshape(-1, S // G, G)
    mn = xf.min(-1, keepdims=True)
    mx = xf.max(-1, keepdims=True)
    sc = (mx - mn) / np.float32(2 ** bits - 1)
    with np.errstate(invalid="ignore", divide="ignore"):
        n = (xf - mn) / sc
    frac = n - np.trunc(n)
    q = np.where(np.isnan(n), 0, np.trunc(n) + (frac >= 0.5)).astype(np.int64)
    q = np.clip(q, 0, 2 ** bits - 1)
    if bits == 3:
        q[..., 10] = np.minimum(q[..., 10], 3)
    qw = q.reshape(-1, S // fpi, fpi)
    if bits == 3:
        w = sum(qw[..., i] << (3 * i) for i in range(10)) | (qw[..., 10] << 30)
    else:
        w = sum(qw[..., i] << (bits * i) for i in range(fpi))
    w = (w & 0xFFFFFFFF).astype(np.uint32).view(np.int32)
    shp = x.shape[:-1]
    stored = (mx - mn) * (np.float32(1) / np.float32(2 ** bits - 1))      # torch: tensor / scalar = tensor * (1/scalar)
    return (w.reshape(shp + (S // fpi,)), stored.astype(x.dtype).reshape(shp + (S // G,)),
            mn.astype(x.dtype).reshape(shp + (S // G,)), q.reshape(x.shape))


@pytest.mark.parametrize("bits,G,S", [(4, 32, 64), (2, 32, 128), (1, 32, 96), (3, 11, 66), (4, 128, 256), (2, 64, 64),
                                      (4, 8, 32), (1, 64, 128)])
@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_quantizer_matches_closed_form(bits, G, S, dtype):
    rng = np.random.default_rng(bits * 100 + G)
    x = rng.standard_normal((2, 3, 17, S)).astype(dtype)
    x[0, 0, 0] = 0.5                                   # constant groups
    c, s, m = oracle.quantize_pack_last_dim(x, G, bits)
    cw, sw, mw, _ = np_quant(x, G, bits)
    assert c.dtype == np.int32 and s.dtype == dtype and m.dtype == dtype
    assert (c == cw).all() and (s == sw).all() and (m == mw).all()
    assert (c[0, 0, 0] == 0).all() and (s[0, 0, 0] == 0).all()


def test_round_half_away_from_zero():
    # group min 0, max 15 -> scale 1: values k + 0.5 must round up (roundf), not to even (rint)
    x = np.zeros((1, 1, 1, 32), np.float16)
    x[..., :16] = np.arange(16) * 1.0
    x[..., 16:31] = np.arange(15) + 0.5
    c, s, m = oracle.quantize_pack_last_dim(x, 32, 4)
    codes = [(int(c[0, 0, 0, i // 8]) >> (4 * (i % 8))) & 15 for i in range(32)]
    assert codes[:16] == list(range(16))
    assert codes[16:31] == [k + 1 for k in range(15)]
    assert float(s[0, 0, 0, 0]) == 1.0 and float(m[0, 0, 0, 0]) == 0.0


def test_three_bit_word_format():
    x = np.tile(np.arange(11, dtype=np.float16) * 0.7, (1, 1, 1, 1))
    c, s, m = oracle.quantize_pack_last_dim(x, 11, 3)
    w = int(c[0, 0, 0, 0]) & 0xFFFFFFFF
    fields = [(w >> (3 * i)) & 7 for i in range(10)] + [w >> 30]
    assert fields[:10] == [0, 1, 2, 3, 4, 5, 6, 7, 7, 7][:10] or fields[0] == 0
    assert fields[10] == 3                             # 11th element saturates at 3 of 7


@pytest.mark.parametrize("args,msg", [
    (((1, 1, 4, 64), 32, 3), "group_length must be 11"),
    (((1, 1, 4, 65), 11, 3), "divisible by 11"),
    (((1, 1, 4, 48), 32, 4), "divisible by group_length"),
    (((1, 1, 4, 16), 16, 1), r"divisible by \(32 / quant_bits\)"),
])
def test_quantizer_argument_errors(args, msg):
    shape, G, bits = args
    with pytest.raises(RuntimeError, match=msg):
        oracle.quantize_pack_last_dim(np.zeros(shape, np.float16), G, bits)
    with pytest.raises(RuntimeError, match="4D"):
        oracle.quantize_pack_last_dim(np.zeros((4, 64), np.float16), 32, 4)


@pytest.mark.parametrize("bits,G", [(4, 32), (2, 32), (1, 32), (3, 11), (2, 64)])
@pytest.mark.parametrize("nh,nh_kv", [(2, 2), (4, 2)])
def test_gemv_matches_dense_dequant(bits, G, nh, nh_kv):
    rng = np.random.default_rng(bits)
    T = 66 if bits == 3 else 128
    kt = rng.standard_normal((2, nh_kv, 128, T)).astype(np.float16)
    c, s, m = oracle.quantize_pack_last_dim(kt, G, bits)
    _, _, _, q = np_quant(kt, G, bits)
    deq = (s.astype(np.float32)[..., None] * q.reshape(2, nh_kv, 128, T // G, G) +
           m.astype(np.float32)[..., None]).reshape(2, nh_kv, 128, T)
    x = rng.standard_normal((2, nh, 1, 128)).astype(np.float16)
    out = oracle.quantized_gemm(G, x, c, s, m, bits)
    rep = nh // nh_kv
    want = np.einsum("bhk,bhkn->bhn", x[:, :, 0].astype(np.float64), np.repeat(deq, rep, axis=1).astype(np.float64))
    assert out.shape == (2, nh, 1, T)
    err = np.abs(out[:, :, 0].astype(np.float64) - want)
    assert (err <= 1e-3 * np.abs(want) + 2e-2).all()    # one fp16 rounding of an O(30) value


def test_gemv_rejects_bad_heads():
    z = np.zeros((1, 3, 1, 128), np.float16)
    with pytest.raises(RuntimeError, match="divisible by KV heads"):
        oracle.quantized_gemm(32, z, np.zeros((1, 2, 128, 4), np.int32), np.zeros((1, 2, 128, 1), np.float16),
                              np.zeros((1, 2, 128, 1), np.float16), 4)


@pytest.mark.parametrize("bits,G", [(4, 32), (2, 32), (1, 32), (3, 11)])
def test_append_forms_are_concatenation(bits, G):
    rng = np.random.default_rng(5)
    T0, T1 = (66, 33) if bits == 3 else (64, 32)
    k0 = rng.standard_normal((1, 2, 128, T0)).astype(np.float16)
    k1 = rng.standard_normal((1, 2, 128, T1)).astype(np.float16)
    c0, s0, m0 = oracle.quantize_pack_last_dim(k0, G, bits)
    c1, s1, m1 = oracle.quantize_pack_last_dim(k1, G, bits)
    c, s, m = oracle.process_key_quantization(k1, c0, s0, m0, G, bits)
    assert (c == np.concatenate([c0, c1], 3)).all() and (s == np.concatenate([s0, s1], 3)).all()
    assert (m == np.concatenate([m0, m1], 3)).all()
    if bits != 3:
        v0 = rng.standard_normal((1, 2, 6, 128)).astype(np.float16)
        v1 = rng.standard_normal((1, 2, 3, 128)).astype(np.float16)
        a0 = oracle.quantize_pack_last_dim(v0, G, bits)
        a1 = oracle.quantize_pack_last_dim(v1, G, bits)
        got = oracle.process_value_quantization(v1, *a0, G, bits)
        for g, x0, x1 in zip(got, a0, a1):
            assert (g == np.concatenate([x0, x1], 2)).all()


def test_split_point_policy():
    # ratio policy, modeling_llama_KVmix.py:118-126
    assert split_point(1024, 32, ratio=0.2) == ((1024 - 204) // 32) * 32 == 800
    assert split_point(31, 32, ratio=0.2) == 0
    assert split_point(40, 32, ratio=0.2) == 32
    assert split_point(224, 11, ratio=0.3) == ((224 - 67) // 11) * 11
    # fixed window
    assert split_point(1024, 32, residual_length=128) == 896
    assert split_point(159, 32, residual_length=128) == 0
    assert split_point(160, 32, residual_length=128) == 32
    assert split_point(100, 32, residual_length=128) == 0


def test_glue_fixed_window_tail_and_prefix():
    k, v = make_kv(3, 1, 2, 300)
    c = RefLayerCache(4, 2, 32, residual_length=128)
    c.prefill(k[:, :, :200], v[:, :, :200])
    assert c.tkq == 64 and c.tvq == 64 and c.kfull.shape[2] == 136
    for t in range(200, 300):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
        assert 128 <= c.kfull.shape[2] <= 159 and c.tkq + c.kfull.shape[2] == t + 1
    # the packed prefix equals quantizing the same tokens in one go (groups are independent)
    kc, ks, km = oracle.quantize_pack_last_dim(np.ascontiguousarray(k[:, :, :c.tkq].transpose(0, 1, 3, 2)), 32, 4)
    assert (kc == c.kcode).all() and (ks == c.kscale).all() and (km == c.kmn).all()
    vc, vs, vm = oracle.quantize_pack_last_dim(v[:, :, :c.tvq], 32, 2)
    assert (vc == c.vcode).all() and (vs == c.vscale).all()


def test_glue_ratio_policy_independent_boundaries():
    k, v = make_kv(4, 1, 2, 400)
    c = RefLayerCache(3, 4, 32, k_residual_ratio=0.2, v_residual_ratio=0.3)
    c.prefill(k[:, :, :330], v[:, :, :330])
    assert c.k_group == 11 and c.tkq == ((330 - 66) // 11) * 11 and c.tvq == ((330 - 99) // 32) * 32
    for t in range(330, 400):
        c.append(k[:, :, t:t + 1], v[:, :, t:t + 1])
    assert c.tkq != c.tvq and c.tkq + c.kfull.shape[2] == 400 == c.tvq + c.vfull.shape[2]


@pytest.mark.parametrize("kb,vb,G,nh,hkv", [(4, 2, 32, 4, 4), (2, 2, 32, 4, 2), (3, 4, 32, 2, 2), (2, 1, 64, 8, 2)])
def test_decode_attention_against_dense(kb, vb, G, nh, hkv):
    T = 352 + 128
    k, v = make_kv(6, 1, hkv, T)
    q = make_q(6, 1, nh)
    c = RefLayerCache(kb, vb, G, residual_length=128)
    c.prefill(k, v)
    out_ref = c.attend(q, ref_rounding=True)
    out_f32 = c.attend(q, ref_rounding=False)
    # dense attention over the dequantized cache, float64
    fk, fv = oracle.features_per_int(kb), oracle.features_per_int(vb)

    def unpack(code, bits, f):
        w = code.astype(np.int64) & 0xFFFFFFFF
        if bits == 3:
            parts = [(w >> (3 * i)) & 7 for i in range(10)] + [w >> 30]
        else:
            parts = [(w >> (bits * i)) & (2 ** bits - 1) for i in range(f)]
        return np.stack(parts, -1).reshape(code.shape[:-1] + (-1,))
    kq = unpack(c.kcode, kb, fk).astype(np.float64)           # [B,H,D,Tkq]
    kd = kq * np.repeat(c.kscale.astype(np.float64), c.k_group, -1) + np.repeat(c.kmn.astype(np.float64), c.k_group, -1)
    K = np.concatenate([kd.transpose(0, 1, 3, 2), c.kfull.astype(np.float64)], 2)
    vq = unpack(c.vcode, vb, fv).astype(np.float64)           # [B,H,Tvq,D]
    vd = vq * np.repeat(c.vscale.astype(np.float64), c.v_group, -1) + np.repeat(c.vmn.astype(np.float64), c.v_group, -1)
    V = np.concatenate([vd, c.vfull.astype(np.float64)], 2)
    rep = nh // hkv
    K, V = np.repeat(K, rep, 1), np.repeat(V, rep, 1)
    s = np.einsum("bhd,bhtd->bht", q[:, :, 0].astype(np.float64), K) / np.sqrt(128.0)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bht,bhtd->bhd", p, V)[:, :, None]
    assert_attn_close(out_f32, want, 1e-3)
    assert_attn_close(out_ref, want, 2e-3)


def _left_pad_mask(B, T, starts, dtype=np.float32, neg=None):
    """Upstream's additive padding mask [B,1,1,T]: `neg` (default finfo(dtype).min) before each sequence's start."""
    neg = np.finfo(dtype).min if neg is None else neg
    m = np.zeros((B, 1, 1, T), dtype)
    for b, s in enumerate(starts):
        m[b, 0, 0, :s] = neg
    return m


@pytest.mark.parametrize("kb,vb,G,nh,hkv", [(4, 2, 32, 4, 4), (2, 2, 32, 4, 2), (3, 4, 32, 2, 2)])
def test_decode_attention_mask_equals_attention_over_the_unmasked_suffix(kb, vb, G, nh, hkv):
    """models/modeling_llama_KVmix.py:188-193: with a left-padding mask the result is attention over the
    unmasked positions only; the oracle's masked output must equal a float64 dense evaluation of that."""
    T, B = 352 + 128, 2
    k, v = make_kv(9, B, hkv, T)
    q = make_q(9, B, nh)
    c = RefLayerCache(kb, vb, G, residual_length=128)
    c.prefill(k, v)
    starts = [0, 133]
    mask = _left_pad_mask(B, T, starts)
    got = c.attend(q, ref_rounding=0, attention_mask=mask)
    assert np.array_equal(c.attend(q, ref_rounding=0, attention_mask=np.zeros_like(mask)), c.attend(q, ref_rounding=0))
    assert np.array_equal(got[0], c.attend(q, ref_rounding=0)[0])           # sequence 0 has no padding
    fk, fv = oracle.features_per_int(kb), oracle.features_per_int(vb)

    def unpack(code, bits, f):
        w = code.astype(np.int64) & 0xFFFFFFFF
        parts = ([(w >> (3 * i)) & 7 for i in range(10)] + [w >> 30]) if bits == 3 else \
            [(w >> (bits * i)) & (2 ** bits - 1) for i in range(f)]
        return np.stack(parts, -1).reshape(code.shape[:-1] + (-1,))
    kd = unpack(c.kcode, kb, fk) * np.repeat(c.kscale.astype(np.float64), c.k_group, -1) + np.repeat(c.kmn.astype(np.float64), c.k_group, -1)
    K = np.concatenate([kd.transpose(0, 1, 3, 2), c.kfull.astype(np.float64)], 2)
    vd = unpack(c.vcode, vb, fv) * np.repeat(c.vscale.astype(np.float64), c.v_group, -1) + np.repeat(c.vmn.astype(np.float64), c.v_group, -1)
    V = np.concatenate([vd, c.vfull.astype(np.float64)], 2)
    rep = nh // hkv
    K, V = np.repeat(K, rep, 1), np.repeat(V, rep, 1)
    s = np.einsum("bhd,bhtd->bht", q[:, :, 0].astype(np.float64), K) / np.sqrt(128.0)
    for b, st in enumerate(starts):
        s[b, :, :st] = -np.inf
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    want = np.einsum("bht,bhtd->bhd", p, V)[:, :, None]
    assert_attn_close(got, want, 1e-3)


def test_decode_attention_fully_masked_row_is_uniform():
    """weights + mask clamped at finfo.min makes every position equal: softmax is uniform (upstream :191-193)."""
    T = 160
    k, v = make_kv(10, 1, 2, T)
    q = make_q(10, 1, 2)
    c = RefLayerCache(4, 4, 32, residual_length=128)
    c.prefill(k, v)
    got = c.attend(q, ref_rounding=0, attention_mask=_left_pad_mask(1, T, [T]))
    zero_q = c.attend(np.zeros_like(q), ref_rounding=0)                      # all scores 0: uniform weights
    assert_attn_close(got, zero_q, 1e-3)
