"""Seeded random configurations of the whole hot path against the oracle: prefill, a run of appends (with the group
quantizations they trigger), then one fused attention -- every bit width, group size, window, grouped-query ratio,
context length from one window to 12k tokens, with and without a left-padding mask.  Codes must stay bit-exact
through the appends; attention is held to 2e-3 per row twice: score narrowing off against the oracle without
narrowing, and the default mode (narrowing on) against the oracle with every one of upstream's narrowing points."""
import random

import numpy as np
import pytest
import torch

from oracle.glue import RefLayerCache
from util import REL_TOL, assert_close_to_upstream, make_kv, make_q, row_rel

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)


@pytest.mark.parametrize("case", range(32))
def test_random_case(cuda, case):
    import kvmix_b200 as kv
    rnd = random.Random(7000 + case)
    kb, vb, G = rnd.choice([1, 2, 3, 4]), rnd.choice([1, 2, 4]), rnd.choice([32, 64, 128])
    hkv = rnd.choice([1, 2, 4])
    nh = hkv * rnd.choice([1, 1, 2, 4])
    B, W = rnd.choice([1, 2, 3]), rnd.choice([128, 128, 256, 32])
    T = rnd.choice([rnd.randint(W + 1, 600), rnd.randint(600, 3000), rnd.randint(3000, 12000)])
    steps = rnd.randint(0, 40)
    k, v = make_kv(case, B, hkv, T + steps)
    q = make_q(case, B, nh)
    ref = RefLayerCache(kb, vb, G, residual_length=W)
    ref.prefill(k[:, :, :T], v[:, :, :T])
    dut = kv.KVmixLayerCache(B, hkv, 128, T + steps + 64, kb, vb, G, residual_length=W, device=cuda)
    dut.prefill(_t(k[:, :, :T], cuda), _t(v[:, :, :T], cuda))
    for s in range(steps):
        ref.append(k[:, :, T + s:T + s + 1], v[:, :, T + s:T + s + 1])
        dut.append(_t(k[:, :, T + s:T + s + 1], cuda), _t(v[:, :, T + s:T + s + 1], cuda))
    Tn = T + steps
    mask = None
    if rnd.random() < 0.5:
        mask = np.zeros((B, 1, 1, Tn), np.float32)
        for b in range(B):
            mask[b, 0, 0, :rnd.randint(0, Tn - 1)] = np.finfo(np.float32).min
    tup = dut.as_tuple()
    for got, want in [(tup[0], ref.kcode), (tup[4], ref.vcode)]:
        assert (got is None and want is None) or np.array_equal(got.cpu().numpy(), want)
    for got, want in [(tup[2], ref.kscale), (tup[3], ref.kmn), (tup[6], ref.vscale), (tup[7], ref.vmn)]:
        assert (got is None and want is None) or np.array_equal(got.cpu().numpy().view(np.uint16), want.view(np.uint16))
    want = ref.attend(q, ref_rounding=0, attention_mask=mask)
    got = dut.attend(_t(q, cuda), round_scores=False, attention_mask=_t(mask, cuda)).cpu().numpy()
    assert np.isfinite(got.astype(np.float32)).all()
    assert row_rel(got, want).max() <= REL_TOL
    want_up = ref.attend(q, ref_rounding=7, attention_mask=mask)
    got_up = dut.attend(_t(q, cuda), attention_mask=_t(mask, cuda)).cpu().numpy()
    assert_close_to_upstream(got_up, want_up, want)
