"""GPU parity of the stand-alone dequant GEMV (upstream quantized_gemm contract) against the oracle."""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def _close(got, want):
    g = got.float().cpu().numpy().astype(np.float64)
    w = want.astype(np.float64)
    # both sides round an fp32 sum to fp16 once; summation order differs
    return (np.abs(g - w) <= 2e-3 * np.abs(w) + 2e-3 * np.abs(w).max()).all()


@pytest.mark.parametrize("bits,G", [(4, 32), (2, 32), (1, 32), (3, 11), (4, 64), (2, 128)])
@pytest.mark.parametrize("nh,hkv", [(4, 4), (8, 2)])
def test_q_times_packed_keys(cuda, bits, G, nh, hkv):
    import kvmix_b200 as kv
    rng = np.random.default_rng(bits + G + nh)
    T = 11 * 40 if bits == 3 else 3 * 128
    kt = rng.standard_normal((2, hkv, 128, T)).astype(np.float16)
    kt[:, :, 5] *= 8
    c, s, m = oracle.quantize_pack_last_dim(kt, G, bits)
    q = rng.standard_normal((2, nh, 1, 128)).astype(np.float16)
    want = oracle.quantized_gemm(G, q, c, s, m, bits)
    got = kv.quantized_gemm(G, _t(q, cuda), _t(c, cuda), _t(s, cuda), _t(m, cuda), bits)
    assert got.shape == (2, nh, 1, T) and got.dtype == torch.float16
    assert _close(got, want)


@pytest.mark.parametrize("bits,G,D", [(4, 32, 128), (2, 32, 128), (1, 32, 128), (3, 11, 132), (2, 64, 128), (1, 128, 128)])
def test_p_times_packed_values(cuda, bits, G, D):
    import kvmix_b200 as kv
    rng = np.random.default_rng(bits + G)
    Tv = 7 * 32 + 32
    v = rng.standard_normal((2, 2, Tv, D)).astype(np.float16)
    c, s, m = oracle.quantize_pack_last_dim(v, G, bits)
    p = np.abs(rng.standard_normal((2, 4, 1, Tv))).astype(np.float16)
    p = (p / p.sum(-1, keepdims=True)).astype(np.float16)
    want = oracle.quantized_gemm(G, p, c, s, m, bits)
    got = kv.quantized_gemm(G, _t(p, cuda), _t(c, cuda), _t(s, cuda), _t(m, cuda), bits)
    assert got.shape == (2, 4, 1, D)
    assert _close(got, want)


def test_gemv_errors(cuda):
    import kvmix_b200 as kv
    z = lambda *s, dt=torch.float16: torch.zeros(s, dtype=dt, device=cuda)
    with pytest.raises(RuntimeError, match="divisible by KV heads"):
        kv.quantized_gemm(32, z(1, 3, 1, 128), z(1, 2, 128, 4, dt=torch.int32), z(1, 2, 128, 1), z(1, 2, 128, 1), 4)
    with pytest.raises(RuntimeError, match="4-dimensional"):
        kv.quantized_gemm(32, z(3, 1, 128), z(1, 2, 128, 4, dt=torch.int32), z(1, 2, 128, 1), z(1, 2, 128, 1), 4)
    with pytest.raises(RuntimeError, match="bits"):
        kv.quantized_gemm(32, z(1, 2, 1, 128), z(1, 2, 128, 4, dt=torch.int32), z(1, 2, 128, 1), z(1, 2, 128, 1), 5)
    with pytest.raises(RuntimeError, match="group size must be 11|group_length must be 11"):
        kv.quantized_gemm(32, z(1, 2, 1, 128), z(1, 2, 128, 3, dt=torch.int32), z(1, 2, 128, 3), z(1, 2, 128, 3), 3)
