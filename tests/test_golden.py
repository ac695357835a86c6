"""Pins against vectors produced by the upstream CUDA extension itself (tests/golden/ref_vectors.npz,
made by tests/golden/make_golden.py on a B200 from the unmodified upstream sources, IEEE build).

CPU part: the oracle reproduces upstream's codes/scale/min bit for bit and its GEMV outputs.
GPU part: the sm_100a library reproduces the same vectors."""
import os

import numpy as np
import pytest

import oracle

PATH = os.path.join(os.path.dirname(__file__), "golden", "ref_vectors.npz")
needs_vectors = pytest.mark.skipif(not os.path.exists(PATH), reason="golden vectors not generated yet")


def _load():
    return np.load(PATH)


def _cases(prefix):
    if not os.path.exists(PATH):
        return []
    keys = sorted({k.rsplit("_", 1)[0] for k in _load().files if k.startswith(prefix)})
    return keys


def _parse(key):
    parts = key.split("_")
    bits = int([p for p in parts if p.startswith("b") and p[1:].isdigit()][0][1:])
    G = int([p for p in parts if p.startswith("g") and p[1:].isdigit()][0][1:])
    return bits, G


def _bits_equal(a, b):
    if a.dtype == np.float16:
        return (a.view(np.uint16) == b.view(np.uint16)).all()
    return (a == b).all()


@needs_vectors
@pytest.mark.parametrize("key", _cases("quant_"))
def test_oracle_quantizer_equals_upstream(key):
    z = _load()
    bits, G = _parse(key)
    c, s, m = oracle.quantize_pack_last_dim(z[key + "_x"], G, bits)
    assert _bits_equal(c, z[key + "_code"]) and _bits_equal(s, z[key + "_scale"]) and _bits_equal(m, z[key + "_mn"])


@needs_vectors
@pytest.mark.parametrize("key", _cases("gemv_qk_") + _cases("gemv_pv_"))
def test_oracle_gemv_equals_upstream(key):
    z = _load()
    bits, G = _parse(key)
    base = key.replace("_nh4", "_nh2")
    x = z[key + "_q"] if "_qk_" in key else z[key + "_p"]
    out = oracle.quantized_gemm(G, x, z[base + "_code"], z[base + "_scale"], z[base + "_mn"], bits)
    want = z[key + "_out"]
    assert out.shape == want.shape
    d = np.abs(out.astype(np.float32) - want.astype(np.float32))
    assert (d <= 2e-3 * np.abs(want.astype(np.float32)) + 1e-3 * np.abs(want.astype(np.float32)).max()).all()


@needs_vectors
@pytest.mark.parametrize("key", _cases("appendk_") + _cases("appendv_"))
def test_oracle_append_equals_upstream(key):
    z = _load()
    bits, G = _parse(key)
    p = oracle.quantize_pack_last_dim(z[key + "_x0"], G, bits)
    fn = oracle.process_key_quantization if key.startswith("appendk") else oracle.process_value_quantization
    c, s, m = fn(z[key + "_x1"], *p, G, bits)
    assert _bits_equal(c, z[key + "_code"]) and _bits_equal(s, z[key + "_scale"]) and _bits_equal(m, z[key + "_mn"])


@needs_vectors
@pytest.mark.gpu
def test_library_equals_upstream_vectors(cuda):
    import torch
    import kvmix_b200 as kv
    z = _load()
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    for key in _cases("quant_"):
        bits, G = _parse(key)
        c, s, m = kv.quantize_pack_last_dim_cuda(t(z[key + "_x"]), G, bits)
        assert _bits_equal(c.cpu().numpy(), z[key + "_code"]), key
        assert _bits_equal(s.cpu().numpy(), z[key + "_scale"]) and _bits_equal(m.cpu().numpy(), z[key + "_mn"]), key
    for key in _cases("gemv_qk_") + _cases("gemv_pv_"):
        bits, G = _parse(key)
        base = key.replace("_nh4", "_nh2")
        x = z[key + "_q"] if "_qk_" in key else z[key + "_p"]
        out = kv.quantized_gemm(G, t(x), t(z[base + "_code"]), t(z[base + "_scale"]), t(z[base + "_mn"]), bits)
        want = z[key + "_out"].astype(np.float32)
        d = np.abs(out.float().cpu().numpy() - want)
        assert (d <= 2e-3 * np.abs(want) + 2e-3 * np.abs(want).max()).all(), key
    for key in _cases("appendk_") + _cases("appendv_"):
        bits, G = _parse(key)
        p = kv.quantize_pack_last_dim_cuda(t(z[key + "_x0"]), G, bits)
        fn = kv.process_key_quantization_cuda if key.startswith("appendk") else kv.process_value_quantization_cuda
        c, s, m = fn(t(z[key + "_x1"]), *p, G, bits)
        assert _bits_equal(c.cpu().numpy(), z[key + "_code"]), key
        assert _bits_equal(s.cpu().numpy(), z[key + "_scale"]) and _bits_equal(m.cpu().numpy(), z[key + "_mn"]), key
