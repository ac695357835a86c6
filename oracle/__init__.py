"""TEST INFRASTRUCTURE: CPU oracle for the KVmix KV-cache hot path.

Only tests, the smoke check and the CPU-baseline legs of the benchmark may import this package;
the product (``kvmix_b200``) never does.  ``kvmix_oracle.c`` restates the upstream CUDA kernels
in plain C; this module compiles it with gcc and wraps it for numpy arrays, and ``glue.py``
restates the cache-update logic of the upstream attention forward.

fp16 arrays are ``numpy.float16``; packed codes are ``numpy.int32``.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "kvmix_oracle.c")
_OUT = os.path.join(_HERE, "_build", "libkvmix_oracle.so")
_lib = None

ERRORS = {
    -1: "Supported quantization bits: 1, 2, 3, 4",
    -2: "For 3-bit quantization, group_length must be 11",
    -3: "For 3-bit quantization, steps must be divisible by 11",
    -4: "steps must be divisible by group_length",
    -5: "steps must be divisible by (32 / quant_bits)",
    -6: "Total heads must be divisible by KV heads",
    -7: "packed width smaller than groups * group_size",
    -8: "group_length must be a multiple of (32 / quant_bits)",
    -9: "K and V token counts differ",
}


def build(force=False):
    """gcc -O2 -fopenmp -ffp-contract=off kvmix_oracle.c -> _build/libkvmix_oracle.so"""
    if not force and os.path.exists(_OUT) and os.path.getmtime(_OUT) >= os.path.getmtime(_SRC):
        return _OUT
    os.makedirs(os.path.dirname(_OUT), exist_ok=True)
    subprocess.check_call(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-mf16c", "-mfma",
                           "-shared", "-fPIC", "-o", _OUT, _SRC, "-lm"])
    return _OUT


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def set_threads(n):
    """Use n OpenMP threads in the C kernels from now on (overrides OMP_NUM_THREADS); returns the count in effect."""
    lib().orc_set_threads(int(n))
    return int(lib().orc_max_threads())


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _check(rc):
    if rc != 0:
        raise RuntimeError(ERRORS.get(rc, f"oracle error {rc}"))


def features_per_int(bits):
    return 11 if bits == 3 else 32 // bits


def quantize_pack_last_dim(x, group_length, quant_bits):
    """quantize_pack_last_dim_cuda (quant_cuda/csrc/quantization_cuda.cu:631-721) on a 4-D array."""
    if x.ndim != 4:
        raise RuntimeError("input_tensor must be a 4D tensor")
    if quant_bits not in (1, 2, 3, 4):
        _check(-1)
    B, H, A, S = x.shape
    G = group_length
    _check(int(lib().orc_quant_check(ctypes.c_int64(S), ctypes.c_int(G), ctypes.c_int(quant_bits))))
    fpi = features_per_int(quant_bits)
    rows = B * H * A
    code = np.empty((B, H, A, S // fpi), np.int32)
    x = np.ascontiguousarray(x)
    if x.dtype == np.float16:
        scale = np.empty((B, H, A, S // G), np.float16)
        mn = np.empty_like(scale)
        rc = lib().orc_quant_lastdim_f16(_p(x), ctypes.c_int64(rows), ctypes.c_int64(S), G, quant_bits,
                                         _p(code), _p(scale), _p(mn))
    elif x.dtype == np.float32:
        scale = np.empty((B, H, A, S // G), np.float32)
        mn = np.empty_like(scale)
        rc = lib().orc_quant_lastdim_f32(_p(x), ctypes.c_int64(rows), ctypes.c_int64(S), G, quant_bits,
                                         _p(code), _p(scale), _p(mn))
    else:
        raise RuntimeError("input must be float16 or float32")
    _check(rc)
    return code, scale, mn


def quantize_ragged3(x, scale_by_division=False):
    """EXTENSION (no upstream counterpart, parity unpinned): 3-bit groups of 11 along the last axis with a short last
    group, for rows whose length is not a multiple of 11 (3-bit values at head_dim 128: 12 words per token, the last
    one holding 7 codes).  x [B,H,A,S] fp16 -> code int32, scale, mn fp16, all [B,H,A,ceil(S/11)]."""
    if x.ndim != 4 or x.dtype != np.float16:
        raise RuntimeError("input must be a 4D float16 array")
    B, H, A, S = x.shape
    nw = (S + 10) // 11
    code = np.empty((B, H, A, nw), np.int32)
    scale = np.empty((B, H, A, nw), np.float16)
    mn = np.empty_like(scale)
    x = np.ascontiguousarray(x)
    _check(lib().orc_quant_ragged3_f16(_p(x), ctypes.c_int64(B * H * A), ctypes.c_int64(S), _p(code), _p(scale), _p(mn),
                                       int(bool(scale_by_division))))
    return code, scale, mn


def quantized_gemm(group_size, fA, qB, scales, zeros, bits):
    """quantized_gemm (quant_cuda/csrc/dequantization_gemv_cuda.cu:127-248), M = 1."""
    if fA.ndim != 4 or qB.ndim != 4:
        raise RuntimeError("Input tensors must be 4-dimensional")
    B, nh, M, K = fA.shape
    if M != 1:
        raise RuntimeError("only M = 1 is meaningful (upstream kernel ignores blockIdx.z)")
    nh_kv = qB.shape[1]
    n_words, n_groups = qB.shape[3], zeros.shape[3]
    N = n_groups * group_size
    out = np.empty((B, nh, 1, N), np.float16)
    fA, qB, scales, zeros = (np.ascontiguousarray(a) for a in (fA, qB, scales, zeros))
    rc = lib().orc_gemv(group_size, _p(fA), _p(qB), _p(scales), _p(zeros), bits, ctypes.c_int64(B),
                        ctypes.c_int64(nh), ctypes.c_int64(nh_kv), ctypes.c_int64(K),
                        ctypes.c_int64(n_words), ctypes.c_int64(n_groups), _p(out))
    _check(rc)
    return out


def process_key_quantization(x, prev_code, prev_scale, prev_mn, group_length, quant_bits):
    """process_key_quantization_cuda (quantization_cuda.cu:298-411): x [B,H,D,Tn] fp16."""
    B, H, D, Tn = x.shape
    fpi = features_per_int(quant_bits)
    old_w, old_g = prev_code.shape[3], prev_scale.shape[3]
    rows = B * H * D
    code = np.empty((B, H, D, old_w + Tn // fpi), np.int32)
    scale = np.empty((B, H, D, old_g + Tn // group_length), np.float16)
    mn = np.empty_like(scale)
    x, prev_code, prev_scale, prev_mn = (np.ascontiguousarray(a) for a in (x, prev_code, prev_scale, prev_mn))
    rc = lib().orc_append_k_f16(_p(x), ctypes.c_int64(rows), ctypes.c_int64(Tn), _p(prev_code),
                                ctypes.c_int64(old_w), _p(prev_scale), _p(prev_mn), ctypes.c_int64(old_g),
                                group_length, quant_bits, _p(code), _p(scale), _p(mn))
    _check(rc)
    return code, scale, mn


def process_value_quantization(x, prev_code, prev_scale, prev_mn, group_length, quant_bits):
    """process_value_quantization_cuda (quantization_cuda.cu:413-537): x [B,H,Tn,D] fp16."""
    B, H, Tn, D = x.shape
    _check(int(lib().orc_quant_check(ctypes.c_int64(D), group_length, quant_bits)))
    fpi = features_per_int(quant_bits)
    Told = prev_code.shape[2]
    code = np.empty((B, H, Told + Tn, D // fpi), np.int32)
    scale = np.empty((B, H, Told + Tn, D // group_length), np.float16)
    mn = np.empty_like(scale)
    x, prev_code, prev_scale, prev_mn = (np.ascontiguousarray(a) for a in (x, prev_code, prev_scale, prev_mn))
    rc = lib().orc_append_v_f16(_p(x), ctypes.c_int64(B * H), ctypes.c_int64(Tn), ctypes.c_int64(D),
                                _p(prev_code), _p(prev_scale), _p(prev_mn), ctypes.c_int64(Told),
                                group_length, quant_bits, _p(code), _p(scale), _p(mn))
    _check(rc)
    return code, scale, mn


def decode_attention(q, kcode, kscale, kmn, kfull, vcode, vscale, vmn, vfull, k_bits, k_group, v_bits,
                     v_group, ref_rounding=True, attention_mask=None):
    """Cached-branch attention of one query token (models/modeling_llama_KVmix.py:170-211).
    attention_mask: optional additive mask [B,1,1,T] or [B,nh,1,T] (upstream :188-193).

    q [B,nh,1,D]; kcode [B,Hkv,D,Tkq/fpi] (or None), kfull [B,Hkv,Rk,D]; vcode [B,Hkv,Tvq,D/fpi]
    (or None), vfull [B,Hkv,Rv,D].  Returns [B,nh,1,D] fp16.
    """
    B, nh, _, D = q.shape
    Hkv = kfull.shape[1]
    Rk, Rv = kfull.shape[2], vfull.shape[2]
    fk, fv = features_per_int(k_bits), features_per_int(v_bits)
    Tkq = 0 if kcode is None else kcode.shape[3] * fk
    Tvq = 0 if vcode is None else vcode.shape[2]
    z32 = np.zeros(1, np.int32)
    z16 = np.zeros(1, np.float16)
    arrs = [q, kcode if Tkq else z32, kscale if Tkq else z16, kmn if Tkq else z16, kfull,
            vcode if Tvq else z32, vscale if Tvq else z16, vmn if Tvq else z16, vfull]
    arrs = [np.ascontiguousarray(a) for a in arrs]
    out = np.empty((B, nh, 1, D), np.float16)
    i64 = ctypes.c_int64
    if attention_mask is not None:
        m = np.ascontiguousarray(np.asarray(attention_mask, np.float32).reshape(B, -1, Tkq + Rk))
        mp, mh = _p(m), m.shape[1]
    else:
        mp, mh = None, 1
    rc = lib().orc_decode_attn(*[_p(a) for a in arrs], i64(B), i64(nh), i64(Hkv), i64(D), i64(Tkq), i64(Rk),
                               i64(Tvq), i64(Rv), k_bits, k_group, v_bits, v_group, (7 if ref_rounding is True else int(ref_rounding)),
                               mp, i64(mh), _p(out))
    _check(rc)
    return out
