"""Operators of the upstream ``KVmix`` extension module, served by the sm_100a C-ABI library.

The four upstream functions keep their names, positional arguments, shapes, dtypes and error
behaviour (quant_cuda/csrc/pybind.cpp:6-15):

    quantize_pack_last_dim_cuda(input, group_length, quant_bits) -> (code, scale, mn)
    quantized_gemm(group_size, fA, qB, scales, zeros, bits) -> Tensor
    process_key_quantization_cuda(input, prev_code, prev_scale, prev_min, group_length, quant_bits)
    process_value_quantization_cuda(...same...)

plus the fused call the cache uses (``decode_attention``) and the in-place quantizer
(``quantize_into``).  torch is used for device memory and the current stream only; all arithmetic
happens in the library.  Inputs are never mutated and outputs are fresh tensors, as upstream.
"""
import ctypes as C
import math

import torch

from . import _lib
from ._lib import AppendFormArgs, AttnArgs, GemvArgs, QuantArgs, check


LAUNCHES = [0]     # kernels of this library launched through this module (benchmark bookkeeping)


def features_per_int(bits):
    return 11 if bits == 3 else 32 // bits


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("kvmix_b200 operators need CUDA tensors (there is no CPU path)")


def _check_quant_rules(S, group_length, quant_bits):
    if quant_bits == 3:
        if group_length != 11:
            check(-2)
        if S % 11 != 0:
            check(-3)
    else:
        if quant_bits not in (1, 2, 4):
            check(-1)
        if group_length <= 0 or S % group_length != 0:
            check(-4)
        if S % (32 // quant_bits) != 0:
            check(-5)


def quantize_into(x, group_length, quant_bits, code, scale, mn, scale_by_division=False, ragged_tail=False):
    """Quantize 4-D ``x`` (any strides) along its last dim into preallocated views.

    ``code`` [B,H,A,S/fpi] int32, ``scale``/``mn`` [B,H,A,S/G] (dtype of x); their last dim must be
    contiguous, other strides are free, so they may be slices of a larger cache.
    ``scale_by_division`` selects how the stored scale is rounded (see include/kvmix_b200.h): False
    reproduces quantize_pack_last_dim_cuda, True the upstream append kernels.
    ``ragged_tail`` (an extension upstream does not have, 3 bits only): S need not be a multiple of 11; outputs
    hold ceil(S/11) words / groups per row, the last group being short.
    """
    _need_cuda(x, code, scale, mn)
    if x.dim() != 4:
        raise RuntimeError("input_tensor must be a 4D tensor")
    if x.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("input must be float16 or float32")
    B, H, A, S = x.shape
    ragged = bool(ragged_tail) and quant_bits == 3 and group_length == 11 and S % 11 != 0
    if not ragged:
        _check_quant_rules(S, group_length, quant_bits)
    fpi = features_per_int(quant_bits)
    nw, ng = (-(-S // 11), -(-S // 11)) if ragged else (S // fpi, S // group_length)
    assert code.dtype == torch.int32 and tuple(code.shape) == (B, H, A, nw)
    assert scale.dtype == x.dtype and mn.dtype == x.dtype
    assert tuple(scale.shape) == (B, H, A, ng) == tuple(mn.shape)
    assert scale.stride() == mn.stride()
    if x.numel() == 0:
        return
    assert code.stride(3) == 1 and scale.stride(3) == 1
    a = QuantArgs(x.data_ptr(), int(x.dtype == torch.float32), B, H, A, S, x.stride(0), x.stride(1), x.stride(2),
                  x.stride(3), group_length, quant_bits, int(bool(scale_by_division)), code.data_ptr(), code.stride(0), code.stride(1),
                  code.stride(2), scale.data_ptr(), mn.data_ptr(), scale.stride(0), scale.stride(1),
                  scale.stride(2), int(ragged))
    check(_lib.lib().kvq_quant_lastdim(C.byref(a), _stream()))
    LAUNCHES[0] += 1


def quantize_pack_last_dim_cuda(input_tensor, group_length, quant_bits):
    """Upstream quantize_pack_last_dim_cuda (quant_cuda/csrc/quantization_cuda.cu:631-721).

    Unlike upstream the input may be a strided view: ``k[:, :, :n].transpose(2, 3)`` is read in
    place, no ``.contiguous()`` copy is needed (one is still accepted).
    """
    if quant_bits == 3 and group_length != 11:
        check(-2)
    _need_cuda(input_tensor)
    if input_tensor.dim() != 4:
        raise RuntimeError("input_tensor must be a 4D tensor")
    B, H, A, S = input_tensor.shape
    _check_quant_rules(S, group_length, quant_bits)
    fpi = features_per_int(quant_bits)
    dev, dt = input_tensor.device, input_tensor.dtype
    code = torch.empty((B, H, A, S // fpi), dtype=torch.int32, device=dev)
    scale = torch.empty((B, H, A, S // group_length), dtype=dt, device=dev)
    mn = torch.empty_like(scale)
    quantize_into(input_tensor, group_length, quant_bits, code, scale, mn)
    return code, scale, mn


def quantized_gemm(group_size, fA, qB, scales, zeros, bits, out=None):
    """Upstream quantized_gemm (quant_cuda/csrc/dequantization_gemv_cuda.cu:127-248), M = 1.

    fA [B,nh,1,K] fp16, qB [B,nh_kv,K,N/fpi] int32, scales/zeros [B,nh_kv,K,N/G] fp16 ->
    [B,nh,1,N] fp16 with N = zeros.size(3) * group_size.  Operands are read where they are (no
    transposed copies); nh may exceed nh_kv (grouped-query attention without repeat copies).
    """
    _need_cuda(fA, qB, scales, zeros)
    if fA.dim() != 4 or qB.dim() != 4:
        raise RuntimeError("Input tensors must be 4-dimensional")
    if bits not in (1, 2, 3, 4):
        check(-1)
    B, nh, M, K = fA.shape
    nh_kv = qB.shape[1]
    if nh % nh_kv != 0:
        check(-6)
    if fA.dtype != torch.float16 or scales.dtype != torch.float16 or zeros.dtype != torch.float16:
        raise RuntimeError("quantized_gemm needs float16 inputs, scales and zeros")
    if qB.dtype != torch.int32:
        raise RuntimeError("quantized_gemm needs int32 packed weights")
    if M != 1:
        raise RuntimeError("quantized_gemm supports one query token (M == 1), as the upstream kernel does")
    if bits == 3 and group_size != 11:
        check(-2)
    if fA.stride(3) != 1:
        fA = fA.contiguous()
    if qB.stride(3) != 1:
        qB = qB.contiguous()
    if scales.stride(3) != 1:
        scales = scales.contiguous()
    if zeros.stride() != scales.stride() or zeros.stride(3) != 1:
        zeros = zeros.contiguous()
        scales = scales.contiguous()
    if qB.shape[0] != B or qB.shape[2] != K or tuple(scales.shape[:3]) != (B, nh_kv, K) or zeros.shape != scales.shape:
        check(-7)
    n_words, n_groups = qB.shape[3], zeros.shape[3]
    N = n_groups * group_size
    if out is None:
        out = torch.empty((B, nh, 1, N), dtype=torch.float16, device=fA.device)
    a = GemvArgs(fA.data_ptr(), fA.stride(0), fA.stride(1), qB.data_ptr(), qB.stride(0), qB.stride(1), qB.stride(2),
                 scales.data_ptr(), zeros.data_ptr(), scales.stride(0), scales.stride(1), scales.stride(2),
                 out.data_ptr(), out.stride(0), out.stride(1), B, nh, nh_kv, K, n_words, n_groups, group_size, bits)
    check(_lib.lib().kvq_gemv(C.byref(a), _stream()))
    LAUNCHES[0] += 1
    return out


def process_key_quantization_cuda(input_tensor, previous_code, previous_scale, previous_min, group_length,
                                  quant_bits):
    """Upstream process_key_quantization_cuda (quantization_cuda.cu:298-411).

    input [B,H,D,Tn]; returns fresh (code, scale, mn) = previous ++ quantize(input) along the last
    dim.  The previous 3-bit code words are copied too (upstream's fused 3-bit kernel leaves them
    uninitialised, quantization_cuda.cu:131-134).
    """
    _need_cuda(input_tensor, previous_code, previous_scale, previous_min)
    B, H, D, Tn = input_tensor.shape
    if quant_bits == 3:
        if group_length != 11:
            check(-2)
        if Tn % 11 != 0:
            raise RuntimeError("new_steps must be divisible by 11 for 3-bit quantization")
    elif Tn % group_length != 0:
        raise RuntimeError("new_steps must be divisible by group_length")
    fpi = features_per_int(quant_bits)
    previous_code, previous_scale, previous_min = (t.contiguous() for t in (previous_code, previous_scale, previous_min))
    old_w, old_g = previous_code.shape[3], previous_scale.shape[3]
    dev, dt = input_tensor.device, input_tensor.dtype
    code = torch.empty((B, H, D, old_w + Tn // fpi), dtype=torch.int32, device=dev)
    scale = torch.empty((B, H, D, old_g + Tn // group_length), dtype=dt, device=dev)
    mn = torch.empty_like(scale)
    a = AppendFormArgs(input_tensor.data_ptr(), int(dt == torch.float32), B, H, D, Tn, *input_tensor.stride(),
                       group_length, quant_bits, previous_code.data_ptr(), previous_scale.data_ptr(),
                       previous_min.data_ptr(), old_w, old_g, 0, code.data_ptr(), scale.data_ptr(), mn.data_ptr())
    check(_lib.lib().kvq_append_k(C.byref(a), _stream()))
    LAUNCHES[0] += 1
    return code, scale, mn


def process_value_quantization_cuda(input_tensor, previous_code, previous_scale, previous_min, group_length,
                                    quant_bits):
    """Upstream process_value_quantization_cuda (quantization_cuda.cu:413-537).

    input [B,H,Tn,D]; returns fresh (code, scale, mn) = previous ++ quantize(input) along dim 2.
    """
    _need_cuda(input_tensor, previous_code, previous_scale, previous_min)
    B, H, Tn, D = input_tensor.shape
    if quant_bits == 3:
        if group_length != 11:
            check(-2)
        if D % 11 != 0:
            raise RuntimeError("head_dim must be divisible by 11 for 3-bit quantization")
    elif D % group_length != 0:
        raise RuntimeError("head_dim must be divisible by group_length")
    fpi = features_per_int(quant_bits)
    previous_code, previous_scale, previous_min = (t.contiguous() for t in (previous_code, previous_scale, previous_min))
    Told = previous_code.shape[2]
    dev, dt = input_tensor.device, input_tensor.dtype
    code = torch.empty((B, H, Told + Tn, D // fpi), dtype=torch.int32, device=dev)
    scale = torch.empty((B, H, Told + Tn, D // group_length), dtype=dt, device=dev)
    mn = torch.empty_like(scale)
    a = AppendFormArgs(input_tensor.data_ptr(), int(dt == torch.float32), B, H, Tn, D, *input_tensor.stride(),
                       group_length, quant_bits, previous_code.data_ptr(), previous_scale.data_ptr(),
                       previous_min.data_ptr(), 0, 0, Told, code.data_ptr(), scale.data_ptr(), mn.data_ptr())
    check(_lib.lib().kvq_append_v(C.byref(a), _stream()))
    LAUNCHES[0] += 1
    return code, scale, mn


# ---------------------------------------------------------------------------------------------
_workspaces = {}


def attn_workspace(device, B, nh, T):
    """A per-(device, stream) scratch buffer for the split partials of decode_attention."""
    need = int(_lib.lib().kvq_decode_attn_workspace_bytes(B, nh, T))
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _s(t, i):
    return 0 if t is None else t.stride(i)


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def mask_fields(mask, B, nh, T):
    """(pointer, batch stride, head stride, is_f32) of an additive attention mask for kvq_attn_args; the caller
    keeps `mask` alive until the launch is enqueued.  Accepts [B,T], [B,1,1,T] or [B,nh,1,T]."""
    if mask is None:
        return 0, 0, 0, 0
    _need_cuda(mask)
    if mask.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("attention_mask must be float16 or float32")
    if mask.dim() == 4:
        if mask.shape[2] != 1:
            raise RuntimeError(f"Attention mask shape {tuple(mask.shape)} does not match weights shape {(B, nh, 1, T)}")
        mask = mask[:, :, 0, :]
    elif mask.dim() == 2:
        mask = mask[:, None, :]
    if mask.dim() != 3 or mask.shape[0] != B or mask.shape[1] not in (1, nh) or mask.shape[2] != T:
        raise RuntimeError(f"Attention mask shape {tuple(mask.shape)} does not match weights shape {(B, nh, 1, T)}")
    if mask.stride(2) != 1:
        raise RuntimeError("attention_mask must be contiguous along the key positions")
    return mask.data_ptr(), mask.stride(0), (0 if mask.shape[1] == 1 else mask.stride(1)), int(mask.dtype == torch.float32)


def decode_attention(q, kcode, kscale, kmn, kfull, vcode, vscale, vmn, vfull, k_bits, k_group, v_bits, v_group,
                     Tkq=None, Tvq=None, Rk=None, Rv=None, kf_start=0, vf_start=0, round_scores=True, out=None,
                     workspace=None, softmax_scale=None, attention_mask=None):
    """Fused decode attention (one launch) over [packed prefix | fp16 tail] keys and values.

    attention_mask: optional additive mask over the T key positions, [B,1,1,T] / [B,nh,1,T] / [B,T], fp16 or
    fp32 (upstream models/modeling_llama_KVmix.py:188-193: added to the scaled scores, clamped at the fp32 floor).

    q [B,nh,1,D] fp16.  kcode [B,Hkv,D,>=Tkq/fpi], kscale/kmn [B,Hkv,D,>=Tkq/Gk]; kfull
    [B,Hkv,cap,D] holding Rk tokens starting at row kf_start (ring).  vcode [B,Hkv,>=Tvq,D/fpi],
    vscale/vmn [B,Hkv,>=Tvq,D/Gv]; vfull [B,Hkv,cap,D] likewise.  Tkq/Tvq default to everything the
    packed tensors hold, Rk/Rv to all rows of the tails.  Returns [B,nh,1,D] fp16.
    """
    _need_cuda(q)
    B, nh, M, D = q.shape
    if M != 1:
        raise RuntimeError("decode_attention takes one query token per sequence")
    fk, fv = features_per_int(k_bits), features_per_int(v_bits)
    if Tkq is None:
        Tkq = 0 if kcode is None else kcode.shape[3] * fk
    if Tvq is None:
        Tvq = 0 if vcode is None else vcode.shape[2]
    if Rk is None:
        Rk = 0 if kfull is None else kfull.shape[2]
    if Rv is None:
        Rv = 0 if vfull is None else vfull.shape[2]
    if Tkq + Rk != Tvq + Rv:
        check(-9)
    T = Tkq + Rk
    Hkv = (kfull if kfull is not None else kcode).shape[1]
    if q.stride(3) != 1:
        q = q.contiguous()

    def _rows(t):                                # packed tensors are indexed with unit stride along their last dim
        return t if t is None or t.stride(3) == 1 else t.contiguous()

    kcode, vcode, kfull, vfull = _rows(kcode), _rows(vcode), _rows(kfull), _rows(vfull)
    if kscale is not None and (kscale.stride(3) != 1 or kmn.stride() != kscale.stride() or kmn.shape != kscale.shape):
        kscale, kmn = kscale.contiguous(), kmn.contiguous()      # one set of strides serves scale and minimum
    if vscale is not None and (vscale.stride(3) != 1 or vmn.stride() != vscale.stride() or vmn.shape != vscale.shape):
        vscale, vmn = vscale.contiguous(), vmn.contiguous()
    if kcode is not None and (kcode.shape[3] * fk < Tkq or kscale.shape[3] * k_group < Tkq):
        check(-7)
    if vcode is not None and (vcode.shape[2] < Tvq or vscale.shape[2] < Tvq):
        check(-7)
    if out is None:
        out = torch.empty((B, nh, 1, D), dtype=torch.float16, device=q.device)
    if workspace is None:
        workspace = attn_workspace(q.device, B, nh, T)
    a = AttnArgs(B, nh, Hkv, D, T, Tkq, Tvq, k_bits, k_group, v_bits, v_group, int(bool(round_scores)),
                 softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(D),
                 q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0), out.stride(1),
                 _ptr(kcode), _s(kcode, 0), _s(kcode, 1), _s(kcode, 2),
                 _ptr(kscale), _ptr(kmn), _s(kscale, 0), _s(kscale, 1), _s(kscale, 2),
                 _ptr(kfull), _s(kfull, 0), _s(kfull, 1), _s(kfull, 2),
                 0 if kfull is None else kfull.shape[2], kf_start,
                 _ptr(vcode), _s(vcode, 0), _s(vcode, 1), _s(vcode, 2),
                 _ptr(vscale), _ptr(vmn), _s(vscale, 0), _s(vscale, 1), _s(vscale, 2),
                 _ptr(vfull), _s(vfull, 0), _s(vfull, 1), _s(vfull, 2),
                 0 if vfull is None else vfull.shape[2], vf_start,
                 workspace.data_ptr(), workspace.numel(), *mask_fields(attention_mask, B, nh, T))
    check(_lib.lib().kvq_decode_attn(C.byref(a), _stream()))
    LAUNCHES[0] += 1
    return out
