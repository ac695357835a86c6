"""TEST INFRASTRUCTURE: upstream's attention forward, cache update included, as plain torch around the *unmodified*
upstream extension built by ``oracle/build_ref.py`` (GPU only: the extension has no CPU path).

Upstream's decode-time attention (models/modeling_llama_KVmix.py:105-211; Mistral twin
models/modeling_mistral_KVmix.py:150-262) is torch glue around two calls into its extension, so it can be executed
without the HuggingFace model classes.  ``upstream_step`` performs the same tensor operations in the same order with
the same dtypes -- cat onto the fp16 tails (:111-112), the split decision (:115-126, :152-157), the extension's
quantizer on the transposed key copy (:131) and on the values (:159), cat of the packed tensors (:134-139, :162-167),
repeat copies for grouped queries (:19-28, :176-178), ``quantized_gemm`` for q.Kq (:180), fp16 matmul for the tail
(:185), fp32 concat and 1/sqrt(D) (:68-75), additive mask and clamp (:189-193), fp32 softmax narrowed to fp16 (:194),
``quantized_gemm`` for p.Vq (:205) plus fp16 matmul for the value tail and the fp16 sum (:209-211).
``upstream_prefill`` is the quantization half of the no-cache branch (:213-254).

Used by tests/golden/make_attn_golden.py (golden vectors) and by bench.py's ``upstream_gpu`` leg (the kernel to beat,
timed on the same GPU).  The fixed-window policy is this project's addition: upstream keeps
``int(ratio * current_fp16_len)`` tokens (:118-119); everything downstream of that decision is upstream's either way.
"""
import importlib
import math
import os
import sys

import torch

_REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def load_extension(variant="ieee"):
    """The upstream extension module: ``ieee`` (upstream sources without --use_fast_math) or ``fast`` (upstream's flags)."""
    if _REF_DIR not in sys.path:
        sys.path.insert(0, _REF_DIR)
    return importlib.import_module(f"KVmix_ref_{variant}")


def keep_of(policy, cur, which):
    if policy[0] == "window":
        return int(policy[1])
    return int(policy[1 + which] * cur)


def rep(t, n_rep):
    if t is None or n_rep == 1:
        return t
    B, H = t.shape[:2]
    return t[:, :, None].expand(B, H, n_rep, *t.shape[2:]).reshape(B, H * n_rep, *t.shape[2:])


def absorb(ext, st, kb, vb, Gk, Gv, policy):
    """The split decision and quantization shared by upstream's two branches."""
    cur = st["kfull"].shape[-2]
    keep = keep_of(policy, cur, 0)
    if cur > keep and keep >= 0:
        n = ((cur - keep) // Gk) * Gk
        if n > 0:
            to_q = st["kfull"][:, :, :n, :]
            st["kfull"] = st["kfull"][:, :, n:, :]
            c, s, m = ext.quantize_pack_last_dim_cuda(to_q.transpose(2, 3).contiguous(), Gk, kb)
            st["kq"] = c if st["kq"] is None else torch.cat([st["kq"], c], dim=3)
            st["ks"] = s if st["ks"] is None else torch.cat([st["ks"], s], dim=3)
            st["km"] = m if st["km"] is None else torch.cat([st["km"], m], dim=3)
    cur = st["vfull"].shape[-2]
    keep = keep_of(policy, cur, 1)
    if cur > keep and keep >= 0:
        n = ((cur - keep) // Gv) * Gv
        if n > 0:
            to_q = st["vfull"][:, :, :n, :]
            st["vfull"] = st["vfull"][:, :, n:, :]
            c, s, m = ext.quantize_pack_last_dim_cuda(to_q.contiguous(), Gv, vb)
            st["vq"] = c if st["vq"] is None else torch.cat([st["vq"], c], dim=2)
            st["vs"] = s if st["vs"] is None else torch.cat([st["vs"], s], dim=2)
            st["vm"] = m if st["vm"] is None else torch.cat([st["vm"], m], dim=2)


def upstream_prefill(ext, k, v, kb, vb, Gk, Gv, policy):
    st = dict(kq=None, ks=None, km=None, vq=None, vs=None, vm=None, kfull=k, vfull=v, seen=k.shape[-2])
    absorb(ext, st, kb, vb, Gk, Gv, policy)
    st["kfull"], st["vfull"] = st["kfull"].contiguous(), st["vfull"].contiguous()
    return st


def upstream_step(ext, st, q, k_new, v_new, kb, vb, Gk, Gv, policy, n_rep, mask):
    D = q.shape[-1]
    st["kfull"] = k_new if st["kfull"] is None else torch.cat([st["kfull"], k_new], dim=2)
    st["vfull"] = v_new if st["vfull"] is None else torch.cat([st["vfull"], v_new], dim=2)
    st["seen"] += 1
    absorb(ext, st, kb, vb, Gk, Gv, policy)
    att_q = ext.quantized_gemm(Gk, q, rep(st["kq"], n_rep), rep(st["ks"], n_rep), rep(st["km"], n_rep), kb) \
        if st["kq"] is not None else None
    att_full = torch.matmul(q, rep(st["kfull"], n_rep).transpose(2, 3))
    if att_q is not None:
        w = torch.cat([att_q.to(torch.float32), att_full.to(torch.float32)], dim=-1)
    else:
        w = att_full.to(torch.float32)
    w = w / math.sqrt(D)
    if mask is not None:
        w = w + mask
        w = torch.clamp(w, min=torch.finfo(w.dtype).min)
    w = torch.nn.functional.softmax(w, dim=-1, dtype=torch.float32).to(q.dtype)
    if st["vq"] is None:
        out = torch.matmul(w, rep(st["vfull"], n_rep))
    else:
        r = st["vfull"].shape[-2]
        out_q = ext.quantized_gemm(Gv, w[:, :, :, :-r], rep(st["vq"], n_rep), rep(st["vs"], n_rep),
                                   rep(st["vm"], n_rep), vb)
        out_f = torch.matmul(w[:, :, :, -r:], rep(st["vfull"], n_rep))
        out = out_q + out_f
    return out                    # (the extension's GEMV runs on the legacy default stream: callers synchronise)
