"""Preallocated mixed-precision KV cache for one attention layer, plus the upstream 9-tuple protocol.

``KVmixLayerCache`` holds what upstream threads through ``past_key_value`` as a 9-tuple
(models/modeling_llama_KVmix.py:269-273) in buffers allocated once:

    packed keys    kcode [B,Hkv,D,words]  kscale/kmn [B,Hkv,D,groups]     (upstream layout, with spare capacity)
    packed values  vcode [B,Hkv,T,D/fpi]  vscale/vmn [B,Hkv,T,D/G]
    fp16 tails     kfull/vfull [B,Hkv,cap,D] used as rings

so a decode step writes one row per tail and, when a group of the oldest tail tokens is due,
quantizes it in place behind the packed prefix -- no ``torch.cat``, no transposed or repeated
copies.  The policy deciding *when* tokens are due is upstream's (:115-129, :152-157): keep
``int(ratio * current_tail_len)`` newest tokens in fp16, or a fixed ``residual_length`` window.

``attention_step`` is the functional drop-in for the body of upstream's attention forward between
RoPE and ``o_proj``: it takes and returns the 9-tuple itself (contiguous tensors in upstream's
layout), calling the same kernels.
"""
import math

import torch

from . import ops
from .ops import features_per_int


def split_point(cur_len, group, ratio=None, residual_length=None):
    """How many of the oldest fp16 tokens to quantize now (modeling_llama_KVmix.py:118-126)."""
    keep = int(residual_length) if residual_length is not None else int(ratio * cur_len)
    if cur_len > keep and keep >= 0:
        return ((cur_len - keep) // group) * group
    return 0


def _round_up(x, m):
    return (x + m - 1) // m * m


class KVmixLayerCache:
    def __init__(self, batch, kv_heads, head_dim, max_tokens, k_bits, v_bits, group_size, k_residual_ratio=None,
                 v_residual_ratio=None, residual_length=None, device="cuda", max_tail=None):
        if residual_length is None and (k_residual_ratio is None or v_residual_ratio is None):
            raise ValueError("give residual ratios (upstream policy) or residual_length (fixed window)")
        self.B, self.Hkv, self.D = batch, kv_heads, head_dim
        self.k_bits, self.v_bits = k_bits, v_bits
        self.v_group = group_size
        self.k_group = 11 if k_bits == 3 else group_size       # modeling_llama_KVmix.py:49-52
        self.rk, self.rv, self.window = k_residual_ratio, v_residual_ratio, residual_length
        self.fk, self.fv = features_per_int(k_bits), features_per_int(v_bits)
        max_tokens = _round_up(max_tokens, 32)                  # keeps every per-head base 16-byte aligned
        self.max_tokens = max_tokens
        dev = torch.device(device)
        B, H, D = batch, kv_heads, head_dim
        kw = _round_up(max_tokens // self.fk + 1, 4)            # rows stay 16-byte aligned
        kg = _round_up(max_tokens // self.k_group + 1, 8)
        self.kcode = torch.empty((B, H, D, kw), dtype=torch.int32, device=dev)
        self.kscale = torch.empty((B, H, D, kg), dtype=torch.float16, device=dev)
        self.kmn = torch.empty_like(self.kscale)
        self.vcode = torch.empty((B, H, max_tokens, D // self.fv), dtype=torch.int32, device=dev)
        self.vscale = torch.empty((B, H, max_tokens, D // self.v_group), dtype=torch.float16, device=dev)
        self.vmn = torch.empty_like(self.vscale)
        if max_tail is None:
            if residual_length is not None:
                max_tail = residual_length + max(self.k_group, self.v_group)
            else:
                max_tail = int(max(k_residual_ratio, v_residual_ratio) * max_tokens) + \
                    2 * max(self.k_group, self.v_group)
        # ring capacities are multiples of the group so that a group never wraps around
        self.k_cap = _round_up(max_tail + 1, self.k_group)
        self.v_cap = _round_up(max_tail + 1, self.v_group)
        self.kfull = torch.empty((B, H, self.k_cap, D), dtype=torch.float16, device=dev)
        self.vfull = torch.empty((B, H, self.v_cap, D), dtype=torch.float16, device=dev)
        self.reset()

    def reset(self):
        self.tkq = self.tvq = 0          # tokens in the packed prefixes
        self.k_start = self.k_len = 0    # fp16 key ring
        self.v_start = self.v_len = 0    # fp16 value ring
        self.kv_seq_len = 0

    # -- cache update --------------------------------------------------------------------------------
    def _quant_k(self, src, n):
        """src: [B,Hkv,n,D] view of the n oldest fp16 keys; appended behind the packed prefix."""
        w0, g0 = self.tkq // self.fk, self.tkq // self.k_group
        ops.quantize_into(src.transpose(2, 3), self.k_group, self.k_bits,
                          self.kcode[..., w0:w0 + n // self.fk], self.kscale[..., g0:g0 + n // self.k_group],
                          self.kmn[..., g0:g0 + n // self.k_group])
        self.tkq += n

    def _quant_v(self, src, n):
        t0 = self.tvq
        ops.quantize_into(src, self.v_group, self.v_bits, self.vcode[:, :, t0:t0 + n], self.vscale[:, :, t0:t0 + n],
                          self.vmn[:, :, t0:t0 + n])
        self.tvq += n

    def _absorb_ring(self):
        nk = split_point(self.k_len, self.k_group, self.rk, self.window)
        while nk > 0:
            run = min(nk, self.k_cap - self.k_start)            # up to the wrap point (a group multiple)
            self._quant_k(self.kfull[:, :, self.k_start:self.k_start + run], run)
            self.k_start = (self.k_start + run) % self.k_cap
            self.k_len -= run
            nk -= run
        nv = split_point(self.v_len, self.v_group, self.rv, self.window)
        while nv > 0:
            run = min(nv, self.v_cap - self.v_start)
            self._quant_v(self.vfull[:, :, self.v_start:self.v_start + run], run)
            self.v_start = (self.v_start + run) % self.v_cap
            self.v_len -= run
            nv -= run

    def prefill(self, k, v):
        """k, v: [B,Hkv,L,D] fp16 (rotated keys).  Upstream prefill branch, :213-254."""
        assert self.kv_seq_len == 0, "prefill needs an empty cache"
        L = k.shape[2]
        if L > self.max_tokens:
            raise RuntimeError("prompt longer than the cache capacity")
        nk = split_point(L, self.k_group, self.rk, self.window)
        nv = split_point(L, self.v_group, self.rv, self.window)
        if L - nk > self.k_cap or L - nv > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        if nk > 0:
            self._quant_k(k[:, :, :nk], nk)
        if nv > 0:
            self._quant_v(v[:, :, :nv], nv)
        self.kfull[:, :, :L - nk].copy_(k[:, :, nk:])
        self.vfull[:, :, :L - nv].copy_(v[:, :, nv:])
        self.k_start = self.v_start = 0
        self.k_len, self.v_len = L - nk, L - nv
        self.kv_seq_len = L

    def append(self, k_new, v_new):
        """k_new, v_new: [B,Hkv,1,D] fp16.  Upstream decode branch, :111-167."""
        if self.kv_seq_len + 1 > self.max_tokens:
            raise RuntimeError("cache capacity exceeded")
        if self.k_len + 1 > self.k_cap or self.v_len + 1 > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        ks = (self.k_start + self.k_len) % self.k_cap
        vs = (self.v_start + self.v_len) % self.v_cap
        self.kfull[:, :, ks:ks + 1].copy_(k_new)
        self.vfull[:, :, vs:vs + 1].copy_(v_new)
        self.k_len += 1
        self.v_len += 1
        self.kv_seq_len += 1
        self._absorb_ring()

    # -- attention -----------------------------------------------------------------------------------
    def attend(self, q, out=None, round_scores=True):
        """q: [B,nh,1,D] fp16 -> [B,nh,1,D] fp16 over everything cached (upstream :170-211)."""
        return ops.decode_attention(q, self.kcode, self.kscale, self.kmn, self.kfull, self.vcode, self.vscale,
                                    self.vmn, self.vfull, self.k_bits, self.k_group, self.v_bits, self.v_group,
                                    Tkq=self.tkq, Tvq=self.tvq, Rk=self.k_len, Rv=self.v_len,
                                    kf_start=self.k_start, vf_start=self.v_start, round_scores=round_scores, out=out)

    def decode_step(self, q, k_new, v_new, out=None):
        self.append(k_new, v_new)
        return self.attend(q, out=out)

    # -- export in upstream's layout -----------------------------------------------------------------
    def _ring(self, buf, start, n, cap):
        idx = (torch.arange(n, device=buf.device) + start) % cap
        return buf.index_select(2, idx)

    def as_tuple(self):
        """The upstream 9-tuple (contiguous copies; None where upstream holds None)."""
        kq = self.tkq > 0
        vq = self.tvq > 0
        return (self.kcode[..., :self.tkq // self.fk].contiguous() if kq else None,
                self._ring(self.kfull, self.k_start, self.k_len, self.k_cap),
                self.kscale[..., :self.tkq // self.k_group].contiguous() if kq else None,
                self.kmn[..., :self.tkq // self.k_group].contiguous() if kq else None,
                self.vcode[:, :, :self.tvq].contiguous() if vq else None,
                self._ring(self.vfull, self.v_start, self.v_len, self.v_cap),
                self.vscale[:, :, :self.tvq].contiguous() if vq else None,
                self.vmn[:, :, :self.tvq].contiguous() if vq else None,
                self.kv_seq_len)

    def load_tuple(self, past_key_value):
        """Adopt an upstream 9-tuple (any of its tensors may be None): copies into the preallocated buffers."""
        kq, kfull, ksc, kmn, vq, vfull, vsc, vmn, seen = past_key_value
        self.reset()
        if kq is not None:
            self.tkq = kq.shape[3] * self.fk
            self.kcode[..., :kq.shape[3]].copy_(kq)
            self.kscale[..., :ksc.shape[3]].copy_(ksc)
            self.kmn[..., :kmn.shape[3]].copy_(kmn)
        if vq is not None:
            self.tvq = vq.shape[2]
            self.vcode[:, :, :self.tvq].copy_(vq)
            self.vscale[:, :, :self.tvq].copy_(vsc)
            self.vmn[:, :, :self.tvq].copy_(vmn)
        self.k_len = 0 if kfull is None else kfull.shape[2]
        self.v_len = 0 if vfull is None else vfull.shape[2]
        if self.k_len > self.k_cap or self.v_len > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        if self.k_len:
            self.kfull[:, :, :self.k_len].copy_(kfull)
        if self.v_len:
            self.vfull[:, :, :self.v_len].copy_(vfull)
        self.kv_seq_len = int(seen)

    def packed_bytes(self):
        """Bytes one attend() must read: codes + scale/zero + fp16 tails (the roofline numerator)."""
        per_head = kv_bytes_per_head(self.tkq, self.tvq, self.k_len, self.v_len, self.D, self.k_bits, self.k_group,
                                     self.v_bits, self.v_group)
        return per_head * self.B * self.Hkv


def kv_bytes_per_head(tkq, tvq, rk, rv, D, k_bits, k_group, v_bits, v_group):
    """Algorithmic cache bytes per (sequence, kv head) for one decode-attention pass."""
    fk, fv = features_per_int(k_bits), features_per_int(v_bits)
    kcodes = (tkq // fk) * 4 * D
    ksz = (tkq // k_group) * D * 4
    vcodes = tvq * (D // fv) * 4
    vsz = tvq * (D // v_group) * 4
    resid = (rk + rv) * D * 2
    return kcodes + ksz + vcodes + vsz + resid


def attention_step(query_states, key_states, value_states, past_key_value, k_bits, v_bits, group_size,
                   k_residual_ratio=None, v_residual_ratio=None, residual_length=None, use_cache=True):
    """Functional drop-in for upstream's attention body (modeling_llama_KVmix.py:105-273).

    query_states [B,nh,q_len,D], key_states/value_states [B,Hkv,q_len,D] (after RoPE);
    past_key_value is upstream's 9-tuple or None.  Returns (attn_output [B,nh,q_len,D], new 9-tuple).
    Decode (tuple given, q_len == 1) runs the fused kernel; prefill (None) quantizes the prompt
    prefix and computes exact fp16 attention over the prompt with torch's SDPA, which stands in
    for upstream's eager softmax(QK^T)V (:256-266) and is outside the accelerated path.
    """
    B, nh, q_len, D = query_states.shape
    Hkv = key_states.shape[1]
    k_group = 11 if k_bits == 3 else group_size
    v_group = group_size
    if past_key_value is not None:
        kq, kfull, ksc, kmn, vq, vfull, vsc, vmn, seen = past_key_value
        kv_seq_len = seen + q_len
        kfull = key_states if kfull is None else torch.cat([kfull, key_states], dim=2)
        vfull = value_states if vfull is None else torch.cat([vfull, value_states], dim=2)
    else:
        kq = ksc = kmn = vq = vsc = vmn = None
        kfull, vfull = key_states, value_states
        kv_seq_len = q_len
    nk = split_point(kfull.shape[2], k_group, k_residual_ratio, residual_length)
    if nk > 0:
        c, s, m = ops.quantize_pack_last_dim_cuda(kfull[:, :, :nk].transpose(2, 3), k_group, k_bits)
        kfull = kfull[:, :, nk:]
        kq = c if kq is None else torch.cat([kq, c], dim=3)
        ksc = s if ksc is None else torch.cat([ksc, s], dim=3)
        kmn = m if kmn is None else torch.cat([kmn, m], dim=3)
    nv = split_point(vfull.shape[2], v_group, v_residual_ratio, residual_length)
    if nv > 0:
        c, s, m = ops.quantize_pack_last_dim_cuda(vfull[:, :, :nv], v_group, v_bits)
        vfull = vfull[:, :, nv:]
        vq = c if vq is None else torch.cat([vq, c], dim=2)
        vsc = s if vsc is None else torch.cat([vsc, s], dim=2)
        vmn = m if vmn is None else torch.cat([vmn, m], dim=2)
    if past_key_value is not None:
        if q_len != 1:
            raise RuntimeError("cached attention takes one new token per step")
        kfull = kfull.contiguous()
        vfull = vfull.contiguous()
        attn = ops.decode_attention(query_states, kq, ksc, kmn, kfull, vq, vsc, vmn, vfull, k_bits, k_group,
                                    v_bits, v_group)
    else:
        attn = torch.nn.functional.scaled_dot_product_attention(
            query_states, key_states, value_states, is_causal=q_len > 1, enable_gqa=nh != Hkv,
            scale=1.0 / math.sqrt(D))
        kfull = kfull.contiguous()
        vfull = vfull.contiguous()
    new_past = (kq, kfull, ksc, kmn, vq, vfull, vsc, vmn, kv_seq_len) if use_cache else None
    return attn, new_past
