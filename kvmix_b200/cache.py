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
import ctypes as C
import math

import torch

from . import _lib, ops
from ._lib import AppendArgs, AttnArgs
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
                 v_residual_ratio=None, residual_length=None, device="cuda", max_tail=None, device_state=False):
        if residual_length is None and (k_residual_ratio is None or v_residual_ratio is None):
            raise ValueError("give residual ratios (upstream policy) or residual_length (fixed window)")
        self.B, self.Hkv, self.D = batch, kv_heads, head_dim
        self.k_bits, self.v_bits = k_bits, v_bits
        self.v_group = group_size                               # values are quantized group_size tokens at a time
        self.k_group = 11 if k_bits == 3 else group_size       # modeling_llama_KVmix.py:49-52
        # channel groups of the values.  3-bit values are an extension upstream does not have (its 3-bit rule needs
        # head_dim % 11 == 0, quantization_cuda.cu:433-434): groups of 11 channels, one word each, the last one short
        self.v_cgroup = 11 if v_bits == 3 else group_size
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
        self.vcode = torch.empty((B, H, max_tokens, -(-D // self.fv)), dtype=torch.int32, device=dev)
        self.vscale = torch.empty((B, H, max_tokens, -(-D // self.v_cgroup)), dtype=torch.float16, device=dev)
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
        # argument blocks of the two per-step launches, filled once; a step only patches what changes
        kf, vf = self.kfull, self.vfull
        self._app = AppendArgs(B, H, D, 0, 0, 0, 0, 0, 0, kf.data_ptr(), kf.stride(0), kf.stride(1), kf.stride(2), 0,
                               vf.data_ptr(), vf.stride(0), vf.stride(1), vf.stride(2), 0)
        kc, ks, vc, vs = self.kcode, self.kscale, self.vcode, self.vscale
        self._att = AttnArgs(B, 0, H, D, 0, 0, 0, k_bits, self.k_group, v_bits, self.v_cgroup, 1, 1.0 / math.sqrt(D),
                             0, 0, 0, 0, 0, 0,
                             kc.data_ptr(), kc.stride(0), kc.stride(1), kc.stride(2),
                             ks.data_ptr(), self.kmn.data_ptr(), ks.stride(0), ks.stride(1), ks.stride(2),
                             kf.data_ptr(), kf.stride(0), kf.stride(1), kf.stride(2), self.k_cap, 0,
                             vc.data_ptr(), vc.stride(0), vc.stride(1), vc.stride(2),
                             vs.data_ptr(), self.vmn.data_ptr(), vs.stride(0), vs.stride(1), vs.stride(2),
                             vf.data_ptr(), vf.stride(0), vf.stride(1), vf.stride(2), self.v_cap, 0, 0, 0)
        self._ws = {}
        self._fused = None               # None: not tried yet; False: the library does not fuse this geometry
        # device_state=True: lengths and ring starts also live in device memory ({T, Tkq, Tvq, k_start, v_start}, then the
        # grid-completion counter) and fused decode steps read and advance them there; the attributes of this object are
        # then a host mirror of that state (advance_mirror() moves it along after graph replays)
        self.state = torch.zeros(8, dtype=torch.int32, device=dev) if device_state else None
        self._lib = _lib.lib()
        self.reset()

    def reset(self):
        self.tkq = self.tvq = 0          # tokens in the packed prefixes
        self.k_start = self.k_len = 0    # fp16 key ring
        self.v_start = self.v_len = 0    # fp16 value ring
        self.kv_seq_len = 0
        self._push_state()

    def _push_state(self):
        """Host mirror -> device state (after prefill / load / a step made of separate launches)."""
        if getattr(self, "state", None) is not None:
            self.state.copy_(torch.tensor([self.kv_seq_len, self.tkq, self.tvq, self.k_start, self.v_start, 0, 0, 0],
                                          dtype=torch.int32), non_blocking=False)

    def steady(self):
        """True when the next step quantizes at most one group of keys and of values (what a device-driven step does)."""
        nk = split_point(self.k_len + 1, self.k_group, self.rk, self.window)
        nv = split_point(self.v_len + 1, self.v_group, self.rv, self.window)
        return nk in (0, self.k_group) and nv in (0, self.v_group) and nk <= self.k_len and nv <= self.v_len

    def advance_mirror(self, steps=1):
        """Move the host mirror along by `steps` device-driven decode steps (e.g. replays of a captured graph)."""
        for _ in range(steps):
            nk = split_point(self.k_len + 1, self.k_group, self.rk, self.window)
            nv = split_point(self.v_len + 1, self.v_group, self.rv, self.window)
            nk, nv = min(nk, self.k_group), min(nv, self.v_group)
            self.tkq, self.tvq = self.tkq + nk, self.tvq + nv
            self.k_start, self.v_start = (self.k_start + nk) % self.k_cap, (self.v_start + nv) % self.v_cap
            self.k_len, self.v_len = self.k_len + 1 - nk, self.v_len + 1 - nv
            self.kv_seq_len += 1

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
        ops.quantize_into(src, self.v_cgroup, self.v_bits, self.vcode[:, :, t0:t0 + n], self.vscale[:, :, t0:t0 + n],
                          self.vmn[:, :, t0:t0 + n], ragged_tail=self.v_bits == 3)
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
        self._push_state()

    def prefill_projected(self, k_proj, v_proj, cos=None, sin=None):
        """Prefill straight from the projections (upstream :213-254 plus the rotary embedding before it).
        k_proj, v_proj: the k_proj / v_proj outputs of the prompt, [B, L, Hkv*D] (or [B, L, Hkv, D]) fp16, keys NOT yet
        rotated; cos, sin: the rotary tables [L, D] or [B, L, D] fp16 as HF's rotary embedding returns them (None: the
        keys arrive rotated).  Rotation, the split into packed prefix and fp16 tail, both quantizers and the tail
        copies run in three launches of the library; no rotated, transposed or sliced temporary is made."""
        assert self.kv_seq_len == 0, "prefill needs an empty cache"
        B, L = k_proj.shape[0], k_proj.shape[1]
        k4, v4 = k_proj.reshape(B, L, self.Hkv, self.D), v_proj.reshape(B, L, self.Hkv, self.D)
        if B != self.B or k4.dtype != torch.float16 or v4.dtype != torch.float16 or k4.stride(3) != 1 or v4.stride(3) != 1:
            raise RuntimeError("prefill_projected takes fp16 projections [B, L, Hkv*D] of the cache's batch")
        if L > self.max_tokens:
            raise RuntimeError("prompt longer than the cache capacity")
        nk = split_point(L, self.k_group, self.rk, self.window)
        nv = split_point(L, self.v_group, self.rv, self.window)
        if L - nk > self.k_cap or L - nv > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        a = _lib.PrefillArgs()
        a.k, a.k_sB, a.k_sT, a.k_sH = k4.data_ptr(), k4.stride(0), k4.stride(1), k4.stride(2)
        a.v, a.v_sB, a.v_sT, a.v_sH = v4.data_ptr(), v4.stride(0), v4.stride(1), v4.stride(2)
        if cos is not None:
            if cos.dtype != torch.float16 or sin.dtype != torch.float16 or cos.stride(-1) != 1 or sin.stride() != cos.stride():
                raise RuntimeError("rotary tables must be fp16 with the same layout, contiguous along head_dim")
            c3 = cos if cos.dim() == 3 else cos[None]
            if c3.shape[-2] < L or c3.shape[-1] != self.D or c3.shape[0] not in (1, B):
                raise RuntimeError("rotary tables must cover [L, head_dim]")
            a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
            a.r_sB, a.r_sT = (c3.stride(0) if c3.shape[0] == B and B > 1 else 0), c3.stride(1)
        a.B, a.Hkv, a.L, a.D, a.nk, a.nv = B, self.Hkv, L, self.D, nk, nv
        a.k_bits, a.k_group, a.v_bits, a.v_group = self.k_bits, self.k_group, self.v_bits, self.v_cgroup
        kc, ks, vc, vs, kf, vf = self.kcode, self.kscale, self.vcode, self.vscale, self.kfull, self.vfull
        a.kcode, a.kc_sB, a.kc_sH, a.kc_sD = kc.data_ptr(), kc.stride(0), kc.stride(1), kc.stride(2)
        a.kscale, a.kmn, a.ks_sB, a.ks_sH, a.ks_sD = ks.data_ptr(), self.kmn.data_ptr(), ks.stride(0), ks.stride(1), ks.stride(2)
        a.vcode, a.vc_sB, a.vc_sH, a.vc_sT = vc.data_ptr(), vc.stride(0), vc.stride(1), vc.stride(2)
        a.vscale, a.vmn, a.vs_sB, a.vs_sH, a.vs_sT = vs.data_ptr(), self.vmn.data_ptr(), vs.stride(0), vs.stride(1), vs.stride(2)
        a.kfull, a.kf_sB, a.kf_sH, a.kf_sT = kf.data_ptr(), kf.stride(0), kf.stride(1), kf.stride(2)
        a.vfull, a.vf_sB, a.vf_sH, a.vf_sT = vf.data_ptr(), vf.stride(0), vf.stride(1), vf.stride(2)
        _lib.check(self._lib.kvq_prefill(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        ops.LAUNCHES[0] += (nk > 0) + (nv > 0) + (nk < L or nv < L)
        self.tkq, self.tvq = nk, nv
        self.k_start = self.v_start = 0
        self.k_len, self.v_len = L - nk, L - nv
        self.kv_seq_len = L
        self._push_state()

    def append(self, k_new, v_new):
        """k_new, v_new: [B,Hkv,1,D] fp16.  Upstream decode branch, :111-167."""
        if self.kv_seq_len + 1 > self.max_tokens:
            raise RuntimeError("cache capacity exceeded")
        if self.k_len + 1 > self.k_cap or self.v_len + 1 > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        a = self._app
        if k_new.stride(3) != 1 or v_new.stride(3) != 1 or k_new.dtype != torch.float16 or v_new.dtype != torch.float16:
            k_new, v_new = k_new.to(torch.float16).contiguous(), v_new.to(torch.float16).contiguous()
        a.k_new, a.kn_sB, a.kn_sH = k_new.data_ptr(), k_new.stride(0), k_new.stride(1)
        a.v_new, a.vn_sB, a.vn_sH = v_new.data_ptr(), v_new.stride(0), v_new.stride(1)
        a.k_slot = (self.k_start + self.k_len) % self.k_cap
        a.v_slot = (self.v_start + self.v_len) % self.v_cap
        _lib.check(self._lib.kvq_append_kv(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        ops.LAUNCHES[0] += 1
        self.k_len += 1
        self.v_len += 1
        self.kv_seq_len += 1
        self._absorb_ring()
        self._push_state()

    # -- attention -----------------------------------------------------------------------------------
    def _workspace(self, nh, stream, device):
        ws = self._ws.get((nh, stream))
        if ws is None:
            need = int(self._lib.kvq_decode_attn_workspace_bytes(self.B, nh, self.max_tokens))
            # zeroed once: the kernels leave the per-head counters at zero, so a step needs no clearing launch
            # (the layout is fixed for this cache: same B and nh on every call)
            ws = self._ws[(nh, stream)] = torch.zeros(need, dtype=torch.uint8, device=device)
        return ws

    def attend(self, q, out=None, round_scores=True, attention_mask=None, peers=None):
        """q: [B,nh,1,D] fp16 -> [B,nh,1,D] fp16 over everything cached (upstream :170-211).  attention_mask:
        optional additive mask over the kv_seq_len cached positions ([B,1,1,T], [B,nh,1,T] or [B,T]; upstream
        :188-193), e.g. the left-padding mask of a ragged batch."""
        B, nh, M, D = q.shape
        if M != 1 or B != self.B or D != self.D or not q.is_cuda:
            raise RuntimeError("attend takes q [B, nh, 1, D] on the cache's device")
        if self.tkq + self.k_len != self.tvq + self.v_len:
            _lib.check(-9)
        if q.stride(3) != 1 or q.dtype != torch.float16:
            q = q.to(torch.float16).contiguous()
        if out is None:
            out = torch.empty((B, nh, 1, D), dtype=torch.float16, device=q.device)
        stream = torch.cuda.current_stream().cuda_stream
        ws = self._workspace(nh, stream, q.device)
        a = self._att
        a.nh, a.T, a.Tkq, a.Tvq = nh, self.tkq + self.k_len, self.tkq, self.tvq
        a.round_scores = int(bool(round_scores))
        a.q, a.q_sB, a.q_sH = q.data_ptr(), q.stride(0), q.stride(1)
        a.out, a.o_sB, a.o_sH = out.data_ptr(), out.stride(0), out.stride(1)
        a.kf_start, a.vf_start = self.k_start, self.v_start
        a.workspace, a.workspace_bytes, a.flags = ws.data_ptr(), ws.numel(), _lib.ATTN_WORKSPACE_READY
        a.mask, a.mask_sB, a.mask_sH, a.mask_is_f32 = ops.mask_fields(attention_mask, B, nh, a.T)
        if peers is not None:
            peers.fill(a)
        rc = self._lib.kvq_decode_attn(C.byref(a), C.c_void_p(stream))
        a.n_peers = 0
        _lib.check(rc)
        ops.LAUNCHES[0] += 1
        return out

    def decode_step(self, q, k_new, v_new, out=None, attention_mask=None, round_scores=True, peers=None, plan_tokens=None):
        """Upstream's decode branch for one new token (:105-211): cache update, then attention over everything cached.
        One launch when the library can fuse the update into the attention kernel (one CTA per kv head and segment:
        MHA, or grouped queries with 2 or 4 query heads per kv head, on the tensor-core kernels); otherwise the ring
        append, the group quantizers and the attention are launched one after the other (``append`` + ``attend``)."""
        if self._fused is not False:
            res = self._decode_step_fused(q, k_new, v_new, out, attention_mask, round_scores, peers, plan_tokens)
            if res is not None:
                return res
        if plan_tokens is not None:
            raise RuntimeError("plan_tokens needs a device-driven fused step (device_state=True, steady state, fused geometry)")
        self.append(k_new, v_new)
        return self.attend(q, out=out, attention_mask=attention_mask, round_scores=round_scores, peers=peers)

    def _decode_step_fused(self, q, k_new, v_new, out, attention_mask, round_scores, peers=None, plan_tokens=None):
        B, nh, M, D = q.shape
        if M != 1 or B != self.B or D != self.D or not q.is_cuda:
            raise RuntimeError("decode_step takes q [B, nh, 1, D] on the cache's device")
        if self.kv_seq_len + 1 > self.max_tokens:
            raise RuntimeError("cache capacity exceeded")
        if self.k_len + 1 > self.k_cap or self.v_len + 1 > self.v_cap:
            raise RuntimeError("fp16 tail larger than the ring capacity (raise max_tail)")
        if self.tkq + self.k_len != self.tvq + self.v_len:
            _lib.check(-9)
        # the state after the update, by upstream's policy (the host mirrors what the kernel is told to do)
        nk = split_point(self.k_len + 1, self.k_group, self.rk, self.window)
        nv = split_point(self.v_len + 1, self.v_group, self.rv, self.window)
        if nk not in (0, self.k_group) or nv not in (0, self.v_group) or nk > self.k_len or nv > self.v_len:
            return None                                         # more than one group due (a freshly adopted cache): unfused
        fix = lambda t: t if (t.stride(3) == 1 and t.dtype == torch.float16) else t.to(torch.float16).contiguous()
        q, k_new, v_new = fix(q), fix(k_new), fix(v_new)
        if out is None:
            out = torch.empty((B, nh, 1, D), dtype=torch.float16, device=q.device)
        stream = torch.cuda.current_stream().cuda_stream
        ws = self._workspace(nh, stream, q.device)
        a = self._att
        a.nh, a.T, a.Tkq, a.Tvq = nh, self.kv_seq_len + 1, self.tkq + nk, self.tvq + nv
        if self.state is not None:
            # device-driven: the kernel takes the lengths from self.state and advances them; T only lays out the grid
            # (plan_tokens: an upper bound valid for every replay of a captured step)
            if plan_tokens is not None:
                if plan_tokens < a.T or plan_tokens > self.max_tokens:
                    raise RuntimeError("plan_tokens must cover the step and fit the cache")
                if attention_mask is not None:
                    raise RuntimeError("a step planned for later lengths cannot carry a mask of a fixed length")
                a.T = int(plan_tokens)
            a.state = self.state.data_ptr()
            a.window = -1 if self.window is None else int(self.window)
            a.k_ratio, a.v_ratio = float(self.rk or 0.0), float(self.rv or 0.0)
        a.round_scores = int(bool(round_scores))
        a.q, a.q_sB, a.q_sH = q.data_ptr(), q.stride(0), q.stride(1)
        a.out, a.o_sB, a.o_sH = out.data_ptr(), out.stride(0), out.stride(1)
        a.kf_start, a.vf_start = (self.k_start + nk) % self.k_cap, (self.v_start + nv) % self.v_cap
        a.workspace, a.workspace_bytes, a.flags = ws.data_ptr(), ws.numel(), _lib.ATTN_WORKSPACE_READY
        a.mask, a.mask_sB, a.mask_sH, a.mask_is_f32 = ops.mask_fields(attention_mask, B, nh, self.kv_seq_len + 1)
        a.k_new, a.kn_sB, a.kn_sH = k_new.data_ptr(), k_new.stride(0), k_new.stride(1)
        a.v_new, a.vn_sB, a.vn_sH = v_new.data_ptr(), v_new.stride(0), v_new.stride(1)
        a.k_quant, a.v_quant, a.k_quant_slot, a.v_quant_slot = nk, nv, self.k_start, self.v_start
        if peers is not None:
            peers.fill(a)
        rc = self._lib.kvq_decode_attn(C.byref(a), C.c_void_p(stream))
        a.k_new = a.v_new = a.state = None
        a.k_quant = a.v_quant = a.n_peers = 0
        if rc == -11:                                           # this geometry is not served fused: remember and fall back
            self._fused = False
            return None
        _lib.check(rc)
        ops.LAUNCHES[0] += 1
        self._fused = True
        self.tkq, self.tvq = self.tkq + nk, self.tvq + nv
        self.k_start, self.v_start = a.kf_start, a.vf_start
        self.k_len, self.v_len = self.k_len + 1 - nk, self.v_len + 1 - nv
        self.kv_seq_len += 1
        return out

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

    def view_tuple(self):
        """The upstream 9-tuple as views into the preallocated buffers (no copies of the packed tensors; the small
        fp16 tails are gathered out of their rings).  The views are overwritten by later appends."""
        kq = self.tkq > 0
        vq = self.tvq > 0
        return (self.kcode[..., :self.tkq // self.fk] if kq else None,
                self._ring(self.kfull, self.k_start, self.k_len, self.k_cap),
                self.kscale[..., :self.tkq // self.k_group] if kq else None,
                self.kmn[..., :self.tkq // self.k_group] if kq else None,
                self.vcode[:, :, :self.tvq] if vq else None,
                self._ring(self.vfull, self.v_start, self.v_len, self.v_cap),
                self.vscale[:, :, :self.tvq] if vq else None,
                self.vmn[:, :, :self.tvq] if vq else None,
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
        if self.tkq + self.k_len != self.kv_seq_len or self.tvq + self.v_len != self.kv_seq_len:
            self.reset()
            raise RuntimeError("inconsistent token counts")
        self._push_state()

    def packed_bytes(self):
        """Bytes one attend() must read: codes + scale/zero + fp16 tails (the roofline numerator)."""
        per_head = kv_bytes_per_head(self.tkq, self.tvq, self.k_len, self.v_len, self.D, self.k_bits, self.k_group,
                                     self.v_bits, self.v_cgroup)
        return per_head * self.B * self.Hkv


def kv_bytes_per_head(tkq, tvq, rk, rv, D, k_bits, k_group, v_bits, v_group):
    """Algorithmic cache bytes per (sequence, kv head) for one decode-attention pass."""
    fk, fv = features_per_int(k_bits), features_per_int(v_bits)
    kcodes = (tkq // fk) * 4 * D
    ksz = (tkq // k_group) * D * 4
    vcodes = tvq * -(-D // fv) * 4                             # ceil: 3-bit values hold 12 words / groups per token
    vsz = tvq * -(-D // v_group) * 4
    resid = (rk + rv) * D * 2
    return kcodes + ksz + vcodes + vsz + resid


class CapturedDecodeStep:
    """One decode step of a stack of layer caches -- every layer's fused launch and, for head-sharded caches, its
    exchange wait -- captured once in a CUDA graph and replayed for the following tokens with no host work per layer.

    The caches must hold their state on the device (``device_state=True``), be in steady state (``steady()``) and have
    a geometry the library fuses.  ``q``, ``k_new``, ``v_new``, ``out`` are per-layer lists of static tensors: write
    the next token's inputs into them, call ``replay()``, read ``out`` (or, head-sharded, ``gathered``).  The grids are
    laid out for ``max_replays`` further tokens; replaying more often than that raises.  Upstream has no counterpart
    (its forward decides on the host, per layer and step, how many tokens to quantize: modeling_llama_KVmix.py:115-126).
    """

    def __init__(self, caches, q, k_new, v_new, out, max_replays, peers=None):
        if not caches or any(c.state is None for c in caches):
            raise RuntimeError("a captured decode step needs caches made with device_state=True")
        if any(not c.steady() for c in caches):
            raise RuntimeError("a captured decode step needs caches in steady state (at most one group due per step)")
        if peers is not None and len(caches) % peers.depth:
            raise RuntimeError("the layers of a step must use the exchange buffers a whole number of rounds")
        self.caches, self.left, self.peers = list(caches), int(max_replays), peers
        self.gathered = [None] * len(caches)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        for c, ql in zip(caches, q):                            # nothing may be allocated while capturing
            c._workspace(ql.shape[1], side.cuda_stream, ql.device)
        torch.cuda.synchronize()
        mirrors = [(c.kv_seq_len, c.tkq, c.tvq, c.k_start, c.v_start, c.k_len, c.v_len) for c in caches]
        layer0 = peers.layer if peers is not None else 0
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(self.graph, stream=side):
                for l, c in enumerate(caches):
                    r = c.decode_step(q[l], k_new[l], v_new[l], out=out[l], peers=peers,
                                      plan_tokens=c.kv_seq_len + self.left)
                    if r is None or c._fused is not True:
                        raise RuntimeError(f"layer {l}: the library does not fuse this geometry")
                    if peers is not None:
                        self.gathered[l] = peers.wait()
        torch.cuda.current_stream().wait_stream(side)
        # capturing launched nothing: put the host mirrors (and the exchange's layer counter) back
        for c, m in zip(caches, mirrors):
            c.kv_seq_len, c.tkq, c.tvq, c.k_start, c.v_start, c.k_len, c.v_len = m
        if peers is not None:
            peers.layer = layer0

    def replay(self, steps=1):
        if steps > self.left:
            raise RuntimeError("captured decode step replayed beyond the context it was laid out for")
        for _ in range(steps):
            self.graph.replay()
        self.left -= steps
        for c in self.caches:
            c.advance_mirror(steps)


class KVmixPast(tuple):
    """Upstream's past_key_value 9-tuple backed by a preallocated KVmixLayerCache (``.cache``): element [8] is
    kv_seq_len as upstream reads it, elements [0..7] are lazily built views for whoever indexes them.
    ``attention_step(..., in_place=True)`` returns it and, given it back, appends in place and runs the fused
    tensor-core attention instead of re-concatenating the packed tensors every step."""

    def __new__(cls, cache):
        self = super().__new__(cls, (None,) * 8 + (cache.kv_seq_len,))
        self.cache = cache
        self._views = None
        return self

    def __getitem__(self, i):
        if isinstance(i, int) and (i == 8 or i == -1):
            return tuple.__getitem__(self, 8)
        if self._views is None:
            self._views = self.cache.view_tuple()
        return self._views[i]

    def __iter__(self):
        return iter(self[0:9])


def _grown(cache, need_tokens):
    """A cache with at least ``need_tokens`` capacity holding the same state (capacity doubles when it runs out)."""
    if need_tokens <= cache.max_tokens:
        return cache
    pol = dict(residual_length=cache.window) if cache.window is not None else \
        dict(k_residual_ratio=cache.rk, v_residual_ratio=cache.rv)
    big = KVmixLayerCache(cache.B, cache.Hkv, cache.D, max(2 * cache.max_tokens, need_tokens + 1024), cache.k_bits,
                          cache.v_bits, cache.v_group, device=cache.kfull.device, **pol)
    big.load_tuple(cache.view_tuple())
    return big


def attention_step(query_states, key_states, value_states, past_key_value, k_bits, v_bits, group_size,
                   k_residual_ratio=None, v_residual_ratio=None, residual_length=None, use_cache=True,
                   attention_mask=None, in_place=False):
    """Functional drop-in for upstream's attention body (modeling_llama_KVmix.py:105-273).
    attention_mask is upstream's additive mask ([B,1,q_len,kv_seq_len]); None means causal prefill / no padding.
    in_place=True keeps the state in a preallocated KVmixLayerCache carried by the returned tuple (a KVmixPast): no
    per-step concatenation, aligned buffers, the tensor-core kernel on every step.  The tuple's tensors are then
    views that later steps overwrite; with in_place=False (default) every step returns fresh tensors as upstream does.

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
    if in_place or isinstance(past_key_value, KVmixPast):
        # same contract, but the state lives in a preallocated cache carried by the returned tuple
        pol = dict(residual_length=residual_length) if residual_length is not None else \
            dict(k_residual_ratio=k_residual_ratio, v_residual_ratio=v_residual_ratio)
        if past_key_value is None:
            cache = KVmixLayerCache(B, Hkv, D, max(2 * q_len, q_len + 1024), k_bits, v_bits, group_size,
                                    device=key_states.device, **pol)
            cache.prefill(key_states, value_states)
            attn = torch.nn.functional.scaled_dot_product_attention(
                query_states, key_states, value_states, attn_mask=attention_mask,
                is_causal=attention_mask is None and q_len > 1, enable_gqa=nh != Hkv, scale=1.0 / math.sqrt(D))
        else:
            if q_len != 1:
                raise RuntimeError("cached attention takes one new token per step")
            if isinstance(past_key_value, KVmixPast):
                cache = past_key_value.cache
            else:                                                  # a plain upstream tuple: adopt it once
                seen = int(past_key_value[8])
                cache = KVmixLayerCache(B, Hkv, D, max(2 * seen, seen + 1024), k_bits, v_bits, group_size,
                                        device=key_states.device, **pol)
                cache.load_tuple(past_key_value)
            cache = _grown(cache, cache.kv_seq_len + 1)
            attn = cache.decode_step(query_states, key_states, value_states, attention_mask=attention_mask)
        return attn, (KVmixPast(cache) if use_cache else None)
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
                                    v_bits, v_group, attention_mask=attention_mask)
    else:
        attn = torch.nn.functional.scaled_dot_product_attention(
            query_states, key_states, value_states, attn_mask=attention_mask,
            is_causal=attention_mask is None and q_len > 1, enable_gqa=nh != Hkv, scale=1.0 / math.sqrt(D))
        kfull = kfull.contiguous()
        vfull = vfull.contiguous()
    new_past = (kq, kfull, ksc, kmn, vq, vfull, vsc, vmn, kv_seq_len) if use_cache else None
    return attn, new_past
