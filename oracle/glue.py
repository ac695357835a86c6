"""TEST INFRASTRUCTURE: numpy restatement of the cache update in the upstream attention forward.

Follows ``LlamaAttention_KVmix.forward`` (models/modeling_llama_KVmix.py:105-211 decode branch,
:213-254 prefill branch; the Mistral twin at models/modeling_mistral_KVmix.py:150-262 is the same
logic with 8 KV heads).  The 9-tuple upstream threads through ``past_key_value`` (:269-273) is
held here as attributes of one object per layer.  RoPE, projections and the attention mask are
outside the path and are not restated: K, V and q enter already rotated.

``keep`` policy: upstream keeps ``int(ratio * current_fp16_len)`` newest tokens in fp16
(:118-119); with ``residual_length`` set, a fixed window of that many tokens is kept instead
(the benchmark configurations ask for fixed windows).  Everything else is identical.
"""
import numpy as np

from . import decode_attention, features_per_int, quantize_pack_last_dim, quantize_ragged3


def split_point(cur_len, group, ratio=None, residual_length=None):
    """Number of oldest fp16 tokens to quantize now (modeling_llama_KVmix.py:118-126)."""
    keep = int(residual_length) if residual_length is not None else int(ratio * cur_len)
    if cur_len > keep and keep >= 0:
        return ((cur_len - keep) // group) * group
    return 0


class RefLayerCache:
    """One layer's cache: (Kcode, Kfull, Kscale, Kmn, Vcode, Vfull, Vscale, Vmn, kv_seq_len)."""

    def __init__(self, k_bits, v_bits, group_size, k_residual_ratio=None, v_residual_ratio=None,
                 residual_length=None):
        self.k_bits, self.v_bits = k_bits, v_bits
        self.v_group = group_size                                  # values are quantized group_size tokens at a time
        self.k_group = 11 if k_bits == 3 else group_size          # modeling_llama_KVmix.py:49-52
        # channel groups of the values.  3-bit values are an extension upstream does not have (its 3-bit rule needs
        # head_dim % 11 == 0, quantization_cuda.cu:433-434): groups of 11 channels with a short last group
        self.v_cgroup = 11 if v_bits == 3 else group_size
        self.rk, self.rv, self.window = k_residual_ratio, v_residual_ratio, residual_length
        self.kcode = self.kscale = self.kmn = None
        self.vcode = self.vscale = self.vmn = None
        self.kfull = self.vfull = None
        self.kv_seq_len = 0

    # -- cache update ------------------------------------------------------------------------
    def _absorb(self):
        nk = split_point(self.kfull.shape[2], self.k_group, self.rk, self.window)
        if nk > 0:                                                   # :127-139 / :223-231
            to_q = np.ascontiguousarray(self.kfull[:, :, :nk, :].transpose(0, 1, 3, 2))
            self.kfull = np.ascontiguousarray(self.kfull[:, :, nk:, :])
            c, s, m = quantize_pack_last_dim(to_q, self.k_group, self.k_bits)
            cat = lambda a, b: b if a is None else np.concatenate([a, b], axis=3)
            self.kcode, self.kscale, self.kmn = cat(self.kcode, c), cat(self.kscale, s), cat(self.kmn, m)
        nv = split_point(self.vfull.shape[2], self.v_group, self.rv, self.window)
        if nv > 0:                                                   # :152-167 / :240-248
            to_q = np.ascontiguousarray(self.vfull[:, :, :nv, :])
            self.vfull = np.ascontiguousarray(self.vfull[:, :, nv:, :])
            if self.v_bits == 3 and to_q.shape[3] % 11:
                c, s, m = quantize_ragged3(to_q)
            else:
                c, s, m = quantize_pack_last_dim(to_q, self.v_cgroup, self.v_bits)
            cat = lambda a, b: b if a is None else np.concatenate([a, b], axis=2)
            self.vcode, self.vscale, self.vmn = cat(self.vcode, c), cat(self.vscale, s), cat(self.vmn, m)

    def prefill(self, k, v):
        """k, v: [B, Hkv, L, D] fp16, already rotated (:213-254)."""
        assert self.kv_seq_len == 0
        self.kfull, self.vfull = np.ascontiguousarray(k), np.ascontiguousarray(v)
        self.kv_seq_len = k.shape[2]
        self._absorb()

    def append(self, k_new, v_new):
        """k_new, v_new: [B, Hkv, 1, D] (:111-112 then the quantize decision)."""
        self.kfull = k_new if self.kfull is None else np.concatenate([self.kfull, k_new], axis=2)
        self.vfull = v_new if self.vfull is None else np.concatenate([self.vfull, v_new], axis=2)
        self.kv_seq_len += k_new.shape[2]
        self._absorb()

    # -- attention ---------------------------------------------------------------------------
    def attend(self, q, ref_rounding=True, attention_mask=None):
        """q: [B, nh, 1, D] fp16 -> [B, nh, 1, D] fp16 (:170-211); attention_mask as upstream's (:188-193)."""
        return decode_attention(q, self.kcode, self.kscale, self.kmn, self.kfull, self.vcode, self.vscale,
                                self.vmn, self.vfull, self.k_bits, self.k_group, self.v_bits, self.v_cgroup,
                                ref_rounding, attention_mask=attention_mask)

    def decode_step(self, q, k_new, v_new, ref_rounding=True, attention_mask=None):
        self.append(k_new, v_new)
        return self.attend(q, ref_rounding, attention_mask=attention_mask)

    @property
    def tkq(self):
        return 0 if self.kcode is None else self.kcode.shape[3] * features_per_int(self.k_bits)

    @property
    def tvq(self):
        return 0 if self.vcode is None else self.vcode.shape[2]
