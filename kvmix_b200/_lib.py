"""ctypes binding of libkvmix_b200.so (declared in include/kvmix_b200.h).

There is no fallback: if the library has not been built (``python -m kvmix_b200.build``) importing
any operator raises.  Struct layouts below mirror the header field for field.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libkvmix_b200.so")

i32, i64, u64, vp = C.c_int32, C.c_int64, C.c_uint64, C.c_void_p


class QuantArgs(C.Structure):
    _fields_ = [("x", vp), ("x_is_f32", i32),
                ("B", i64), ("H", i64), ("A", i64), ("S", i64),
                ("x_sB", i64), ("x_sH", i64), ("x_sA", i64), ("x_sS", i64),
                ("group", i32), ("bits", i32), ("scale_by_division", i32),
                ("code", vp), ("c_sB", i64), ("c_sH", i64), ("c_sA", i64),
                ("scale", vp), ("mn", vp), ("z_sB", i64), ("z_sH", i64), ("z_sA", i64), ("ragged_tail", i32)]


class GemvArgs(C.Structure):
    _fields_ = [("fA", vp), ("a_sB", i64), ("a_sH", i64),
                ("qB", vp), ("q_sB", i64), ("q_sH", i64), ("q_sK", i64),
                ("scale", vp), ("zero", vp), ("s_sB", i64), ("s_sH", i64), ("s_sK", i64),
                ("out", vp), ("o_sB", i64), ("o_sH", i64),
                ("B", i64), ("nh", i64), ("nh_kv", i64), ("K", i64), ("n_words", i64), ("n_groups", i64),
                ("group", i32), ("bits", i32)]


class AppendArgs(C.Structure):
    _fields_ = [("B", i32), ("Hkv", i32), ("D", i32),
                ("k_new", vp), ("kn_sB", i64), ("kn_sH", i64),
                ("v_new", vp), ("vn_sB", i64), ("vn_sH", i64),
                ("kfull", vp), ("kf_sB", i64), ("kf_sH", i64), ("kf_sT", i64), ("k_slot", i32),
                ("vfull", vp), ("vf_sB", i64), ("vf_sH", i64), ("vf_sT", i64), ("v_slot", i32)]


class AppendFormArgs(C.Structure):
    _fields_ = [("x", vp), ("x_is_f32", i32), ("B", i64), ("H", i64), ("A", i64), ("S", i64),
                ("x_sB", i64), ("x_sH", i64), ("x_sA", i64), ("x_sS", i64), ("group", i32), ("bits", i32),
                ("prev_code", vp), ("prev_scale", vp), ("prev_mn", vp),
                ("old_words", i64), ("old_groups", i64), ("old_tokens", i64),
                ("code", vp), ("scale", vp), ("mn", vp)]


class AttnArgs(C.Structure):
    _fields_ = [("B", i32), ("nh", i32), ("nh_kv", i32), ("D", i32),
                ("T", i32), ("Tkq", i32), ("Tvq", i32),
                ("k_bits", i32), ("k_group", i32), ("v_bits", i32), ("v_group", i32),
                ("round_scores", i32), ("softmax_scale", C.c_float),
                ("q", vp), ("q_sB", i64), ("q_sH", i64),
                ("out", vp), ("o_sB", i64), ("o_sH", i64),
                ("kcode", vp), ("kc_sB", i64), ("kc_sH", i64), ("kc_sD", i64),
                ("kscale", vp), ("kmn", vp), ("ks_sB", i64), ("ks_sH", i64), ("ks_sD", i64),
                ("kfull", vp), ("kf_sB", i64), ("kf_sH", i64), ("kf_sT", i64),
                ("kf_cap", i32), ("kf_start", i32),
                ("vcode", vp), ("vc_sB", i64), ("vc_sH", i64), ("vc_sT", i64),
                ("vscale", vp), ("vmn", vp), ("vs_sB", i64), ("vs_sH", i64), ("vs_sT", i64),
                ("vfull", vp), ("vf_sB", i64), ("vf_sH", i64), ("vf_sT", i64),
                ("vf_cap", i32), ("vf_start", i32),
                ("workspace", vp), ("workspace_bytes", u64),
                ("mask", vp), ("mask_sB", i64), ("mask_sH", i64), ("mask_is_f32", i32), ("flags", i32),
                ("k_new", vp), ("v_new", vp), ("kn_sB", i64), ("kn_sH", i64), ("vn_sB", i64), ("vn_sH", i64),
                ("k_quant", i32), ("v_quant", i32), ("k_quant_slot", i32), ("v_quant_slot", i32),
                ("state", vp), ("window", i32), ("k_ratio", C.c_double), ("v_ratio", C.c_double),
                ("n_peers", i32), ("peer_head0", i32), ("peer_out", vp * 8), ("peer_flag", vp * 8),
                ("peer_sB", i64), ("peer_sH", i64)]


class PrefillArgs(C.Structure):
    _fields_ = [("k", vp), ("v", vp), ("k_sB", i64), ("k_sT", i64), ("k_sH", i64), ("v_sB", i64), ("v_sT", i64), ("v_sH", i64),
                ("cos", vp), ("sin", vp), ("r_sB", i64), ("r_sT", i64),
                ("B", i32), ("Hkv", i32), ("L", i32), ("D", i32), ("nk", i32), ("nv", i32),
                ("k_bits", i32), ("k_group", i32), ("v_bits", i32), ("v_group", i32),
                ("kcode", vp), ("kc_sB", i64), ("kc_sH", i64), ("kc_sD", i64),
                ("kscale", vp), ("kmn", vp), ("ks_sB", i64), ("ks_sH", i64), ("ks_sD", i64),
                ("vcode", vp), ("vc_sB", i64), ("vc_sH", i64), ("vc_sT", i64),
                ("vscale", vp), ("vmn", vp), ("vs_sB", i64), ("vs_sH", i64), ("vs_sT", i64),
                ("kfull", vp), ("kf_sB", i64), ("kf_sH", i64), ("kf_sT", i64),
                ("vfull", vp), ("vf_sB", i64), ("vf_sH", i64), ("vf_sT", i64)]


class AttnPlan(C.Structure):
    _fields_ = [("kernel", i32), ("heads_per_cta", i32), ("unit", i32), ("units_per_head", i32), ("n_ctas", i32),
                ("n_whole", i32), ("n_cut", i32), ("segments", i32), ("segment_units", i32), ("max_segment_tokens", i32)]


ATTN_WORKSPACE_READY = 1


_lib = None


def lib():
    """The loaded C-ABI library; raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m kvmix_b200.build` (needs nvcc). "
                "kvmix_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        L.kvq_version.restype = C.c_int
        L.kvq_error_string.restype = C.c_char_p
        L.kvq_error_string.argtypes = [C.c_int]
        L.kvq_last_cuda_error.restype = C.c_char_p
        L.kvq_features_per_int.restype = C.c_int
        L.kvq_features_per_int.argtypes = [C.c_int]
        L.kvq_quant_lastdim.restype = C.c_int
        L.kvq_quant_lastdim.argtypes = [C.POINTER(QuantArgs), vp]
        L.kvq_append_kv.restype = C.c_int
        L.kvq_append_kv.argtypes = [C.POINTER(AppendArgs), vp]
        L.kvq_gemv.restype = C.c_int
        L.kvq_gemv.argtypes = [C.POINTER(GemvArgs), vp]
        L.kvq_decode_attn.restype = C.c_int
        L.kvq_decode_attn.argtypes = [C.POINTER(AttnArgs), vp]
        L.kvq_decode_attn_static.restype = C.c_int
        L.kvq_decode_attn_static.argtypes = [C.POINTER(AttnArgs), vp]
        for fn in (L.kvq_append_k, L.kvq_append_v):
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(AppendFormArgs), vp]
        L.kvq_decode_attn_plan.restype = C.c_int
        L.kvq_decode_attn_plan.argtypes = [C.POINTER(AttnArgs), i32, C.POINTER(AttnPlan)]
        L.kvq_peer_wait.restype = C.c_int
        L.kvq_peer_wait.argtypes = [vp, C.c_uint32, C.c_uint32, vp, vp]
        L.kvq_peer_wait_next.restype = C.c_int
        L.kvq_peer_wait_next.argtypes = [vp, C.c_uint32, vp, C.c_uint32, vp, vp]
        L.kvq_prefill.restype = C.c_int
        L.kvq_prefill.argtypes = [C.POINTER(PrefillArgs), vp]
        L.kvq_decode_attn_workspace_init.restype = C.c_int
        L.kvq_decode_attn_workspace_init.argtypes = [vp, u64, i32, i32, vp]
        L.kvq_decode_attn_workspace_bytes.restype = u64
        L.kvq_decode_attn_workspace_bytes.argtypes = [i32, i32, i32]
        _lib = L
    return _lib


EXPORTS = ["kvq_version", "kvq_error_string", "kvq_last_cuda_error", "kvq_features_per_int",
           "kvq_quant_lastdim", "kvq_append_kv", "kvq_gemv", "kvq_decode_attn", "kvq_decode_attn_workspace_bytes",
           "kvq_decode_attn_static", "kvq_decode_attn_plan", "kvq_decode_attn_workspace_init", "kvq_prefill", "kvq_peer_wait", "kvq_peer_wait_next", "kvq_append_k", "kvq_append_v"]


def check(rc):
    """Negative status -> RuntimeError carrying the upstream TORCH_CHECK wording where one exists."""
    if rc == 0:
        return
    msg = lib().kvq_error_string(rc).decode()
    if rc == -100:
        msg += ": " + lib().kvq_last_cuda_error().decode()
    raise RuntimeError(msg)
