"""The C-ABI library loads and exports every symbol include/kvmix_b200.h declares (no GPU needed)."""
import ctypes
import os
import re

import pytest

from kvmix_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(kvq_[a-z0-9_]+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    L = _lib.lib()
    decl = declared_symbols()
    assert decl, "no declarations found"
    assert decl == set(_lib.EXPORTS) | (decl - set(_lib.EXPORTS))
    for name in sorted(decl):
        assert hasattr(L, name), f"{name} declared in include/ but not exported"
    for name in _lib.EXPORTS:
        assert name in decl, f"{name} bound in Python but not declared in include/"


def test_version_and_error_strings():
    L = _lib.lib()
    assert L.kvq_version() >= 100
    assert L.kvq_error_string(0) == b"ok"
    assert b"group_length must be 11" in L.kvq_error_string(-2)
    assert [L.kvq_features_per_int(b) for b in (1, 2, 3, 4)] == [32, 16, 11, 8]


def test_struct_sizes_match_header():
    """Compile a tiny C program against the header and compare sizeof() with the ctypes mirrors."""
    import subprocess, tempfile
    src = r'''
#include <stdio.h>
#include "kvmix_b200.h"
int main(void){ printf("%zu %zu %zu %zu %zu %zu %zu\n", sizeof(kvq_quant_args), sizeof(kvq_gemv_args), sizeof(kvq_attn_args), sizeof(kvq_append_args), sizeof(kvq_append_form_args), sizeof(kvq_prefill_args), sizeof(kvq_attn_plan)); return 0; }
'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    assert sizes == [ctypes.sizeof(_lib.QuantArgs), ctypes.sizeof(_lib.GemvArgs), ctypes.sizeof(_lib.AttnArgs),
                     ctypes.sizeof(_lib.AppendArgs), ctypes.sizeof(_lib.AppendFormArgs), ctypes.sizeof(_lib.PrefillArgs),
                     ctypes.sizeof(_lib.AttnPlan)]


def test_argument_errors_need_no_gpu():
    """Host-side argument checks return before any CUDA call."""
    L = _lib.lib()
    a = _lib.QuantArgs()
    a.bits, a.group, a.B, a.H, a.A, a.S = 3, 32, 1, 1, 1, 34
    assert L.kvq_quant_lastdim(ctypes.byref(a), None) == -2
    a.group = 11
    assert L.kvq_quant_lastdim(ctypes.byref(a), None) == -3
    a.bits, a.group, a.S = 4, 32, 48
    assert L.kvq_quant_lastdim(ctypes.byref(a), None) == -4
    a.bits, a.group, a.S = 1, 16, 16
    assert L.kvq_quant_lastdim(ctypes.byref(a), None) == -5
    a.bits = 5
    assert L.kvq_quant_lastdim(ctypes.byref(a), None) == -1
    g = _lib.GemvArgs()
    g.bits, g.group, g.nh, g.nh_kv = 4, 32, 3, 2
    assert L.kvq_gemv(ctypes.byref(g), None) == -6
    t = _lib.AttnArgs()
    t.D = 64
    assert L.kvq_decode_attn(ctypes.byref(t), None) == -11


def _plan(B, nh, T, kb, tc, nh_kv=None, G=32, vb=2):
    import ctypes
    a = _lib.AttnArgs()
    a.B, a.nh, a.nh_kv, a.D, a.T = B, nh, nh_kv or nh, 128, T
    a.k_bits, a.k_group, a.v_bits, a.v_group = kb, 11 if kb == 3 else G, vb, G
    p = _lib.AttnPlan()
    assert _lib.lib().kvq_decode_attn_plan(ctypes.byref(a), tc, ctypes.byref(p)) == 0
    return p


def _walk(p, T):
    """Every (head, t0, t1, segment, count) the tensor-core kernels run under plan p, CTA by CTA (the arithmetic of
    kvmix_b200/csrc/attn_plan.cuh restated)."""
    out = []
    for c in range(p.n_ctas):
        if c < p.n_whole:
            out.append((c, 0, T, 0, 1))
            continue
        cc = c - p.n_whole
        seg = cc // p.n_cut
        t0 = seg * p.segment_units * p.unit
        out.append((p.n_whole + cc % p.n_cut, t0, min(T, t0 + p.segment_units * p.unit), seg, p.segments))
    return out


def test_split_plan_invariants_and_workspace_bound():
    """Host-only: every plan covers every head's T tokens exactly once with segments in token order, respects the
    score buffer of its kernel, and never needs more workspace than kvq_decode_attn_workspace_bytes promises for any
    shorter context (a cache sizes its workspace once, for its maximum length)."""
    L = _lib.lib()
    for B, nh, nh_kv in [(1, 1, 1), (1, 32, 32), (3, 8, 8), (8, 32, 32), (14, 32, 32), (64, 32, 32), (256, 32, 32),
                         (1, 32, 8), (8, 32, 8), (5, 16, 8), (64, 64, 8)]:
        for Tmax in (1, 31, 352, 1024, 4096, 4119, 9000, 32768, 131072 + 300):
            ws = L.kvq_decode_attn_workspace_bytes(B, nh, Tmax)
            for T in sorted({1, Tmax // 3 + 1, Tmax - 1 if Tmax > 1 else 1, Tmax}):
                for kb in (1, 2, 3, 4):
                    heads = B * nh
                    g = _plan(B, nh, T, kb, 0, nh_kv, 128)
                    assert g.kernel == 0 and g.unit > 0 and g.segments >= 1
                    assert (g.segments - 1) * g.unit < T <= g.segments * g.unit <= g.segments * 4224
                    assert g.unit % (352 if kb == 3 else 128) == 0 and g.n_ctas == heads * g.segments
                    need = 0 if g.segments == 1 else ((heads * 4 + 255) // 256) * 256 + heads * g.segments * 132 * 4
                    assert need <= ws
                    p = _plan(B, nh, T, kb, 1, nh_kv, 128)
                    grouped = nh // nh_kv in (2, 4, 8)
                    assert p.kernel == (2 if grouped else 1) and p.heads_per_cta == (min(4, nh // nh_kv) if grouped else 1)
                    groups = heads // p.heads_per_cta
                    assert p.unit == (352 if kb == 3 else 256) and p.units_per_head == -(-T // p.unit)
                    assert p.n_whole + p.n_cut == groups and p.n_ctas == p.n_whole + p.n_cut * p.segments
                    slots, cap = (148 * 2, 2816 if kb == 3 else 2048) if grouped else (148 * 3, 8096 if kb == 3 else 8192)
                    assert p.n_whole % slots == 0 and p.max_segment_tokens <= cap
                    assert (p.segments - 1) * p.segment_units < p.units_per_head <= p.segments * p.segment_units
                    if p.n_ctas <= 40000:                                    # walk the small and medium plans fully
                        seen = {}
                        for hd, t0, t1, seg, cnt in _walk(p, T):
                            assert 0 <= t0 < t1 <= T and t0 % p.unit == 0 and t1 - t0 <= p.max_segment_tokens
                            assert len(seen.setdefault(hd, [])) == seg and (seg == 0 or seen[hd][-1][1] == t0)
                            seen[hd].append((t0, t1, cnt))
                        assert sorted(seen) == list(range(groups))
                        for segs in seen.values():
                            assert segs[0][0] == 0 and segs[-1][1] == T and len(segs) == segs[0][2]
                    partials = 0 if p.segments == 1 else p.n_cut * p.segments * p.heads_per_cta
                    need = 0 if partials == 0 else ((heads * 4 + 255) // 256) * 256 + partials * 132 * 4
                    assert need <= ws, (B, nh, nh_kv, Tmax, T, kb, p.kernel, p.segments)


def test_split_plan_prefers_one_split_for_full_grids():
    p = _plan(64, 32, 4119, 2, 1)                            # 2048 heads of 4119 tokens: one CTA per head
    assert (p.n_whole, p.n_cut, p.segments) == (1776, 272, 1) and p.max_segment_tokens == 4128
    p = _plan(8, 32, 4096, 2, 1)                             # 256 heads for 444 slots: cutting would need a second round
    assert (p.n_whole, p.n_cut, p.segments) == (0, 256, 1)
    p = _plan(1, 32, 4096, 2, 1)                             # 32 heads: cut, the slots are mostly empty otherwise
    assert p.segments > 1 and p.n_ctas <= 444
    assert _plan(1, 32, 131072, 4, 1).segments > 8           # one long sequence: many segments per head
    p = _plan(8, 32, 32768, 2, 1, nh_kv=8, G=64)             # grouped queries: 64 head groups of 4 query heads
    assert (p.kernel, p.heads_per_cta, p.n_whole + p.n_cut) == (2, 4, 64) and p.max_segment_tokens <= 2048
    assert _plan(8, 32, 32768, 2, 1, nh_kv=8, G=32).kernel == 1      # 2-bit keys in groups of 32: one head per CTA
    assert _plan(8, 32, 32768, 2, 1, nh_kv=8, G=64, vb=1).kernel == 2     # 1-bit values at group 64: two groups per block
    assert _plan(8, 32, 32768, 4, 1, nh_kv=8, G=64, vb=2).kernel == 2
    assert _plan(8, 32, 32768, 4, 1, nh_kv=8, G=32, vb=2).kernel == 1     # 2-bit values at group 32: one head per CTA
    with pytest.raises(Exception):
        _lib.check(_lib.lib().kvq_decode_attn_plan(None, 1, None))
