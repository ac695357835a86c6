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
int main(void){ printf("%zu %zu %zu %zu %zu\n", sizeof(kvq_quant_args), sizeof(kvq_gemv_args), sizeof(kvq_attn_args), sizeof(kvq_append_args), sizeof(kvq_append_form_args)); return 0; }
'''
    with tempfile.TemporaryDirectory() as d:
        c = os.path.join(d, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(d, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = [int(x) for x in subprocess.check_output([exe]).split()]
    assert sizes == [ctypes.sizeof(_lib.QuantArgs), ctypes.sizeof(_lib.GemvArgs), ctypes.sizeof(_lib.AttnArgs),
                     ctypes.sizeof(_lib.AppendArgs), ctypes.sizeof(_lib.AppendFormArgs)]


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


def _plan(B, nh, T, kb, tc):
    import ctypes
    c, n = ctypes.c_int32(), ctypes.c_int32()
    assert _lib.lib().kvq_decode_attn_plan(B, nh, T, kb, tc, ctypes.byref(c), ctypes.byref(n)) == 0
    return c.value, n.value


def test_split_plan_invariants_and_workspace_bound():
    """Host-only: every plan covers T with its last split running to T, respects the score buffer of its kernel, and
    never needs more workspace than kvq_decode_attn_workspace_bytes promises for any shorter context (a cache sizes
    its workspace once, for its maximum length)."""
    L = _lib.lib()
    for B, nh in [(1, 1), (1, 32), (3, 8), (8, 32), (16, 32), (64, 32), (256, 32)]:
        for Tmax in (1, 31, 352, 1024, 4096, 4119, 9000, 32768, 131072 + 300):
            ws = L.kvq_decode_attn_workspace_bytes(B, nh, Tmax)
            for T in sorted({1, Tmax // 3 + 1, Tmax - 1 if Tmax > 1 else 1, Tmax}):
                for kb in (1, 2, 3, 4):
                    for tc in (0, 1):
                        chunk, n = _plan(B, nh, T, kb, tc)
                        assert chunk > 0 and n >= 1
                        assert (n - 1) * chunk < T
                        last = T - (n - 1) * chunk
                        unit = (352 if kb == 3 else 1024) if tc else (352 if kb == 3 else 128)
                        assert chunk % unit == 0
                        if tc:
                            assert last <= (8096 if kb == 3 else 8192) + unit // 4 and chunk <= 8192
                        else:
                            assert last <= chunk <= 4224
                        heads = B * nh
                        need = 0 if n == 1 else ((heads * 4 + 255) // 256) * 256 + heads * n * 130 * 4
                        assert need <= ws, (B, nh, Tmax, T, kb, tc, chunk, n)


def test_split_plan_prefers_one_split_for_full_grids():
    assert _plan(64, 32, 4119, 2, 1) == (4096, 1)          # the last split absorbs the 23-token remainder
    assert _plan(64, 32, 4119, 3, 1)[1] == 1
    assert _plan(1, 32, 131072, 4, 1)[1] > 8               # one long sequence: many splits
    with pytest.raises(Exception):
        _lib.check(_lib.lib().kvq_decode_attn_plan(1, 1, 16, 5, 1, None, None))
