"""kvq_decode_attn_static: the attention entry point for callers that cannot hand over device memory
(a foreign-function host with no device allocator of its own, or an engine whose HBM is fully committed
to its KV-cache pool).  It must give exactly what kvq_decode_attn gives with a caller workspace, call
after call, although every call reuses the same library-resident scratch.

Collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _args(cache, q, out, workspace):
    """kvq_attn_args for `cache` (a KVmixLayerCache), filled the way the library's own host code fills it."""
    from kvmix_b200._lib import AttnArgs
    c = cache
    B, nh, _, D = q.shape
    T = c.tkq + c.k_len
    return AttnArgs(B, nh, c.Hkv, D, T, c.tkq, c.tvq, c.k_bits, c.k_group, c.v_bits, c.v_group, 1, 1.0 / math.sqrt(D),
                    q.data_ptr(), q.stride(0), q.stride(1), out.data_ptr(), out.stride(0), out.stride(1),
                    c.kcode.data_ptr(), c.kcode.stride(0), c.kcode.stride(1), c.kcode.stride(2),
                    c.kscale.data_ptr(), c.kmn.data_ptr(), c.kscale.stride(0), c.kscale.stride(1), c.kscale.stride(2),
                    c.kfull.data_ptr(), c.kfull.stride(0), c.kfull.stride(1), c.kfull.stride(2), c.k_cap, c.k_start,
                    c.vcode.data_ptr(), c.vcode.stride(0), c.vcode.stride(1), c.vcode.stride(2),
                    c.vscale.data_ptr(), c.vmn.data_ptr(), c.vscale.stride(0), c.vscale.stride(1), c.vscale.stride(2),
                    c.vfull.data_ptr(), c.vfull.stride(0), c.vfull.stride(1), c.vfull.stride(2), c.v_cap, c.v_start,
                    0 if workspace is None else workspace.data_ptr(), 0 if workspace is None else workspace.numel())


# tensor-core kernel / grouped-query tensor-core kernel / generic CUDA-core kernel (groups of 16 are not a tensor-core layout)
@pytest.mark.parametrize("nh,hkv,kb,vb,G,kernel", [(4, 4, 2, 2, 32, 1), (8, 2, 4, 2, 64, 2), (4, 2, 2, 2, 16, 0)])
def test_static_scratch_matches_workspace_entry_point_twice(cuda, nh, hkv, kb, vb, G, kernel):
    import kvmix_b200 as kv
    from kvmix_b200 import _lib, configs
    L = _lib.lib()
    B, T = 1, 20000                                   # few heads + long context: many splits, so the scratch is really used
    cache = kv.KVmixLayerCache(B, hkv, 128, T + 64, kb, vb, G, residual_length=128, device=cuda)
    k, v = configs.synth_kv(B, hkv, T, 128, cuda, seed=5)
    cache.prefill(k, v)
    need = int(L.kvq_decode_attn_workspace_bytes(B, nh, T))
    assert 256 < need <= (8 << 20)
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device=cuda).manual_seed(1)
    plan = _lib.AttnPlan()                                     # the kernel this case is meant to exercise, cut into several pieces
    probe = _args(cache, torch.zeros((B, nh, 1, 128), device=cuda, dtype=torch.float16),
                  torch.zeros((B, nh, 1, 128), device=cuda, dtype=torch.float16), ws)
    assert L.kvq_decode_attn_plan(C.byref(probe), -1, C.byref(plan)) == 0
    assert plan.kernel == kernel and plan.segments > 1
    for call in range(2):                             # two calls in a row: the second sees the first one's leftovers
        q = torch.randn((B, nh, 1, 128), generator=g, device=cuda, dtype=torch.float16)
        want = torch.zeros_like(q)
        got = torch.zeros_like(q)
        a_ws = _args(cache, q, want, ws)
        a_st = _args(cache, q, got, None)             # no workspace at all
        assert L.kvq_decode_attn(C.byref(a_ws), stream) == 0
        assert L.kvq_decode_attn_static(C.byref(a_st), stream) == 0
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same kernel, same split plan, deterministic merge order: bit-identical, well inside the 2e-3 tolerance
        assert torch.equal(got, want), f"call {call}: max diff {(got.float() - want.float()).abs().max().item():.3e}"
        assert want.float().abs().max().item() > 0


def test_static_scratch_rejects_oversize_problems(cuda):
    from kvmix_b200 import _lib
    L = _lib.lib()
    a = _lib.AttnArgs()
    a.B, a.nh, a.nh_kv, a.D, a.T = 64, 32, 32, 128, 131072     # 2048 heads x 16+ splits: far beyond 8 MiB of partials
    assert int(L.kvq_decode_attn_workspace_bytes(a.B, a.nh, a.T)) > (8 << 20)
    assert L.kvq_decode_attn_static(C.byref(a), None) == -14
    assert b"built-in scratch" in L.kvq_error_string(-14)
