"""Single-operator timings on one GPU (CUDA events, inputs larger than L2): the commands the ncu captures summarised
under profiles/ run.

    python -m kvmix_b200.microbench attn  KB VB G [B] [T] [reps] [heads] [kv_heads] [window]   one layer of fused decode attention
    python -m kvmix_b200.microbench step  KB VB G [B] [T] [reps] [heads] [kv_heads] [window]   one layer's fused decode step:
                                                                        append + quantize when due + attention, device-driven
    python -m kvmix_b200.microbench quant BITS G STYLE [B] [T] [reps]   STYLE k: [B,32,T,128] keys, groups over tokens
                                                                        STYLE v: values, groups over channels
    python -m kvmix_b200.microbench gemv  BITS G [B] [T] [reps]         the stand-alone quantized_gemm (q.K^T form)

Each line reports microseconds per launch and algorithmic GB/s (bytes the operator must move / time).  The
quantize-on-append sweep of benchmark configuration 4 is ``bench.py --config 4``.
"""
import sys

import torch

from . import configs, ops
from .cache import KVmixLayerCache


def _time(fn, reps, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def attn(kb, vb, G, B=16, T=4096, reps=3, heads=32, kv_heads=None, window=128):
    dev = torch.device("cuda:0")
    kv_heads = kv_heads or heads
    c = KVmixLayerCache(B, kv_heads, 128, T + 64, kb, vb, G, residual_length=window, device=dev)
    k, v = configs.synth_kv(B, kv_heads, T, 128, dev, 0)
    c.prefill(k, v)
    del k, v
    q = torch.randn((B, heads, 1, 128), device=dev, dtype=torch.float16)
    out = torch.empty_like(q)
    ms = _time(lambda: c.attend(q, out=out), reps)
    by = c.packed_bytes() + 2 * B * heads * 128 * 2
    print(f"attn K{kb}V{vb} G{G} B{B} H{heads}/{kv_heads} T{T}: {ms * 1e3:.1f} us/launch, {by / 1e6:.1f} MB, "
          f"{by / ms / 1e6:.0f} GB/s")
    return by / ms / 1e6


def step(kb, vb, G, B=16, T=4096, reps=3, heads=32, kv_heads=None, window=128):
    """The product's per-layer launch: one fused decode step with the cache lengths read from device memory."""
    dev = torch.device("cuda:0")
    kv_heads = kv_heads or heads
    c = KVmixLayerCache(B, kv_heads, 128, T + 2 * reps + 64, kb, vb, G, residual_length=window, device=dev, device_state=True)
    k, v = configs.synth_kv(B, kv_heads, T, 128, dev, 0)
    c.prefill(k, v)
    del k, v
    q = torch.randn((B, heads, 1, 128), device=dev, dtype=torch.float16)
    kn = torch.randn((B, kv_heads, 1, 128), device=dev, dtype=torch.float16)
    vn = torch.randn((B, kv_heads, 1, 128), device=dev, dtype=torch.float16)
    out = torch.empty_like(q)
    ms = _time(lambda: c.decode_step(q, kn, vn, out=out), reps)
    if c._fused is not True:
        raise SystemExit("this geometry is not served by the fused decode step")
    by = c.packed_bytes() + 2 * B * heads * 128 * 2
    print(f"step K{kb}V{vb} G{G} B{B} H{heads}/{kv_heads} T{T}: {ms * 1e3:.1f} us/launch, {by / 1e6:.1f} MB, "
          f"{by / ms / 1e6:.0f} GB/s")
    return by / ms / 1e6


def quant(bits, G, style, B=16, T=8192, reps=3, heads=32):
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn((B, heads, T, 128), generator=g, device=dev, dtype=torch.float16)
    chi = torch.randn((B, heads, T, 4, 3), generator=g, device=dev).pow(2).sum(-1).div(3.0).sqrt()
    x[..., :4] = (x[..., :4].float() / chi).to(torch.float16)                          # Student-t(3) outlier channels
    fpi = 11 if bits == 3 else 32 // bits
    if style == "k":
        Tq = (T // (11 * 32)) * 11 * 32 if bits == 3 else T
        Gk = 11 if bits == 3 else G
        src = x[:, :, :Tq].transpose(2, 3)
        code = torch.empty((B, heads, 128, Tq // fpi), dtype=torch.int32, device=dev)
        sc = torch.empty((B, heads, 128, Tq // Gk), dtype=torch.float16, device=dev)
        n, grp = B * heads * Tq * 128, Gk
    else:
        if bits == 3:
            raise SystemExit("3-bit values need head_dim % 11 == 0 (not 128)")
        src = x
        code = torch.empty((B, heads, T, 128 // fpi), dtype=torch.int32, device=dev)
        sc = torch.empty((B, heads, T, 128 // G), dtype=torch.float16, device=dev)
        n, grp = B * heads * T * 128, G
    mn = torch.empty_like(sc)
    ms = _time(lambda: ops.quantize_into(src, grp, bits, code, sc, mn), reps)
    by = n * 2 + code.numel() * 4 + 2 * sc.numel() * 2
    print(f"quant b{bits} G{grp} {style} B{B} T{T}: {ms * 1e3:.1f} us/launch, {by / 1e6:.1f} MB, {by / ms / 1e6:.0f} GB/s")
    return by / ms / 1e6


def gemv(bits, G, B=64, T=4096, reps=3, heads=32):
    """upstream's quantized_gemm contract (q.K^T over packed keys), operands read in place."""
    dev = torch.device("cuda:0")
    fpi = 11 if bits == 3 else 32 // bits
    grp = 11 if bits == 3 else G
    Tq = (T // 352) * 352 if bits == 3 else T
    k, _ = configs.synth_kv(B, heads, Tq, 128, dev, 0)
    code, sc, mn = ops.quantize_pack_last_dim_cuda(k.transpose(2, 3), grp, bits)
    del k
    q = torch.randn((B, heads, 1, 128), device=dev, dtype=torch.float16)
    out = torch.empty((B, heads, 1, Tq), device=dev, dtype=torch.float16)
    ms = _time(lambda: ops.quantized_gemm(grp, q, code, sc, mn, bits, out=out), reps)
    by = code.numel() * 4 + 2 * sc.numel() * 2 + q.numel() * 2 + out.numel() * 2
    print(f"gemv b{bits} G{grp} B{B} H{heads} T{Tq}: {ms * 1e3:.1f} us/launch, {by / 1e6:.1f} MB, {by / ms / 1e6:.0f} GB/s")
    return by / ms / 1e6


if __name__ == "__main__":
    a = sys.argv[1:]
    if not a:
        raise SystemExit(__doc__)
    if a[0] == "attn":
        attn(*[int(x) for x in a[1:]])
    elif a[0] == "step":
        step(*[int(x) for x in a[1:]])
    elif a[0] == "quant":
        quant(int(a[1]), int(a[2]), a[3], *[int(x) for x in a[4:]])
    elif a[0] == "gemv":
        gemv(*[int(x) for x in a[1:]])
    else:
        raise SystemExit(__doc__)
