"""Single-operator timings on one GPU (CUDA events, inputs larger than L2), for profiling and for the
stand-alone quantize-on-append sweep.

    python -m kvmix_b200.microbench attn  KB VB G [B] [T] [reps]       one layer of fused decode attention
    python -m kvmix_b200.microbench quant BITS G STYLE [B] [T] [reps]  STYLE k: [B,32,T,128] keys, groups over tokens
                                                                       STYLE v: values, groups over channels
    python -m kvmix_b200.microbench quant-sweep                        the sweep of benchmark configuration 4
    python -m kvmix_b200.microbench phases KB VB G [B] [T]             per-CTA phase durations of the attention kernel
                                                                       (needs `python -m kvmix_b200.build --phase-timing`)

Each line reports microseconds per launch and algorithmic GB/s (bytes the operator must move / time).
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


def phases(kb, vb, G, B=64, T=4096, heads=32):
    """Mean / p10 / p90 duration of each phase of the tensor-core attention kernel over its first 4096 CTAs, from the
    kernel's optional %globaltimer stamps (the per-line view of a profiler's source page is not used in this project)."""
    import ctypes

    import numpy as np

    from . import _lib
    lib = _lib.lib()
    if not hasattr(lib, "kvq_debug_phases"):
        raise SystemExit("the library was built without the phase clock: python -m kvmix_b200.build --phase-timing")
    dev = torch.device("cuda:0")
    c = KVmixLayerCache(B, heads, 128, T + 64, kb, vb, G, residual_length=128, device=dev)
    k, v = configs.synth_kv(B, heads, T, 128, dev, 0)
    c.prefill(k, v)
    del k, v
    q = torch.randn((B, heads, 1, 128), device=dev, dtype=torch.float16)
    out = torch.empty_like(q)
    for _ in range(3):
        c.attend(q, out=out)
    torch.cuda.synchronize()
    buf = np.zeros(4096 * 8, dtype=np.uint64)
    if lib.kvq_debug_phases(buf.ctypes.data_as(ctypes.c_void_p)) != 0:
        raise SystemExit("could not read the phase stamps")
    raw = buf.reshape(4096, 8).astype(np.int64)
    raw = raw[(raw[:, 0] > 0) & (raw[:, 5] > 0)]
    p = raw[:, :6]
    d = np.diff(p, axis=1) / 1000.0
    print(f"phases K{kb}V{vb} G{G} B{B} T{T}: {len(p)} CTAs, mean life {(p[:, 5] - p[:, 0]).mean() / 1000:.1f} us, "
          f"first start to last end {(p[:, 5].max() - p[:, 0].min()) / 1000:.1f} us")
    for i, name in enumerate(["q store", "scores (packed + fp16 tail keys)", "softmax (+ tail value loads)",
                              "fp16 tail values", "packed values"]):
        print(f"  {name:34s} mean {d[:, i].mean():6.2f} us  p10 {np.percentile(d[:, i], 10):6.2f}  "
              f"p90 {np.percentile(d[:, i], 90):6.2f}")
    print(f"  warp 0 waiting on its ring: keys {raw[:, 6].mean() / 1000:6.2f} us, values {raw[:, 7].mean() / 1000:6.2f} us")


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


def quant_sweep():
    free = torch.cuda.mem_get_info()[0]
    for T in (512, 2048, 8192, 32768):
        for B in (1, 16, 64, 256):
            if B * 32 * T * 128 * 2 * 1.7 > free:
                print(f"quant sweep: B{B} T{T} skipped (does not fit one GPU with its outputs)")
                continue
            for bits in (1, 2, 3, 4):
                for G in (32, 128):
                    for style in ("k", "v"):
                        if bits == 3 and (style == "v" or G == 128):
                            continue
                        quant(bits, G, style, B, T, reps=2)


if __name__ == "__main__":
    a = sys.argv[1:]
    if not a:
        raise SystemExit(__doc__)
    if a[0] == "attn":
        attn(*[int(x) for x in a[1:]])
    elif a[0] == "quant":
        quant(int(a[1]), int(a[2]), a[3], *[int(x) for x in a[4:]])
    elif a[0] == "phases":
        phases(*[int(x) for x in a[1:]])
    elif a[0] == "quant-sweep":
        quant_sweep()
    else:
        raise SystemExit(__doc__)
