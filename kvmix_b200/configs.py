"""The five benchmark configurations of the KV-cache hot path, as data: attention geometry, the
seeded per-layer bit maps (the ``quant_bits[layer] = {k_bits, v_bits, k_residual_ratio,
v_residual_ratio}`` schema of upstream myprofileKV.py:99-104) and synthetic-state builders.

Synthetic stand-ins: upstream measures throughput on real checkpoints and prompts; here K/V/q are
seeded N(0,1) tensors of the same shapes with a seeded set of outlier key channels per head.
"""
import random
from dataclasses import dataclass, field

import torch

RESIDUAL_RATIO = {4: 0.3, 3: 0.2, 2: 0.2, 1: 0.1}      # upstream myprofileKV.py:75-80


def _entry(kb, vb):
    return {"k_bits": kb, "v_bits": vb, "k_residual_ratio": RESIDUAL_RATIO[kb], "v_residual_ratio": RESIDUAL_RATIO[vb]}


def seeded_bit_map(n_layers, plan, seed=0):
    """plan: list of (count, k_bits, v_bits); layers are assigned in a seeded shuffle order."""
    order = list(range(n_layers))
    random.Random(seed).shuffle(order)
    out, i = {}, 0
    for count, kb, vb in plan:
        for layer in order[i:i + count]:
            out[layer] = _entry(kb, vb)
        i += count
    assert i == n_layers
    return out


@dataclass
class HotPathConfig:
    name: str
    n_layers: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    group_size: int
    residual_length: int
    batch: int
    context: int
    decode_steps: int
    quant_bits: dict = field(default_factory=dict)
    shard: str = "batch"           # "batch": sequences split across GPUs; "kv_head": heads split + all-gather


def config1():
    return HotPathConfig("cfg1-micro-K4V2-g32-ctx1024", 1, 32, 32, 128, 32, 128, 1, 1024, 1, {0: _entry(4, 2)})


def config2():
    qb = seeded_bit_map(32, [(8, 4, 4), (12, 3, 2), (12, 2, 2)])
    return HotPathConfig("cfg2-llama2-7b-b64-ctx4096-g32-w128", 32, 32, 32, 128, 32, 128, 64, 4096, 256, qb)


def config3(v3_as_v4=True):
    # upstream cannot hold 3-bit values for head_dim 128 (128 % 11 != 0): by default those layers run V4 (the map
    # upstream could run); v3_as_v4=False runs them with the 3-bit-value extension of this library
    qb = seeded_bit_map(32, [(4, 4, 4), (12, 3, 4 if v3_as_v4 else 3), (12, 2, 2), (4, 2, 1)])
    name = "cfg3-mistral-7b-b8-ctx32768-g64-w128" + ("" if v3_as_v4 else "-v3ext")
    return HotPathConfig(name, 32, 32, 8, 128, 64, 128, 8, 32768, 128, qb)


def config5():
    qb = {i: _entry(4, 4) if i < 4 else _entry(3, 2) for i in range(32)}
    return HotPathConfig("cfg5-llama3-8b-b1-ctx131072-g128-w256", 32, 32, 8, 128, 128, 256, 1, 131072, 64, qb,
                         shard="kv_head")


def synth_kv(batch, kv_heads, tokens, head_dim, device, seed, outliers=4, outlier_scale=8.0):
    """Seeded K, V [B,Hkv,T,D] fp16 ~ N(0,1), ``outliers`` key channels per head scaled."""
    g = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn((batch, kv_heads, tokens, head_dim), generator=g, device=device, dtype=torch.float16)
    v = torch.randn((batch, kv_heads, tokens, head_dim), generator=g, device=device, dtype=torch.float16)
    ch = torch.rand((kv_heads, head_dim), generator=g, device=device).argsort(dim=1)[:, :outliers]
    scale = torch.ones((kv_heads, head_dim), device=device, dtype=torch.float16)
    scale.scatter_(1, ch, outlier_scale)
    k.mul_(scale[None, :, None, :])
    return k, v


def build_layer_caches(cfg, batch, device, extra_tokens, kv_heads=None, seed=0, use_ratio_policy=False,
                       device_state=False):
    """One prefilled KVmixLayerCache per layer, holding ``cfg.context`` synthetic tokens."""
    from .cache import KVmixLayerCache
    kv_heads = kv_heads or cfg.n_kv_heads
    caches = []
    for layer in range(cfg.n_layers):
        qb = cfg.quant_bits[layer]
        pol = (dict(k_residual_ratio=qb["k_residual_ratio"], v_residual_ratio=qb["v_residual_ratio"])
               if use_ratio_policy else dict(residual_length=cfg.residual_length))
        c = KVmixLayerCache(batch, kv_heads, cfg.head_dim, cfg.context + extra_tokens, qb["k_bits"], qb["v_bits"],
                            cfg.group_size, device=device, device_state=device_state, **pol)
        k, v = synth_kv(batch, kv_heads, cfg.context, cfg.head_dim, device, seed * 1000 + layer)
        c.prefill(k, v)
        del k, v
        caches.append(c)
    return caches
