"""Hand-off from upstream's gradient profiler to the cache: ``myprofileKV.profile_model`` stays upstream's Python and
only supplies the per-layer bit map (myprofileKV.py:108-115 -> ``quant_bits[layer] = {k_bits, v_bits,
k_residual_ratio, v_residual_ratio}``, :99-104), which upstream's model constructors consume
(models/modeling_llama_KVmix.py:36-39, 49-52).  This module loads that function without needing the plotting stack
the upstream file imports at its top (matplotlib, seaborn: :4-10, used only by its heat-map helpers), checks the map
against what the cache format can hold, and turns it into one preallocated ``KVmixLayerCache`` per layer.
"""
import importlib.util
import os
import sys
import types

from .configs import RESIDUAL_RATIO

_PLOTTING = ("matplotlib", "matplotlib.pyplot", "matplotlib.gridspec", "matplotlib.colors", "seaborn")


class _Missing:
    """Any name taken from a stand-in module: importing it is fine, calling or using it says what is missing."""

    def __init__(self, name):
        self._name = name

    def _fail(self, *a, **k):
        raise ImportError(f"{self._name} is not installed: only upstream's plotting helpers need it, "
                          f"profile_model does not")

    __call__ = __getattr__ = _fail


class _Lazy(types.ModuleType):
    """Stand-in for a plotting module that is not installed."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return sys.modules.get(f"{self.__name__}.{name}") or _Missing(f"{self.__name__}.{name}")


def load_profile_model(upstream_root):
    """``profile_model`` from ``<upstream_root>/myprofileKV.py``.  Plotting modules that are missing are replaced by
    stand-ins for the duration of the import, so the profiler itself (torch + numpy only) is usable without them."""
    path = os.path.join(upstream_root, "myprofileKV.py")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    added = []
    for name in _PLOTTING:
        if name in sys.modules:
            continue
        try:
            found = importlib.util.find_spec(name) is not None
        except (ImportError, ValueError):
            found = False
        if not found:
            sys.modules[name] = _Lazy(name)
            added.append(name)
    try:
        spec = importlib.util.spec_from_file_location("myprofileKV", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for name in added:
            sys.modules.pop(name, None)
    return mod.profile_model


def check_quant_bits(quant_bits, n_layers, head_dim=128, allow_v3_extension=False):
    """Validate a profiler bit map for ``n_layers`` layers; returns it with integer layer keys in order.
    3-bit values are refused for the reason upstream's own quantizer refuses them: its 3-bit format packs groups of 11
    and head_dim % 11 != 0 (quant_cuda/csrc/quantization_cuda.cu:637-639, 649) -- unless ``allow_v3_extension`` opts
    into this library's own layout for them (12 words per token, a short last group), which upstream cannot read."""
    out = {}
    for layer in range(n_layers):
        e = quant_bits.get(layer, quant_bits.get(str(layer)))
        if e is None:
            raise ValueError(f"quant_bits has no entry for layer {layer}")
        missing = {"k_bits", "v_bits", "k_residual_ratio", "v_residual_ratio"} - set(e)
        if missing:
            raise ValueError(f"layer {layer}: missing {sorted(missing)}")
        kb, vb = int(e["k_bits"]), int(e["v_bits"])
        if kb not in (1, 2, 3, 4) or vb not in (1, 2, 3, 4):
            raise ValueError(f"layer {layer}: Supported quantization bits: 1, 2, 3, 4")
        if vb == 3 and head_dim % 11 != 0 and not allow_v3_extension:
            raise ValueError(f"layer {layer}: 3-bit values need head_dim % 11 == 0 (upstream's 3-bit format packs groups of 11)")
        rk, rv = float(e["k_residual_ratio"]), float(e["v_residual_ratio"])
        if not (0.0 <= rk < 1.0 and 0.0 <= rv < 1.0):
            raise ValueError(f"layer {layer}: residual ratios must lie in [0, 1)")
        out[layer] = {"k_bits": kb, "v_bits": vb, "k_residual_ratio": rk, "v_residual_ratio": rv}
    return out


def default_entry(k_bits, v_bits):
    """A bit-map entry with upstream's residual ratios for these widths (myprofileKV.py:75-80)."""
    return {"k_bits": k_bits, "v_bits": v_bits, "k_residual_ratio": RESIDUAL_RATIO[k_bits],
            "v_residual_ratio": RESIDUAL_RATIO[v_bits]}


def caches_from_profile(quant_bits, batch, kv_heads, head_dim, max_tokens, group_size, device="cuda",
                        residual_length=None, allow_v3_extension=False):
    """One ``KVmixLayerCache`` per layer of the (checked) bit map.  Upstream's window policy -- keep
    ``int(ratio * current_fp16_len)`` tokens in fp16, with the ratio the profiler chose per layer -- is the default; a
    fixed ``residual_length`` replaces it when given."""
    from .cache import KVmixLayerCache
    qb = check_quant_bits(quant_bits, len(quant_bits), head_dim, allow_v3_extension)
    caches = []
    for layer in range(len(qb)):
        e = qb[layer]
        pol = dict(residual_length=residual_length) if residual_length is not None else \
            dict(k_residual_ratio=e["k_residual_ratio"], v_residual_ratio=e["v_residual_ratio"])
        caches.append(KVmixLayerCache(batch, kv_heads, head_dim, max_tokens, e["k_bits"], e["v_bits"], group_size,
                                      device=device, **pol))
    return caches
