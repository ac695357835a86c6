"""Profiler hand-off (host logic, no GPU): a profiler module shaped like upstream's myprofileKV.py -- plotting imports
at the top, ``profile_model`` returning the per-layer dict -- loads without the plotting stack, and its bit map is
checked against what the cache format holds."""
import textwrap

import pytest

from kvmix_b200 import profiler

FAKE = textwrap.dedent('''
    import torch
    import numpy as np
    import matplotlib.pyplot as plt
    import seaborn as sns
    import matplotlib.gridspec as gridspec
    from matplotlib.colors import LinearSegmentedColormap, to_rgb

    def profile_model(model, input_ids_list, attention_mask_list, labels_list, num_layers):
        ratios = {4: 0.3, 2: 0.2, 1: 0.1, 3: 0.2}
        out = {}
        for layer in range(num_layers):
            kb, vb = (3, 4) if layer % 4 == 0 else (2, 2)
            out[layer] = {'k_bits': kb, 'v_bits': vb, 'k_residual_ratio': ratios[kb], 'v_residual_ratio': ratios[vb]}
        return out

    def plot_something():
        return plt.figure()
''')


def test_profile_model_loads_without_plotting_stack(tmp_path):
    (tmp_path / "myprofileKV.py").write_text(FAKE)
    fn = profiler.load_profile_model(str(tmp_path))
    qb = fn(None, [], [], [], 8)
    checked = profiler.check_quant_bits(qb, 8)
    assert checked[0] == {"k_bits": 3, "v_bits": 4, "k_residual_ratio": 0.2, "v_residual_ratio": 0.3}
    assert checked[1]["k_bits"] == 2 and list(checked) == list(range(8))
    with pytest.raises(FileNotFoundError):
        profiler.load_profile_model(str(tmp_path / "nowhere"))
    import importlib.util
    if importlib.util.find_spec("matplotlib") is None:           # the plotting helpers then say what they need
        with pytest.raises(ImportError, match="not installed"):
            fn.__globals__["plot_something"]()


def test_bit_map_checks():
    good = {i: profiler.default_entry(2, 2) for i in range(4)}
    assert profiler.check_quant_bits({str(k): v for k, v in good.items()}, 4)[3]["k_residual_ratio"] == 0.2
    with pytest.raises(ValueError, match="no entry for layer 4"):
        profiler.check_quant_bits(good, 5)
    bad = dict(good)
    bad[2] = dict(good[2], v_bits=3)
    with pytest.raises(ValueError, match="3-bit values"):
        profiler.check_quant_bits(bad, 4)
    assert profiler.check_quant_bits(bad, 4, allow_v3_extension=True)[2]["v_bits"] == 3
    bad[2] = dict(good[2], k_bits=5)
    with pytest.raises(ValueError, match="Supported quantization bits"):
        profiler.check_quant_bits(bad, 4)
    bad[2] = {"k_bits": 2, "v_bits": 2}
    with pytest.raises(ValueError, match="missing"):
        profiler.check_quant_bits(bad, 4)


@pytest.mark.gpu
def test_caches_from_profile_run_a_decode_step(cuda):
    import torch
    qb = {0: profiler.default_entry(3, 4), 1: profiler.default_entry(2, 2), 2: profiler.default_entry(4, 2)}
    caches = profiler.caches_from_profile(qb, 1, 2, 128, 700, 32, device=cuda)
    assert [(c.k_bits, c.v_bits, c.rk, c.rv) for c in caches] == [(3, 4, 0.2, 0.3), (2, 2, 0.2, 0.2), (4, 2, 0.3, 0.2)]
    g = torch.Generator(device=cuda).manual_seed(0)
    k = torch.randn((1, 2, 600, 128), generator=g, device=cuda, dtype=torch.float16)
    q = torch.randn((1, 2, 1, 128), generator=g, device=cuda, dtype=torch.float16)
    for c in caches:
        c.prefill(k, k.flip(2))
        out = c.decode_step(q, k[:, :, :1], k[:, :, 1:2])
        assert torch.isfinite(out.float()).all() and c.kv_seq_len == 601 and c.tkq > 0
