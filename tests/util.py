"""Shared helpers for the parity tests: seeded synthetic K/V in the shapes the benchmark
configurations name, and the comparison rule for attention outputs."""
import numpy as np


def make_kv(seed, B, H, T, D=128, outlier_scale=8.0, n_outliers=4, heavy_tail=False):
    """K, V [B,H,T,D] fp16 ~ N(0,1); per head a seeded choice of ``n_outliers`` K channels is scaled
    (or, with heavy_tail, drawn Student-t nu=3)."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((B, H, T, D)).astype(np.float32)
    v = rng.standard_normal((B, H, T, D)).astype(np.float32)
    for b in range(B):
        for h in range(H):
            ch = rng.choice(D, n_outliers, replace=False)
            if heavy_tail:
                k[b, h][:, ch] = rng.standard_t(3, size=(T, n_outliers))
            else:
                k[b, h][:, ch] *= outlier_scale
    return k.astype(np.float16), v.astype(np.float16)


def make_q(seed, B, nh, D=128):
    rng = np.random.default_rng(seed + 1000)
    return rng.standard_normal((B, nh, 1, D)).astype(np.float16)


REL_TOL = 2e-3   # per (batch, head) row: ||a-b||_2 / ||b||_2, and element-wise atol = REL_TOL * max|b|


def assert_attn_close(got, want, tol=REL_TOL):
    g = got.astype(np.float64).reshape(-1, got.shape[-1])
    w = want.astype(np.float64).reshape(-1, want.shape[-1])
    assert np.isfinite(g).all()
    num = np.linalg.norm(g - w, axis=1)
    den = np.linalg.norm(w, axis=1)
    rel = num / np.maximum(den, 1e-30)
    assert rel.max() <= tol, f"row-relative error {rel.max():.3e} > {tol}"
    atol = tol * np.abs(w).max(axis=1, keepdims=True)
    assert (np.abs(g - w) <= atol + 1e-7).all(), f"element error {np.abs(g - w).max():.3e}"
    return rel.max()
