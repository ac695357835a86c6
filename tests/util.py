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


def row_rel(a, b):
    a = a.astype(np.float64).reshape(-1, a.shape[-1])
    b = b.astype(np.float64).reshape(-1, b.shape[-1])
    return np.linalg.norm(a - b, axis=1) / np.maximum(np.linalg.norm(b, axis=1), 1e-30)


def assert_attn_parity(kernel, ref_cache, q, tol=REL_TOL):
    """The two parity statements for fused attention.

    ``kernel(round_scores)`` returns the library's output as numpy; ``ref_cache`` is the oracle cache.

    1. fp32-accumulate parity: with score narrowing off, the kernel is within ``tol`` (2e-3 relative
       per row, the stated tolerance) of the oracle evaluated without intermediate narrowing.
    2. closeness to upstream's rounding: upstream narrows every raw score to fp16 before the softmax.
       A score that lies near a rounding midpoint falls one way or the other depending on the fp32
       summation order, which a fused kernel cannot share with upstream's lane/shuffle order, and
       one flipped dominant score moves a row by a full fp16 ulp of that score.  So with narrowing
       on, each row must be within ``tol`` plus upstream's own rounding noise on that row (the
       distance between the oracle with and without upstream's narrowing points).
    """
    want32 = ref_cache.attend(q, ref_rounding=0)
    want_up = ref_cache.attend(q, ref_rounding=7)
    got32 = kernel(False)
    assert_attn_close(got32, want32, tol)
    got_up = kernel(True)
    assert np.isfinite(got_up.astype(np.float32)).all()
    noise = row_rel(want32, want_up)
    err = row_rel(got_up, want_up)
    assert (err <= tol + noise).all(), f"rows beyond tol + upstream rounding noise: {err.max():.3e} (noise {noise.max():.3e})"
    return err.max()


def assert_close_to_upstream(got, want_up, want32, tol=REL_TOL):
    """Statement 2 of assert_attn_parity for an output computed with score narrowing on."""
    noise = row_rel(want32, want_up)
    err = row_rel(got, want_up)
    assert np.isfinite(got.astype(np.float32)).all()
    assert (err <= tol + noise).all(), f"{err.max():.3e} beyond tol + upstream rounding noise {noise.max():.3e}"
