"""Shared helpers for the parity tests: seeded synthetic K/V in the shapes the benchmark
configurations name, and the comparison rule for attention outputs."""
import os

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


ROUNDING_DOMINATED = []     # (test id, rows, worst error, upstream's own noise on that row): reported by conftest.py


def _assert_rows_within(got, want, tol, noise=None, what="", dominated_rows=0):
    """Every (batch, head) row of ``got`` within ``tol`` relative of ``want``; the failure message names how many rows
    miss, by how much, and (when given) upstream's own rounding noise on the worst row.

    ``dominated_rows`` > 0 (only the small-context tests that need it pass it, each naming its count) admits that many
    rounding-dominated rows: rows on which upstream's own fp16 narrowing of the scores moves the result by at least
    0.5 tol.  There one dominant score sitting next to an fp16 rounding midpoint falls to one side in upstream's
    summation order and to the other in any other order, and that single ulp is worth more than tol; such a row must
    still be within tol + that noise.  Every use is recorded in ROUNDING_DOMINATED and listed at the end of the run."""
    assert np.isfinite(got.astype(np.float32)).all()
    err = row_rel(got, want)
    bad = np.flatnonzero(err > tol)
    if bad.size and noise is not None and bad.size <= dominated_rows and \
            (noise[bad] >= 0.5 * tol).all() and (err[bad] <= tol + noise[bad]).all():
        w = int(bad[np.argmax(err[bad])])
        ROUNDING_DOMINATED.append((os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0], int(bad.size), float(err[w]), float(noise[w])))
        bad = bad[:0]
    if bad.size:
        w = int(bad[np.argmax(err[bad])])
        extra = "" if noise is None else f", upstream's own narrowing moves that row by {noise[w]:.3e}"
        raise AssertionError(f"{what}{bad.size} of {err.size} rows beyond {tol:.1e}: worst row {w} at {err[w]:.3e}{extra}")
    ok = err <= tol
    g = got.astype(np.float64).reshape(-1, got.shape[-1])[ok]
    w_ = want.astype(np.float64).reshape(-1, want.shape[-1])[ok]
    atol = tol * np.abs(w_).max(axis=1, keepdims=True)
    assert (np.abs(g - w_) <= atol + 1e-7).all(), f"{what}element error {np.abs(g - w_).max():.3e}"
    return err.max()


def assert_attn_parity(kernel, ref_cache, q, tol=REL_TOL, dominated_rows=0):
    """The parity statements for fused attention.

    ``kernel(round_scores)`` returns the library's output as numpy; ``ref_cache`` is the oracle cache.

    1. fp32-accumulate parity: with score narrowing off, the kernel is within ``tol`` (2e-3 relative per row, the
       stated tolerance) of the oracle evaluated without intermediate narrowing.
    2. reference parity: in the default mode (score narrowing on, what ``attend`` and the benchmark run) the kernel is
       within the same ``tol`` of the oracle evaluated with every one of upstream's narrowing points
       (``ref_rounding=7``) -- the plain statement, no allowance for upstream's rounding noise.
    """
    want32 = ref_cache.attend(q, ref_rounding=0)
    want_up = ref_cache.attend(q, ref_rounding=7)
    _assert_rows_within(kernel(False), want32, tol, what="fp32-accumulate parity: ")
    return _assert_rows_within(kernel(True), want_up, tol, noise=row_rel(want32, want_up), what="reference parity: ",
                               dominated_rows=dominated_rows)


def assert_close_to_upstream(got, want_up, want32=None, tol=REL_TOL, dominated_rows=0):
    """Statement 2 of assert_attn_parity for an output computed with score narrowing on."""
    noise = None if want32 is None else row_rel(want32, want_up)
    return _assert_rows_within(got, want_up, tol, noise=noise, what="reference parity: ", dominated_rows=dominated_rows)
