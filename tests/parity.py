"""Error measures shared by the parity tests."""
import numpy as np

# tolerances stated by the north star: f32 max relative error 1e-5, bf16/f16 2e-2
TOL_F32 = 1e-5
TOL_BF16 = 2e-2


def ref_is_equal(a, b, rel=1e-3, abs_tol=2e-7):
    """The reference's own Scalar::is_equal (zyx/src/scalar.rs:1194-1209), elementwise."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    diff = np.abs(a - b)
    mx = np.maximum(np.abs(a), np.abs(b))
    ok = (a == b) | (diff < rel * mx) | (diff < abs_tol) | (np.isnan(a) & np.isnan(b))
    return bool(ok.all())


F16_MIN_NORMAL = 6.103515625e-05   # the reference's f32tof16 flushes anything smaller to zero


def max_rel_err(got, want, row_axis=-1, floor=1e-2, abs_floor=0.0):
    """max |got-want| / max(|want|, floor * max|want| over the row); floor defaults to 1e-2.

    Reductions are compared relative to the row's scale: the reference accumulates
    sequentially in f32 while the GPU reduces as a tree, so an element much smaller than
    its row's largest magnitude carries rounding error proportional to the row scale.
    Matmul tests pass floor=0.1: an f32 dot product of k terms has an absolute error of about
    sqrt(k) * 2^-24 * |partial sums| whatever its own value, so entries that cancel to nearly
    zero are measured against a tenth of the row's largest entry.
    """
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if want.size == 0:
        return 0.0
    scale = np.max(np.abs(want), axis=row_axis, keepdims=True) if want.ndim else np.abs(want)
    denom = np.maximum(np.maximum(np.abs(want), floor * scale), abs_floor)
    denom = np.where(denom == 0, 1.0, denom)
    err = np.abs(got - want) / denom
    err = np.where(np.isnan(got) & np.isnan(want), 0.0, err)
    return float(np.max(err))


# Every comparison that did not meet the tolerance against the oracle directly and was decided by the float64 attribution
# instead: (test id, what, tolerance, floor, gpu-vs-oracle, gpu-vs-float64, oracle-vs-float64).  tests/conftest.py writes the
# table out at the end of a session so that it can be read beside the results.
FALLBACKS = []


def record_fallback(what, tol, floor, e_go, e_ge, e_oe):
    import os
    test = os.environ.get("PYTEST_CURRENT_TEST", "?").split(" ")[0]
    FALLBACKS.append((test, what, tol, floor, e_go, e_ge, e_oe))


def assert_parity(got, oracle, exact, tol, floor=1e-2, row_axis=-1, what="", abs_floor=0.0):
    """The parity bar for reductions whose order differs between the reference and the GPU.

    The reference accumulates sequentially in f32 (zyx/src/kernel/linearize.rs:920-950), so over
    tens of thousands of terms its own result drifts from the exact one by more than `tol`.
    The GPU result must be within `tol` of the oracle; or else it must be as close to the exact
    (float64) value of the same formula as `tol` — or as the oracle itself is, where the formula's
    own f32 conditioning (cancellation) is worse than `tol` — with the remaining distance to the
    oracle no larger than `tol` plus the oracle's own distance from exact.
    """
    e_go = max_rel_err(got, oracle, row_axis, floor, abs_floor)
    if e_go <= tol:
        return
    e_ge = max_rel_err(got, exact, row_axis, floor, abs_floor)
    e_oe = max_rel_err(oracle, exact, row_axis, floor, abs_floor)
    record_fallback(what, tol, floor, e_go, e_ge, e_oe)
    assert (e_ge <= tol or e_ge <= 1.05 * e_oe) and e_go <= tol + e_oe, "%s: gpu-vs-oracle %.3g, gpu-vs-exact %.3g, oracle-vs-exact %.3g, tol %.3g" % (
        what, e_go, e_ge, e_oe, tol)


# ---- exact (float64) restatements used only for error attribution ----------------------------------
def exact_softmax(x, log=False, scale=1.0, causal=False, period=0):
    x = np.asarray(x, np.float64) * scale
    if causal:
        r = np.arange(x.shape[0]) % period
        x = np.where(np.arange(x.shape[1])[None, :] > r[:, None], -np.inf, x)
    m = x - x.max(1, keepdims=True)
    e = np.exp(m)
    s = e.sum(1, keepdims=True)
    return m - np.log(s) if log else e / s


def exact_layernorm(x, w=None, b=None, eps=1e-5, n_cast=None, d_cast=None):
    x = np.asarray(x, np.float64)
    n = x.shape[1]
    mean = x.sum(1, keepdims=True) / (n_cast or n)
    var = ((x - mean) ** 2).sum(1, keepdims=True) / (d_cast or (n - 1))
    y = (x - mean) / np.sqrt(var + eps)
    if w is not None:
        y = y * np.asarray(w, np.float64)
    if b is not None:
        y = y + np.asarray(b, np.float64)
    return y
