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


def max_rel_err(got, want, row_axis=-1, floor=1e-2):
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
    denom = np.maximum(np.abs(want), floor * scale)
    denom = np.where(denom == 0, 1.0, denom)
    err = np.abs(got - want) / denom
    err = np.where(np.isnan(got) & np.isnan(want), 0.0, err)
    return float(np.max(err))
