"""Parity of the CUDA row kernels (through the C ABI) with the CPU oracle and the reference's
golden vectors.  f32: max relative error <= 1e-5; bf16/f16: <= 2e-2; integers bit-exact."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import F16_MIN_NORMAL, TOL_BF16, TOL_F32, assert_parity, exact_layernorm, exact_softmax, max_rel_err, ref_is_equal
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu

RNG = np.random.default_rng(7)
TOL = {L.F32: TOL_F32, L.BF16: TOL_BF16, L.F16: TOL_BF16}
# shapes that exercise every geometry: warp rows, CTA rows, register-resident long rows,
# the streaming form, ragged (non multiple of the vector width) and single-column rows
SHAPES = [(1, 1), (3, 2), (2, 3), (64, 10), (5, 37), (7, 255), (33, 256), (4, 1000), (9, 1024), (3, 4099), (5, 8192), (2, 16384),
          (3, 32768), (2, 40000), (2, 70001)]


def rand(shape, dtype, scale=1.0):
    x = (RNG.standard_normal(shape) * scale).astype(np.float32)
    return zo.to_bits(x, dtype) if dtype != L.F32 else x


def f(x, dtype):
    return zo.to_f32(x, dtype)


def f32(x):
    return np.asarray(x, np.float32)


# ---- golden vectors of the reference's own tests, run on the GPU path ------------------------------
def test_golden_softmax(sess, golden):
    for case in golden["softmax"]:
        assert ref_is_equal(sess.softmax(L.F32, f32(case["x"])), f32(case["y"])), case["src"]


def test_golden_layernorm(sess, golden):
    for case in golden["layernorm"]:
        y = sess.layernorm(L.F32, f32(case["x"]), w=f32(case["weight"]), eps=case["eps"])
        assert ref_is_equal(y, f32(case["y"])), case["src"]


def test_golden_cross_entropy(sess, golden):
    for case in golden["cross_entropy"]:
        logits, labels = f32(case["logits"]), np.asarray(case["labels"], np.int32)
        want = f32(case["neg_ln_softmax_times_onehot"])
        per, mean = sess.cross_entropy(logits, labels)
        assert ref_is_equal(per, want.sum(1)) and ref_is_equal(mean, [want.sum() / len(labels)])
        onehot = (labels[:, None] == np.arange(logits.shape[1])[None, :]).astype(np.float32)
        assert ref_is_equal(-sess.softmax(L.F32, logits, log=True) * onehot, want)


def test_golden_reduce(sess, golden):
    ops = {"sum": L.RR_SUM, "max": L.RR_MAX, "mean": L.RR_MEAN, "var": L.RR_VAR}
    for case in golden["reduce_f32"]:
        y = sess.row_reduce(ops[case["op"]], L.F32, f32(case["x"]), correction=case["correction"])
        assert ref_is_equal(y, f32(case["y"])), case["src"]
    for case in golden["reduce_i32"]:
        rows, cols = case["rows"], case["cols"]
        x = np.full((rows, cols), case["x_fill"], np.int32) if "x_fill" in case else \
            (np.arange(rows * cols, dtype=np.int32) + case["x_arange_from"]).reshape(rows, cols)
        assert sess.row_reduce(ops[case["op"]], L.I32, x).tolist() == case["y"], case["src"]


# ---- randomised parity against the oracle -------------------------------------------------------------
@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16])
@pytest.mark.parametrize("shape", SHAPES)
def test_softmax_and_ln_softmax(sess, dtype, shape):
    x = rand(shape, dtype, 3.0)
    xf = f(x, dtype)
    # f16 stores flush results below 2^-14 to zero: near that edge one last-bit difference decides
    # between 0 and 6.1e-5, so f16 outputs carry an absolute allowance of one minimum normal
    af = F16_MIN_NORMAL / TOL_BF16 if dtype == L.F16 else 0.0
    assert_parity(f(sess.softmax(dtype, x), dtype), f(zo.softmax(dtype, x), dtype), exact_softmax(xf), TOL[dtype], what="softmax", abs_floor=af)
    assert_parity(f(sess.softmax(dtype, x, log=True), dtype), f(zo.ln_softmax(dtype, x), dtype), exact_softmax(xf, log=True), TOL[dtype],
                  what="ln_softmax")


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_softmax_scaled_causal(sess, dtype):
    T = 96
    x = rand((4 * T, T), dtype, 4.0)
    got = f(sess.softmax(dtype, x, scale=0.125, causal=True, period=T), dtype)
    want = f(zo.softmax(dtype, x, scale=0.125, causal=True, period=T), dtype)
    assert max_rel_err(got, want) <= TOL[dtype]
    r = np.arange(4 * T) % T
    assert np.all(got[np.arange(T)[None, :] > r[:, None]] == 0.0)     # masked columns are exactly zero


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("T", [40, 96, 2048, 4100])
def test_causal_softmax_forward_backward_skip_masked_columns(sess, dtype, T):
    """Columns past the diagonal are never read: poison them with NaN bit patterns and the results must not change."""
    rows = 2 * T
    x, dp = rand((rows, T), dtype, 4.0), rand((rows, T), dtype)
    masked = np.arange(T)[None, :] > (np.arange(rows) % T)[:, None]
    p_want = zo.softmax(dtype, x, causal=True, period=T)
    ds_want = f(zo.softmax_bwd(dtype, p_want, dp), dtype)
    nan = np.float32(np.nan) if dtype == L.F32 else np.uint16(0x7fc0)
    xp, dpp = x.copy(), dp.copy()
    xp[masked], dpp[masked] = nan, nan
    p_got = sess.softmax(dtype, xp, causal=True, period=T)
    exact = exact_softmax(np.where(masked, -np.inf, f(x, dtype).astype(np.float64)))
    assert_parity(f(p_got, dtype), f(p_want, dtype), exact, TOL[dtype], what="causal softmax")
    assert np.all(f(p_got, dtype)[masked] == 0.0)
    ds_got = f(sess.softmax_bwd(dtype, p_want, dpp, causal=True, period=T), dtype)
    assert np.all(ds_got[masked] == 0.0)
    # rows just under the diagonal hold one dominant probability, so dp - sum(p*dp) cancels down to the rounding noise of
    # the f32 sum: the error is bounded relative to |dp| (order 1), not to the result, hence the absolute floor
    assert max_rel_err(ds_got, ds_want, floor=1e-2, abs_floor=5e-3) <= TOL[dtype] * (20 if dtype == L.F32 else 1)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16])
@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] >= 2])
@pytest.mark.parametrize("affine", [False, True])
def test_layernorm(sess, dtype, shape, affine):
    if dtype == L.F16 and shape[1] > 65504:
        pytest.skip("the column count itself overflows f16 (the divisor is a scalar of the tensor dtype)")
    x = rand(shape, dtype, 2.0)
    w = rand((shape[1],), dtype) if affine else None
    b = rand((shape[1],), dtype) if affine else None
    got, want = f(sess.layernorm(dtype, x, w, b, 1e-5), dtype), f(zo.layernorm(dtype, x, w, b, 1e-5), dtype)
    cc = lambda v: zo.const_cast(dtype, float(v))      # n, n-1 and eps enter as scalars of the tensor dtype
    exact = exact_layernorm(f(x, dtype), None if w is None else f(w, dtype), None if b is None else f(b, dtype), cc(1e-5),
                            cc(shape[1]), cc(shape[1] - 1))
    assert_parity(got, want, exact, TOL[dtype], what="layernorm")


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("shape", [(3, 5), (64, 10), (5, 37), (4, 1000), (3, 4099), (2, 16384), (2, 32768), (2, 70001)])
def test_backward_rows(sess, dtype, shape):
    x, dy, w = rand(shape, dtype, 2.0), rand(shape, dtype), rand((shape[1],), dtype)
    got, want = f(sess.layernorm_bwd(dtype, x, dy, w, 1e-5), dtype), f(zo.layernorm_bwd(dtype, x, dy, w, 1e-5), dtype)
    assert max_rel_err(got, want, floor=1e-2) <= TOL[dtype] * (20 if dtype == L.F32 else 1)   # three chained f32 sums
    got, want = f(sess.layernorm_dyxhat(dtype, x, dy, 1e-5), dtype), f(zo.layernorm_dyxhat(dtype, x, dy, 1e-5), dtype)
    assert max_rel_err(got, want, floor=1e-2) <= TOL[dtype] * (20 if dtype == L.F32 else 1)
    p = zo.softmax(dtype, rand(shape, dtype, 2.0))
    got, want = f(sess.softmax_bwd(dtype, p, dy), dtype), f(zo.softmax_bwd(dtype, p, dy), dtype)
    assert max_rel_err(got, want, floor=1e-2) <= TOL[dtype] * (20 if dtype == L.F32 else 1)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16])
@pytest.mark.parametrize("shape", SHAPES)
def test_scalar_reductions(sess, dtype, shape):
    if dtype == L.F16 and shape[1] > 65504:
        pytest.skip("the column count itself overflows f16 (the divisor is a scalar of the tensor dtype)")
    x = rand(shape, dtype, 2.0)
    ops = [(L.RR_SUM, zo.RR_SUM), (L.RR_MAX, zo.RR_MAX), (L.RR_MIN, zo.RR_MIN), (L.RR_MEAN, zo.RR_MEAN)]
    if shape[1] >= 2:
        ops += [(L.RR_VAR, zo.RR_VAR), (L.RR_STD, zo.RR_STD)]
    for gop, oop in ops:
        got, want = f(sess.row_reduce(gop, dtype, x), dtype), f(zo.row_reduce(oop, dtype, x), dtype)
        if gop in (L.RR_MAX, L.RR_MIN):
            assert np.array_equal(got, want)                       # order-independent: bit-exact
        else:
            # a sum is compared relative to the magnitude of what was summed
            # a sum is compared relative to the magnitude of what was summed; where the oracle's own
            # sequential f32 sum has drifted from the exact sum by more than the tolerance, the GPU
            # must be within tolerance of the exact value instead
            xf = f(x, dtype).astype(np.float64)
            n, nc, dc = shape[1], zo.const_cast(dtype, float(shape[1])), zo.const_cast(dtype, float(shape[1] - 1))
            if gop in (L.RR_SUM, L.RR_MEAN):
                exact = xf.sum(1) / (nc if gop == L.RR_MEAN else 1.0)
                scale = 100.0 * np.sqrt((xf ** 2).sum(1)) / (n if gop == L.RR_MEAN else 1)   # floor = 0.1 * |x|_2
            else:
                mean = xf.sum(1, keepdims=True) / nc
                exact = ((xf - mean) ** 2).sum(1) / dc
                exact = np.sqrt(exact) if gop == L.RR_STD else exact
                scale = np.abs(exact)
            denom = lambda ref: np.maximum(np.abs(ref), 1e-3 * np.maximum(scale, 1e-30))
            e_go = float(np.max(np.abs(got - want) / denom(want)))
            e_ge = float(np.max(np.abs(got - exact) / denom(exact)))
            e_oe = float(np.max(np.abs(want - exact) / denom(exact)))
            assert e_go <= TOL[dtype] or (e_ge <= TOL[dtype] and e_go <= TOL[dtype] + e_oe), (gop, shape, e_go, e_ge, e_oe)


@pytest.mark.parametrize("shape", SHAPES)
def test_integer_reductions_bit_exact(sess, shape):
    x = RNG.integers(-2**31, 2**31 - 1, size=shape, dtype=np.int64).astype(np.int32)
    for gop, oop in [(L.RR_SUM, zo.RR_SUM), (L.RR_MAX, zo.RR_MAX), (L.RR_MIN, zo.RR_MIN)]:
        assert np.array_equal(sess.row_reduce(gop, L.I32, x), zo.row_reduce(oop, zo.I32, x)), (gop, shape)


@pytest.mark.parametrize("shape", [(1, 2), (64, 10), (128, 1000), (3, 50257)])
def test_cross_entropy_forward_backward(sess, shape):
    logits = rand(shape, L.F32, 3.0)
    labels = RNG.integers(0, shape[1], size=shape[0]).astype(np.int32)
    per, mean = sess.cross_entropy(logits, labels)
    wper, wmean = zo.cross_entropy(logits, labels)
    ls = exact_softmax(logits, log=True)
    eper = -ls[np.arange(shape[0]), labels]
    assert_parity(per, wper, eper, TOL_F32, row_axis=0, what="ce per-sample")
    assert_parity(mean, wmean, np.array([eper.mean()]), TOL_F32, row_axis=0, what="ce mean")
    got, want = sess.cross_entropy_bwd(logits, labels), zo.cross_entropy_bwd(logits, labels)
    onehot = (labels[:, None] == np.arange(shape[1])[None, :])
    assert_parity(got, want, (exact_softmax(logits) - onehot) / shape[0], TOL_F32, what="ce backward")
    # bit-exact indexing: the only negative entry of each row sits at the label
    assert np.array_equal(np.argmin(got, axis=1), labels) or shape[1] == 1


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("shape", [(1, 1), (5, 3), (1000, 10), (64, 128), (777, 130), (4096, 4096), (300, 16384)])
def test_colsum_and_mse(sess, dtype, shape):
    x, t = rand(shape, dtype), rand(shape, dtype)
    got, want = f(sess.colsum(dtype, x), dtype), f(zo.colsum(dtype, x), dtype)
    xf = f(x, dtype).astype(np.float64)
    # a sum that cancels is measured against a tenth of the 2-norm of what was summed
    exact, scale = xf.sum(0), np.sqrt((xf ** 2).sum(0))
    denom = lambda ref: np.maximum(np.abs(ref), 1e-1 * np.maximum(scale, 1e-30))
    e_go, e_ge, e_oe = (float(np.max(np.abs(a - b) / denom(b))) for a, b in ((got, want), (got, exact), (want, exact)))
    assert e_go <= TOL[dtype] or (e_ge <= TOL[dtype] and e_go <= TOL[dtype] + e_oe), (e_go, e_ge, e_oe)
    assert abs(sess.mse(dtype, x, t) - zo.mse(dtype, x, t)) <= 1e-5 * abs(zo.mse(dtype, x, t))


def test_baseline_shape_properties(sess):
    """The [8192, 32768] f32 configuration: rows of a softmax sum to 1, a layernorm row has zero
    mean and unit (unbiased) variance, and sampled rows match the oracle."""
    rows, cols = 8192, 32768
    x = np.random.default_rng(1).standard_normal((rows, cols), dtype=np.float32)
    pick = np.array([0, 1, 17, 4095, 4096, 8190, 8191])
    y = sess.softmax(L.F32, x)
    assert np.max(np.abs(y.sum(1, dtype=np.float64) - 1.0)) < 1e-5
    assert max_rel_err(y[pick], zo.softmax(zo.F32, x[pick])) <= TOL_F32
    g, b = np.ones(cols, np.float32), np.zeros(cols, np.float32)
    z = sess.layernorm(L.F32, x, g, b, 1e-5)
    assert np.max(np.abs(z.mean(1, dtype=np.float64))) < 1e-5
    assert np.max(np.abs(z.var(1, dtype=np.float64, ddof=1) - 1.0)) < 1e-4
    assert max_rel_err(z[pick], zo.layernorm(zo.F32, x[pick], g, b, 1e-5)) <= TOL_F32


def test_bad_arguments_are_reported_not_faulted(sess):
    from zyx_b200 import BackendError
    from zyx_b200 import backend as B
    prog = sess.device.create_program(B.rowreduce_desc(L.RR_SOFTMAX, L.F32, 8, 8))
    small, _ = sess.pool.allocate(16)
    with pytest.raises(BackendError) as e:
        sess.device.launch(prog, [small, small])
    assert e.value.status_name == "IncorrectKernelArg"
    with pytest.raises(BackendError):
        sess.device.launch(prog, [small])
    with pytest.raises(BackendError) as e:
        sess.device.create_program(B.rowreduce_desc(L.RR_SOFTMAX, L.F32, 0, 8))
    assert e.value.status_name == "KernelCompilation"
    sess.pool.deallocate(small)
    sess.device.release(prog)


@pytest.mark.parametrize("dtype,cols", [(L.F32, 4096), (L.F32, 20000), (L.F32, 32768), (L.BF16, 8192), (L.BF16, 32768), (L.F16, 16384)])
def test_long_rows_staged_through_shared_memory(sess, dtype, cols):
    """Enough rows (>= 2 per SM) of 16..128 KB each select the persistent kernel that stages rows with bulk copies:
    softmax, ln_softmax, scaled + causal softmax and layernorm without affine parameters, against the oracle."""
    rows = 333
    x = rand((rows, cols), dtype, 3.0)
    xf = f(x, dtype)
    af = F16_MIN_NORMAL / TOL_BF16 if dtype == L.F16 else 0.0
    assert_parity(f(sess.softmax(dtype, x), dtype), f(zo.softmax(dtype, x), dtype), exact_softmax(xf), TOL[dtype], what="softmax", abs_floor=af)
    assert_parity(f(sess.softmax(dtype, x, log=True), dtype), f(zo.ln_softmax(dtype, x), dtype), exact_softmax(xf, log=True), TOL[dtype],
                  what="ln_softmax")
    period = 111
    got = f(sess.softmax(dtype, x, scale=0.25, causal=True, period=period), dtype)
    want = f(zo.softmax(dtype, x, scale=0.25, causal=True, period=period), dtype)
    assert max_rel_err(got, want, abs_floor=af) <= TOL[dtype]
    assert np.all(got[np.arange(cols)[None, :] > (np.arange(rows) % period)[:, None]] == 0.0)
    cc = lambda v: zo.const_cast(dtype, float(v))
    assert_parity(f(sess.layernorm(dtype, x), dtype), f(zo.layernorm(dtype, x), dtype),
                  exact_layernorm(xf, None, None, cc(1e-5), cc(cols), cc(cols - 1)), TOL[dtype], what="layernorm")
    assert sess.device.status() == 0


@pytest.mark.parametrize("dtype,shape", [(L.F32, (300, 32768)), (L.F32, (150, 8192)), (L.F32, (149, 32760)), (L.BF16, (200, 16384)),
                                         (L.F16, (160, 65536 - 16))])
def test_affine_layernorm_of_long_rows_on_cluster_pairs(sess, dtype, shape):
    """Rows of 16 .. 128 KB with weight and bias: two CTAs of a cluster share each row and combine their halves' statistics."""
    if dtype == L.F16 and shape[1] > 65504:
        pytest.skip("the column count itself overflows f16")
    x = rand(shape, dtype, 2.0)
    x[::7] = zo.to_bits(f(x[::7], dtype) + 3.0, dtype)             # rows with a mean far from zero: the halves' means differ from the row's
    w, b = rand((shape[1],), dtype), rand((shape[1],), dtype)
    got, want = f(sess.layernorm(dtype, x, w, b, 1e-5), dtype), f(zo.layernorm(dtype, x, w, b, 1e-5), dtype)
    assert sess.device.status() == 0
    cc = lambda v: zo.const_cast(dtype, float(v))
    exact = exact_layernorm(f(x, dtype), f(w, dtype), f(b, dtype), cc(1e-5), cc(shape[1]), cc(shape[1] - 1))
    assert_parity(got, want, exact, TOL[dtype], what="layernorm on cluster pairs")
