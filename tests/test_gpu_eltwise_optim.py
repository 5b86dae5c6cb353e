"""Parity of the elementwise and fused optimizer kernels with the CPU oracle."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, TOL_F32, assert_parity, max_rel_err, ref_is_equal
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(11)
TOL = {L.F32: TOL_F32, L.BF16: TOL_BF16, L.F16: TOL_BF16}


def rand(shape, dtype, scale=1.0):
    x = (RNG.standard_normal(shape) * scale).astype(np.float32)
    return zo.to_bits(x, dtype) if dtype != L.F32 else x


def f(x, dtype):
    return zo.to_f32(x, dtype)


def test_golden_relu(sess, golden):
    for case in golden["relu"]:
        y = sess.eltwise(L.EW_RELU, L.F32, np.asarray(case["x"], np.float32))
        assert ref_is_equal(y, np.asarray(case["y"], np.float32)), case["src"]


UNARY = [(L.EW_RELU, zo.EW_RELU), (L.EW_GELU, zo.EW_GELU), (L.EW_TANH, zo.EW_TANH), (L.EW_SIGMOID, zo.EW_SIGMOID), (L.EW_EXP, zo.EW_EXP),
         (L.EW_SCALE, zo.EW_SCALE)]
BINARY = [(L.EW_ADD, zo.EW_ADD), (L.EW_SUB, zo.EW_SUB), (L.EW_MUL, zo.EW_MUL), (L.EW_RELU_BWD, zo.EW_RELU_BWD),
          (L.EW_GELU_BWD, zo.EW_GELU_BWD), (L.EW_MSE_BWD, zo.EW_MSE_BWD)]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16])
@pytest.mark.parametrize("n", [1, 7, 1024, 4099, 1 << 20])
def test_eltwise(sess, dtype, n):
    # |x| <= 6: the tanh-by-exp GELU overflows to inf/inf = NaN near |x| = 10 in f32, in the reference as here
    # (and the reference C code is compiled with -ffast-math, which leaves inf/NaN results unspecified)
    a, b = rand((n,), dtype, 2.0), rand((n,), dtype, 2.0)
    if dtype == L.F32:
        a, b = np.clip(a, -6, 6), np.clip(b, -6, 6)
    else:
        a, b = zo.to_bits(np.clip(f(a, dtype), -6, 6), dtype), zo.to_bits(np.clip(f(b, dtype), -6, 6), dtype)
    # the tanh-by-exp formulas cancel near zero (the reference notes the instability,
    # zyx/tests/11_autograd.rs:476): compare against the scale of the whole tensor
    # The oracle is built with the reference's -ffast-math, whose vectorised expf is good to a few
    # ulp only; where it and the GPU differ by more than the tolerance the float64 value of the
    # same formula arbitrates (tests/parity.py::assert_parity).
    af64, bf64 = f(a, dtype).astype(np.float64), f(b, dtype).astype(np.float64)
    cc = lambda v: zo.const_cast(dtype, v)
    tanh = lambda u: (np.exp(u + u) - 1) / (np.exp(u + u) + 1)
    u_of = lambda x: (x + x * x * x * cc(0.044715)) * cc(0.7978845608028654)
    gelu = lambda x: x * cc(0.5) * (tanh(u_of(x)) + 1)
    dgelu = lambda x: cc(0.5) * (tanh(u_of(x)) + 1) + x * cc(0.5) * (1 - tanh(u_of(x)) ** 2) * (1 + 3 * cc(0.044715) * x * x) * cc(0.7978845608028654)
    exact_unary = {L.EW_RELU: (af64 > 0) * af64, L.EW_GELU: gelu(af64), L.EW_TANH: tanh(af64), L.EW_SIGMOID: np.exp(af64) / (np.exp(af64) + 1),
                   L.EW_EXP: np.exp(af64), L.EW_SCALE: af64 * cc(0.37)}
    exact_binary = {L.EW_ADD: af64 + bf64, L.EW_SUB: af64 - bf64, L.EW_MUL: af64 * bf64, L.EW_RELU_BWD: af64 * (bf64 > 0),
                    L.EW_GELU_BWD: af64 * dgelu(bf64), L.EW_MSE_BWD: (af64 - bf64) * 2.0 * np.float32(0.01)}
    for gop, oop in UNARY:
        got, want = f(sess.eltwise(gop, dtype, a, p0=0.37), dtype), f(zo.eltwise(oop, dtype, a, p0=0.37), dtype)
        assert_parity(got, want, exact_unary[gop], TOL[dtype], floor=3e-2, what="unary %d" % gop)
    for gop, oop in BINARY:
        got, want = f(sess.eltwise(gop, dtype, a, b, p0=0.01), dtype), f(zo.eltwise(oop, dtype, a, b, p0=0.01), dtype)
        assert_parity(got, want, exact_binary[gop], TOL[dtype], floor=3e-2, what="binary %d" % gop)


def test_relu_is_bit_exact_and_follows_the_formula(sess):
    x = np.array([-0.0, 0.0, -1.5, 2.5, 3e38, -3e38, 1e-38, -1e-38], np.float32)
    got, want = sess.eltwise(L.EW_RELU, L.F32, x), zo.eltwise(zo.EW_RELU, zo.F32, x)
    # equal as numbers: the sign of a zero product is left open by the reference's -ffast-math build
    assert np.array_equal(got, want) and np.all(got[[0, 1, 2, 5, 7]] == 0)
    assert np.array_equal(got.view(np.uint32)[[3, 4, 6]], x.view(np.uint32)[[3, 4, 6]])   # positive inputs pass through bit for bit


@pytest.mark.parametrize("src,dst", [(L.F32, L.BF16), (L.F32, L.F16), (L.BF16, L.F32), (L.F16, L.F32), (L.BF16, L.F16)])
def test_cast_truncates_like_the_reference(sess, src, dst):
    a = rand((5000,), src, 10.0)
    got = sess.eltwise(L.EW_CAST, src, a, dtype_out=dst)
    want = zo.eltwise(zo.EW_CAST, src, a, dtype_out=dst)
    assert np.array_equal(got, want)     # bit-exact: bits >> 16 for bf16, truncating f16


def test_bias_add(sess):
    for dtype in (L.F32, L.BF16):
        for rows, cols in [(3, 5), (64, 128), (100, 1000)]:
            x, b = rand((rows, cols), dtype), rand((cols,), dtype)
            got = sess.eltwise(L.EW_BIAS_ADD, dtype, x, b, cols=cols)
            want = zo.eltwise(zo.EW_BIAS_ADD, dtype, x, b, cols=cols)
            assert max_rel_err(f(got, dtype), f(want, dtype)) <= TOL[dtype]


# ---- optimizers ---------------------------------------------------------------------------------------
SIZES = [1, 7, 4096, 100480, 128, 1280 + 3]


def _tensors(dtype, with_state, n_state):
    out = []
    for n in SIZES:
        grp = [rand((n,), dtype), rand((n,), dtype, 0.1)]
        for _ in range(n_state):
            grp.append(np.zeros(n, grp[0].dtype) if not with_state else np.abs(rand((n,), dtype, 0.01)))
        out.append(grp)
    return out


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("kw", [dict(lr=0.01), dict(lr=0.01, weight_decay=0.1), dict(lr=0.05, momentum=0.9),
                                dict(lr=0.05, momentum=0.9, dampening=0.1, nesterov=True, weight_decay=0.01), dict(lr=0.01, maximize=True)])
def test_sgd_steps(sess, dtype, kw):
    mom = kw.get("momentum", 0.0) != 0.0
    gpu = _tensors(dtype, False, 1 if mom else 0)
    cpu = [[a.copy() for a in grp] for grp in gpu]
    for step in (1, 2, 3):
        for grp_g, grp_c in zip(gpu, cpu):      # fresh gradients each step, same on both sides
            g = rand(grp_g[1].shape, dtype, 0.1)
            grp_g[1][...] = g
            grp_c[1][...] = g
        sess.optim_step(kw, dtype, L.OPT_SGD, gpu, t=step)
        for grp in cpu:
            zo.sgd(dtype, grp[0], grp[1], grp[2] if mom else None, lr=kw["lr"], wd=kw.get("weight_decay", 0.0),
                   momentum=kw.get("momentum", 0.0), dampening=kw.get("dampening", 0.0), nesterov=kw.get("nesterov", False),
                   maximize=kw.get("maximize", False), first=(step == 1))
        for grp_g, grp_c in zip(gpu, cpu):
            for a, b in zip(grp_g, grp_c):
                assert max_rel_err(f(a, dtype), f(b, dtype), row_axis=0) <= TOL[dtype], (step, kw)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("algo,mode,kw", [(L.OPT_ADAMW, 1, dict(lr=1e-3, weight_decay=0.01)), (L.OPT_ADAMW, 2, dict(lr=1e-3, weight_decay=0.01, standard=True)),
                                          (L.OPT_ADAM, 0, dict(lr=1e-3, weight_decay=0.01)), (L.OPT_ADAM, 0, dict(lr=1e-3))])
def test_adam_family_steps(sess, dtype, algo, mode, kw):
    """AdamW as the reference writes it divides the step by lr (zyx-optim/src/adamw.rs:88-89);
    `standard` selects the textbook form.  Compared after 1..4 steps, state included."""
    gpu = _tensors(dtype, False, 2)
    cpu = [[a.copy() for a in grp] for grp in gpu]
    for step in (1, 2, 3, 4):
        for grp_g, grp_c in zip(gpu, cpu):
            g = rand(grp_g[1].shape, dtype, 0.1)
            grp_g[1][...] = g
            grp_c[1][...] = g
        sess.optim_step(kw, dtype, algo, gpu, t=step)
        for grp in cpu:
            zo.adam(dtype, grp[0], grp[1], grp[2], grp[3], step, lr=kw["lr"], wd=kw.get("weight_decay", 0.0), mode=mode)
        for grp_g, grp_c in zip(gpu, cpu):
            for a, b in zip(grp_g, grp_c):
                assert max_rel_err(f(a, dtype), f(b, dtype), row_axis=0) <= TOL[dtype] * (10 if dtype == L.F32 else 1), (step, kw)


def test_grad_scale_and_step_counter(sess):
    dtype = L.F32
    gpu = _tensors(dtype, False, 2)
    cpu = [[a.copy() for a in grp] for grp in gpu]
    sess.optim_step(dict(lr=1e-3, weight_decay=0.01, grad_scale=0.125, standard=True), dtype, L.OPT_ADAMW, gpu, t=1)
    for grp in cpu:
        zo.adam(dtype, grp[0], grp[1], grp[2], grp[3], 1, lr=1e-3, wd=0.01, mode=2, grad_scale=0.125)
    for grp_g, grp_c in zip(gpu, cpu):
        assert max_rel_err(grp_g[0], grp_c[0], row_axis=0) <= 1e-4
