"""Parity of the matmul programs (through the C ABI) with the CPU oracle and the reference's
golden vectors.  Integer matmul is bit-exact; f32 <= 1e-5 and bf16/f16 <= 2e-2 relative to the
scale of the output row."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, TOL_F32, max_rel_err, ref_is_equal
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(13)
TOL = {L.F32: TOL_F32, L.BF16: TOL_BF16, L.F16: TOL_BF16}


def rand(shape, dtype, lo=-1.0, hi=1.0):
    x = RNG.uniform(lo, hi, size=shape).astype(np.float32)
    return zo.to_bits(x, dtype) if dtype != L.F32 else x


def f(x, dtype):
    return zo.to_f32(x, dtype)


def gemm_err(got, want, dtype):
    return max_rel_err(f(got, dtype), f(want, dtype), floor=0.1)


def test_golden_matmul(sess, golden):
    for case in golden["matmul_i32"]:
        c = sess.gemm(L.I32, np.asarray(case["a"], np.int32), np.asarray(case["b"], np.int32))
        assert c.tolist() == case["c"], case["src"]
    for case in golden["matmul_f32"]:
        c = sess.gemm(L.F32, np.asarray(case["a"], np.float32), np.asarray(case["b"], np.float32))
        assert ref_is_equal(c, np.asarray(case["c"], np.float32)), case["src"]


def test_golden_matmul_i32_procedural(sess, golden):
    g = golden["matmul_i32_procedural"]
    for m in g["m"]:
        for k in g["k"]:
            for n in g["n"]:
                x = (np.arange(m)[:, None] + np.arange(k)[None, :]).astype(np.int32)
                y = (np.arange(k)[:, None] - np.arange(n)[None, :]).astype(np.int32)
                want = (x.astype(np.int64) @ y.astype(np.int64)).astype(np.int32)
                assert np.array_equal(sess.gemm(L.I32, x, y), want), (m, k, n)


def test_golden_batched_matmul_i32_procedural(sess, golden):
    g = golden["batched_matmul_i32_procedural"]
    for b in g["b"]:
        for m in g["m"]:
            for k in g["k"]:
                for n in g["n"]:
                    bb = np.arange(b)[:, None, None]
                    x = (bb + np.arange(m)[None, :, None] + np.arange(k)[None, None, :]).astype(np.int32)
                    y = (bb + np.arange(k)[None, :, None] - np.arange(n)[None, None, :]).astype(np.int32)
                    want = np.einsum("bmk,bkn->bmn", x.astype(np.int64), y.astype(np.int64)).astype(np.int32)
                    assert np.array_equal(sess.gemm(L.I32, x, y), want), (b, m, k, n)


def test_golden_bf16_matmul(sess, golden):
    g = golden["bf16_matmul_procedural"]
    m, k, n = g["m"], g["k"], g["n"]
    xf = np.fmod(np.arange(m)[:, None] + np.arange(k)[None, :], 10).astype(np.float32)
    yf = np.fmod((np.arange(k)[:, None] - np.arange(n)[None, :]).astype(np.float32), 10).astype(np.float32)
    want = np.zeros((m, n), np.float32)
    for kk in range(k):
        want = zo.to_f32(zo.to_bits(want + xf[:, kk:kk + 1] * yf[kk:kk + 1, :], zo.BF16), zo.BF16)
    got = f(sess.gemm(L.BF16, zo.to_bits(xf, zo.BF16), zo.to_bits(yf, zo.BF16)), L.BF16)
    assert ref_is_equal(got, want, rel=0.01, abs_tol=0.001)


def test_golden_integer_mlp_forward_backward(sess, golden):
    """grad_linear_2 (zyx/tests/11_autograd.rs:409-465) through GEMM + epilogue + elementwise + colsum programs."""
    g = golden["mlp_fwd_bwd_i32"]
    a = lambda v: np.asarray(v, np.float32)
    x, y, w1, b1, w2, b2 = a([g["x"]]), a([g["y"]]), a(g["w1"]), a(g["b1"]), a(g["w2"]), a(g["b2"])
    h, z1 = sess.gemm(L.F32, x, w1, bias=b1, epi=L.EPI_BIAS_RELU, want_preact=True)
    o = sess.gemm(L.F32, h, w2, bias=b2, epi=L.EPI_BIAS)
    do = sess.eltwise(L.EW_MSE_BWD, L.F32, o, y, p0=1.0)
    dw2, db2 = sess.gemm(L.F32, h, do, ta=True), sess.colsum(L.F32, do)
    dz1 = sess.eltwise(L.EW_RELU_BWD, L.F32, sess.gemm(L.F32, do, w2, tb=True), z1)
    dw1, db1 = sess.gemm(L.F32, x, dz1, ta=True), sess.colsum(L.F32, dz1)
    assert dw1.astype(np.int64).tolist() == g["w1_grad"] and db1.astype(np.int64).tolist() == g["b1_grad"]
    assert dw2.astype(np.int64).tolist() == g["w2_grad"] and db2.astype(np.int64).tolist() == g["b2_grad"]


SHAPES = [(1, 1, 1), (2, 3, 4), (17, 19, 2), (64, 128, 784), (64, 10, 128), (128, 128, 16), (129, 131, 17), (200, 300, 100), (256, 512, 333)]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16])
@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(sess, dtype, m, n, k, ta, tb):
    a = rand((k, m) if ta else (m, k), dtype)
    b = rand((n, k) if tb else (k, n), dtype)
    assert gemm_err(sess.gemm(dtype, a, b, ta=ta, tb=tb), zo.gemm(dtype, a, b, ta=ta, tb=tb), dtype) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("epi", [L.EPI_BIAS, L.EPI_BIAS_RELU, L.EPI_BIAS_GELU])
def test_gemm_epilogues(sess, dtype, epi):
    m, n, k = 96, 160, 200
    a, w, bias = rand((m, k), dtype), rand((n, k), dtype), rand((n,), dtype)
    got, gpre = sess.gemm(dtype, a, w, tb=True, bias=bias, epi=epi, alpha=0.5, want_preact=True)
    want, wpre = zo.gemm(dtype, a, w, tb=True, bias=bias, epi=epi, alpha=0.5, want_preact=True)
    assert gemm_err(got, want, dtype) <= TOL[dtype]
    assert gemm_err(gpre, wpre, dtype) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_batched_gemm(sess, dtype):
    bsz, m, n, k = 5, 70, 50, 33
    a, b = rand((bsz, m, k), dtype), rand((bsz, k, n), dtype)
    assert gemm_err(sess.gemm(dtype, a, b), zo.gemm(dtype, a, b), dtype) <= TOL[dtype]
    bt = rand((bsz, n, k), dtype)
    assert gemm_err(sess.gemm(dtype, a, bt, tb=True, alpha=0.25), zo.gemm(dtype, a, bt, tb=True, alpha=0.25), dtype) <= TOL[dtype]
    shared = rand((k, n), dtype)        # one B for every batch (stride 0)
    assert gemm_err(sess.gemm(dtype, a, shared), zo.gemm(dtype, a, shared), dtype) <= TOL[dtype]


def test_f32_gemm_1024_against_float64(sess):
    """The reference cross-checks a 1024^3 f32 matmul against a CPU sgemm (zyx/tests/05_misc.rs:820-842)."""
    a, b = rand((1024, 1024), L.F32), rand((1024, 1024), L.F32)
    got = sess.gemm(L.F32, a, b)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert max_rel_err(got, want, floor=0.1) <= TOL_F32


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(512, 512, 256), (640, 772, 1028), (1536, 516, 4096)])
def test_f32_tensor_core_path_meets_the_f32_bar(sess, ta, tb, m, n, k):
    """Large f32 matmuls run as three TF32 tensor-core products per k-step on operands split into hi + lo, with the k-chunks
    added in f32 outside the tensor core.  The bar is the f32 one (1e-5 relative to max(|c|, 0.1 * the row's largest |c|)),
    checked against float64; plain TF32 would miss it by two orders of magnitude.  Ragged edges, all four layouts, alpha
    and bias."""
    a = rand((k, m) if ta else (m, k), L.F32)
    b = rand((n, k) if tb else (k, n), L.F32)
    bias = rand((n,), L.F32)
    af, bf = (a.T if ta else a).astype(np.float64), (b.T if tb else b).astype(np.float64)
    exact = af @ bf
    got = sess.gemm(L.F32, a, b, ta=ta, tb=tb)
    assert sess.device.status() == 0
    # the f32 bar, or - where sequential f32 accumulation itself misses it on this data - as close as the reference gets
    bar = max(TOL_F32, max_rel_err(zo.gemm(L.F32, a, b, ta=ta, tb=tb), exact, floor=0.1))
    assert max_rel_err(got, exact, floor=0.1) <= bar
    got = sess.gemm(L.F32, a, b, ta=ta, tb=tb, bias=bias, epi=L.EPI_BIAS, alpha=0.5)
    assert max_rel_err(got, 0.5 * exact + bias.astype(np.float64), floor=0.1) <= bar


def test_f32_tensor_core_path_survives_cancellation_and_scale(sess):
    """Operands spanning many binades and a product that cancels: the hi / lo split must not lose the small terms."""
    m = n = 512
    k = 2048
    a = (RNG.standard_normal((m, k)) * np.exp(RNG.uniform(-8, 8, size=(m, 1)))).astype(np.float32)
    b = RNG.standard_normal((k, n)).astype(np.float32)
    b[1::2] = -b[0::2] * (1 + 1e-3 * RNG.standard_normal((k // 2, n))).astype(np.float32)      # pairs of rows nearly cancel
    a[:, 1::2] = a[:, 0::2]
    exact = a.astype(np.float64) @ b.astype(np.float64)
    got = sess.gemm(L.F32, a, b)
    # the reference's own f32 accumulation on the same data, as the yardstick for what f32 can deliver here
    ref = zo.gemm(L.F32, a, b)
    e_got, e_ref = max_rel_err(got, exact, floor=0.1), max_rel_err(ref, exact, floor=0.1)
    assert e_got <= max(TOL_F32, 4.0 * e_ref), (e_got, e_ref)      # within a small factor of sequential f32 accumulation


@pytest.mark.parametrize("epi", [L.EPI_MUL_RELU_GRAD, L.EPI_MUL_GELU_GRAD])
def test_activation_gradient_epilogue_f32(sess, epi):
    m, n, k = 70, 50, 33
    dz, w = rand((m, k), L.F32), rand((k, n), L.F32)
    z = RNG.normal(0, 1.5, size=(m, n)).astype(np.float32)
    assert gemm_err(sess.gemm(L.F32, dz, w, bias=z, epi=epi), zo.gemm(L.F32, dz, w, bias=z, epi=epi), L.F32) <= TOL[L.F32] * 3


def test_f32_4096_cubed_sampled_rows(sess):
    """The M=N=K=4096 f32 configuration at its stated size (A, B uniform(-1, 1), seeds 2 and 3, row-major): 24 sampled rows
    against the oracle's product of the same rows (rows of A.B are independent, so the oracle on A[rows] is the oracle's
    own answer for those rows) and against float64, at the f32 bar; and C(A, -B) == -C(A, B) over the whole matrix (a
    size-independent property; the tensor core's accumulator rounding need not be symmetric, so it is held to the bar, not to bits)."""
    n = 4096
    a = np.random.default_rng(2).uniform(-1, 1, (n, n)).astype(np.float32)
    b = np.random.default_rng(3).uniform(-1, 1, (n, n)).astype(np.float32)
    got = sess.gemm(L.F32, a, b)
    assert sess.device.status() == 0
    rows = np.array([0, 1, 127, 128, 129, 255, 256, 1000, 2047, 2048, 2049, 3000, 3071, 3072, 3967, 3968, 4000, 4094, 4095, 3, 777, 1535, 1536, 2500])
    exact = a[rows].astype(np.float64) @ b.astype(np.float64)
    want = zo.gemm(L.F32, np.ascontiguousarray(a[rows]), b)
    e_ge, e_go, e_oe = (max_rel_err(got[rows], exact, floor=0.1), max_rel_err(got[rows], want, floor=0.1), max_rel_err(want, exact, floor=0.1))
    assert e_ge <= TOL_F32, (e_ge, e_go, e_oe)
    assert e_go <= TOL_F32 + e_oe, (e_ge, e_go, e_oe)        # the oracle's sequential f32 sum of 4096 terms is itself about 1e-5 from exact
    neg = sess.gemm(L.F32, a, -b)
    assert max_rel_err(neg, -got.astype(np.float64), floor=0.1) <= TOL_F32
