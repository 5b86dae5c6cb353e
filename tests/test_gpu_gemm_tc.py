"""Parity of the tensor-core (tcgen05 / TMEM / TMA) matmul with the CPU oracle: every operand
layout, both 16-bit dtypes, ragged edges, epilogues, batches; and the 8192^3 bf16 configuration
checked on sampled rows against float64."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, max_rel_err
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(17)


def rand(shape, dtype):
    return zo.to_bits(RNG.uniform(-1, 1, size=shape).astype(np.float32), dtype)


def f(x, dtype):
    return zo.to_f32(x, dtype)


def err(got, want, dtype):
    return max_rel_err(f(got, dtype), f(want, dtype), floor=0.1)


def test_status_word_is_clear(sess):
    assert sess.device.status() == 0


# m, n, k: multiples of the tile, ragged in every dimension, n <= 128 (the 128-wide tile), k below one k-block
SHAPES = [(128, 256, 64), (256, 512, 320), (130, 264, 72), (384, 128, 256), (200, 96, 136), (1024, 1024, 1024), (64, 2048, 40), (4096, 16, 512)]


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, False), (True, True)])
def test_tc_layouts(sess, dtype, m, n, k, ta, tb):
    if (ta and m % 8) or ((not ta) and k % 8) or (tb and k % 8) or ((not tb) and n % 8):
        pytest.skip("row pitch not a multiple of 16 bytes: served by the SIMT kernel")
    a = rand((k, m) if ta else (m, k), dtype)
    b = rand((n, k) if tb else (k, n), dtype)
    got = sess.gemm(dtype, a, b, ta=ta, tb=tb)
    assert sess.device.status() == 0
    assert err(got, zo.gemm(dtype, a, b, ta=ta, tb=tb), dtype) <= TOL_BF16


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("epi", [L.EPI_NONE, L.EPI_BIAS, L.EPI_BIAS_RELU, L.EPI_BIAS_GELU])
def test_tc_epilogues(sess, dtype, epi):
    m, n, k = 192, 328, 264
    a, w = rand((m, k), dtype), rand((n, k), dtype)
    bias = rand((n,), dtype) if epi != L.EPI_NONE else None
    got, gpre = sess.gemm(dtype, a, w, tb=True, bias=bias, epi=epi, alpha=0.25, want_preact=True)
    want, wpre = zo.gemm(dtype, a, w, tb=True, bias=bias, epi=epi, alpha=0.25, want_preact=True)
    assert err(got, want, dtype) <= TOL_BF16 and err(gpre, wpre, dtype) <= TOL_BF16


def test_tc_mostly_bit_identical_with_truncating_stores(sess):
    """Both sides accumulate exact products in f32 and truncate to bf16: apart from sums that land
    on opposite sides of a bf16 boundary because of the summation order, results are identical."""
    a, b = rand((256, 512), L.BF16), rand((384, 512), L.BF16)
    got, want = sess.gemm(L.BF16, a, b, tb=True), zo.gemm(L.BF16, a, b, tb=True)
    assert np.mean(got == want) > 0.97
    big = np.abs(f(want, L.BF16)) >= 0.1 * np.abs(f(want, L.BF16)).max(1, keepdims=True)   # sums that did not cancel
    assert np.max(np.abs(got.astype(np.int32) - want.astype(np.int32))[big]) <= 1          # differ by at most one bf16 ulp


@pytest.mark.parametrize("dtype", [L.BF16])
def test_tc_batched(sess, dtype):
    bsz, m, n, k = 6, 256, 136, 128
    a, b = rand((bsz, m, k), dtype), rand((bsz, n, k), dtype)
    assert err(sess.gemm(dtype, a, b, tb=True, alpha=0.088), zo.gemm(dtype, a, b, tb=True, alpha=0.088), dtype) <= TOL_BF16
    b2 = rand((bsz, k, n), dtype)
    assert err(sess.gemm(dtype, a, b2), zo.gemm(dtype, a, b2), dtype) <= TOL_BF16
    shared = rand((k, n), dtype)
    assert err(sess.gemm(dtype, a, shared), zo.gemm(dtype, a, shared), dtype) <= TOL_BF16


def test_tc_8192_cubed_sampled_rows(sess):
    """The M=N=K=8192 bf16 configuration: 24 sampled rows against a float64 product of the same bf16 inputs,
    and linearity C(A, B) + C(A, -B) == 0 exactly (a size-independent property of truncating stores)."""
    n = 8192
    rng = np.random.default_rng(2)
    a = zo.to_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32), zo.BF16)
    b = zo.to_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32), zo.BF16)
    got = sess.gemm(L.BF16, a, b)
    assert sess.device.status() == 0
    rows = np.array([0, 1, 127, 128, 129, 255, 256, 1000, 2047, 2048, 4095, 4096, 4097, 5000, 6143, 6144, 7000, 8000, 8063, 8064, 8190, 8191, 3, 777])
    want = f(a[rows], zo.BF16).astype(np.float64) @ f(b, zo.BF16).astype(np.float64)
    assert max_rel_err(f(got[rows], zo.BF16), want, floor=0.1) <= TOL_BF16
    neg = sess.gemm(L.BF16, a, b ^ np.uint16(0x8000))
    assert np.array_equal(neg, got ^ np.uint16(0x8000)) or np.array_equal(f(neg, zo.BF16), -f(got, zo.BF16))


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("epi", [L.EPI_MUL_RELU_GRAD, L.EPI_MUL_GELU_GRAD])
def test_tc_activation_gradient_epilogue(sess, dtype, epi):
    """dZ_prev = (dZ . W) * act'(z): the input-gradient matmul with the activation's adjoint in its epilogue."""
    m, n, k = 192, 264, 136
    dz, w = rand((m, k), dtype), rand((k, n), dtype)
    z = zo.to_bits(RNG.normal(0, 1.5, size=(m, n)).astype(np.float32), dtype)
    got = sess.gemm(dtype, dz, w, bias=z, epi=epi)
    want = zo.gemm(dtype, dz, w, bias=z, epi=epi)
    assert err(got, want, dtype) <= TOL_BF16


@pytest.mark.parametrize("dtype,T,D", [(L.BF16, 256, 64), (L.BF16, 200, 128), (L.F32, 48, 16)])
def test_attention_shaped_strided_batches(sess, dtype, T, D):
    """q, k, v live as [B, T, H*D] (what the q/k/v projections write); the per-head matmuls read them in place through
    row pitches and a two-level batch (B, H), and the P.V product writes straight back into [B, T, H*D]:
    the reshapes and transposes of MultiheadAttention::forward (zyx-nn/src/multi_head_attention.rs:160-226) without a copy."""
    from zyx_b200 import backend as Bk
    Bsz, H = 2, 4
    E = H * D
    mk = (lambda shape: rand(shape, dtype)) if dtype != L.F32 else (lambda shape: RNG.uniform(-1, 1, size=shape).astype(np.float32))
    tof = (lambda x: f(x, dtype)) if dtype != L.F32 else (lambda x: x)
    tol = TOL_BF16 if dtype != L.F32 else 1e-5
    q, k, v = mk((Bsz, T, E)), mk((Bsz, T, E)), mk((Bsz, T, E))
    heads = lambda x: np.ascontiguousarray(x.reshape(Bsz, T, H, D).transpose(0, 2, 1, 3)).reshape(Bsz * H, T, D)
    scale = 1.0 / np.sqrt(D)
    # scores[b, h] = q[b, :, h, :] . k[b, :, h, :]^T * scale  -> [B*H, T, T] packed
    d = Bk.gemm_desc(dtype, T, T, D, batch=Bsz, trans_b=True, stride_a=T * E, stride_b=T * E, stride_c=H * T * T, alpha=scale,
                     lda=E, ldb=E, batch_inner=H, stride_a_inner=D, stride_b_inner=D, stride_c_inner=T * T)
    s_got = sess.run(d, [q, k], [((Bsz * H, T, T), q.dtype)])[0]
    s_want = zo.gemm(dtype, heads(q), heads(k), tb=True, alpha=scale)
    assert max_rel_err(tof(s_got), tof(s_want), floor=0.1) <= tol
    # out[b, :, h, :] = p[b, h] . v[b, :, h, :]   -> written into [B, T, H*D]
    p = zo.softmax(dtype, s_want.reshape(-1, T)).reshape(Bsz * H, T, T)
    d = Bk.gemm_desc(dtype, T, D, T, batch=Bsz, stride_a=H * T * T, stride_b=T * E, stride_c=T * E, ldb=E, ldc=E, batch_inner=H,
                     stride_a_inner=T * T, stride_b_inner=D, stride_c_inner=D)
    o_got = sess.run(d, [p, v], [((Bsz, T, E), q.dtype)])[0]
    o_want = zo.gemm(dtype, p, heads(v)).reshape(Bsz, H, T, D).transpose(0, 2, 1, 3).reshape(Bsz, T, E)
    assert max_rel_err(tof(o_got), tof(o_want), floor=0.1) <= tol
    # dV[b, :, h, :] = p[b, h]^T . dO[b, :, h, :]: transposed A, strided B and C
    do = mk((Bsz, T, E))
    d = Bk.gemm_desc(dtype, T, D, T, batch=Bsz, trans_a=True, stride_a=H * T * T, stride_b=T * E, stride_c=T * E, ldb=E, ldc=E,
                     batch_inner=H, stride_a_inner=T * T, stride_b_inner=D, stride_c_inner=D)
    dv_got = sess.run(d, [p, do], [((Bsz, T, E), q.dtype)])[0]
    dv_want = zo.gemm(dtype, p, heads(do), ta=True).reshape(Bsz, H, T, D).transpose(0, 2, 1, 3).reshape(Bsz, T, E)
    assert max_rel_err(tof(dv_got), tof(dv_want), floor=0.1) <= tol
    assert sess.device.status() == 0


def test_residual_add_epilogue(sess):
    m, n, k = 256, 264, 128
    a, w, r = rand((m, k), L.BF16), rand((n, k), L.BF16), rand((m, n), L.BF16)
    got = sess.gemm(L.BF16, a, w, tb=True, bias=r, epi=L.EPI_ADD)
    acc = f(a, L.BF16).astype(np.float64) @ f(w, L.BF16).astype(np.float64).T + f(r, L.BF16)
    assert max_rel_err(f(got, L.BF16), acc, floor=0.1) <= TOL_BF16


# ---- causal (lower-triangular) structure ---------------------------------------------------------------
@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("T,d", [(128, 64), (384, 128), (1024, 128), (520, 72)])
def test_tc_triangular_modes(sess, dtype, T, d):
    """The three declarations a causal attention makes: results equal the plain matmul wherever they are defined."""
    batch = 3
    q, k = rand((batch, T, d), dtype), rand((batch, T, d), dtype)
    # OUT_LOWER: scores = q.k^T; entries on and below the diagonal are defined, tiles wholly above it keep the buffer's content
    sentinel = np.full((batch, T, T), 0x4321, np.uint16)
    got = sess.gemm(dtype, q, k, tb=True, alpha=0.125, tri=L.TRI_OUT_LOWER, out_init=sentinel)
    want = zo.gemm(dtype, q, k, tb=True, alpha=0.125)
    lower = np.tril(np.ones((T, T), bool))
    assert max_rel_err(np.where(lower, f(got, dtype), 0.0), np.where(lower, f(want, dtype), 0.0), floor=0.1) <= TOL_BF16
    if T >= 384:   # a 128 x 256 tile wholly above the diagonal exists and was left alone
        assert np.all(got[:, :128, 256:] == 0x4321)
    # A_LOWER: p.v with p zero above the diagonal (k range cut per row tile)
    p = np.where(lower, rand((batch, T, T), dtype), np.uint16(0)).astype(np.uint16)
    nan = np.uint16(0x7fc0 if dtype == L.BF16 else 0x7e00)
    v = rand((batch, T, d), dtype)
    want = zo.gemm(dtype, p, v)
    assert err(sess.gemm(dtype, p, v, tri=L.TRI_A_LOWER), want, dtype) <= TOL_BF16
    if T % 128 == 0 and T > 128:   # whole k-blocks right of the diagonal tile are not even read: NaN there changes nothing
        poisoned = p.copy()
        for r0 in range(0, T, 128):
            poisoned[:, r0:r0 + 128, r0 + 128:] = nan
        assert err(sess.gemm(dtype, poisoned, v, tri=L.TRI_A_LOWER), want, dtype) <= TOL_BF16
    # AT_LOWER: p^T.dO (k range starts at the row tile)
    want = zo.gemm(dtype, p, v, ta=True)
    assert err(sess.gemm(dtype, p, v, ta=True, tri=L.TRI_AT_LOWER), want, dtype) <= TOL_BF16
    assert sess.device.status() == 0


def test_triangular_declarations_are_validated(sess):
    from zyx_b200 import backend as B
    for kw in (dict(m=128, n=256, k=64, tri=L.TRI_OUT_LOWER), dict(m=128, n=64, k=256, tri=L.TRI_A_LOWER),
               dict(m=128, n=64, k=128, tri=L.TRI_AT_LOWER), dict(m=128, n=64, k=128, tri=L.TRI_A_LOWER, trans_a=True), dict(m=8, n=8, k=8, tri=7)):
        with pytest.raises(B.BackendError):
            sess.device.create_program(B.gemm_desc(L.BF16, **kw))
