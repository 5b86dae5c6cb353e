"""Out-of-bounds writes, checked by the library itself: a context opened with debug bit 2 puts guard words behind every
allocation (the reference gives every buffer a spare trailing element, zyx/src/runtime.rs:622-625) and zyxb_check_guards
verifies them after every launch.  Ragged shapes - the ones whose last tile, vector or row hangs over the edge - run through
every kernel family; results are compared with the oracle as usual, and no guard word may change."""
import numpy as np
import pytest

from oracle import models as zm
from oracle import oracle as zo
from tests.parity import TOL_BF16, assert_parity, exact_layernorm, exact_softmax, max_rel_err
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def guarded():
    from zyx_b200 import build
    from zyx_b200.ops import Session
    build.build()
    s = Session(device_ids=[0], debug=2)
    assert s.check_guards
    yield s
    s.close()


def bits(rng, shape, dtype, scale=1.0):
    return zo.to_bits((rng.standard_normal(shape) * scale).astype(np.float32), dtype)


def test_matmuls_with_ragged_edges_stay_inside_their_buffers(guarded):
    rng = np.random.default_rng(41)
    for m, n, k in [(130, 260, 72), (257, 136, 200), (1, 8, 8), (129, 8, 4104), (640, 776, 1032)]:
        a, b = bits(rng, (m, k), zo.BF16), bits(rng, (k, n), zo.BF16)
        got = zo.to_f32(guarded.gemm(L.BF16, a, b), zo.BF16)
        assert max_rel_err(got, zo.to_f32(zo.gemm(zo.BF16, a, b), zo.BF16), floor=0.1) <= TOL_BF16, (m, n, k)
    for m, n, k in [(640, 772, 1028), (70, 50, 33)]:                 # f32: three-TF32 tensor-core path and the FFMA path
        a, b = rng.uniform(-1, 1, (m, k)).astype(np.float32), rng.uniform(-1, 1, (k, n)).astype(np.float32)
        assert max_rel_err(guarded.gemm(L.F32, a, b), a.astype(np.float64) @ b.astype(np.float64), floor=0.1) <= 2e-5
    a, b = rng.integers(-9, 9, (33, 17)).astype(np.int32), rng.integers(-9, 9, (17, 5)).astype(np.int32)
    assert np.array_equal(guarded.gemm(L.I32, a, b), a @ b)
    bias = bits(rng, (260,), zo.BF16)
    a, b = bits(rng, (130, 72), zo.BF16), bits(rng, (260, 72), zo.BF16)
    y, z = guarded.gemm(L.BF16, a, b, tb=True, bias=bias, epi=L.EPI_BIAS_GELU, want_preact=True)
    wy, wz = zo.gemm(zo.BF16, a, b, tb=True, bias=bias, epi=zo.EPI_BIAS_GELU, want_preact=True)
    assert max_rel_err(zo.to_f32(z, zo.BF16), zo.to_f32(wz, zo.BF16), floor=0.1) <= TOL_BF16


def test_row_eltwise_and_optimizer_kernels_stay_inside_their_buffers(guarded):
    rng = np.random.default_rng(42)
    for rows, cols in [(3, 1031), (129, 4096), (300, 32768), (5, 7), (64, 40000)]:
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        assert_parity(guarded.softmax(L.F32, x), zo.softmax(zo.F32, x), exact_softmax(x), 1e-5, what="guarded softmax")
        w, b = np.ones(cols, np.float32), np.zeros(cols, np.float32)
        assert_parity(guarded.layernorm(L.F32, x, w, b, 1e-5), zo.layernorm(zo.F32, x, w, b, 1e-5), exact_layernorm(x, w, b, 1e-5), 1e-5, what="guarded layernorm")
        xb = zo.to_bits(x, zo.BF16)
        guarded.softmax(L.BF16, xb)
        guarded.colsum(L.BF16, xb)
        guarded.row_reduce(L.RR_SUM, L.F32, x)
    for n in (1, 7, 1025, 100003):
        a = rng.standard_normal(n).astype(np.float32)
        guarded.eltwise(L.EW_GELU, L.F32, a)
        guarded.eltwise(L.EW_ADD, L.BF16, zo.to_bits(a, zo.BF16), zo.to_bits(a, zo.BF16))
        grp = [a.copy(), a.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)]
        guarded.optim_step(dict(lr=1e-3, weight_decay=0.01), L.F32, L.OPT_ADAMW, [grp], t=1)


def test_convolution_and_attention_stay_inside_their_buffers(guarded):
    rng = np.random.default_rng(43)
    x, w = bits(rng, (2, 72, 15, 17), zo.BF16), bits(rng, (136, 72, 3, 3), zo.BF16, 0.05)
    got = zo.to_f32(guarded.conv(L.BF16, x, w, None, 1, 1, 1), zo.BF16)
    want = zo.to_f32(zo.conv(zo.BF16, x, w, None, 1, 1, 1), zo.BF16)
    assert max_rel_err(got.reshape(2 * 136, -1), want.reshape(2 * 136, -1), floor=0.1) <= TOL_BF16
    dy = bits(rng, got.shape, zo.BF16)
    guarded.conv_weight_grad(L.BF16, x, dy, w.shape, 1, 1, 1)
    guarded.conv_input_grad(L.BF16, dy, w, (15, 17), 1, 1, 1)
    guarded.conv(L.BF16, x, w, None, 2, 1, 1)                        # stride 2: the direct kernel for the gradient
    q, k, v, do = (bits(rng, (1, 384, 256), zo.BF16) for _ in range(4))
    o, lse = guarded.attention(L.BF16, q, k, v, 2, causal=True)
    want_o, _, exact = zm.attention(zo.BF16, q, k, v, 2, True)
    assert max_rel_err(zo.to_f32(o, zo.BF16), exact, floor=1.0) <= TOL_BF16
    guarded.attention_bwd(L.BF16, q, k, v, o, do, lse, 2, causal=True)
    assert guarded.device.status() == 0


def test_an_unguarded_context_says_so(sess):
    from zyx_b200 import backend as B
    with pytest.raises(B.BackendError) as e:
        sess.device.check_guards()
    assert "debug bit 2" in e.value.context
