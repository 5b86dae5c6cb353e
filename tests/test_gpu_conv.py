"""Parity of the convolution program (Tensor::conv, groups = 1) with the oracle: the direct kernel (f32, i32, small
problems) and the implicit GEMM on the tensor cores (bf16 / f16), over strides, dilations, paddings and channel counts."""
import numpy as np
import pytest
import torch

from oracle import oracle as zo
from tests.parity import TOL_BF16, TOL_F32, assert_parity
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(41)


def exact_conv(x, w, b, stride, dilation, padding):
    """float64 convolution of the same stored values: the third party for error attribution."""
    pad = (padding,) * 4 if isinstance(padding, int) else ((padding[0], padding[0], padding[1], padding[1]) if len(padding) == 2 else padding)
    xt = torch.nn.functional.pad(torch.from_numpy(np.asarray(x, np.float64)), (pad[2], pad[3], pad[0], pad[1]))
    bt = None if b is None else torch.from_numpy(np.asarray(b, np.float64))
    return torch.nn.functional.conv2d(xt, torch.from_numpy(np.asarray(w, np.float64)), bt, stride=stride, dilation=dilation).numpy()


def test_reference_golden_vector(sess):
    """zyx/tests/05_misc.rs:880-888 (conv1): arange(9) as [1,1,3,3] with a 2x2 filter of ones."""
    t = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3)
    y = sess.conv(L.F32, t, np.ones((1, 1, 2, 2), np.float32))
    assert y.tolist() == [[[[8.0, 12.0], [20.0, 24.0]]]]


@pytest.mark.parametrize("stride,dilation,padding", [(1, 1, 0), (2, 1, 1), ((2, 1), (1, 2), (1, 2)), (1, 2, (0, 2, 1, 3)), (3, 1, 2)])
def test_f32_direct_kernel(sess, stride, dilation, padding):
    x = RNG.standard_normal((2, 5, 19, 23)).astype(np.float32)
    w = RNG.standard_normal((7, 5, 3, 2)).astype(np.float32)
    b = RNG.standard_normal(7).astype(np.float32)
    got = sess.conv(L.F32, x, w, b, stride, dilation, padding)
    want = zo.conv(zo.F32, x, w, b, stride, dilation, padding)
    assert got.shape == want.shape
    assert_parity(got, want, exact_conv(x, w, b, stride, dilation, padding), TOL_F32, floor=0.1, what="conv f32")


def test_i32_is_bit_exact(sess):
    x = RNG.integers(-50, 50, (2, 3, 9, 8)).astype(np.int32)
    w = RNG.integers(-9, 9, (4, 3, 3, 3)).astype(np.int32)
    b = RNG.integers(-100, 100, 4).astype(np.int32)
    got = sess.conv(L.I32, x, w, b, 2, 1, 1)
    assert np.array_equal(got, zo.conv(zo.I32, x, w, b, 2, 1, 1))
    assert np.array_equal(got, exact_conv(x, w, b, 2, 1, 1).astype(np.int64))


# (n, c, h, w, o, kh, kw, stride, dilation, padding): every case has enough work for the tensor-core path
TC_CASES = [
    (2, 64, 56, 56, 64, 3, 3, 1, 1, 1),               # a ResNet 3x3 layer: 64-wide patches, two rows each
    (1, 32, 57, 57, 96, 3, 3, 2, 1, 1),               # stride 2 through the tensor map's element strides
    (2, 3, 64, 64, 64, 7, 7, 2, 1, 3),                # 3 channels (padded to 8), 7x7 stride 2
    (3, 128, 14, 14, 256, 3, 3, 1, 1, 1),             # 256 filters per tile, 16 x 8 patches
    (1, 72, 20, 300, 40, 1, 3, 1, 2, (0, 0, 2, 2)),   # rows wider than a patch, dilation 2, channels not a multiple of 64
    (2, 40, 31, 29, 24, 3, 3, (2, 1), (1, 2), (0, 2, 1, 3)),   # mixed strides / dilations, asymmetric padding
    (1, 256, 28, 28, 128, 1, 1, 1, 1, 0),             # 1x1: a plain matmul over channels
    (4, 16, 9, 7, 512, 5, 5, 1, 1, 2),                # images smaller than a tile: a tile spans several images
    (1, 16, 12, 20, 32, 3, 3, 1, 1, (1, 1, 130, 2)),  # padding beyond the 8-bit corners of an im2col-mode map: patch mode
]


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("case", TC_CASES)
def test_implicit_gemm_on_tensor_cores(sess, dtype, case):
    n, c, h, w_, o, kh, kw, stride, dilation, padding = case
    x = zo.to_bits(RNG.standard_normal((n, c, h, w_)).astype(np.float32), dtype)
    w = zo.to_bits((RNG.standard_normal((o, c, kh, kw)) / np.sqrt(c * kh * kw)).astype(np.float32), dtype)
    b = zo.to_bits(RNG.standard_normal(o).astype(np.float32), dtype)
    before = sess.device.launch_count()
    got = sess.conv(dtype, x, w, b, stride, dilation, padding)
    assert sess.device.launch_count() - before == 3, "expected the two layout kernels and the tensor-core kernel"
    assert sess.device.status() == 0
    want = zo.conv(dtype, x, w, b, stride, dilation, padding)
    assert got.shape == want.shape
    exact = exact_conv(zo.to_f32(x, dtype), zo.to_f32(w, dtype), zo.to_f32(b, dtype), stride, dilation, padding)
    # tolerance 2e-2 relative to max(|want|, a tenth of the largest |want| along the row): sums of hundreds of products
    assert_parity(zo.to_f32(got, dtype), zo.to_f32(want, dtype), exact, TOL_BF16, floor=0.1, what="conv %s" % (case,))


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("case", [TC_CASES[0], TC_CASES[1], TC_CASES[4], TC_CASES[8], (2, 36, 20, 20, 20, 3, 3, 1, 1, 1)])
def test_channels_last_reads_and_writes_in_place(sess, dtype, case):
    """x [n,h,w,c] -> y [n,oh,ow,o]: no layout kernel when c is a multiple of 8 (two launches), and the same values as the
    channels-first oracle on the transposed tensors.  The last case (c = 36, o = 20) takes the direct kernel."""
    n, c, h, w_, o, kh, kw, stride, dilation, padding = case
    x = zo.to_bits(RNG.standard_normal((n, c, h, w_)).astype(np.float32), dtype)
    w = zo.to_bits((RNG.standard_normal((o, c, kh, kw)) / np.sqrt(c * kh * kw)).astype(np.float32), dtype)
    b = zo.to_bits(RNG.standard_normal(o).astype(np.float32), dtype)
    before = sess.device.launch_count()
    got = sess.conv(dtype, np.ascontiguousarray(x.transpose(0, 2, 3, 1)), w, b, stride, dilation, padding, channels_last=True)
    assert sess.device.launch_count() - before == (2 if c % 8 == 0 else 1)
    assert sess.device.status() == 0
    want = zo.conv(dtype, x, w, b, stride, dilation, padding)
    assert got.shape == tuple(np.array(want.shape)[[0, 2, 3, 1]])
    exact = exact_conv(zo.to_f32(x, dtype), zo.to_f32(w, dtype), zo.to_f32(b, dtype), stride, dilation, padding)
    assert_parity(zo.to_f32(got, dtype).transpose(0, 3, 1, 2), zo.to_f32(want, dtype), exact, TOL_BF16, floor=0.1, what="conv nhwc %s" % (case,))


def test_channels_last_f32_and_i32(sess):
    x = RNG.integers(-50, 50, (2, 3, 9, 8)).astype(np.int32)
    w = RNG.integers(-9, 9, (4, 3, 3, 3)).astype(np.int32)
    got = sess.conv(L.I32, np.ascontiguousarray(x.transpose(0, 2, 3, 1)), w, None, 2, 1, 1, channels_last=True)
    assert np.array_equal(got.transpose(0, 3, 1, 2), zo.conv(zo.I32, x, w, None, 2, 1, 1))
    xf = RNG.standard_normal((2, 5, 11, 7)).astype(np.float32)
    wf = RNG.standard_normal((6, 5, 3, 3)).astype(np.float32)
    got = sess.conv(L.F32, np.ascontiguousarray(xf.transpose(0, 2, 3, 1)), wf, None, 1, 1, 1, channels_last=True)
    assert_parity(got.transpose(0, 3, 1, 2), zo.conv(zo.F32, xf, wf, None, 1, 1, 1), exact_conv(xf, wf, None, 1, 1, 1), TOL_F32, floor=0.1, what="conv nhwc f32")


def test_without_bias_and_small_problem_takes_the_direct_kernel(sess):
    x = zo.to_bits(RNG.standard_normal((1, 4, 8, 8)).astype(np.float32), L.BF16)
    w = zo.to_bits(RNG.standard_normal((4, 4, 3, 3)).astype(np.float32), L.BF16)
    before = sess.device.launch_count()
    got = sess.conv(L.BF16, x, w, None, 1, 1, 1)
    assert sess.device.launch_count() - before == 1
    want = zo.conv(zo.BF16, x, w, None, 1, 1, 1)
    exact = exact_conv(zo.to_f32(x, L.BF16), zo.to_f32(w, L.BF16), None, 1, 1, 1)
    assert_parity(zo.to_f32(got, L.BF16), zo.to_f32(want, L.BF16), exact, TOL_BF16, floor=0.1, what="conv direct bf16")


def test_bad_arguments_are_errors(sess):
    from zyx_b200 import backend as B
    with pytest.raises(B.BackendError):
        sess.device.create_program(B.conv_desc(L.F32, (1, 1, 2, 2), (1, 1, 3, 3)))      # filter larger than the input
    with pytest.raises(B.BackendError):
        sess.device.create_program(B.conv_desc(L.F64, (1, 1, 4, 4), (1, 1, 3, 3)))


@pytest.mark.parametrize("dtype", [L.BF16, L.F32])
@pytest.mark.parametrize("case", [(2, 64, 28, 28, 96, 3, 3, 1, 1), (1, 32, 20, 24, 48, 3, 2, 2, (2, 1, 0, 2)), (1, 4, 9, 9, 6, 2, 3, 1, (0, 1, 2, 0))])
def test_input_gradient_of_a_stride_one_convolution(sess, dtype, case):
    """flip_filter: dx = conv(dy, filter transposed in (o, c) and reversed in (r, s), padding d*(k-1) - p), read from the
    forward filter's buffer as it is.  Held against the oracle's convolution with an explicitly flipped filter, and
    against autograd in float64."""
    n, c, h, w_, o, kh, kw, dil, padding = case
    pads = (padding,) * 4 if isinstance(padding, int) else padding
    oh, ow = h + pads[0] + pads[1] - dil * (kh - 1), w_ + pads[2] + pads[3] - dil * (kw - 1)
    wt = zo.to_bits((RNG.standard_normal((o, c, kh, kw)) / np.sqrt(o * kh * kw)).astype(np.float32), dtype)
    dy = zo.to_bits(RNG.standard_normal((n, o, oh, ow)).astype(np.float32), dtype)
    got = sess.conv_input_grad(dtype, dy, wt, (h, w_), 1, dil, padding)
    assert got.shape == (n, c, h, w_)
    flipped = np.ascontiguousarray(wt.transpose(1, 0, 2, 3)[:, :, ::-1, ::-1])
    back = (dil * (kh - 1) - pads[0], dil * (kh - 1) - pads[1], dil * (kw - 1) - pads[2], dil * (kw - 1) - pads[3])
    want = zo.conv(dtype, dy, flipped, None, 1, dil, back)
    x = torch.zeros((n, c, h, w_), dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.conv2d(torch.nn.functional.pad(x, (pads[2], pads[3], pads[0], pads[1])),
                                   torch.from_numpy(zo.to_f32(wt, dtype).astype(np.float64)), dilation=dil)
    y.backward(torch.from_numpy(zo.to_f32(dy, dtype).astype(np.float64)))
    exact = x.grad.numpy()
    tol = TOL_F32 if dtype == L.F32 else TOL_BF16
    assert_parity(zo.to_f32(got, dtype), zo.to_f32(want, dtype), exact, tol, floor=0.1, what="conv dgrad %s" % (case,))


def exact_weight_grad(x, dy, w_shape, stride, dilation, padding):
    pad = (padding,) * 4 if isinstance(padding, int) else ((padding[0], padding[0], padding[1], padding[1]) if len(padding) == 2 else padding)
    w = torch.zeros(tuple(w_shape), dtype=torch.float64, requires_grad=True)
    xt = torch.nn.functional.pad(torch.from_numpy(np.asarray(x, np.float64)), (pad[2], pad[3], pad[0], pad[1]))
    torch.nn.functional.conv2d(xt, w, stride=stride, dilation=dilation).backward(torch.from_numpy(np.asarray(dy, np.float64)))
    return w.grad.numpy()


WG_CASES = [
    (2, 64, 28, 28, 64, 3, 3, 1, 1, 1),                # 1568 positions, one 128 x 128 tile per tap
    (2, 160, 20, 20, 200, 3, 3, 1, 1, 1),              # two filter blocks, 256-wide channel block with a ragged tail
    (3, 24, 33, 31, 40, 3, 2, (2, 1), (1, 2), (1, 0, 2, 1)),   # strides, dilations, asymmetric padding, odd plane
    (16, 8, 32, 32, 8, 5, 5, 2, 1, 2),                 # one chunk of 64 in each operand mostly empty
    (4, 128, 14, 14, 128, 1, 1, 1, 1, 0),              # 1x1
]


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("case", WG_CASES)
def test_weight_gradient_on_tensor_cores(sess, dtype, case):
    n, c, h, w_, o, kh, kw, stride, dilation, padding = case
    from zyx_b200 import backend as B
    shape = B.conv_out_shape((n, c, h, w_), (o, c, kh, kw), stride, dilation, padding)
    x = zo.to_bits(RNG.standard_normal((n, c, h, w_)).astype(np.float32), dtype)
    dy = zo.to_bits((RNG.standard_normal(shape) / np.sqrt(shape[0] * shape[2] * shape[3])).astype(np.float32), dtype)
    before = sess.device.launch_count()
    got = sess.conv_weight_grad(dtype, x, dy, (o, c, kh, kw), stride, dilation, padding)
    assert sess.device.launch_count() - before == 4, "expected two layout kernels, the tensor-core kernel and the split sum"
    assert sess.device.status() == 0
    want = zo.conv_weight_grad(dtype, x, dy, (o, c, kh, kw), stride, dilation, padding)
    exact = exact_weight_grad(zo.to_f32(x, dtype), zo.to_f32(dy, dtype), (o, c, kh, kw), stride, dilation, padding)
    # sums over thousands of positions: measured per filter [c*kh*kw] against a tenth of its largest entry
    g, w, e = (a.reshape(o, -1) for a in (zo.to_f32(got, dtype), zo.to_f32(want, dtype), exact))
    assert_parity(g, w, e, TOL_BF16, floor=0.1, what="conv wgrad %s" % (case,))
    if c % 8 == 0 and o % 8 == 0:
        got_cl = sess.conv_weight_grad(dtype, np.ascontiguousarray(x.transpose(0, 2, 3, 1)), np.ascontiguousarray(dy.transpose(0, 2, 3, 1)),
                                       (o, c, kh, kw), stride, dilation, padding, channels_last=True)
        assert np.array_equal(got_cl, got)                 # the same tiles, the same order of sums


def test_weight_gradient_direct_kernel(sess):
    x = RNG.integers(-20, 20, (2, 3, 9, 8)).astype(np.int32)
    dy = RNG.integers(-9, 9, (2, 4, 5, 4)).astype(np.int32)
    got = sess.conv_weight_grad(L.I32, x, dy, (4, 3, 3, 3), 2, 1, 1)
    assert np.array_equal(got, zo.conv_weight_grad(zo.I32, x, dy, (4, 3, 3, 3), 2, 1, 1))
    assert np.array_equal(got, exact_weight_grad(x, dy, (4, 3, 3, 3), 2, 1, 1).astype(np.int64))
    xf = RNG.standard_normal((2, 5, 11, 7)).astype(np.float32)
    dyf = RNG.standard_normal((2, 6, 11, 7)).astype(np.float32)
    got = sess.conv_weight_grad(L.F32, xf, dyf, (6, 5, 3, 3), 1, 1, 1)
    want = zo.conv_weight_grad(zo.F32, xf, dyf, (6, 5, 3, 3), 1, 1, 1)
    assert_parity(got.reshape(6, -1), want.reshape(6, -1), exact_weight_grad(xf, dyf, (6, 5, 3, 3), 1, 1, 1).reshape(6, -1), TOL_F32, floor=0.1, what="wgrad f32")
    got_cl = sess.conv_weight_grad(L.F32, np.ascontiguousarray(xf.transpose(0, 2, 3, 1)), np.ascontiguousarray(dyf.transpose(0, 2, 3, 1)), (6, 5, 3, 3), 1, 1, 1,
                                   channels_last=True)
    assert np.array_equal(got_cl, got)


@pytest.mark.parametrize("dtype", [L.BF16, L.F32, L.I32])
@pytest.mark.parametrize("channels_last", [False, True])
def test_input_gradient_with_strides_takes_the_direct_kernel(sess, dtype, channels_last):
    """Stride 2 x 3 with dilation and asymmetric padding: dx against float64 autograd (integers exactly)."""
    n, c, h, w_, o, kh, kw, stride, dil, pads = 2, 5, 13, 17, 6, 3, 2, (2, 3), (1, 2), (1, 0, 2, 1)
    from zyx_b200 import backend as B
    shape = B.conv_out_shape((n, c, h, w_), (o, c, kh, kw), stride, dil, pads)
    if dtype == L.I32:
        wt, dy = RNG.integers(-9, 9, (o, c, kh, kw)).astype(np.int32), RNG.integers(-20, 20, shape).astype(np.int32)
        f = lambda a: a
    else:
        wt = zo.to_bits(RNG.standard_normal((o, c, kh, kw)).astype(np.float32), dtype)
        dy = zo.to_bits(RNG.standard_normal(shape).astype(np.float32), dtype)
        f = lambda a: zo.to_f32(a, dtype)
    dy_in = np.ascontiguousarray(dy.transpose(0, 2, 3, 1)) if channels_last else dy
    got = sess.conv_input_grad(dtype, dy_in, wt, (h, w_), stride, dil, pads, channels_last=channels_last)
    if channels_last:
        got = got.transpose(0, 3, 1, 2)
    x = torch.zeros((n, c, h, w_), dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.conv2d(torch.nn.functional.pad(x, (pads[2], pads[3], pads[0], pads[1])), torch.from_numpy(np.asarray(f(wt), np.float64)),
                                   stride=stride, dilation=dil)
    y.backward(torch.from_numpy(np.asarray(f(dy), np.float64)))
    exact = x.grad.numpy()
    if dtype == L.I32:
        assert np.array_equal(got, exact.astype(np.int64))
    else:
        tol = TOL_F32 if dtype == L.F32 else TOL_BF16
        from tests.parity import max_rel_err
        assert max_rel_err(f(got), exact, floor=0.1) <= tol


STRIDED_DGRAD_CASES = [
    (2, 64, 56, 56, 128, 3, 3, 2, 1, 1),                          # the down-sampling 3x3 of a residual network: four phases of 1, 2, 2, 4 taps
    (4, 64, 57, 55, 128, 1, 1, 2, 1, 0),                          # 1x1 stride 2: three of the four phases have no tap (zero gradient)
    (1, 24, 64, 64, 64, 7, 7, 2, 1, 3),                           # 7x7 stride 2, 24 channels
    (6, 40, 31, 29, 24, 3, 3, (2, 1), (1, 2), (0, 2, 1, 3)),      # stride only in h, dilation only in w, asymmetric padding
    (8, 48, 30, 30, 64, 3, 3, 3, 1, 0),                           # stride = filter size: nine one-tap phases
    (4, 32, 40, 40, 64, 3, 3, 2, 2, 2),                           # stride 2 with dilation 2: only the even input positions are ever read
]


@pytest.mark.parametrize("dtype,channels_last", [(L.BF16, False), (L.BF16, True), (L.F16, False)])
@pytest.mark.parametrize("case", STRIDED_DGRAD_CASES)
def test_strided_input_gradient_on_tensor_cores(sess, dtype, channels_last, case):
    """Stride > 1: one stride-1 convolution per residue class of the input positions, each with the sub-filter of the taps
    that reach the class, written to the class's positions of dx.  Oracle: the transposed-convolution identity through the
    oracle's own convolution - dy with stride-1 zeros inserted between its elements, convolved with the filter transposed in
    (o, c) and reversed in (r, s) - and float64 autograd as the third party."""
    from zyx_b200 import backend as B
    n, c, h, w_, o, kh, kw, stride, dil, padding = case
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    dh, dw = (dil, dil) if isinstance(dil, int) else dil
    pads = (padding,) * 4 if isinstance(padding, int) else padding
    shape = B.conv_out_shape((n, c, h, w_), (o, c, kh, kw), stride, dil, pads)
    wt = zo.to_bits((RNG.standard_normal((o, c, kh, kw)) / np.sqrt(o * kh * kw)).astype(np.float32), dtype)
    dy = zo.to_bits(RNG.standard_normal(shape).astype(np.float32), dtype)
    dy_in = np.ascontiguousarray(dy.transpose(0, 2, 3, 1)) if channels_last else dy
    before = sess.device.launch_count()
    got = sess.conv_input_grad(dtype, dy_in, wt, (h, w_), stride, dil, pads, channels_last=channels_last)
    launches = sess.device.launch_count() - before
    assert sess.device.status() == 0
    if channels_last:
        got = np.ascontiguousarray(got.transpose(0, 3, 1, 2))
    assert got.shape == (n, c, h, w_)
    assert launches >= 2, "the phases launch a filter layout kernel and a matmul kernel each; the direct kernel is one launch"
    oh, ow = shape[2], shape[3]
    up = np.zeros((n, o, (oh - 1) * sh + 1, (ow - 1) * sw + 1), dy.dtype)
    up[:, :, ::sh, ::sw] = dy
    flipped = np.ascontiguousarray(wt.transpose(1, 0, 2, 3)[:, :, ::-1, ::-1])
    top, left = dh * (kh - 1) - pads[0], dw * (kw - 1) - pads[2]
    back = (top, h + pads[0] - up.shape[2], left, w_ + pads[2] - up.shape[3])
    assert min(back) >= 0
    want = zo.conv(dtype, up, flipped, None, 1, dil, back)
    x = torch.zeros((n, c, h, w_), dtype=torch.float64, requires_grad=True)
    y = torch.nn.functional.conv2d(torch.nn.functional.pad(x, (pads[2], pads[3], pads[0], pads[1])),
                                   torch.from_numpy(zo.to_f32(wt, dtype).astype(np.float64)), stride=stride, dilation=dil)
    y.backward(torch.from_numpy(zo.to_f32(dy, dtype).astype(np.float64)))
    exact = x.grad.numpy()
    assert_parity(zo.to_f32(got, dtype), zo.to_f32(want, dtype), exact, TOL_BF16, floor=0.1, what="strided conv dgrad %s" % (case,))
    never_read = exact == 0.0            # positions no window element covers
    assert np.all(zo.to_f32(got, dtype)[never_read] == 0.0)
