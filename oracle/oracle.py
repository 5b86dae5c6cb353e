"""ctypes loader for the CPU oracle (oracle/zyx_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the bench's CPU-baseline leg may import this module; the
shipped package never does.  bf16 / f16 tensors are carried as numpy uint16 bit patterns.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libzyx_oracle.so")

BF16, F16, F32, I32 = 0, 1, 2, 10
_NP = {BF16: np.uint16, F16: np.uint16, F32: np.float32, I32: np.int32}


def build(force=False):
    src = os.path.join(_HERE, "zyx_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.zo_rng_next_f32.restype = C.c_float
        _lib.zo_rng_next_u64.restype = C.c_uint64
        _lib.zo_mse.restype = C.c_float
        _lib.zo_const_cast.restype = C.c_float
        _lib.zo_const_cast.argtypes = [C.c_int, C.c_float]
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _u64(v):
    return C.c_uint64(int(v))


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    assert a.dtype == _NP[dtype], (a.dtype, dtype)
    return a


# ---- dtype helpers -----------------------------------------------------------------------
def to_bits(x_f32, dtype):
    """f32 array -> storage array of `dtype` exactly as a store in the reference C backend."""
    x = np.ascontiguousarray(x_f32, dtype=np.float32)
    if dtype == F32:
        return x.copy()
    y = np.empty(x.shape, np.uint16)
    lib().zo_cast_from_f32(dtype, _p(x), _p(y), _u64(x.size))
    return y


def to_f32(x, dtype):
    x = np.ascontiguousarray(x)
    if dtype in (F32, I32):
        return x.astype(np.float32)
    y = np.empty(x.shape, np.float32)
    lib().zo_cast_to_f32(dtype, _p(x), _p(y), _u64(x.size))
    return y


def const_cast(dtype, v):
    return float(lib().zo_const_cast(dtype, C.c_float(v)))


# ---- rng ---------------------------------------------------------------------------------
class Rng:
    """zyx's global RNG (zyx/src/rng.rs); default seed 42069 (zyx/src/runtime.rs:178)."""

    def __init__(self, seed=42069):
        self.state = (C.c_uint64 * 4)()
        lib().zo_rng_seed(self.state, _u64(seed))

    def next_u64(self):
        return int(lib().zo_rng_next_u64(self.state))

    def rand(self, n):
        out = np.empty(n, np.float32)
        lib().zo_rand_f32(self.state, _p(out), _u64(n))
        return out

    def uniform(self, n, low, high):
        out = np.empty(n, np.float32)
        lib().zo_uniform_f32(self.state, _p(out), _u64(n), C.c_float(low), C.c_float(high))
        return out

    def randn(self, n):
        out = np.empty(n, np.float32)
        lib().zo_randn_f32(self.state, _p(out), _u64(n))
        return out

    def linear_init(self, dtype, in_f, out_f, bias=True):
        w = np.empty((out_f, in_f), _NP[dtype])
        b = np.empty((out_f,), _NP[dtype]) if bias else None
        lib().zo_linear_init(self.state, dtype, _u64(in_f), _u64(out_f), _p(w), _p(b))
        return w, b


# ---- row kernels -------------------------------------------------------------------------
RR_SUM, RR_MAX, RR_MIN, RR_MEAN, RR_VAR, RR_STD = range(6)


def row_reduce(op, dtype, x, correction=1):
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    if dtype == I32:
        y = np.empty(rows, np.int32)
        lib().zo_row_reduce_i32(op, _p(_c(x, I32)), _p(y), _u64(rows), _u64(cols))
        return y
    y = np.empty(rows, _NP[dtype])
    lib().zo_row_reduce(op, dtype, _p(_c(x, dtype)), _p(y), _u64(rows), _u64(cols), int(correction))
    return y


def softmax(dtype, x, scale=0.0, causal=False, period=0):
    x = _c(x, dtype)
    rows, cols = x.shape
    y = np.empty_like(x)
    lib().zo_softmax(dtype, _p(x), _p(y), _u64(rows), _u64(cols), C.c_float(scale), int(causal), _u64(period))
    return y


def ln_softmax(dtype, x):
    x = _c(x, dtype)
    y = np.empty_like(x)
    lib().zo_ln_softmax(dtype, _p(x), _p(y), _u64(x.shape[0]), _u64(x.shape[1]))
    return y


def layernorm(dtype, x, w=None, b=None, eps=1e-5):
    x = _c(x, dtype)
    y = np.empty_like(x)
    w = None if w is None else _c(w, dtype)
    b = None if b is None else _c(b, dtype)
    lib().zo_layernorm(dtype, _p(x), _p(w), _p(b), _p(y), _u64(x.shape[0]), _u64(x.shape[1]), C.c_float(eps))
    return y


def layernorm_bwd(dtype, x, dy, w=None, eps=1e-5):
    x, dy = _c(x, dtype), _c(dy, dtype)
    dx = np.empty_like(x)
    w = None if w is None else _c(w, dtype)
    lib().zo_layernorm_bwd(dtype, _p(x), _p(dy), _p(w), _p(dx), _u64(x.shape[0]), _u64(x.shape[1]), C.c_float(eps))
    return dx


def layernorm_dyxhat(dtype, x, dy, eps=1e-5):
    x, dy = _c(x, dtype), _c(dy, dtype)
    out = np.empty_like(x)
    lib().zo_layernorm_dyxhat(dtype, _p(x), _p(dy), _p(out), _u64(x.shape[0]), _u64(x.shape[1]), C.c_float(eps))
    return out


def softmax_bwd(dtype, p, dp):
    p, dp = _c(p, dtype), _c(dp, dtype)
    ds = np.empty_like(p)
    lib().zo_softmax_bwd(dtype, _p(p), _p(dp), _p(ds), _u64(p.shape[0]), _u64(p.shape[1]))
    return ds


def cross_entropy(logits, labels):
    logits, labels = _c(logits, F32), _c(labels, I32)
    rows, classes = logits.shape
    per = np.empty(rows, np.float32)
    mean = np.empty(1, np.float32)
    lib().zo_cross_entropy(_p(logits), _p(labels), _p(per), _p(mean), _u64(rows), _u64(classes))
    return per, mean


def cross_entropy_bwd(logits, labels):
    logits, labels = _c(logits, F32), _c(labels, I32)
    d = np.empty_like(logits)
    lib().zo_cross_entropy_bwd(_p(logits), _p(labels), _p(d), _u64(logits.shape[0]), _u64(logits.shape[1]))
    return d


def colsum(dtype, x):
    x = _c(x, dtype)
    y = np.empty(x.shape[1], _NP[dtype])
    lib().zo_colsum(dtype, _p(x), _p(y), _u64(x.shape[0]), _u64(x.shape[1]))
    return y


def mse(dtype, y, t):
    y, t = _c(y, dtype), _c(t, dtype)
    return float(lib().zo_mse(dtype, _p(y), _p(t), _u64(y.size)))


# ---- elementwise -------------------------------------------------------------------------
(EW_RELU, EW_GELU, EW_ADD, EW_SUB, EW_MUL, EW_SCALE, EW_RELU_BWD, EW_GELU_BWD, EW_MSE_BWD, EW_CAST, EW_TANH, EW_SIGMOID,
 EW_EXP, EW_BIAS_ADD) = range(14)


def eltwise(op, dtype, a, b=None, p0=0.0, dtype_out=None, cols=1):
    a = _c(a, dtype)
    b = None if b is None else np.ascontiguousarray(b)
    od = dtype_out if (op == EW_CAST and dtype_out is not None) else dtype
    y = np.empty(a.shape, _NP[od])
    lib().zo_eltwise(op, dtype, od, _p(a), _p(b), _p(y), _u64(a.size), _u64(cols), C.c_float(p0))
    return y


# ---- matmul ------------------------------------------------------------------------------
EPI_NONE, EPI_BIAS, EPI_BIAS_RELU, EPI_BIAS_GELU, EPI_MUL_RELU_GRAD, EPI_MUL_GELU_GRAD = range(6)


def gemm(dtype, a, b, ta=False, tb=False, bias=None, epi=EPI_NONE, alpha=0.0, want_preact=False):
    """a: [batch?, m, k] (or [.., k, m] when ta); b: [batch?, k, n] (or [.., n, k] when tb).
    For the MUL_*_GRAD epilogues `bias` is z, shaped like the result."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    batch = a.shape[0] if a.ndim == 3 else 1
    am, ak = (a.shape[-1], a.shape[-2]) if ta else (a.shape[-2], a.shape[-1])
    bk, bn = (b.shape[-1], b.shape[-2]) if tb else (b.shape[-2], b.shape[-1])
    assert ak == bk, (a.shape, b.shape)
    m, n, k = am, bn, ak
    shape = (batch, m, n) if a.ndim == 3 else (m, n)
    if dtype == I32:
        c = np.empty(shape, np.int32)
        lib().zo_gemm_i32(int(ta), int(tb), _u64(m), _u64(n), _u64(k), _u64(batch), _p(_c(a, I32)), _p(_c(b, I32)), _p(c))
        return c
    c = np.empty(shape, _NP[dtype])
    pre = np.empty(shape, _NP[dtype]) if want_preact else None
    sb = 0 if b.ndim == 2 else k * n
    lib().zo_gemm(dtype, int(ta), int(tb), _u64(m), _u64(n), _u64(k), _u64(batch), _p(_c(a, dtype)), _p(_c(b, dtype)),
                  _p(None if bias is None else _c(bias, dtype)), _p(c), _p(pre), C.c_int64(m * k), C.c_int64(sb),
                  C.c_int64(m * n), int(epi), C.c_float(alpha))
    return (c, pre) if want_preact else c


# ---- convolution -------------------------------------------------------------------------
def conv(dtype, x, w, bias=None, stride=1, dilation=1, padding=0):
    """Tensor::conv with groups = 1: x [n,c,h,w], w [o,c,kh,kw], bias [o] -> y [n,o,oh,ow].
    padding: int, (pad_h, pad_w) or (top, bottom, left, right)."""
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    dh, dw = (dilation, dilation) if isinstance(dilation, int) else dilation
    pad = (padding,) * 4 if isinstance(padding, int) else ((padding[0], padding[0], padding[1], padding[1]) if len(padding) == 2 else tuple(padding))
    n, c, h, wd = x.shape
    o, c2, kh, kw = w.shape
    assert c == c2, (x.shape, w.shape)
    oh = (h + pad[0] + pad[1] - dh * (kh - 1) - 1) // sh + 1
    ow = (wd + pad[2] + pad[3] - dw * (kw - 1) - 1) // sw + 1
    y = np.empty((n, o, oh, ow), _NP[dtype])
    pads = (C.c_int64 * 4)(*pad)
    lib().zo_conv(dtype, _p(_c(x, dtype)), _p(_c(w, dtype)), _p(None if bias is None else _c(bias, dtype)), _p(y), _u64(n), _u64(c), _u64(h),
                  _u64(wd), _u64(o), _u64(kh), _u64(kw), _u64(sh), _u64(sw), _u64(dh), _u64(dw), pads)
    return y


def conv_weight_grad(dtype, x, dy, w_shape, stride=1, dilation=1, padding=0):
    """Filter gradient of conv: x [n,c,h,w], dy [n,o,oh,ow] -> dw [o,c,kh,kw]."""
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    dh, dw = (dilation, dilation) if isinstance(dilation, int) else dilation
    pad = (padding,) * 4 if isinstance(padding, int) else ((padding[0], padding[0], padding[1], padding[1]) if len(padding) == 2 else tuple(padding))
    n, c, h, wd = x.shape
    o, c2, kh, kw = w_shape
    assert c == c2 and dy.shape[:2] == (n, o), (x.shape, dy.shape, w_shape)
    out = np.empty(tuple(w_shape), _NP[dtype])
    pads = (C.c_int64 * 4)(*pad)
    lib().zo_conv_wgrad(dtype, _p(_c(x, dtype)), _p(_c(dy, dtype)), _p(out), _u64(n), _u64(c), _u64(h), _u64(wd), _u64(o), _u64(kh), _u64(kw),
                        _u64(sh), _u64(sw), _u64(dh), _u64(dw), pads)
    return out


# ---- optimizers --------------------------------------------------------------------------
def sgd(dtype, p, g, buf=None, lr=0.01, wd=0.0, momentum=0.0, dampening=0.0, nesterov=False, maximize=False, first=True,
        grad_scale=1.0):
    """In place on p (and buf)."""
    lib().zo_sgd(dtype, _p(p), _p(_c(g, dtype)), _p(buf), _u64(p.size), C.c_float(lr), C.c_float(wd), C.c_float(momentum),
                 C.c_float(dampening), int(nesterov), int(maximize), int(first), C.c_float(grad_scale))


def adam(dtype, p, g, m, v, t, lr=1e-3, wd=0.0, beta1=0.9, beta2=0.999, eps=1e-8, mode=1, grad_scale=1.0):
    """In place on p, m, v.  mode: 0 Adam, 1 AdamW as the reference writes it, 2 textbook AdamW."""
    lib().zo_adam(dtype, _p(p), _p(_c(g, dtype)), _p(m), _p(v), _u64(p.size), C.c_float(lr), C.c_float(wd), C.c_float(beta1),
                  C.c_float(beta2), C.c_float(eps), _u64(t), int(mode), C.c_float(grad_scale))
