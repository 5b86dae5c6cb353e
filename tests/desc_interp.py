"""TEST INFRASTRUCTURE: what a kernel descriptor means, in numpy float64, and a mirror graph that carries values.

`ValGraph` is the matcher's mirror graph (zyx_b200.matcher.MGraph) with a value per class, computed node by node as the graph is
built (leaves get seeded random values): the value of a class is what zyx's graph semantics say it is, independent of any
program.  `run_match` executes a matched program the way its descriptor reads (include/zyxb.h) on the flat values of the matched
input classes - row pitches, batch strides, argument offsets, transposition flags, epilogues, optimizer hyper-parameters and step
- and returns the flat outputs.  tests/test_matcher_semantics.py holds the two against each other for every match of a graph:
a pattern that picks the wrong operand, stride, flag or constant computes something else than the subgraph it replaces.

Float casts do not round here (values stay float64 whatever the class dtype says), so the comparison is about structure, not
about rounding; the rounding of the real kernels is the business of the GPU parity tests."""
import math

import numpy as np

from zyx_b200 import _lib as L
from zyx_b200 import matcher as M

_FLOATS = (L.F32, L.BF16, L.F16, L.F64)


class ValGraph(M.MGraph):
    def __init__(self, seed=0):
        super().__init__()
        self.vals = {}
        self.rng = np.random.default_rng(seed)
        self.int_high = 10                      # integer leaves are class indices below this
        self.scale = 0.5                        # float leaves are scale * N(0, 1) ...
        self.positive = False                   # ... or their absolute values (second moments, variances)

    def _set(self, cls, value):
        self.vals.setdefault(cls, np.asarray(value))
        return cls

    def const(self, dtype, value):
        return self._set(super().const(dtype, value), np.float64(value) if dtype in _FLOATS else np.int64(value))

    def leaf(self, dtype, shape):
        cls = super().leaf(dtype, shape)
        if dtype in _FLOATS:
            value = self.scale * self.rng.standard_normal(shape)
            value = np.abs(value) if self.positive else value
        else:
            value = self.rng.integers(0, self.int_high, shape).astype(np.int64)
        return self._set(cls, value)

    def expand(self, x, shape):
        return self._set(super().expand(x, shape), np.broadcast_to(self.vals[x], tuple(shape)).copy())

    def reshape(self, x, shape):
        return self._set(super().reshape(x, shape), self.vals[x].reshape(tuple(shape)))

    def permute(self, x, axes):
        return self._set(super().permute(x, axes), np.transpose(self.vals[x], axes))

    def pad(self, x, axis, lp, length):
        cls = super().pad(x, axis, lp, length)
        src = self.vals[x]
        shape = list(src.shape)
        shape[axis] = length
        out = np.zeros(shape, src.dtype)
        lo, hi = max(lp, 0), min(lp + src.shape[axis], length)          # destination range that holds source elements
        dst = [slice(None)] * len(shape)
        take = [slice(None)] * len(shape)
        dst[axis], take[axis] = slice(lo, hi), slice(lo - lp, hi - lp)
        out[tuple(dst)] = src[tuple(take)]
        return self._set(cls, out)

    def reduce(self, x, rop, axes):
        fn = {M.B_ADD: np.add, M.B_MAX: np.maximum, M.B_MUL: np.multiply}[rop]
        return self._set(super().reduce(x, rop, axes), fn.reduce(self.vals[x], axis=tuple(axes)))

    def cast(self, x, dtype):
        v = self.vals[x]
        if dtype in _FLOATS:
            out = v.astype(np.float64)
        elif dtype == L.BOOL:
            out = v != 0
        else:
            out = np.trunc(v).astype(np.int64)
        return self._set(super().cast(x, dtype), out)

    def unary(self, x, uop):
        v = self.vals[x]
        fn = {M.U_NEG: np.negative, M.U_BITNOT: np.invert, M.U_EXP: np.exp, M.U_EXP2: np.exp2, M.U_LN: np.log, M.U_LOG2: np.log2,
              M.U_RECIPROCAL: np.reciprocal, M.U_SQRT: np.sqrt, M.U_SIN: np.sin, M.U_COS: np.cos, M.U_FLOOR: np.floor,
              M.U_TRUNC: np.trunc, M.U_ABS: np.abs}[uop]
        return self._set(super().unary(x, uop), fn(v))

    def binary(self, x, y, bop):
        a, b = self.vals[x], self.vals[y]
        if bop == M.B_DIV:
            out = a / b if a.dtype.kind == "f" else np.trunc(a / b).astype(np.int64)
        else:
            out = {M.B_ADD: np.add, M.B_SUB: np.subtract, M.B_MUL: np.multiply, M.B_POW: np.power, M.B_MOD: np.fmod,
                   M.B_CMPLT: np.less, M.B_CMPGT: np.greater, M.B_CMPGE: np.greater_equal, M.B_MAX: np.maximum,
                   M.B_NOTEQ: np.not_equal, M.B_EQ: np.equal}[bop](a, b)
        return self._set(super().binary(x, y, bop), out)


def _gelu(x):
    e = np.exp(2.0 * (x + 0.044715 * x * x * x) * math.sqrt(2.0 / math.pi))
    return x * 0.5 * ((e - 1.0) / (e + 1.0) + 1.0)


def _softmax(x):
    e = np.exp(x - x.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def _gemm(d, ins, offsets, out_numel):
    a, b = ins[0], ins[1]
    extra = ins[2] if len(ins) > 2 else None
    inner = max(int(d.batch_inner), 1)

    def window(rows, cols, ld, base):
        return base + np.arange(rows)[:, None] * (ld or cols) + np.arange(cols)[None, :]

    c = np.zeros(out_numel[0])
    pre = np.zeros(out_numel[1]) if d.store_preact else None
    alpha = d.alpha if d.alpha != 0 else 1.0
    for z in range(int(d.batch) * inner):
        zo, zi = (z // inner, z % inner) if inner > 1 else (z, 0)
        ar, ac = (d.k, d.m) if d.trans_a else (d.m, d.k)
        br, bc = (d.n, d.k) if d.trans_b else (d.k, d.n)
        am = a[window(ar, ac, d.lda, offsets[0] + zo * d.stride_a + zi * d.stride_a_inner)]
        bm = b[window(br, bc, d.ldb, offsets[1] + zo * d.stride_b + zi * d.stride_b_inner)]
        acc = alpha * ((am.T if d.trans_a else am) @ (bm.T if d.trans_b else bm))
        if d.epilogue in (L.EPI_BIAS, L.EPI_BIAS_RELU, L.EPI_BIAS_GELU):
            acc = acc + extra[None, :d.n]
        where = window(d.m, d.n, d.ldc, zo * d.stride_c + zi * d.stride_c_inner)
        if d.epilogue == L.EPI_ADD:
            acc = acc + extra[where]
        if pre is not None:
            pre[where] = acc
        c[where] = np.maximum(acc, 0.0) if d.epilogue == L.EPI_BIAS_RELU else _gelu(acc) if d.epilogue == L.EPI_BIAS_GELU else acc
    return [c] + ([pre] if pre is not None else [])


def _row(d, ins):
    x = ins[0].reshape(d.rows, d.cols)
    n = d.cols
    if d.op == L.RR_SUM: return [x.sum(1)]
    if d.op == L.RR_MAX: return [x.max(1)]
    if d.op == L.RR_MIN: return [x.min(1)]
    if d.op == L.RR_MEAN: return [x.mean(1)]
    if d.op in (L.RR_VAR, L.RR_STD):
        v = ((x - x.mean(1, keepdims=True)) ** 2).sum(1) / (n - d.correction)
        return [np.sqrt(v) if d.op == L.RR_STD else v]
    if d.op == L.RR_SOFTMAX: return [_softmax(x)]
    if d.op == L.RR_LN_SOFTMAX:
        m = x - x.max(1, keepdims=True)
        return [m - np.log(np.exp(m).sum(1, keepdims=True))]
    if d.op == L.RR_LAYERNORM:
        c = x - x.mean(1, keepdims=True)
        y = c / np.sqrt((c * c).sum(1, keepdims=True) / (n - 1) + d.eps)
        i = 1
        if d.has_weight:
            y = y * ins[i][None, :]
            i += 1
        if d.has_bias:
            y = y + ins[i][None, :]
        return [y]
    if d.op == L.RR_CROSS_ENTROPY:
        m = x - x.max(1, keepdims=True)
        per = -(m - np.log(np.exp(m).sum(1, keepdims=True)))[np.arange(d.rows), ins[1].astype(np.int64)]
        return [per, np.array([per.mean()])]
    if d.op == L.RR_COLSUM: return [x.sum(0)]
    if d.op == L.RR_MSE: return [np.array([((x - ins[1].reshape(d.rows, d.cols)) ** 2).mean()])]
    raise NotImplementedError(d.op)


def _eltwise(d, ins):
    x = ins[0]
    if d.op == L.EW_RELU: return [(x > 0) * x]
    if d.op == L.EW_GELU: return [_gelu(x)]
    if d.op == L.EW_ADD: return [x + ins[1]]
    if d.op == L.EW_SUB: return [x - ins[1]]
    if d.op == L.EW_MUL: return [x * ins[1]]
    if d.op == L.EW_SCALE: return [x * d.p0]
    if d.op == L.EW_CAST: return [x]
    if d.op == L.EW_TANH:
        e = np.exp(2.0 * x)
        return [(e - 1.0) / (e + 1.0)]
    if d.op == L.EW_SIGMOID:
        e = np.exp(x)
        return [e / (e + 1.0)]
    if d.op == L.EW_EXP: return [np.exp(x)]
    if d.op == L.EW_BIAS_ADD: return [(x.reshape(-1, d.cols) + ins[1][None, :]).reshape(-1)]
    raise NotImplementedError(d.op)


def _attention(d, ins):
    b, h, t, hd = int(d.batch), int(d.heads), int(d.seq), int(d.head_dim)
    q, k, v = (a.reshape(b, t, h, hd).transpose(0, 2, 1, 3) for a in ins)
    s = np.einsum("bhqd,bhkd->bhqk", q, k) * (d.scale if d.scale != 0 else hd ** -0.5)
    if d.causal:
        s = np.where(np.tril(np.ones((t, t), bool)), s, -np.inf)
    return [np.einsum("bhqk,bhkd->bhqd", _softmax(s), v).transpose(0, 2, 1, 3).reshape(-1)]


def _conv(d, ins):
    x = ins[0].reshape(d.n, d.c, d.h, d.w)
    w = ins[1].reshape(d.o, d.c, d.kh, d.kw)
    sh, sw, dh, dw = (max(int(v), 1) for v in (d.stride_h, d.stride_w, d.dil_h, d.dil_w))
    oh = (d.h + d.pad_top + d.pad_bottom - dh * (d.kh - 1) - 1) // sh + 1
    ow = (d.w + d.pad_left + d.pad_right - dw * (d.kw - 1) - 1) // sw + 1
    xp = np.pad(x, ((0, 0), (0, 0), (d.pad_top, d.pad_bottom + sh), (d.pad_left, d.pad_right + sw)))
    y = np.zeros((d.n, d.o, oh, ow))
    for r in range(d.kh):
        for s in range(d.kw):
            win = xp[:, :, r * dh:r * dh + oh * sh:sh, s * dw:s * dw + ow * sw:sw]
            y += np.einsum("nchw,oc->nohw", win, w[:, :, r, s])
    if d.has_bias:
        y += ins[2][None, :, None, None]
    return [y.reshape(-1)]


def _optim(d, ins, step):
    n = d.n_tensors
    p, g = ins[:n], ins[n:2 * n]
    state = ins[2 * n:]
    outs = []
    for i in range(n):
        grad = g[i]
        if d.algo == L.OPT_SGD:
            if d.weight_decay != 0:
                grad = grad + p[i] * d.weight_decay
            if state:                                        # a later step of SGD with momentum: the buffer is read
                buf = state[i] * d.momentum + grad * (1.0 - d.dampening)
                grad = grad + buf * d.momentum if d.nesterov else buf
                outs += [p[i] - grad * d.lr, buf]
            else:
                outs += [p[i] - grad * d.lr]
            continue
        if d.algo == L.OPT_ADAM and d.weight_decay != 0:
            grad = grad + p[i] * d.weight_decay
        m = (state[i] * d.beta1 if state else 0.0) + grad * (1.0 - d.beta1)
        v = (state[n + i] * d.beta2 if state else 0.0) + grad * grad * (1.0 - d.beta2)
        mh, vh = m / (1.0 - float(d.beta1) ** step), v / (1.0 - float(d.beta2) ** step)
        if d.algo == L.OPT_ADAM:
            q = p[i] - d.lr * mh / (np.sqrt(vh) + d.eps)
        else:                                                # AdamW as the reference writes it: the step is divided by lr
            q = p[i] - mh / ((np.sqrt(vh) + d.eps) * d.lr)
            if d.weight_decay != 0:
                q = q * (1.0 - d.lr * d.weight_decay)
        outs += [q, m, v]
    return outs


def run_match(g, m):
    """-> the flat float64 outputs of the matched program on the values of its input classes, in the order of m.outputs"""
    ins = [np.asarray(g.vals[c], np.float64).reshape(-1) for c in m.inputs[:m.n_inputs]]
    out_numel = [int(np.prod(g.info(c)[1]) or 1) for c in m.outputs[:m.n_outputs]]
    kind, u = m.desc.kind, m.desc.u
    if kind == L.KIND_GEMM: outs = _gemm(u.gemm, ins, list(m.input_offsets[:m.n_inputs]), out_numel)
    elif kind == L.KIND_ROWREDUCE: outs = _row(u.rowreduce, ins)
    elif kind == L.KIND_ELTWISE: outs = _eltwise(u.eltwise, ins)
    elif kind == L.KIND_ATTENTION: outs = _attention(u.attention, ins)
    elif kind == L.KIND_CONV: outs = _conv(u.conv, ins)
    elif kind == L.KIND_OPTIM: outs = _optim(u.optim, ins, int(m.optim_step))
    else: raise NotImplementedError(kind)
    return [np.asarray(o, np.float64).reshape(-1) for o in outs]
