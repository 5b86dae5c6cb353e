"""A tracer that records, into the matcher's mirror graph, the nodes the reference's Tensor methods push in graph mode.
TEST INFRASTRUCTURE: each method restates the decomposition of the reference method it is named after.

    binary ops     Tensor::broadcast (zyx/src/tensor/mod.rs:3033-3113): a rank-0 operand is cast to the other's dtype, both are
                   expanded to the common shape, then one Binary node
    reductions     Tensor::reduce_impl (tensor/reduce_ops.rs:45-157): cast to the accumulator dtype (f32 for floats), Reduce,
                   cast back when the dtype changed, reshape for keepdim; Mean = sum / const(n).cast(dtype); Var with correction 1
    dot            tensor/mod.rs:1469-1490;  softmax / ln_softmax 1427-1461;  relu / gelu / tanh / exp / sqrt elementwise.rs
    Linear         zyx-nn/src/linear.rs:39-45;  LayerNorm zyx-nn/src/layer_norm.rs:95-135
    SGD / AdamW    zyx-optim/src/sgd.rs:45-84, adamw.rs:51-97
    index helpers  pad_zeros / rpad_zeros (tensor/mod.rs:1120-1226: one Pad node per padded axis, negative amounts cut),
                   slice (index_ops.rs:84-160: negative paddings, then squeeze's reshape), repeat (2766-2783), pool (2442-2543),
                   cumsum (reduce_ops.rs:1076-1091), full (745-754), arange (773-781), one_hot_along_dim (1920-1946),
                   cross_entropy with class-index targets (1639-1656), tri (2396-2414), conv (2583-2680)
Every `.cast(dtype)` pushes a Cast node, also when the dtype does not change (zyx/src/runtime.rs:696-700)."""
import math

from zyx_b200 import _lib as L
from zyx_b200 import matcher as M


# DType::least_upper_dtype (zyx/src/dtype.rs:121-129): the later of the two in this order
_ORDER = [L.BOOL, L.U8, L.U16, L.U32, L.U64, L.I8, L.I16, L.I32, L.I64, L.BF16, L.F16, L.F32, L.F64]
_UINTS, _INTS = (L.U8, L.U16, L.U32, L.U64), (L.I8, L.I16, L.I32, L.I64)


def _least_upper(a, b):
    return _ORDER[max(_ORDER.index(a), _ORDER.index(b))]


class T:
    def __init__(self, g, cls):
        self.g, self.cls = g, cls

    # ---- introspection
    @property
    def dtype(self):
        return self.g.info(self.cls)[0]

    @property
    def shape(self):
        return self.g.info(self.cls)[1]

    # ---- constructors
    @staticmethod
    def leaf(g, dtype, shape):
        return T(g, g.leaf(dtype, shape))

    @staticmethod
    def scalar(g, value, dtype=L.F32):
        return T(g, g.const(dtype, value))

    # ---- movement / dtype
    def cast(self, dtype):
        return T(self.g, self.g.cast(self.cls, dtype))

    def reshape(self, shape):
        return T(self.g, self.g.reshape(self.cls, list(shape)))

    def expand(self, shape):
        return T(self.g, self.g.expand(self.cls, list(shape)))

    def permute(self, axes):
        if list(axes) == list(range(len(axes))):
            return self                                   # runtime.rs:1134-1137: the identity permutation returns the tensor itself
        return T(self.g, self.g.permute(self.cls, list(axes)))

    def t(self):
        r = len(self.shape)
        axes = list(range(r))
        axes[-1], axes[-2] = axes[-2], axes[-1]
        return self.permute(axes)

    def transpose(self, d0, d1):
        axes = list(range(len(self.shape)))
        d0, d1 = d0 % len(axes), d1 % len(axes)
        axes[d0], axes[d1] = axes[d1], axes[d0]
        return self.permute(axes)

    def unsqueeze(self, dim):
        shape = list(self.shape)
        dim = dim if dim >= 0 else len(shape) + dim + 1
        return self.reshape(shape[:dim] + [1] + shape[dim:])

    def squeeze(self, axes):
        shape = list(self.shape)
        axes = [a % len(shape) for a in axes]
        return self.reshape([d for a, d in enumerate(shape) if d != 1 or a not in axes] or [1])

    def _pad_axis(self, axis, left, right):
        orig = self.shape[axis]
        return T(self.g, self.g.pad(self.cls, axis, left, orig + left + right))

    def pad_zeros(self, padding):
        """(left, right) per axis from the first axis on; axes with (0, 0) push no node"""
        cur = self
        for axis, (left, right) in enumerate(padding):
            if left != 0 or right != 0:
                cur = cur._pad_axis(axis, left, right)
        return cur

    def rpad_zeros(self, padding):
        """the same from the last axis backwards"""
        rank = len(self.shape)
        padding = list(padding) + [(0, 0)] * (rank - len(padding))
        padding.reverse()
        return self.pad_zeros(padding)

    def slice(self, ranges):
        """ranges: (start, end) per leading axis, 0 <= start <= end <= extent"""
        shape = self.shape
        return self.pad_zeros([(-s, -(d - e)) for (s, e), d in zip(ranges, shape)]).squeeze([])

    def split(self, sizes, axis):
        """consecutive slices along one axis (tensor/mod.rs:2340-2381)"""
        shape = self.shape
        axis = axis % len(shape)
        out, acc = [], 0
        for size in sizes:
            out.append(self.slice([(0, d) for d in shape[:axis]] + [(acc, acc + size)]))
            acc += size
        return out

    def dropout(self, p, training=False):
        """outside training: x / (1 - p) (tensor/mod.rs:822-828); the training branch draws a random mask and is not transcribed"""
        assert not training
        return self / (1.0 - p)

    def repeat(self, repeats):
        shape = list(self.shape)
        lead = len(repeats) - len(shape)
        base = [1] * lead + shape
        new_shape = [d for b in base for d in (1, b)]
        expand_shape = [d for r, b in zip(repeats, base) for d in (r, b)]
        return self.reshape(new_shape).expand(expand_shape).reshape([r * b for r, b in zip(repeats, base)])

    def pool(self, kernel_size, stride=1, dilation=1):
        """the last len(kernel_size) axes become (output positions.., kernel offsets..)"""
        k_ = list(kernel_size)
        s_ = [stride] * len(k_) if isinstance(stride, int) else list(stride)
        d_ = [dilation] * len(k_) if isinstance(dilation, int) else list(dilation)
        shape = list(self.shape)
        rank = len(shape)
        nb = rank - len(k_)
        i_ = shape[nb:]
        o_ = [-(-(i - d * (k - 1)) // s) for i, d, k, s in zip(i_, d_, k_, s_)]
        full = [(0, d) for d in shape[:nb]]
        sh_b = shape[:nb]
        xup = self.repeat([1] * nb + [-(-(k * (i + d)) // i) for k, i, d in zip(k_, i_, d_)])
        xup = xup.slice(full + [(0, k * (i + d)) for k, i, d in zip(k_, i_, d_)])
        xup = xup.reshape(sh_b + [e for k, i, d in zip(k_, i_, d_) for e in (k, i + d)])
        xup = xup.slice(full + [r for k, o, s in zip(k_, o_, s_) for r in ((0, k), (0, o * s))])
        xup = xup.reshape(sh_b + [e for k, o, s in zip(k_, o_, s_) for e in (k, o, s)])
        xup = xup.slice(full + [r for k, o in zip(k_, o_) for r in ((0, k), (0, o), (0, 1))])
        xup = xup.reshape(sh_b + [e for k, o in zip(k_, o_) for e in (k, o)])
        return xup.permute(list(range(nb)) + [nb + 2 * i + 1 for i in range(len(i_))] + [nb + 2 * i for i in range(len(i_))])

    def conv(self, weight, bias=None, groups=1, stride=(1,), dilation=(1,), padding=(0,)):
        """padding: one value, one per spatial axis, or (before, after) per axis starting from the LAST axis"""
        bs, cin_ = self.shape[:2]
        cout, cin = weight.shape[:2]
        hw = list(weight.shape[2:])
        padding = list(padding)
        if len(padding) == 1:
            pads = padding * (2 * len(hw))
        elif len(padding) == 2 * len(hw):
            pads = padding
        else:
            pads = (padding + padding)[::-1]                                    # resolve_pool_pads, as written
        assert groups * cin == cin_ and len(self.shape) == len(weight.shape)
        stride, dilation = list(stride), list(dilation)
        x = self.rpad_zeros([(pads[2 * i], pads[2 * i + 1]) for i in range(len(hw))])
        x = x.pool(hw, stride[0] if len(stride) == 1 else stride, dilation[0] if len(dilation) == 1 else dilation)
        rcout = cout // groups
        oyx = list(x.shape[2:len(x.shape) - len(hw)])
        x = x.reshape([bs, groups, cin, 1] + oyx + hw).expand([bs, groups, cin, rcout] + oyx + hw)
        x = x.permute([0, 1, 3] + [4 + i for i in range(len(oyx))] + [2] + [4 + len(oyx) + i for i in range(len(hw))])
        w = weight.reshape([1, groups, rcout] + [1] * len(oyx) + [cin] + hw)
        ret = (x * w).sum([-1 - i for i in range(len(oyx) + 1)], keepdim=True).reshape([bs, cout] + oyx)
        if bias is not None:
            n = 1
            for d in bias.shape:
                n *= d
            ret = ret + bias.reshape([1, n] + [1] * len(hw))
        return ret

    def cumsum(self, axis):
        n = self.shape[axis % len(self.shape)]
        x = self.transpose(axis, -1).rpad_zeros([(n - 1, 0)]).pool([n], 1, 1).sum([-1])
        return x.transpose(axis, -1)

    @staticmethod
    def full(g, shape, value, dtype):
        return T.scalar(g, value, dtype).expand(list(shape))            # Runtime::new_full: the constant, expanded

    @staticmethod
    def arange(g, start, stop, step, dtype=L.I64):
        n = (stop - start) // step
        return T.full(g, [n], step, dtype).cumsum(0) + T.scalar(g, start, dtype) - T.scalar(g, step, dtype)

    @staticmethod
    def tri(g, r, c, diagonal, dtype):
        """ones where column >= row + diagonal (tensor/mod.rs:2396-2414): a padded square of ones re-read with a longer pitch"""
        if diagonal >= c:
            return T.full(g, [r, c], 0, dtype)
        if r + diagonal <= 0:
            return T.full(g, [r, c], 1, dtype)
        s = r + c - 1
        t = T.full(g, [s, s], 1, dtype).rpad_zeros([(0, s)]).reshape([2 * s * s]).rpad_zeros([(0, -s)])
        t = t.reshape([s, 2 * s - 1]).rpad_zeros([(0, -(s - 1))])
        if diagonal <= 0:
            return t.slice([(0, r), (-diagonal, c - diagonal)])
        return t.slice([(diagonal, r + diagonal), (0, c)])

    def equal(self, rhs): return self._binary(rhs, M.B_EQ)

    def one_hot_along_dim(self, num_classes, dim):
        rank = len(self.shape)
        dim = dim % rank
        offset = rank - dim - 1
        arange = T.arange(self.g, 0, num_classes, 1).cast(L.I32).reshape([num_classes] + [1] * offset)
        return self.equal(arange)

    def cross_entropy(self, target):
        """ReduceOp::Mean; -> (loss, per-sample losses)"""
        classes_dim = 0 if len(self.shape) <= 1 else 1
        if tuple(self.shape) != tuple(target.shape):
            target = target.unsqueeze(classes_dim).one_hot_along_dim(self.shape[classes_dim], classes_dim)
        per_sample = (self.ln_softmax([classes_dim]).neg() * target).sum([classes_dim])
        return per_sample.mean_all(), per_sample

    # ---- binary with broadcasting
    def _lift(self, other):
        return other if isinstance(other, T) else T.scalar(self.g, other)

    def _binary(self, other, bop):
        x, y = self, self._lift(other)
        xd, yd, xs, ys = x.dtype, y.dtype, x.shape, y.shape
        if xd != yd:
            if len(xs) == 0 and len(ys) != 0:
                x = x.cast(yd)
            elif len(ys) == 0 and len(xs) != 0:
                y = y.cast(xd)
            else:
                common = _least_upper(xd, yd)
                x = x.cast(common) if xd != common else x
                y = y.cast(common) if yd != common else y
        rx, ry = len(xs), len(ys)
        nx, ny = (1,) * max(ry - rx, 0) + tuple(xs), (1,) * max(rx - ry, 0) + tuple(ys)
        eshape = tuple(max(a, b) for a, b in zip(nx, ny))
        if tuple(xs) != eshape:
            x = x.expand(eshape)
        if tuple(ys) != eshape:
            y = y.expand(eshape)
        return T(self.g, self.g.binary(x.cls, y.cls, bop))

    def __add__(self, o): return self._binary(o, M.B_ADD)
    def __sub__(self, o): return self._binary(o, M.B_SUB)
    def __mul__(self, o): return self._binary(o, M.B_MUL)
    def __truediv__(self, o): return self._binary(o, M.B_DIV)
    def cmpgt(self, o): return self._binary(o, M.B_CMPGT)

    # ---- unary
    def _unary(self, uop):
        return T(self.g, self.g.unary(self.cls, uop))

    def neg(self): return self._unary(M.U_NEG)
    def exp(self): return self._unary(M.U_EXP)
    def ln(self): return self._unary(M.U_LN)
    def sqrt(self): return self._unary(M.U_SQRT)

    def relu(self):
        return self.cmpgt(0.0) * self

    def tanh(self):
        e = (self + self).exp()
        return (e - 1) / (e + 1)

    def gelu(self):
        return self * 0.5 * (((self + self * self * self * 0.044715) * math.sqrt(2.0 / math.pi)).tanh() + 1.0)

    # ---- reductions (reduce_impl)
    def _reduce(self, rop, axes, keepdim):
        shape = list(self.shape)
        axes = [a % len(shape) for a in axes]
        xd = self.dtype
        acc = _least_upper(xd, L.U32 if xd in _UINTS else L.I32 if xd in _INTS or xd == L.BOOL else L.F32)   # reduce_acc_dtype
        t = T(self.g, self.g.reduce(self.cast(acc).cls, rop, axes))
        if t.dtype != xd:
            t = t.cast(xd)
        if keepdim:
            for a in axes:
                shape[a] = 1
            t = t.reshape(shape)
        return t

    def sum(self, axes, keepdim=False): return self._reduce(M.B_ADD, axes, keepdim)
    def max(self, axes, keepdim=False): return self._reduce(M.B_MAX, axes, keepdim)

    def min(self, axes, keepdim=False):
        """ReduceOp::Min = inverse().max().inverse() (reduce_ops.rs:33-42, 93-99); the keepdim reshape comes last"""
        inv = (lambda t: t._unary(M.U_NEG)) if self.dtype in (L.F32, L.BF16, L.F16, L.F64) else (lambda t: t._unary(M.U_BITNOT))
        t = inv(inv(self).max(axes))
        if keepdim:
            shape = list(self.shape)
            for a in axes:
                shape[a % len(shape)] = 1
            t = t.reshape(shape)
        return t

    def mean(self, axes, keepdim=False):
        shape = list(self.shape)
        n = 1
        for a in axes:
            n *= shape[a % len(shape)]
        t = self.sum(axes) / T.scalar(self.g, n, L.I64).cast(self.dtype)
        if keepdim:
            for a in axes:
                shape[a % len(shape)] = 1
            t = t.reshape(shape)
        return t

    def mean_all(self):
        return self.mean(list(range(len(self.shape))))          # reduce_impl with no axes: every axis (reduce_ops.rs:286-288)

    def mse_loss(self, target):
        d = self - target                                       # tensor/mod.rs:1999-2003
        return (d * d).mean_all()

    def var(self, axes, keepdim=False, correction=1):
        shape = list(self.shape)
        n = 1
        for a in axes:
            n *= shape[a % len(shape)]
        x = self - self.mean(axes, keepdim=True)
        t = (x * x).sum(axes) / T.scalar(self.g, n - correction, L.I64).cast(self.dtype)
        if keepdim:
            for a in axes:
                shape[a % len(shape)] = 1
            t = t.reshape(shape)
        return t

    def std(self, axes, keepdim=False, correction=1):
        return self.var(axes, keepdim=keepdim, correction=correction).sqrt()     # reduce_ops.rs:124-130

    def softmax(self, axes=(-1,)):
        e = (self - self.max(list(axes), keepdim=True)).exp()
        return e / e.sum(list(axes), keepdim=True)

    def ln_softmax(self, axes=(-1,)):
        m = self - self.max(list(axes), keepdim=True)
        return m - m.exp().sum(list(axes), keepdim=True).ln()

    def dot(self, rhs):
        y = rhs.t()
        xs, ys = self.shape, y.shape
        assert xs[-1] == ys[-1]
        x_shape = list(xs[:-1]) + [1, xs[-1]]
        y_shape = list(ys[:-2]) + [1] + list(ys[-2:])
        out_shape = list(xs[:-1]) + [ys[-2]]
        return (self.reshape(x_shape) * y.reshape(y_shape)).sum([-1]).reshape(out_shape)


class Linear:
    def __init__(self, g, dtype, in_f, out_f, bias=True):
        self.weight = T.leaf(g, dtype, (out_f, in_f))
        self.bias = T.leaf(g, dtype, (out_f,)) if bias else None

    def forward(self, x):
        y = x.dot(self.weight.t())
        return y + self.bias if self.bias is not None else y


class LayerNorm:
    def __init__(self, g, dtype, n, eps=1e-5, weight=True, bias=True):
        self.eps = eps
        self.weight = T.leaf(g, dtype, (n,)) if weight else None
        self.bias = T.leaf(g, dtype, (n,)) if bias else None

    def forward(self, x):
        mean = x.mean([-1], keepdim=True)
        var = x.var([-1], keepdim=True)
        out = (x - mean) / (var + T.scalar(x.g, self.eps, L.F64)).sqrt()
        if self.weight is not None:
            out = out * self.weight
        if self.bias is not None:
            out = out + self.bias
        return out


def sgd_update(params, grads, lr, weight_decay=0.0, momentum=0.0, dampening=0.0, nesterov=False, bufs=None):
    """SGD::update (zyx-optim/src/sgd.rs:45-84) without `maximize`.  bufs: the momentum buffers of the earlier steps, or None on
    the first step, when the reference stores the (decayed) gradient itself as the buffer.  -> new params, or (new params, new bufs)
    when momentum != 0."""
    new_p, new_b = [], []
    for i, (p, g) in enumerate(zip(params, grads)):
        if weight_decay != 0.0:
            g = g + p * weight_decay
        if momentum != 0.0:
            b = bufs[i] * momentum + g * (1.0 - dampening) if bufs is not None else g
            new_b.append(b)
            g = g + b * momentum if nesterov else b
        new_p.append((p - g * lr).cast(p.dtype))
    return (new_p, new_b) if momentum != 0.0 else new_p


def adamw_update(params, grads, m, v, t, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01):
    """-> (new params, new m, new v); m / v are None on the first step."""
    new_p, new_m, new_v = [], [], []
    for i, (p, g) in enumerate(zip(params, grads)):
        mi = m[i] * betas[0] + g * (1.0 - betas[0]) if m is not None else g * (1.0 - betas[0])
        vi = v[i] * betas[1] + g * g * (1.0 - betas[1]) if v is not None else g * g * (1.0 - betas[1])
        mh = mi / (1.0 - betas[0] ** t)
        vh = vi / (1.0 - betas[1] ** t)
        q = (p - mh / ((vh.sqrt() + eps) * lr)).cast(p.dtype)
        if weight_decay != 0.0:
            q = q * (1.0 - lr * weight_decay)
        new_p.append(q); new_m.append(mi); new_v.append(vi)
    return new_p, new_m, new_v


def adam_update(params, grads, m, v, t, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
    """Adam::update without amsgrad (zyx-optim/src/adam.rs:66-101).  -> (new params, new m, new v); m / v are None on the first step.
    `self.learning_rate * mh` is scalar * tensor: the constant is the left operand of the Mul."""
    new_p, new_m, new_v = [], [], []
    for i, (p, g) in enumerate(zip(params, grads)):
        if weight_decay != 0.0:
            g = g + p * weight_decay
        mi = m[i] * betas[0] + g * (1.0 - betas[0]) if m is not None else g * (1.0 - betas[0])
        vi = v[i] * betas[1] + g * g * (1.0 - betas[1]) if v is not None else g * g * (1.0 - betas[1])
        mh = mi / (1.0 - betas[0] ** t)
        vh = vi / (1.0 - betas[1] ** t)
        q = (p - (T.scalar(p.g, lr) * mh) / (vh.sqrt() + eps)).cast(p.dtype)
        new_p.append(q); new_m.append(mi); new_v.append(vi)
    return new_p, new_m, new_v


def attention_core(q, k, v, heads):
    """The mask-free core of MultiheadAttention::forward between the projections (zyx-nn/src/multi_head_attention.rs:160-172,
    197-199, 219-226): q, k, v [b, t, e] -> head split, scores * 1/sqrt(d), softmax, .matmul(v), heads merged -> [b, t, e].
    `matmul` is `dot` (tensor/mod.rs:1464-1467); transpose(1, 2) and transpose(-2, -1) are permutes."""
    b, t, e = q.shape
    d = e // heads
    split = lambda x: x.reshape([x.shape[0], x.shape[1], heads, d]).permute([0, 2, 1, 3])
    qh, kh, vh = split(q), split(k), split(v)
    scores = qh.dot(kh.t()) * (1.0 / math.sqrt(d))
    out = scores.softmax().dot(vh)
    return out.permute([0, 2, 1, 3]).reshape([b, t, e])


def causal_self_attention(x, c_attn, c_proj, n_head, dropout_p=0.0):
    """CausalSelfAttention::forward (zyx-nn/src/causal_self_attention.rs:36-71) outside training: one fused q/k/v projection,
    split along the features, head split, scores * scale, softmax, dropout, .dot(v), heads merged, output projection.  (The
    reference's own mask is commented out there.)  -> (y, scores, probabilities after dropout, merged heads, qkv)"""
    b, t, c = x.shape
    qkv = c_attn.forward(x)
    q, k, v = qkv.split([c, c, c], 2)
    heads = lambda z: z.reshape([b, t, n_head, c // n_head]).transpose(1, 2)
    k, q, v = heads(k), heads(q), heads(v)
    scale = 1.0 / math.sqrt(c // n_head)
    scores = q.dot(k.t()) * scale
    att = scores.softmax([-1]).dropout(dropout_p)
    merged = att.dot(v).transpose(1, 2).reshape([b, t, c])
    return c_proj.forward(merged), scores, att, merged, qkv


class MultiheadAttention:
    """zyx-nn/src/multi_head_attention.rs: batch_first, no bias_kv / zero_attn, no masks, need_weights = false, outside training."""

    def __init__(self, g, dtype, embed_dim, num_heads, dropout=0.0, bias=True):
        self.h, self.d, self.dropout = num_heads, embed_dim // num_heads, dropout
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (Linear(g, dtype, embed_dim, embed_dim, bias) for _ in range(4))

    def forward(self, query, key, value):
        b, t_q, _ = query.shape
        t_kv = key.shape[1]
        h, d = self.h, self.d
        q = self.q_proj.forward(query).reshape([b, t_q, h, d]).transpose(1, 2)
        k = self.k_proj.forward(key).reshape([b, t_kv, h, d]).transpose(1, 2)
        v = self.v_proj.forward(value).reshape([b, t_kv, h, d]).transpose(1, 2)
        weights = (q.dot(k.transpose(-2, -1)) * (1.0 / math.sqrt(d))).softmax([-1])
        if self.dropout > 0.0:
            weights = weights.dropout(self.dropout)
        out = weights.dot(v).transpose(1, 2).reshape([b, t_q, h * d])
        return self.out_proj.forward(out)


class TransformerEncoderLayer:
    """zyx-nn/src/transformer_encoder_layer.rs:84-172 without masks, outside training (every dropout is `/ (1 - p)`)."""

    def __init__(self, g, dtype, d_model, nhead, dim_feedforward, dropout=0.0, activation=T.gelu, eps=1e-5, norm_first=True):
        self.self_attn = MultiheadAttention(g, dtype, d_model, nhead, dropout)
        self.linear1, self.linear2 = Linear(g, dtype, d_model, dim_feedforward), Linear(g, dtype, dim_feedforward, d_model)
        self.norm1, self.norm2 = LayerNorm(g, dtype, d_model, eps), LayerNorm(g, dtype, d_model, eps)
        self.dropout, self.activation, self.norm_first = dropout, activation, norm_first

    def _sa(self, x):
        return self.self_attn.forward(x, x, x).dropout(self.dropout)

    def _ff(self, x):
        return self.linear2.forward(self.activation(self.linear1.forward(x)).dropout(self.dropout)).dropout(self.dropout)

    def forward(self, x):
        if self.norm_first:
            x = x + self._sa(self.norm1.forward(x))
            return x + self._ff(self.norm2.forward(x))
        x = self.norm1.forward(x + self._sa(x))
        return self.norm2.forward(x + self._ff(x))
