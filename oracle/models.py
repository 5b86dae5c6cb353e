"""Training steps composed from the CPU oracle's primitives.  TEST INFRASTRUCTURE ONLY.

The composition follows the reference's definitions: Linear::forward = x.dot(W.t()) + b
(zyx-nn/src/linear.rs:39-45), activation, loss (mse of README.md:144-150 or Tensor::cross_entropy,
zyx/src/tensor/mod.rs:1639-1655), reverse-mode adjoints (zyx/src/graph/autograd.rs), optimizer
(zyx-optim).  Values are rounded to the tensor dtype exactly where the GPU plan writes a tensor.
"""
import numpy as np

from oracle import oracle as zo

ACT_NONE, ACT_RELU, ACT_GELU = range(3)
LOSS_MSE, LOSS_CE = range(2)


def init_linears(rng, dtype, dims):
    """[(W, b)] from Linear::new with the given zyx RNG (weight then bias per layer)."""
    return [rng.linear_init(dtype, dims[i], dims[i + 1]) for i in range(len(dims) - 1)]


def forward_backward(dtype, layers, x, target, activation, loss, keep=None):
    """-> (loss, [(dW, db)], y).  `keep` (a dict) receives the stored intermediates: "act" / "pre" / "dz" lists per layer."""
    n = len(layers)
    acts, zs = [x], []
    for i, (w, b) in enumerate(layers):
        last = i == n - 1
        epi = zo.EPI_BIAS if last or activation == ACT_NONE else (zo.EPI_BIAS_RELU if activation == ACT_RELU else zo.EPI_BIAS_GELU)
        a, z = zo.gemm(dtype, acts[-1], w, tb=True, bias=b, epi=epi, want_preact=True)
        acts.append(a)
        zs.append(z)
    y = acts[-1]
    if loss == LOSS_CE:
        _, mean = zo.cross_entropy(y, target)
        lval = float(mean[0])
        dz = zo.cross_entropy_bwd(y, target)
    else:
        lval = zo.mse(dtype, y, target)
        dz = zo.eltwise(zo.EW_MSE_BWD, dtype, y, target, p0=1.0 / y.size)
    grads = [None] * n
    dzs = [None] * n
    for i in range(n - 1, -1, -1):
        w, _ = layers[i]
        dzs[i] = dz
        dw = zo.gemm(dtype, dz, acts[i], ta=True)           # dZ^T . input
        db = zo.colsum(dtype, dz)
        grads[i] = (dw, db)
        if i > 0:
            # (dZ . W) * act'(z): the product is not rounded in between, like the fused GPU epilogue
            if activation == ACT_RELU:
                dz = zo.gemm(dtype, dz, w, bias=acts[i], epi=zo.EPI_MUL_RELU_GRAD)
            elif activation == ACT_GELU:
                dz = zo.gemm(dtype, dz, w, bias=zs[i - 1], epi=zo.EPI_MUL_GELU_GRAD)
            else:
                dz = zo.gemm(dtype, dz, w)
    if keep is not None:
        keep.update(act=acts[1:], pre=zs, dz=dzs)
    return lval, grads, y


class Optim:
    """SGD / Adam / AdamW over the flattened parameter list, state kept like the reference keeps it."""

    def __init__(self, algo, dtype, params, **kw):
        self.algo, self.dtype, self.kw, self.t = algo, dtype, kw, 0
        self.s0 = [np.zeros_like(p) for p in params]
        self.s1 = [np.zeros_like(p) for p in params]

    def update(self, params, grads, grad_scale=1.0):
        self.t += 1
        kw = self.kw
        for p, g, a, b in zip(params, grads, self.s0, self.s1):
            if self.algo == "sgd":
                mom = kw.get("momentum", 0.0)
                zo.sgd(self.dtype, p, g, a if mom else None, lr=kw["lr"], wd=kw.get("weight_decay", 0.0), momentum=mom,
                       dampening=kw.get("dampening", 0.0), nesterov=kw.get("nesterov", False), first=(self.t == 1), grad_scale=grad_scale)
            else:
                mode = 0 if self.algo == "adam" else (2 if kw.get("standard") else 1)
                zo.adam(self.dtype, p, g, a, b, self.t, lr=kw["lr"], wd=kw.get("weight_decay", 0.0), beta1=kw.get("beta1", 0.9),
                        beta2=kw.get("beta2", 0.999), eps=kw.get("eps", 1e-8), mode=mode, grad_scale=grad_scale)


def flat(pairs):
    return [t for pair in pairs for t in pair]


# ---- one transformer block (zyx-examples/examples/readme_test.rs:9-40) ---------------------------------
BLOCK_PARAMS = ["wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "w1", "b1", "w2", "b2", "g1", "be1", "g2", "be2"]


def block_init(nprng, dtype, dim, ffn, std=0.02):
    """Random-init weights N(0, std) (the configuration's choice), biases N(0, std); LayerNorm weight 1, bias 0
    (zyx-nn/src/layer_norm.rs:23-45).  Returned in Module::iter() order as a dict."""
    shapes = {"wq": (dim, dim), "bq": (dim,), "wk": (dim, dim), "bk": (dim,), "wv": (dim, dim), "bv": (dim,), "wo": (dim, dim),
              "bo": (dim,), "w1": (ffn, dim), "b1": (ffn,), "w2": (dim, ffn), "b2": (dim,)}
    p = {k: zo.to_bits((nprng.standard_normal(s) * std).astype(np.float32), dtype) for k, s in shapes.items()}
    for k in ("g1", "g2"):
        p[k] = zo.to_bits(np.ones(dim, np.float32), dtype)
    for k in ("be1", "be2"):
        p[k] = zo.to_bits(np.zeros(dim, np.float32), dtype)
    return p


def attention(dtype, q, k, v, heads, causal, scale=None):
    """Self-attention as MultiheadAttention::forward composes it (zyx-nn/src/multi_head_attention.rs:197-226): per head
    scores = q.k^T * scale, masked softmax, probabilities . v, each tensor stored in `dtype` as the reference's kernels
    store them.  q, k, v: [B, T, H*D] -> (o [B, T, H*D], lse [B*H, T] float64 = ln sum exp(scale * q.k^T) of the stored q, k,
    exact [B, T, H*D] float64 = the same attention of the stored q, k, v without any intermediate rounding)."""
    B, T, E = q.shape
    H, D = heads, E // heads
    scale = float(1.0 / np.sqrt(np.float32(D))) if scale is None else float(scale)
    heads_of = lambda a: np.ascontiguousarray(a.reshape(B, T, H, D).transpose(0, 2, 1, 3)).reshape(B * H, T, D)
    qh, kh, vh = heads_of(q), heads_of(k), heads_of(v)
    s = zo.gemm(dtype, qh, kh, tb=True, alpha=scale)
    pr = zo.softmax(dtype, s.reshape(B * H * T, T), causal=causal, period=T).reshape(B * H, T, T)
    o = zo.gemm(dtype, pr, vh)
    o = np.ascontiguousarray(o.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B, T, E)
    sx = np.einsum("btd,bsd->bts", zo.to_f32(qh, dtype).astype(np.float64), zo.to_f32(kh, dtype).astype(np.float64)) * scale
    if causal:
        sx = np.where(np.arange(T)[None, None, :] > np.arange(T)[None, :, None], -np.inf, sx)
    mx = sx.max(-1, keepdims=True)
    ex = np.exp(sx - mx)
    lse = (mx + np.log(ex.sum(-1, keepdims=True)))[..., 0]
    exact = np.einsum("bts,bsd->btd", ex / ex.sum(-1, keepdims=True), zo.to_f32(vh, dtype).astype(np.float64))
    exact = np.ascontiguousarray(exact.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B, T, E)
    return o, lse, exact


def attention_bwd(dtype, q, k, v, do, heads, causal, scale=None):
    """The adjoint of `attention` as the reference's autograd composes it from stored tensors: dP = dO.V^T,
    dV = P^T.dO, dS = P*(dP - sum(dP*P)), dQ = dS.K*scale, dK = dS^T.Q*scale, every tensor stored in `dtype`.
    -> (dq, dk, dv, exact) with exact = (dq, dk, dv) in float64 from the stored q, k, v, do without intermediate rounding."""
    B, T, E = q.shape
    H, D = heads, E // heads
    scale = float(1.0 / np.sqrt(np.float32(D))) if scale is None else float(scale)
    heads_of = lambda a: np.ascontiguousarray(a.reshape(B, T, H, D).transpose(0, 2, 1, 3)).reshape(B * H, T, D)
    merge = lambda a: np.ascontiguousarray(a.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(B, T, E)
    qh, kh, vh, doh = heads_of(q), heads_of(k), heads_of(v), heads_of(do)
    s = zo.gemm(dtype, qh, kh, tb=True, alpha=scale)
    pr = zo.softmax(dtype, s.reshape(B * H * T, T), causal=causal, period=T).reshape(B * H, T, T)
    dp = zo.gemm(dtype, doh, vh, tb=True)
    dv = zo.gemm(dtype, pr, doh, ta=True)
    ds = zo.softmax_bwd(dtype, pr.reshape(B * H * T, T), dp.reshape(B * H * T, T)).reshape(B * H, T, T)
    dq = zo.gemm(dtype, ds, kh, alpha=scale)
    dk = zo.gemm(dtype, ds, qh, ta=True, alpha=scale)
    f = lambda a: zo.to_f32(a, dtype).astype(np.float64)
    sx = np.einsum("btd,bsd->bts", f(qh), f(kh)) * scale
    if causal:
        sx = np.where(np.arange(T)[None, None, :] > np.arange(T)[None, :, None], -np.inf, sx)
    px = np.exp(sx - sx.max(-1, keepdims=True))
    px /= px.sum(-1, keepdims=True)
    dpx = np.einsum("btd,bsd->bts", f(doh), f(vh))
    dsx = px * (dpx - (dpx * px).sum(-1, keepdims=True))
    exact = (merge(np.einsum("bts,bsd->btd", dsx, f(kh)) * scale), merge(np.einsum("bts,btd->bsd", dsx, f(qh)) * scale),
             merge(np.einsum("bts,btd->bsd", px, f(doh))))
    return merge(dq), merge(dk), merge(dv), exact


def block_forward_backward(dtype, p, x, target, heads, causal, eps=1e-5):
    """x, target: [B, T, E].  -> (loss, grads dict, y, intermediates).  Rounds to `dtype` wherever the GPU plan stores a tensor."""
    B, T, E = x.shape
    H, D, R = heads, E // heads, B * T
    scale = 1.0 / np.sqrt(np.float32(D))
    x2 = np.ascontiguousarray(x.reshape(R, E))
    t2 = np.ascontiguousarray(target.reshape(R, E))
    lin = lambda a, w, b, epi=zo.EPI_BIAS, pre=False: zo.gemm(dtype, a, p[w], tb=True, bias=p[b], epi=epi, want_preact=pre)
    heads_of = lambda a: np.ascontiguousarray(a.reshape(B, T, H, D).transpose(0, 2, 1, 3)).reshape(B * H, T, D)
    merge = lambda a: np.ascontiguousarray(a.reshape(B, H, T, D).transpose(0, 2, 1, 3)).reshape(R, E)
    q, k, v = lin(x2, "wq", "bq"), lin(x2, "wk", "bk"), lin(x2, "wv", "bv")
    qh, kh, vh = heads_of(q), heads_of(k), heads_of(v)
    s = zo.gemm(dtype, qh, kh, tb=True, alpha=float(scale))
    pr = zo.softmax(dtype, s.reshape(B * H * T, T), causal=causal, period=T).reshape(B * H, T, T)
    attn = merge(zo.gemm(dtype, pr, vh))
    o = lin(attn, "wo", "bo")
    s1 = zo.eltwise(zo.EW_ADD, dtype, x2, o)
    x1 = zo.layernorm(dtype, s1, p["g1"], p["be1"], eps)
    h, z1 = lin(x1, "w1", "b1", zo.EPI_BIAS_GELU, True)
    m = lin(h, "w2", "b2")
    s2 = zo.eltwise(zo.EW_ADD, dtype, x1, m)
    y = zo.layernorm(dtype, s2, p["g2"], p["be2"], eps)
    loss = zo.mse(dtype, y, t2)
    # ---- backward ----
    g = {}
    dy = zo.eltwise(zo.EW_MSE_BWD, dtype, y, t2, p0=1.0 / y.size)

    def ln_bwd(xin, dout, w, gw, gb):
        g[gw] = zo.colsum(dtype, zo.layernorm_dyxhat(dtype, xin, dout, eps))
        g[gb] = zo.colsum(dtype, dout)
        return zo.layernorm_bwd(dtype, xin, dout, p[w], eps)

    def lin_grads(dout, xin, gw, gb):
        g[gw] = zo.gemm(dtype, dout, xin, ta=True)
        g[gb] = zo.colsum(dtype, dout)

    ds2 = ln_bwd(s2, dy, "g2", "g2", "be2")
    lin_grads(ds2, h, "w2", "b2")
    dz1 = zo.gemm(dtype, ds2, p["w2"], bias=z1, epi=zo.EPI_MUL_GELU_GRAD)
    lin_grads(dz1, x1, "w1", "b1")
    # (dz1 . W1) + ds2 with a single rounding, like the fused residual epilogue
    acc = _gemm_f32(dtype, dz1, p["w1"]) + zo.to_f32(ds2, dtype)
    dx1 = zo.to_bits(acc, dtype)
    ds1 = ln_bwd(s1, dx1, "g1", "g1", "be1")
    lin_grads(ds1, attn, "wo", "bo")
    dattn = zo.gemm(dtype, ds1, p["wo"])
    dah = heads_of(dattn)
    dp = zo.gemm(dtype, dah, vh, tb=True)
    dv = merge(zo.gemm(dtype, pr, dah, ta=True))
    dsc = zo.softmax_bwd(dtype, pr.reshape(B * H * T, T), dp.reshape(B * H * T, T)).reshape(B * H, T, T)
    dq = merge(zo.gemm(dtype, dsc, kh, alpha=float(scale)))
    dk = merge(zo.gemm(dtype, dsc, qh, ta=True, alpha=float(scale)))
    lin_grads(dv, x2, "wv", "bv")
    lin_grads(dk, x2, "wk", "bk")
    lin_grads(dq, x2, "wq", "bq")
    mid = {"p": pr, "attn": attn, "x1": x1, "q": q, "k": k, "v": v, "o": o, "s1": s1, "z1": z1, "h": h, "m": m, "s2": s2, "dy": dy, "ds2": ds2,
           "dz1": dz1, "dx1": dx1, "ds1": ds1, "dattn": dattn, "dq": dq, "dk": dk, "dv": dv}
    return loss, g, y.reshape(B, T, E), mid


def _gemm_f32(dtype, a, b):
    """a . b with the oracle's sequential f32 accumulation, returned unrounded (f32)."""
    if dtype == zo.F32:
        return zo.gemm(zo.F32, a, b)
    return zo.gemm(zo.F32, zo.to_f32(a, dtype), zo.to_f32(b, dtype))
