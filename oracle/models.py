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


def forward_backward(dtype, layers, x, target, activation, loss):
    """-> (loss, [(dW, db)], y)."""
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
    for i in range(n - 1, -1, -1):
        w, _ = layers[i]
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
