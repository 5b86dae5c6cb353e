"""Parity of the training plans at the configurations' full sizes, stage by stage on sampled rows.  TEST INFRASTRUCTURE ONLY.

The scalar CPU oracle cannot run a whole step of config 4 (batch 8192) or config 5 (seq 2048, d 2048) in reasonable time, but
every stage of those steps is either row-independent (a Linear, a LayerNorm, an activation gradient: row r of the output
needs row r of the input only) or a reduction over the batch whose sampled output rows need a thin slice of one operand
(a weight gradient's row o is column o of dZ against the whole input).  So each stage is checked exactly against the oracle:
the stage's INPUT is the tensor the GPU plan itself stored, the oracle recomputes the sampled rows of the stage's OUTPUT
from it, and the two are compared at the configuration's tolerance.  Attention is checked per sampled (batch, head) over the
whole sequence.  An end-to-end forward of the sampled rows through the oracle alone is compared as well.

Only tests, the smoke check and bench.py's checker leg import this module.  The plan objects are duck-typed
(zyx_b200.host.Mlp / Block): nothing here imports the package.
"""
import numpy as np

from oracle import models as om
from oracle import oracle as zo

ACT_OUT, ACT_PRE, ACT_GRAD = range(3)      # zyxb_mlp_activation's `which`
PARAM, GRAD = 0, 1                         # zyxb_mlp_tensor's `which`


def f64(a, dtype):
    return zo.to_f32(a, dtype).astype(np.float64)


def rel_err(got, want, floor=0.1, row_axis=-1, abs_floor=0.0):
    """max |got - want| / max(|want|, floor * the row's largest |want|, abs_floor), on float64 arrays."""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    scale = np.max(np.abs(want), axis=row_axis, keepdims=True)
    den = np.maximum(np.maximum(np.abs(want), floor * scale), abs_floor)
    den = np.where(den == 0, 1.0, den)
    return float(np.max(np.abs(got - want) / den))


def _c(a):
    return np.ascontiguousarray(a)


def pick_indices(n, count=16):
    """Tile-boundary and spread-out indices in [0, n)."""
    fixed = [0, 1, 127, 128, 129, 255, 256, n // 2 - 1, n // 2, n // 2 + 1, n - 129, n - 128, n - 2, n - 1]
    spread = np.linspace(0, n - 1, max(count - len(fixed), 4)).astype(int).tolist()
    return np.array(sorted({i for i in fixed + spread if 0 <= i < n}))


def mlp_stage_errors(mlp, dtype, layers, x, t, rows=None, activation=om.ACT_GELU, backward=True):
    """`mlp` has just run forward_backward() on (x, t) with parameters `layers` = [(W, b)].  -> {stage: error}; every
    error is relative to max(|want|, 0.1 * the row's largest |want|) unless the key says otherwise."""
    n, B = len(layers), x.shape[0]
    rows = pick_indices(B) if rows is None else np.asarray(rows)
    errs = {}
    inp = _c(x[rows])
    chain = _c(x[rows])                      # the same rows through the oracle alone, end to end
    for i, (w, b) in enumerate(layers):
        last = i == n - 1
        epi = zo.EPI_BIAS if last or activation == om.ACT_NONE else (zo.EPI_BIAS_RELU if activation == om.ACT_RELU else zo.EPI_BIAS_GELU)
        a, z = zo.gemm(dtype, inp, w, tb=True, bias=b, epi=epi, want_preact=True)
        got = mlp.activation(ACT_OUT, i, rows)
        errs["forward_layer%d" % i] = rel_err(f64(got, dtype), f64(a, dtype))
        if not last and activation == om.ACT_GELU:
            errs["preactivation_layer%d" % i] = rel_err(f64(mlp.activation(ACT_PRE, i, rows), dtype), f64(z, dtype))
        inp = got
        chain = zo.gemm(dtype, chain, w, tb=True, bias=b, epi=epi)
    errs["output_end_to_end(floor 0.5)"] = rel_err(f64(inp, dtype), f64(chain, dtype), floor=0.5)
    y = mlp.activation(ACT_OUT, n - 1)
    exact = float(np.mean((f64(y, dtype) - f64(t, dtype)) ** 2))
    got_loss = mlp.read_loss()
    errs["loss_vs_float64"] = abs(got_loss - exact) / exact
    errs["loss_oracle_vs_float64"] = abs(zo.mse(dtype, y, _c(t)) - exact) / exact
    if not backward:
        return errs
    want = zo.eltwise(zo.EW_MSE_BWD, dtype, _c(y[rows]), _c(t[rows]), p0=1.0 / y.size)
    errs["loss_gradient"] = rel_err(f64(mlp.activation(ACT_GRAD, n - 1, rows), dtype), f64(want, dtype))
    for i in range(n - 1, -1, -1):
        w, _ = layers[i]
        dz = mlp.activation(ACT_GRAD, i)                       # [B, out]
        xin = _c(x) if i == 0 else mlp.activation(ACT_OUT, i - 1)
        pick = pick_indices(w.shape[0])
        want_dw = zo.gemm(dtype, _c(dz[:, pick]), xin, ta=True)              # rows `pick` of dZ^T . input
        errs["weight_gradient_layer%d" % i] = rel_err(f64(mlp.get_tensor(GRAD, 2 * i)[pick], dtype), f64(want_dw, dtype))
        errs["bias_gradient_layer%d" % i] = rel_err(f64(mlp.get_tensor(GRAD, 2 * i + 1), dtype), f64(zo.colsum(dtype, dz), dtype), row_axis=None)
        if i > 0:
            if activation == om.ACT_GELU:
                want = zo.gemm(dtype, _c(dz[rows]), w, bias=mlp.activation(ACT_PRE, i - 1, rows), epi=zo.EPI_MUL_GELU_GRAD)
            elif activation == om.ACT_RELU:
                want = zo.gemm(dtype, _c(dz[rows]), w, bias=mlp.activation(ACT_OUT, i - 1, rows), epi=zo.EPI_MUL_RELU_GRAD)
            else:
                want = zo.gemm(dtype, _c(dz[rows]), w)
            errs["input_gradient_layer%d" % i] = rel_err(f64(mlp.activation(ACT_GRAD, i - 1, rows), dtype), f64(want, dtype))
    return errs


def attribution(got, oracle, exact, tol, **kw):
    """The three distances of the attribution rule: GPU to oracle, GPU to the unrounded float64 value of the same formula,
    oracle to that value; and whether the rule holds (within `tol` of the oracle, or as close to exact as the oracle is — within a
    quarter — with the rest of the gap no larger than tol plus the oracle's own distance)."""
    e_go, e_ge, e_oe = rel_err(got, oracle, **kw), rel_err(got, exact, **kw), rel_err(oracle, exact, **kw)
    ok = e_go <= tol or (e_ge <= max(tol, 1.25 * e_oe) and e_go <= tol + e_oe)
    return {"gpu_vs_oracle": e_go, "gpu_vs_float64": e_ge, "oracle_vs_float64": e_oe, "ok": bool(ok)}


def block_stage_errors(blk, dtype, p, x, t, heads, causal, rows=None, head_samples=None, eps=1e-5, tol=2e-2, backward=True):
    """`blk` (zyx_b200.host.Block) has just run forward_backward() on (x, t) [B, T, E] with parameters `p` (dict in
    oracle.models.BLOCK_PARAMS names).  -> ({stage: error}, {attention stage: attribution dict})."""
    B, T, E = x.shape
    H, D, R, F = heads, E // heads, B * T, p["w1"].shape[0]
    rows = pick_indices(R) if rows is None else np.asarray(rows)
    head_samples = head_samples or sorted({(0, 0), (B - 1, H - 1), (B // 2, H // 2)})
    x2, t2 = _c(x.reshape(R, E)), _c(t.reshape(R, E))
    cache = {}

    def act(name):
        if name not in cache:
            cache[name] = blk.activation(name, (R, F) if name in ("z1", "h", "dz1") else (R, E))
        return cache[name]

    e, att = {}, {}
    cmp_rows = lambda name, want, **kw: e.__setitem__(name, rel_err(f64(act(name)[rows], dtype), f64(want, dtype), **kw))
    lin = lambda a, w, b, epi=zo.EPI_BIAS, pre=False: zo.gemm(dtype, _c(a), p[w], tb=True, bias=p[b], epi=epi, want_preact=pre)
    for name, w, b in (("q", "wq", "bq"), ("k", "wk", "bk"), ("v", "wv", "bv")):
        cmp_rows(name, lin(x2[rows], w, b))

    def head(a, b_, h_):
        return _c(a[b_ * T:(b_ + 1) * T, h_ * D:(h_ + 1) * D]).reshape(1, T, D)

    for (b_, h_) in head_samples:
        want, _, exact = om.attention(dtype, head(act("q"), b_, h_), head(act("k"), b_, h_), head(act("v"), b_, h_), 1, causal)
        att["attention_b%d_h%d" % (b_, h_)] = attribution(f64(head(act("attn"), b_, h_), dtype), f64(want, dtype), exact, tol, floor=1.0)
    cmp_rows("o", lin(act("attn")[rows], "wo", "bo"))
    cmp_rows("s1", zo.eltwise(zo.EW_ADD, dtype, _c(x2[rows]), _c(act("o")[rows])))
    cmp_rows("x1", zo.layernorm(dtype, _c(act("s1")[rows]), p["g1"], p["be1"], eps))
    want_h, want_z = lin(act("x1")[rows], "w1", "b1", zo.EPI_BIAS_GELU, True)
    cmp_rows("h", want_h)
    cmp_rows("z1", want_z)
    cmp_rows("m", lin(act("h")[rows], "w2", "b2"))
    cmp_rows("s2", zo.eltwise(zo.EW_ADD, dtype, _c(act("x1")[rows]), _c(act("m")[rows])))
    y = blk.read_output().reshape(R, E)
    e["y"] = rel_err(f64(y[rows], dtype), f64(zo.layernorm(dtype, _c(act("s2")[rows]), p["g2"], p["be2"], eps), dtype))
    exact = float(np.mean((f64(y, dtype) - f64(t2, dtype)) ** 2))
    e["loss_vs_float64"] = abs(blk.read_loss() - exact) / exact
    e["loss_oracle_vs_float64"] = abs(zo.mse(dtype, y, t2) - exact) / exact
    if not backward:
        return e, att

    def grad(name):
        return blk.get_tensor(GRAD, om.BLOCK_PARAMS.index(name))

    def lin_grads(dout, xin, gw, gb):
        pick = pick_indices(p[gw].shape[0])
        e["grad_" + gw] = rel_err(f64(grad(gw)[pick], dtype), f64(zo.gemm(dtype, _c(dout[:, pick]), _c(xin), ta=True), dtype))
        if gb != "bk":      # mathematically zero (softmax ignores a shift of every key score): rounding noise on both sides
            e["grad_" + gb] = rel_err(f64(grad(gb), dtype), f64(zo.colsum(dtype, _c(dout)), dtype), row_axis=None)

    def ln_grads(xin, dout, gw, gb):
        e["grad_" + gw] = rel_err(f64(grad(gw), dtype), f64(zo.colsum(dtype, zo.layernorm_dyxhat(dtype, _c(xin), _c(dout), eps)), dtype), row_axis=None)
        e["grad_" + gb] = rel_err(f64(grad(gb), dtype), f64(zo.colsum(dtype, _c(dout)), dtype), row_axis=None)

    cmp_rows("dy", zo.eltwise(zo.EW_MSE_BWD, dtype, _c(y[rows]), _c(t2[rows]), p0=1.0 / y.size))
    cmp_rows("ds2", zo.layernorm_bwd(dtype, _c(act("s2")[rows]), _c(act("dy")[rows]), p["g2"], eps))
    ln_grads(act("s2"), act("dy"), "g2", "be2")
    lin_grads(act("ds2"), act("h"), "w2", "b2")
    cmp_rows("dz1", zo.gemm(dtype, _c(act("ds2")[rows]), p["w2"], bias=_c(act("z1")[rows]), epi=zo.EPI_MUL_GELU_GRAD))
    lin_grads(act("dz1"), act("x1"), "w1", "b1")
    cmp_rows("dx1", zo.to_bits(om._gemm_f32(dtype, _c(act("dz1")[rows]), p["w1"]) + zo.to_f32(_c(act("ds2")[rows]), dtype), dtype))
    cmp_rows("ds1", zo.layernorm_bwd(dtype, _c(act("s1")[rows]), _c(act("dx1")[rows]), p["g1"], eps))
    ln_grads(act("s1"), act("dx1"), "g1", "be1")
    lin_grads(act("ds1"), act("attn"), "wo", "bo")
    cmp_rows("dattn", zo.gemm(dtype, _c(act("ds1")[rows]), p["wo"]))
    for (b_, h_) in head_samples:
        wq, wk, wv, exact = om.attention_bwd(dtype, head(act("q"), b_, h_), head(act("k"), b_, h_), head(act("v"), b_, h_),
                                             head(act("dattn"), b_, h_), 1, causal)
        for name, want, ex in (("dq", wq, exact[0]), ("dk", wk, exact[1]), ("dv", wv, exact[2])):
            att["%s_b%d_h%d" % (name, b_, h_)] = attribution(f64(head(act(name), b_, h_), dtype), f64(want, dtype), ex, tol, floor=1.0,
                                                           abs_floor=0.05 * float(np.abs(ex).max()))
    lin_grads(act("dv"), x2, "wv", "bv")
    lin_grads(act("dk"), x2, "wk", "bk")
    lin_grads(act("dq"), x2, "wq", "bq")
    return e, att
