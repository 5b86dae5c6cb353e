"""From a traced graph to a launch: the matcher's descriptor goes to zyxb_program_create as it is, the matched input and
output classes name the buffers (loads first, then stores, as Device::launch receives them), and the result is the oracle's.
This is the path a `Node::Kernel` pushed by match_graph takes when the plan is executed (zyx/src/backend/cblas.rs:213-271)."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, TOL_F32, assert_parity, exact_layernorm, max_rel_err
from tests.zyx_trace import LayerNorm, Linear, T, sgd_update
from zyx_b200 import _lib as L
from zyx_b200.matcher import MGraph

pytestmark = pytest.mark.gpu
NP = {L.F32: np.float32, L.BF16: np.uint16, L.F16: np.uint16}


def run_match(sess, g, match, values):
    """values: class id -> host array for every input class.  -> {output class: host array}"""
    prog = sess.device.create_program(match.desc)
    ins = [sess.pool.upload(values[c]) for c in match.inputs[:match.n_inputs]]
    outs, specs = [], []
    for c in match.outputs[:match.n_outputs]:
        dt, shape, _ = g.info(c)
        specs.append((shape, NP[dt]))
        outs.append(sess.pool.allocate(int(np.prod(shape)) * np.dtype(NP[dt]).itemsize)[0])
    try:
        sess.device.launch(prog, ins + outs)
        return {c: sess.pool.download(b, s, t) for c, b, (s, t) in zip(match.outputs[:match.n_outputs], outs, specs)}
    finally:
        for b in ins + outs:
            sess.pool.deallocate(b)
        sess.device.release(prog)


def pick(matches, pattern, out_cls):
    return next(m for m in matches if m.pattern == pattern and m.outputs[0] == out_cls)


@pytest.mark.parametrize("dtype,tol", [(L.F32, TOL_F32), (L.BF16, TOL_BF16)])
def test_linear_gelu_layer_from_graph_to_launch(sess, dtype, tol):
    rng = np.random.default_rng(31)
    g = MGraph()
    try:
        lin = Linear(g, dtype, 320, 264)
        x = T.leaf(g, dtype, (200, 320))
        z = lin.forward(x)
        h = z.gelu()
        m = pick(g.match([h.cls, z.cls]), b"matmul_nt_bias_gelu", h.cls)
        bits = lambda a: zo.to_bits(a.astype(np.float32), dtype)
        vals = {x.cls: bits(rng.standard_normal((200, 320))), lin.weight.cls: bits(rng.uniform(-0.05, 0.05, (264, 320))),
                lin.bias.cls: bits(rng.uniform(-0.05, 0.05, 264))}
        got = run_match(sess, g, m, vals)
        want_h, want_z = zo.gemm(dtype, vals[x.cls], vals[lin.weight.cls], tb=True, bias=vals[lin.bias.cls], epi=zo.EPI_BIAS_GELU, want_preact=True)
        f = lambda a: zo.to_f32(a, dtype)
        assert max_rel_err(f(got[h.cls]), f(want_h), floor=0.1) <= tol
        assert max_rel_err(f(got[z.cls]), f(want_z), floor=0.1) <= tol
    finally:
        g.close()


def test_softmax_layernorm_and_sgd_from_graph_to_launch(sess):
    rng = np.random.default_rng(32)
    g = MGraph()
    try:
        x = T.leaf(g, L.F32, (96, 4096))
        ln = LayerNorm(g, L.F32, 4096, eps=1e-5)
        y_sm, y_ln = x.softmax(), ln.forward(x)
        p, gr = T.leaf(g, L.F32, (50, 30)), T.leaf(g, L.F32, (50, 30))
        new_p = sgd_update([p], [gr], 0.01)[0]
        ms = g.match([y_sm.cls, y_ln.cls, new_p.cls])
        xv = rng.standard_normal((96, 4096)).astype(np.float32)
        wv, bv = (1 + 0.1 * rng.standard_normal(4096)).astype(np.float32), (0.1 * rng.standard_normal(4096)).astype(np.float32)
        got = run_match(sess, g, pick(ms, b"softmax", y_sm.cls), {x.cls: xv})[y_sm.cls]
        assert max_rel_err(got, zo.softmax(zo.F32, xv)) <= TOL_F32
        got = run_match(sess, g, pick(ms, b"layernorm", y_ln.cls), {x.cls: xv, ln.weight.cls: wv, ln.bias.cls: bv})[y_ln.cls]
        # 4096-term f32 sums in another order than the oracle's: the shared parity rule (oracle, or float64 attribution)
        assert_parity(got, zo.layernorm(zo.F32, xv, wv, bv, 1e-5), exact_layernorm(xv, wv, bv, 1e-5), TOL_F32, what="matched layernorm")
        # the optimizer program updates where its arguments lie (the shim's launch copies p into the output buffer first)
        m = pick(ms, b"sgd", new_p.cls)
        pv, gv = rng.standard_normal((50, 30)).astype(np.float32), rng.standard_normal((50, 30)).astype(np.float32)
        prog = sess.device.create_program(m.desc)
        bp, bg = sess.pool.upload(pv), sess.pool.upload(gv)
        try:
            sess.device.launch(prog, [bp, bg])
            got = sess.pool.download(bp, pv.shape, np.float32)
        finally:
            sess.pool.deallocate(bp); sess.pool.deallocate(bg); sess.device.release(prog)
        want = pv.copy()
        zo.sgd(zo.F32, want, gv, None, lr=0.01)
        assert max_rel_err(got, want) <= TOL_F32
    finally:
        g.close()


def test_attention_core_from_graph_to_launch(sess):
    """The mask-free core of MultiheadAttention::forward, traced, matched as one fused program and launched on the three stored
    [b, t, e] tensors (plus the log-sum-exp buffer the program takes behind its output): the oracle's composed attention."""
    from oracle import models as zm
    from tests.zyx_trace import attention_core
    rng = np.random.default_rng(33)
    dtype, b, t, heads, d = L.BF16, 2, 256, 3, 128
    g = MGraph()
    try:
        q, k, v = (T.leaf(g, dtype, (b, t, heads * d)) for _ in range(3))
        out = attention_core(q, k, v, heads)
        m = pick(g.match([out.cls]), b"attention", out.cls)
        vals = {c.cls: zo.to_bits(rng.standard_normal((b, t, heads * d)).astype(np.float32), dtype) for c in (q, k, v)}
        prog = sess.device.create_program(m.desc)
        bufs = [sess.pool.upload(vals[c]) for c in m.inputs[:m.n_inputs]]
        o_buf = sess.pool.allocate(b * t * heads * d * 2)[0]
        lse_buf = sess.pool.allocate(b * heads * t * 4)[0]
        try:
            sess.device.launch(prog, bufs + [o_buf, lse_buf])
            got = sess.pool.download(o_buf, (b, t, heads * d), np.uint16)
            assert sess.device.status() == 0
        finally:
            for x in bufs + [o_buf, lse_buf]:
                sess.pool.deallocate(x)
            sess.device.release(prog)
        want, _, exact = zm.attention(dtype, vals[q.cls], vals[k.cls], vals[v.cls], heads, False)
        assert_parity(zo.to_f32(got, dtype).astype(np.float64), zo.to_f32(want, dtype).astype(np.float64), exact, TOL_BF16, floor=1.0,
                      what="matched attention")
    finally:
        g.close()


@pytest.mark.parametrize("nesterov", [False, True])
def test_sgd_with_momentum_from_graph_to_launch(sess, nesterov):
    """A later step of SGD with weight decay, momentum, dampening (and Nesterov), traced and matched as one program over
    (p, g, buf): the match's step goes into the program's counter so that the kernel reads the buffer; p' and buf' are the oracle's."""
    rng = np.random.default_rng(34)
    g = MGraph()
    try:
        p, gr, buf = (T.leaf(g, L.F32, (70, 33)) for _ in range(3))
        new_p, new_b = sgd_update([p], [gr], 0.05, weight_decay=0.01, momentum=0.9, dampening=0.1, nesterov=nesterov, bufs=[buf])
        m = pick(g.match([new_p[0].cls, new_b[0].cls]), b"sgd_nesterov" if nesterov else b"sgd_momentum", new_p[0].cls)
        assert m.optim_step == 2
        pv, gv, bv = (rng.standard_normal((70, 33)).astype(np.float32) for _ in range(3))
        prog = sess.device.create_program(m.desc)
        sess.device.set_step(prog, m.optim_step - 1)
        bufs = [sess.pool.upload(a) for a in (pv, gv, bv)]
        try:
            sess.device.launch(prog, bufs)
            got_p = sess.pool.download(bufs[0], pv.shape, np.float32)
            got_b = sess.pool.download(bufs[2], bv.shape, np.float32)
        finally:
            for b_ in bufs:
                sess.pool.deallocate(b_)
            sess.device.release(prog)
        want_p, want_b = pv.copy(), bv.copy()
        zo.sgd(zo.F32, want_p, gv, want_b, lr=0.05, wd=0.01, momentum=0.9, dampening=0.1, nesterov=nesterov, first=False)
        assert max_rel_err(got_p, want_p) <= TOL_F32 and max_rel_err(got_b, want_b) <= TOL_F32
    finally:
        g.close()


def test_cross_entropy_from_graph_to_launch(sess):
    """logits.cross_entropy(labels, Mean) traced with class-index labels (the one-hot compares against a folded arange),
    matched as one program: logits, labels -> per-sample losses, mean."""
    rng = np.random.default_rng(35)
    g = MGraph()
    try:
        logits, labels = T.leaf(g, L.F32, (64, 10)), T.leaf(g, L.I32, (64,))
        loss, per_sample = logits.cross_entropy(labels)
        m = next(x for x in g.match([loss.cls]) if x.pattern == b"cross_entropy")
        assert list(m.outputs[:m.n_outputs]) == [per_sample.cls, loss.cls]
        xv = (3.0 * rng.standard_normal((64, 10))).astype(np.float32)
        yv = rng.integers(0, 10, 64).astype(np.int32)
        got = run_match(sess, g, m, {logits.cls: xv, labels.cls: yv})
        want_per, want_mean = zo.cross_entropy(xv, yv)
        x64 = xv.astype(np.float64)
        exact = np.log(np.exp(x64 - x64.max(1, keepdims=True)).sum(1)) + x64.max(1) - x64[np.arange(64), yv]
        assert_parity(got[per_sample.cls], want_per, exact, TOL_F32, row_axis=0, what="matched ce per-sample")
        assert_parity(got[loss.cls].reshape(1), want_mean, np.array([exact.mean()]), TOL_F32, row_axis=0, what="matched ce mean")
    finally:
        g.close()


def test_convolution_from_graph_to_launch(sess):
    """Tensor::conv traced (padding, pooling view, broadcast product, sum over channel and taps, bias), recognised by what the
    view reads, launched as the convolution program: x, w, bias -> y."""
    rng = np.random.default_rng(36)
    g = MGraph()
    try:
        x, w, b = T.leaf(g, L.F32, (2, 5, 19, 23)), T.leaf(g, L.F32, (7, 5, 3, 2)), T.leaf(g, L.F32, (7,))
        y = x.conv(w, b, stride=(2, 1), dilation=(1, 2), padding=(1, 2, 0, 3))         # (left, right, top, bottom)
        m = pick(g.match([y.cls]), b"conv_bias", y.cls)
        xv = rng.standard_normal((2, 5, 19, 23)).astype(np.float32)
        wv = rng.standard_normal((7, 5, 3, 2)).astype(np.float32)
        bv = rng.standard_normal(7).astype(np.float32)
        got = run_match(sess, g, m, {x.cls: xv, w.cls: wv, b.cls: bv})[y.cls]
        want = zo.conv(zo.F32, xv, wv, bv, (2, 1), (1, 2), (0, 3, 1, 2))                # (top, bottom, left, right)
        assert got.shape == want.shape == tuple(y.shape)
        xp = np.pad(xv.astype(np.float64), ((0, 0), (0, 0), (0, 3), (1, 2)))           # the float64 convolution of the same values
        exact = np.zeros(want.shape) + bv.astype(np.float64)[None, :, None, None]
        for r in range(3):
            for s in range(2):
                win = xp[:, :, r:r + 2 * 10:2, 2 * s:2 * s + 24]                        # rows oy*2 + r, columns ox + 2*s
                exact += np.einsum("nchw,oc->nohw", win, wv[:, :, r, s].astype(np.float64))
        assert_parity(got, want, exact, TOL_F32, floor=0.1, what="matched conv")
    finally:
        g.close()


def test_unfused_attention_from_graph_to_launch(sess):
    """Head dimension 32 in f32 is outside the fused kernel's shapes: the traced attention core is three programs - scores,
    softmax, product with v - whose matmuls read q, k, v as per-head views of the stored [b, t, h*d] tensors and write the
    merged [b, t, h*d] result in place (row pitches and a two-level batch; no [b, h, t, d] copy anywhere)."""
    import math
    rng = np.random.default_rng(37)
    nb, t, h, d = 2, 64, 4, 32
    e = h * d
    g = MGraph()
    try:
        q, k, v = (T.leaf(g, L.F32, (nb, t, e)) for _ in range(3))
        split = lambda x: x.reshape([nb, t, h, d]).permute([0, 2, 1, 3])
        scale = 1.0 / math.sqrt(d)
        scores = split(q).dot(split(k).t()) * scale
        probs = scores.softmax()
        merged = probs.dot(split(v)).permute([0, 2, 1, 3]).reshape([nb, t, e])
        ms = g.match([merged.cls])
        m_s, m_p, m_o = pick(ms, b"matmul_nt_batched_heads", scores.cls), pick(ms, b"softmax", probs.cls), pick(ms, b"matmul_nn_batched_heads", merged.cls)
        assert list(m_s.inputs[:2]) == [q.cls, k.cls] and list(m_o.inputs[:2]) == [probs.cls, v.cls]
        qv, kv, vv = (rng.uniform(-1, 1, (nb, t, e)).astype(np.float32) for _ in range(3))
        s_got = run_match(sess, g, m_s, {q.cls: qv, k.cls: kv})[scores.cls]
        p_got = run_match(sess, g, m_p, {scores.cls: s_got})[probs.cls]
        o_got = run_match(sess, g, m_o, {probs.cls: p_got, v.cls: vv})[merged.cls]
        heads = lambda x: np.ascontiguousarray(x.reshape(nb, t, h, d).transpose(0, 2, 1, 3)).reshape(nb * h, t, d)
        s_want = zo.gemm(zo.F32, heads(qv), heads(kv), tb=True, alpha=scale)
        p_want = zo.softmax(zo.F32, s_want.reshape(-1, t)).reshape(nb * h, t, t)
        o_want = zo.gemm(zo.F32, p_want, heads(vv)).reshape(nb, h, t, d).transpose(0, 2, 1, 3).reshape(nb, t, e)
        s64 = np.einsum("bqd,bkd->bqk", heads(qv).astype(np.float64), heads(kv).astype(np.float64)) * scale
        p64 = np.exp(s64 - s64.max(-1, keepdims=True))
        p64 /= p64.sum(-1, keepdims=True)
        exact = np.einsum("bqk,bkd->bqd", p64, heads(vv).astype(np.float64)).reshape(nb, h, t, d).transpose(0, 2, 1, 3).reshape(nb, t, e)
        assert s_got.shape == (nb, h, t, t) and o_got.shape == (nb, t, e)
        assert max_rel_err(s_got.reshape(nb * h, t, t), s_want, floor=0.1) <= TOL_F32
        assert_parity(o_got, o_want, exact, TOL_F32, floor=0.1, what="matched unfused attention")
    finally:
        g.close()
