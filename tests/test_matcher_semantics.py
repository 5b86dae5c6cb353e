"""Soundness of the matcher: every matched program computes what the subgraph it replaces computes.

The mirror graph carries a float64 value per class (tests/desc_interp.py: ValGraph evaluates zyx's graph semantics node by node),
and every match - the covers and the alternatives at inner classes alike - is executed the way its descriptor reads, on the flat
values of its input classes, and held against the values of its output classes.  A wrong operand, row pitch, batch stride,
argument offset, transposition flag, epilogue, convolution geometry, hyper-parameter or step number shows up here, on the CPU,
whatever the shapes are."""
import numpy as np
import pytest

from tests.desc_interp import ValGraph, run_match
from tests.zyx_trace import (LayerNorm, Linear, T, TransformerEncoderLayer, adam_update, adamw_update, attention_core,
                             causal_self_attention, sgd_update)
from zyx_b200 import _lib as L


def check_every_match(g, outputs, expect_patterns=(), tol=2e-6):
    ms = g.match(outputs)
    assert ms, "nothing matched"
    for m in ms:
        got = run_match(g, m)
        assert len(got) == m.n_outputs, m.pattern
        for cls, flat in zip(m.outputs[:m.n_outputs], got):
            want = np.asarray(g.vals[cls], np.float64).reshape(-1)
            scale = max(float(np.abs(want).max()), 1e-30)
            err = float(np.abs(flat - want).max()) / scale
            assert flat.shape == want.shape and err <= tol, (m.pattern, cls, err)       # constants pass through f32 descriptor fields
    seen = {m.pattern.decode() for m in ms}
    assert set(expect_patterns) <= seen, sorted(seen)
    return ms


@pytest.fixture()
def g():
    graph = ValGraph(seed=11)
    yield graph
    graph.close()


def test_matmuls_in_every_layout_and_with_every_epilogue(g):
    a, b = T.leaf(g, L.F32, (24, 40)), T.leaf(g, L.F32, (40, 56))
    w, dz = T.leaf(g, L.F32, (56, 40)), T.leaf(g, L.F32, (24, 56))
    lin = Linear(g, L.BF16, 40, 56)
    x16 = T.leaf(g, L.BF16, (24, 40))
    z = lin.forward(x16)
    a3, b3 = T.leaf(g, L.F32, (3, 24, 40)), T.leaf(g, L.F32, (3, 40, 8))
    outs = [a.dot(b), a.dot(w.t()), dz.t().dot(a), dz.t().dot(T.leaf(g, L.F32, (8, 24)).t()), z.gelu(), z, lin.forward(x16).relu(), a3.dot(b3),
            a3.dot(b), a3.t().dot(T.leaf(g, L.F32, (24, 8))), a3.dot(b3) * 0.125]
    check_every_match(g, [t.cls for t in outs], ["matmul_nn", "matmul_nt", "matmul_tn", "matmul_tt", "matmul_nt_bias_gelu", "matmul_nt_bias_relu",
                                                 "matmul_nn_batched", "matmul_tn_batched"])


def test_row_programs_losses_and_elementwise_programs(g):
    x = T.leaf(g, L.F32, (12, 48))
    ln = LayerNorm(g, L.F32, 48, eps=1e-5)
    labels = T.leaf(g, L.I32, (12,))
    t = T.leaf(g, L.F32, (12, 48))
    loss, _ = T.leaf(g, L.F32, (12, 10)).cross_entropy(labels)
    bias = T.leaf(g, L.F32, (48,))
    outs = [x.softmax(), x.ln_softmax(), ln.forward(x), LayerNorm(g, L.F32, 48, weight=False, bias=False).forward(x), x.sum([-1]),
            x.max([-1]), x.min([-1]), x.mean([-1]), x.var([-1]), x.var([-1], correction=0), x.std([-1]), x.sum([0]), x.mse_loss(t), loss,
            x.gelu(), x.relu(), x.tanh(), x.exp() / (x.exp() + 1), (x * t + x).exp(), x * 0.25, x / 0.8, x - t, x + bias, x.cast(L.BF16)]
    check_every_match(g, [o.cls for o in outs], ["softmax", "ln_softmax", "layernorm", "sum", "max", "min", "mean", "var", "std", "colsum",
                                                 "mse_loss", "cross_entropy", "gelu", "relu", "tanh", "sigmoid", "exp", "add", "mul",
                                                 "scale", "sub", "bias_add", "cast"])


@pytest.mark.parametrize("stride,dilation,padding", [((1,), (1,), (1,)), ((2,), (1,), (3,)), ((2, 1), (1, 2), (1, 2, 0, 3)), ((3,), (2,), (0,))])
def test_convolutions(g, stride, dilation, padding):
    x, w, b = T.leaf(g, L.F32, (2, 3, 13, 11)), T.leaf(g, L.F32, (4, 3, 3, 2)), T.leaf(g, L.F32, (4,))
    check_every_match(g, [x.conv(w, b, stride=stride, dilation=dilation, padding=padding).cls, x.conv(w, stride=stride, padding=padding).cls],
                      ["conv", "conv_bias"])


def test_attention_fused_and_in_three_programs(g):
    q, k, v = (T.leaf(g, L.BF16, (2, 128, 256)) for _ in range(3))
    check_every_match(g, [attention_core(q, k, v, heads=2).cls], ["attention", "matmul_nt_batched_heads", "softmax"])
    q, k, v = (T.leaf(g, L.F32, (2, 24, 64)) for _ in range(3))
    check_every_match(g, [attention_core(q, k, v, heads=4).cls], ["matmul_nt_batched_heads", "matmul_nn_batched_heads", "softmax"])
    # the adjoint's products written by hand: p^T . dO and dS^T . q read the packed scores transposed and the per-head views in place
    nb, t, h, d = 2, 24, 4, 16
    p4, do, qq = T.leaf(g, L.F32, (nb, h, t, t)), T.leaf(g, L.F32, (nb, t, h * d)), T.leaf(g, L.F32, (nb, t, h * d))
    split = lambda z: z.reshape([nb, t, h, d]).permute([0, 2, 1, 3])
    dv = p4.t().dot(split(do)).permute([0, 2, 1, 3]).reshape([nb, t, h * d])
    dp = split(do).dot(split(qq).t())
    ms = check_every_match(g, [dv.cls, dp.cls], ["matmul_tn_batched_heads", "matmul_nt_batched_heads"])
    assert next(m for m in ms if m.pattern == b"matmul_tn_batched_heads" and m.outputs[0] == dv.cls).desc.u.gemm.ldc == h * d
    # q, k, v as slices of one fused projection: row pitch 3c and argument offsets (256-byte aligned slices: c = 128 in f32)
    x = T.leaf(g, L.F32, (2, 16, 128))
    y = causal_self_attention(x, Linear(g, L.F32, 128, 384), Linear(g, L.F32, 128, 128), 4, dropout_p=0.0)[0]
    ms = check_every_match(g, [y.cls], ["matmul_nt_batched_heads", "matmul_nn_batched_heads", "matmul_nt_bias"])
    assert any(list(m.input_offsets[:2]) == [0, 128] for m in ms) and any(list(m.input_offsets[:2]) == [0, 256] for m in ms)


@pytest.mark.parametrize("norm_first,dropout", [(True, 0.0), (False, 0.0), (True, 0.25)])
def test_a_transformer_encoder_layer(g, norm_first, dropout):
    g.scale = 0.05                                   # weights small enough for the tanh-by-exp GELU (it overflows near |x| = 10)
    layer = TransformerEncoderLayer(g, L.BF16, 256, 2, 256, dropout=dropout, norm_first=norm_first)
    y = layer.forward(T.leaf(g, L.BF16, (1, 128, 256)))
    check_every_match(g, [y.cls], ["layernorm", "matmul_nt_bias", "matmul_nt_bias_gelu", "add"] + (["attention"] if dropout == 0.0 else ["scale"]))
    assert g.uncovered([y.cls]) == []


def test_optimizer_updates(g):
    shapes = [(6, 5), (7,)]

    def mk(positive=False):
        g.positive = positive
        return [T.leaf(g, L.F32, s) for s in shapes]

    outs = []
    outs += sgd_update(mk(), mk(), 0.05)
    outs += sgd_update(mk(), mk(), 0.03, weight_decay=0.1)
    for nesterov in (False, True):
        new_p, new_b = sgd_update(mk(), mk(), 0.02, weight_decay=0.01, momentum=0.9, dampening=0.1, nesterov=nesterov, bufs=mk())
        outs += new_p + new_b
    for update, kw in ((adamw_update, dict(lr=2e-3, weight_decay=0.02)), (adam_update, dict(lr=3e-3, weight_decay=0.01))):
        for step in (1, 6):
            m, v = (mk(), mk(positive=True)) if step > 1 else (None, None)          # second moments are not negative
            for group in update(mk(), mk(), m, v, step, betas=(0.8, 0.95), eps=1e-6, **kw):
                outs += group
    ms = check_every_match(g, [t.cls for t in outs], ["sgd", "sgd_momentum", "sgd_nesterov", "adamw", "adamw_first_step", "adam", "adam_first_step"])
    assert sorted(m.optim_step for m in ms if m.pattern in (b"adamw", b"adam")) == [6, 6]


def test_convolutions_over_random_geometries(g):
    """A hundred and fifty seeded geometries (sizes, filter shapes, strides, dilations, four-sided paddings): each is recognised, with the
    geometry it was built with, and computes the graph's value."""
    rng = np.random.default_rng(5)
    done = 0
    while done < 150:
        n, c, o = (int(v) for v in rng.integers(1, 4, 3))
        h, w = (int(v) for v in rng.integers(5, 15, 2))
        kh, kw = (int(v) for v in rng.integers(1, 5, 2))
        stride, dil = tuple(int(v) for v in rng.integers(1, 4, 2)), tuple(int(v) for v in rng.integers(1, 3, 2))
        left, right, top, bottom = (int(v) for v in rng.integers(0, 4, 4))
        oh = (h + top + bottom - dil[0] * (kh - 1) - 1) // stride[0] + 1
        ow = (w + left + right - dil[1] * (kw - 1) - 1) // stride[1] + 1
        if h + top + bottom < dil[0] * (kh - 1) + 1 or w + left + right < dil[1] * (kw - 1) + 1:
            continue
        x, wt = T.leaf(g, L.F32, (n, c, h, w)), T.leaf(g, L.F32, (o, c, kh, kw))
        y = x.conv(wt, stride=stride, dilation=dil, padding=(left, right, top, bottom))
        assert tuple(y.shape) == (n, o, oh, ow)
        m = next(m for m in check_every_match(g, [y.cls], ["conv"]) if m.outputs[0] == y.cls)
        d = m.desc.u.conv
        assert (d.pad_top, d.pad_bottom, d.pad_left, d.pad_right) == (top, bottom, left, right)
        slack = (h + top + bottom - dil[0] * (kh - 1), w + left + right - dil[1] * (kw - 1))
        # a single window never takes its stride: the descriptor names the first stride that gives one window
        assert (d.stride_h, d.stride_w) == tuple(s if e > 1 else max(1, k) for s, e, k in zip(stride, (oh, ow), slack))
        assert (d.dil_h, d.dil_w) == tuple(s if k > 1 else 1 for s, k in zip(dil, (kh, kw)))
        done += 1


@pytest.mark.parametrize("dtype", [L.F32, L.BF16], ids=["f32", "bf16"])
def test_matmuls_over_random_shapes_and_layouts(g, dtype):
    """Eighty seeded products: rank 2 to 4, either operand stored transposed, the right one shared by the batch or not, with and
    without a scale, a bias and an activation - whatever is matched must compute the graph's value, and a matmul ends at each."""
    rng = np.random.default_rng(17)
    for _ in range(80):
        m, n, k = (int(v) for v in rng.integers(1, 9, 3))
        batch = [int(v) for v in rng.integers(1, 4, int(rng.integers(0, 3)))]
        ta, tb, shared = (bool(rng.integers(0, 2)) for _ in range(3))
        a = T.leaf(g, dtype, batch + ([k, m] if ta else [m, k]))
        b = T.leaf(g, dtype, ([] if shared else batch) + ([n, k] if tb else [k, n]))
        out = (a.t() if ta else a).dot(b.t() if tb else b)
        kind = int(rng.integers(0, 5))
        if kind == 1:
            out = out * 0.375
        elif kind == 4:
            out = T.leaf(g, dtype, out.shape) + out                 # a residual
        elif kind >= 2:
            out = out + T.leaf(g, dtype, (n,))
            out = out.relu() if kind == 3 else out
        ms = check_every_match(g, [out.cls])
        # (a residual on a batch of products stays an elementwise addition after them)
        assert any((x.pattern.startswith(b"matmul") or (kind == 4 and x.pattern == b"add")) and x.outputs[0] == out.cls for x in ms), \
            (batch, m, n, k, ta, tb, shared, kind)
        assert g.uncovered([out.cls]) == []


@pytest.mark.parametrize("dtype", [L.F32, L.BF16], ids=["f32", "bf16"])
def test_per_head_views_over_random_shapes(g, dtype):
    """Thirty seeded attention cores outside the fused kernel's shapes (images, heads, lengths, head widths; q, k, v whole tensors
    or slices of one fused projection): three programs each, every one computing the graph's value."""
    rng = np.random.default_rng(23)
    for _ in range(30):
        nb, h, t = (int(v) for v in rng.integers(1, 4, 3))
        t *= 3
        d = int(rng.integers(1, 5)) * (64 if dtype == L.F32 else 128)    # slices of a fused projection must start on 256-byte boundaries
        e = h * d
        if rng.integers(0, 2):
            q, k, v = (T.leaf(g, dtype, (nb, t, e)) for _ in range(3))
        else:
            q, k, v = T.leaf(g, dtype, (nb, t, 3 * e)).split([e, e, e], 2)
        split = lambda z: z.reshape([nb, t, h, d]).permute([0, 2, 1, 3])
        out = (split(q).dot(split(k).t()) * (d ** -0.5)).softmax().dot(split(v)).permute([0, 2, 1, 3]).reshape([nb, t, e])
        ms = check_every_match(g, [out.cls], ["softmax"])
        assert any(x.pattern.startswith(b"matmul_nn") and x.outputs[0] == out.cls and x.desc.u.gemm.ldc == (e if h > 1 or nb > 1 else x.desc.u.gemm.ldc)
                   for x in ms), (nb, h, t, d)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16], ids=["f32", "bf16"])
def test_row_programs_over_random_shapes(g, dtype):
    """Sixty seeded tensors of rank 1 to 4: every reduction (with and without keepdim), softmax, ln_softmax and both layer norms
    end in a row program that computes the graph's value."""
    rng = np.random.default_rng(29)
    for _ in range(60):
        shape = [int(v) for v in rng.integers(1, 6, int(rng.integers(1, 5)))]
        shape[-1] = int(rng.integers(2, 12))
        x = T.leaf(g, dtype, shape)
        keep = bool(rng.integers(0, 2))
        outs = {"sum": x.sum([-1], keepdim=keep), "max": x.max([-1], keepdim=keep), "min": x.min([-1], keepdim=keep),
                "mean": x.mean([-1], keepdim=keep), "var": x.var([-1], keepdim=keep, correction=int(rng.integers(0, 2))),
                "std": x.std([-1], keepdim=keep), "softmax": x.softmax(), "ln_softmax": x.ln_softmax(),
                "layernorm": LayerNorm(g, dtype, shape[-1], eps=1e-5, weight=bool(rng.integers(0, 2)), bias=bool(rng.integers(0, 2))).forward(x)}
        ms = check_every_match(g, [t.cls for t in outs.values()])
        at = {m.outputs[0]: m.pattern.decode() for m in ms}
        assert {name: at.get(t.cls) for name, t in outs.items()} == {name: name for name in outs}, shape


def test_optimizer_updates_over_random_hyper_parameters(g):
    """Forty seeded updates: SGD in all its forms, Adam and AdamW at random steps, random learning rates, decays and momenta."""
    rng = np.random.default_rng(31)
    for _ in range(40):
        g.positive = False
        p, gr = T.leaf(g, L.F32, (5, 3)), T.leaf(g, L.F32, (5, 3))
        lr, wd = float(rng.uniform(1e-3, 0.1)), float(rng.choice([0.0, rng.uniform(0.001, 0.1)]))
        form = int(rng.integers(0, 3))
        if form == 0:
            mom = float(rng.choice([0.0, rng.uniform(0.5, 0.99)]))
            bufs = [T.leaf(g, L.F32, (5, 3))] if mom != 0.0 else None
            res = sgd_update([p], [gr], lr, weight_decay=wd, momentum=mom, dampening=float(rng.choice([0.0, 0.2])), nesterov=bool(rng.integers(0, 2)), bufs=bufs)
            outs = res[0] + res[1] if mom != 0.0 else res
        else:
            step = int(rng.integers(1, 40))
            m = [T.leaf(g, L.F32, (5, 3))] if step > 1 else None
            g.positive = True
            v = [T.leaf(g, L.F32, (5, 3))] if step > 1 else None
            update = adamw_update if form == 1 else adam_update
            outs = [t for group in update([p], [gr], m, v, step, lr=lr, betas=(float(rng.uniform(0.7, 0.95)), float(rng.uniform(0.9, 0.999))),
                                          eps=1e-7, weight_decay=wd) for t in group]
        # beta2 as an f32 descriptor field: 1 - beta2^t carries its rounding several times over
        ms = check_every_match(g, [t.cls for t in outs], tol=1e-4)
        assert any(x.desc.kind == L.KIND_OPTIM for x in ms), (form, lr, wd)


def test_cross_entropy_over_random_shapes(g):
    """Twenty seeded (samples, classes) pairs, square ones among them: the loss program reads the labels along the samples."""
    rng = np.random.default_rng(37)
    for i in range(20):
        n = int(rng.integers(1, 12))
        c = n if i % 4 == 0 else int(rng.integers(2, 12))
        g.int_high = c
        loss, per = T.leaf(g, L.F32, (n, c)).cross_entropy(T.leaf(g, L.I32, (n,)))
        ms = check_every_match(g, [loss.cls], ["cross_entropy"])
        m = next(x for x in ms if x.pattern == b"cross_entropy")
        assert list(m.outputs[:2]) == [per.cls, loss.cls] and (m.desc.u.rowreduce.rows, m.desc.u.rowreduce.cols) == (n, c)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16], ids=["f32", "bf16"])
def test_random_elementwise_expressions_are_covered_and_sound(g, dtype):
    """Fifty seeded expression trees over three tensors and a bias vector (additions, products, activations, scales, casts): the
    on-demand elementwise programs cover each of them completely, and every program computes its class."""
    rng = np.random.default_rng(41)
    g.scale = 0.3
    for _ in range(50):
        shape = (int(rng.integers(1, 5)), int(rng.integers(2, 7)))
        pool = [T.leaf(g, dtype, shape) for _ in range(3)]
        bias = T.leaf(g, dtype, (shape[1],))
        for _ in range(int(rng.integers(1, 7))):
            a, b = pool[int(rng.integers(0, len(pool)))], pool[int(rng.integers(0, len(pool)))]
            op = int(rng.integers(0, 12))
            new = [lambda: a + b, lambda: a - b, lambda: a * b, lambda: a.relu(), lambda: a.gelu(), lambda: a.tanh(), lambda: a.exp(),
                   lambda: a * 0.75, lambda: a / 1.25, lambda: a + bias, lambda: a.exp() / (a.exp() + 1), lambda: a.cast(L.F32 if dtype == L.BF16 else L.BF16).cast(dtype)][op]()
            pool.append(new)
        out = pool[-1]
        check_every_match(g, [out.cls])
        assert g.uncovered([out.cls]) == [], shape


@pytest.mark.parametrize("dtype", [L.F32, L.BF16], ids=["f32", "bf16"])
def test_random_networks_are_covered_and_sound(g, dtype):
    """Forty seeded stacks of Linear layers (with and without bias and activation), layer norms, residual additions, softmaxes and
    scales on [batch, features] or [batch, tokens, features] inputs, closed by a loss: covered without a leftover, every program
    computing its class."""
    rng = np.random.default_rng(43)
    g.scale = 0.2
    for _ in range(40):
        lead = [int(rng.integers(1, 5))] + ([int(rng.integers(1, 4))] if rng.integers(0, 2) else [])
        f = int(rng.integers(2, 9))
        h = T.leaf(g, dtype, lead + [f])
        for _ in range(int(rng.integers(2, 6))):
            op = int(rng.integers(0, 6))
            if op <= 1:
                f2 = int(rng.integers(1, 9))
                z = Linear(g, dtype, f, f2, bias=bool(rng.integers(0, 4))).forward(h)
                act = int(rng.integers(0, 3))
                h, f = (z.relu() if act == 1 else z.gelu() if act == 2 else z), f2
            elif op == 2 and f > 1:
                h = LayerNorm(g, dtype, f, weight=bool(rng.integers(0, 2)), bias=bool(rng.integers(0, 2))).forward(h)
            elif op == 3:
                h = h + Linear(g, dtype, f, f).forward(h)
            elif op == 4:
                h = h.softmax()
            else:
                h = h * 0.5
        # the loss program is f32: a 16-bit output is cast first, as the training plans do
        loss = h.cast(L.F32).mse_loss(T.leaf(g, L.F32, h.shape)) if rng.integers(0, 2) else h.sum([-1])
        check_every_match(g, [loss.cls])
        assert g.uncovered([loss.cls]) == [], (lead, f)


def test_cross_entropy_against_a_stored_one_hot_matrix_is_covered_by_five_programs(g):
    """`logits.cross_entropy(one_hot, Mean)` with a float target of the logits' shape has no program of its own: log-softmax, a
    negation (a scale by -1), the product with the target, the row sums and their mean cover it."""
    logits, target = T.leaf(g, L.F32, (12, 7)), T.leaf(g, L.F32, (12, 7))
    loss, _ = logits.cross_entropy(target)
    ms = check_every_match(g, [loss.cls], ["ln_softmax", "scale", "mul", "sum", "mean"])
    assert g.uncovered([loss.cls]) == [] and b"cross_entropy" not in {m.pattern for m in ms}
