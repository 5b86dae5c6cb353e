"""The e-graph matcher (zyx_b200/csrc/host/matcher.hpp through the C ABI of include/zyxb_host.h) on node lists transcribed from
the reference's Tensor::dot, Linear::forward, MultiheadAttention::forward, Tensor::conv, softmax, ln_softmax, LayerNorm::forward,
the reductions, cross_entropy, mse_loss, the elementwise functions, SGD::update, Adam::update and AdamW::update
(tests/zyx_trace.py): the emitted descriptor must equal the hand-written one the training plans (or a caller of
zyx_b200.backend's descriptor builders) create for the same operation, and the launch arguments must be the stored tensors
(loads first, then stores).  CPU only; the GPU run of a matched descriptor is in tests/test_gpu_matcher.py."""
import math

import pytest

from tests.zyx_trace import LayerNorm, Linear, T, adam_update, adamw_update, sgd_update
from zyx_b200 import _lib as L
from zyx_b200 import backend as B
from zyx_b200.matcher import MGraph


def fields(struct):
    out = {}
    for name, _ in struct._fields_:
        v = getattr(struct, name)
        out[name] = v if isinstance(v, (int, float)) else None
    return out


def assert_same_gemm(got, want):
    a, b = fields(got.u.gemm), fields(want.u.gemm)
    for d in (a, b):
        d["alpha"] = d["alpha"] or 1.0
    assert got.kind == want.kind == L.KIND_GEMM and a == b, (a, b)


def assert_same_row(got, want):
    a, b = fields(got.u.rowreduce), fields(want.u.rowreduce)
    assert abs(a.pop("eps") - b.pop("eps")) <= 1e-12
    assert got.kind == want.kind == L.KIND_ROWREDUCE and a == b, (a, b)


@pytest.fixture()
def g():
    graph = MGraph()
    yield graph
    graph.close()


def by_pattern(matches):
    """pattern -> the last match of that pattern in topological order.  Tensor::dot closes with a reshape to the shape the
    reduce already has, so a matmul is matched at two classes (the Reduce's, as the reference does, and the reshape's, which
    is what the users of the result read); the later one is the reshape's."""
    return {m.pattern.decode(): m for m in matches}


@pytest.mark.parametrize("dtype", [L.F32, L.BF16, L.F16, L.I32])
def test_plain_matmul_is_the_reference_pattern(g, dtype):
    """Tensor::dot of two stored matrices: the NN form Graph::match_matmul recognises (vendor/matmul.rs:43-71)."""
    a, b = T.leaf(g, dtype, (96, 40)), T.leaf(g, dtype, (40, 72))
    out = a.dot(b)
    ms = g.match([out.cls])
    assert [m.pattern for m in ms] == [b"matmul_nn", b"matmul_nn"]      # at the Reduce's class and at the closing reshape's
    m = ms[1]
    assert_same_gemm(m.desc, B.gemm_desc(dtype, 96, 72, 40))
    assert list(m.inputs[:m.n_inputs]) == [a.cls, b.cls] and list(m.outputs[:m.n_outputs]) == [out.cls]
    assert g.info(out.cls)[2] == 1                      # a Node::Kernel alternative now sits in the output class


def test_linear_forward_is_nt_on_the_stored_weight(g):
    """x.dot(W.t()) + b (zyx-nn/src/linear.rs:39-45): b of the matmul is the leaf W with trans_b, not the class W.t();
    the descriptor equals the one the Linear-stack plan creates for a last layer (bias epilogue)."""
    lin = Linear(g, L.BF16, 4096, 16384)
    x = T.leaf(g, L.BF16, (8192, 4096))
    y = lin.forward(x)
    m = by_pattern(g.match([y.cls]))
    assert set(m) == {"matmul_nt", "matmul_nt_bias"}   # the product alone is an alternative too; extraction picks
    mt = m["matmul_nt_bias"]
    assert_same_gemm(mt.desc, B.gemm_desc(L.BF16, 8192, 16384, 4096, trans_b=True, epilogue=L.EPI_BIAS))
    assert list(mt.inputs[:mt.n_inputs]) == [x.cls, lin.weight.cls, lin.bias.cls]
    assert list(mt.outputs[:mt.n_outputs]) == [y.cls]


@pytest.mark.parametrize("dtype,act", [(L.F32, "relu"), (L.BF16, "gelu"), (L.F16, "gelu")])
def test_linear_with_activation_and_the_stored_preactivation(g, dtype, act):
    """Hidden layers of the configurations: bias + ReLU (SimpleNet) and bias + GELU storing the pre-activation the backward
    pass reads (config 4) - exactly the forward descriptors of host/trainer.cpp."""
    lin = Linear(g, dtype, 784, 128)
    x = T.leaf(g, dtype, (64, 784))
    z = lin.forward(x)
    h = z.relu() if act == "relu" else z.gelu()
    m = by_pattern(g.match([h.cls, z.cls]))            # z is wanted too (the backward reads it)
    key = "matmul_nt_bias_" + act
    assert key in m, sorted(m)
    mt = m[key]
    epi = L.EPI_BIAS_RELU if act == "relu" else L.EPI_BIAS_GELU
    assert_same_gemm(mt.desc, B.gemm_desc(dtype, 64, 128, 784, trans_b=True, epilogue=epi, store_preact=act == "gelu"))
    assert list(mt.inputs[:mt.n_inputs]) == [x.cls, lin.weight.cls, lin.bias.cls]
    assert list(mt.outputs[:mt.n_outputs]) == ([h.cls, z.cls] if act == "gelu" else [h.cls])
    # without z among the outputs nothing else reads the pre-activation: one output
    g2 = MGraph()
    try:
        lin2, x2 = Linear(g2, dtype, 784, 128), T.leaf(g2, dtype, (64, 784))
        h2 = lin2.forward(x2).gelu()
        mt2 = by_pattern(g2.match([h2.cls]))["matmul_nt_bias_gelu"]
        assert mt2.desc.u.gemm.store_preact == 0 and mt2.n_outputs == 1
    finally:
        g2.close()


def test_batched_matmul_shared_and_per_batch_operands_and_scale(g):
    """Rank > 2 (attention's per-head products as [B*H, T, D] tensors): batch strides; a shared right operand has stride 0;
    `* 1/sqrt(d)` after the product (multi_head_attention.rs:198-199) becomes alpha."""
    q, k = T.leaf(g, L.BF16, (12, 256, 64)), T.leaf(g, L.BF16, (12, 256, 64))
    s = q.dot(k.t()) * (1.0 / math.sqrt(64.0))
    m = by_pattern(g.match([s.cls]))
    mt = m["matmul_nt_batched"]
    assert mt.outputs[0] == s.cls
    assert g.match([s.cls]) == []                         # a second pass: the classes already hold kernels, nothing new
    want = B.gemm_desc(L.BF16, 256, 256, 64, batch=12, trans_b=True, alpha=1.0 / math.sqrt(64.0))
    a, b = fields(mt.desc.u.gemm), fields(want.u.gemm)
    assert abs(a.pop("alpha") - b.pop("alpha")) <= 1e-3 * b.get("alpha", 1) + 1e-3 and a == b
    assert list(mt.inputs[:2]) == [q.cls, k.cls]
    g3 = MGraph()
    try:
        a3, w3 = T.leaf(g3, L.F32, (6, 40, 24)), T.leaf(g3, L.F32, (24, 56))
        o3 = a3.dot(w3)
        m3 = g3.match([o3.cls])[-1]
        assert m3.pattern == b"matmul_nn" and m3.outputs[0] == o3.cls          # one matrix for the whole batch: 6 * 40 rows
        assert_same_gemm(m3.desc, B.gemm_desc(L.F32, 240, 56, 24))
    finally:
        g3.close()


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_transposed_left_operand_is_read_where_it_lies(g, dtype):
    """`dz.t().dot(x)`, a Linear's weight gradient written by hand: the left operand of the program is the stored dz with
    trans_a, the descriptor the Linear-stack plan creates for its weight-gradient launch (host/trainer.cpp); with `w.t()` on
    the right as well both flags are set; a transposed rank-3 left operand against a shared matrix keeps its batch (stride 0 on
    the right), where an untransposed one folds its batch into the rows."""
    dz, x = T.leaf(g, dtype, (8192, 512)), T.leaf(g, dtype, (8192, 384))
    dw = dz.t().dot(x)
    m = g.match([dw.cls])[-1]
    assert m.pattern == b"matmul_tn" and m.outputs[0] == dw.cls
    assert_same_gemm(m.desc, B.gemm_desc(dtype, 512, 384, 8192, trans_a=True))
    assert list(m.inputs[:m.n_inputs]) == [dz.cls, x.cls]
    w = T.leaf(g, dtype, (640, 8192))
    tt = dz.t().dot(w.t())
    m = g.match([tt.cls])[-1]
    assert m.pattern == b"matmul_tt"
    assert_same_gemm(m.desc, B.gemm_desc(dtype, 512, 640, 8192, trans_a=True, trans_b=True))
    assert list(m.inputs[:m.n_inputs]) == [dz.cls, w.cls]
    a3, w3 = T.leaf(g, dtype, (6, 24, 40)), T.leaf(g, dtype, (24, 56))
    o3 = a3.t().dot(w3)
    m = g.match([o3.cls])[-1]
    assert m.pattern == b"matmul_tn_batched"
    assert_same_gemm(m.desc, B.gemm_desc(dtype, 40, 56, 24, batch=6, trans_a=True, stride_b=0))
    assert list(m.inputs[:m.n_inputs]) == [a3.cls, w3.cls]
    # a permute that is not the exchange of the last two axes stays an operand of its own (the kernel has no such view)
    a4 = T.leaf(g, dtype, (24, 6, 40))
    o4 = a4.permute([1, 0, 2]).dot(T.leaf(g, dtype, (40, 56)))
    m = g.match([o4.cls])[-1]
    assert m.pattern == b"matmul_nn" and m.inputs[0] != a4.cls              # (its 6 x 24 rows folded against the shared right operand)


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_softmax_and_ln_softmax(g, dtype):
    x = T.leaf(g, dtype, (8192, 32768))
    y, z = x.softmax(), x.ln_softmax()
    m = by_pattern(g.match([y.cls, z.cls]))
    assert_same_row(m["softmax"].desc, B.rowreduce_desc(L.RR_SOFTMAX, dtype, 8192, 32768))
    assert_same_row(m["ln_softmax"].desc, B.rowreduce_desc(L.RR_LN_SOFTMAX, dtype, 8192, 32768))
    for key, out in (("softmax", y), ("ln_softmax", z)):
        assert list(m[key].inputs[:m[key].n_inputs]) == [x.cls] and m[key].outputs[0] == out.cls
    # a rank-3 input: rows are every leading extent
    x3 = T.leaf(g, dtype, (4, 16, 128))
    m3 = by_pattern(g.match([x3.softmax().cls]))
    assert_same_row(m3["softmax"].desc, B.rowreduce_desc(L.RR_SOFTMAX, dtype, 64, 128))


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("weight,bias", [(True, True), (True, False), (False, False)])
def test_layernorm(g, dtype, weight, bias):
    """LayerNorm::forward (zyx-nn/src/layer_norm.rs:95-135): two means, the unbiased variance (divisor n - 1), eps, affine."""
    ln = LayerNorm(g, dtype, 32768, eps=1e-5, weight=weight, bias=bias)
    x = T.leaf(g, dtype, (8192, 32768))
    y = ln.forward(x)
    m = by_pattern(g.match([y.cls]))
    assert "layernorm" in m, sorted(m)
    mt = m["layernorm"]
    assert_same_row(mt.desc, B.rowreduce_desc(L.RR_LAYERNORM, dtype, 8192, 32768, eps=1e-5, has_weight=weight, has_bias=bias))
    want_in = [x.cls] + ([ln.weight.cls] if weight else []) + ([ln.bias.cls] if bias else [])
    assert list(mt.inputs[:mt.n_inputs]) == want_in and mt.outputs[0] == y.cls


def test_plain_reductions(g):
    x = T.leaf(g, L.F32, (100, 333))
    s, mx, mean = x.sum([-1]), x.max([-1]), x.mean([-1])
    m = by_pattern(g.match([s.cls, mx.cls, mean.cls]))
    assert_same_row(m["sum"].desc, B.rowreduce_desc(L.RR_SUM, L.F32, 100, 333))
    assert_same_row(m["max"].desc, B.rowreduce_desc(L.RR_MAX, L.F32, 100, 333))
    assert_same_row(m["mean"].desc, B.rowreduce_desc(L.RR_MEAN, L.F32, 100, 333))


def test_min_is_the_inverted_max(g):
    """ReduceOp::Min is `inverse().max().inverse()` (reduce_ops.rs:33-42, 93-99): a negation around the max of the negated
    tensor for floats, a bitwise not for integers; the row program takes the tensor itself."""
    for dtype in (L.F32, L.BF16, L.I32):
        x = T.leaf(g, dtype, (40, 96))
        lo, lo_keep = x.min([-1]), x.min([-1], keepdim=True)
        at = {m.outputs[0]: m for m in g.match([lo.cls, lo_keep.cls])}
        for out in (lo, lo_keep):
            m = at[out.cls]
            assert m.pattern == b"min" and list(m.inputs[:m.n_inputs]) == [x.cls]
            assert_same_row(m.desc, B.rowreduce_desc(L.RR_MIN, dtype, 40, 96))


def test_sgd_update_of_simplenet_is_one_multi_tensor_program(g):
    shapes = [(128, 784), (128,), (10, 128), (10,)]
    params = [T.leaf(g, L.F32, s) for s in shapes]
    grads = [T.leaf(g, L.F32, s) for s in shapes]
    new = sgd_update(params, grads, 0.01)
    ms = g.match([t.cls for t in new])
    assert [m.pattern for m in ms] == [b"sgd"]
    o = ms[0].desc.u.optim
    assert (ms[0].desc.kind, o.algo, o.dtype, o.n_tensors) == (L.KIND_OPTIM, L.OPT_SGD, L.F32, 4)
    assert [o.numel[i] for i in range(4)] == [100352, 128, 1280, 10] and abs(o.lr - 0.01) < 1e-9 and o.momentum == 0 and o.weight_decay == 0
    assert list(ms[0].inputs[:8]) == [t.cls for t in params] + [t.cls for t in grads]
    assert list(ms[0].outputs[:4]) == [t.cls for t in new]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
@pytest.mark.parametrize("step", [1, 7])
def test_adamw_update_is_one_multi_tensor_program(g, dtype, step):
    """AdamW::update (zyx-optim/src/adamw.rs:51-97): hyper-parameters are read back from the graph's constants; on the first
    step the moment buffers do not exist yet (adamw.rs:60-71), so they are outputs only."""
    shapes = [(16384, 4096), (16384,), (4096, 16384), (4096,)]
    params = [T.leaf(g, dtype, s) for s in shapes]
    grads = [T.leaf(g, dtype, s) for s in shapes]
    m = [T.leaf(g, dtype, s) for s in shapes] if step > 1 else None
    v = [T.leaf(g, dtype, s) for s in shapes] if step > 1 else None
    new_p, new_m, new_v = adamw_update(params, grads, m, v, step, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    ms = g.match([t.cls for t in new_p + new_m + new_v])
    assert [x.pattern for x in ms] == [b"adamw" if step > 1 else b"adamw_first_step"]
    mt = ms[0]
    o = mt.desc.u.optim
    assert (o.algo, o.dtype, o.n_tensors) == (L.OPT_ADAMW, dtype, 4)
    assert [o.numel[i] for i in range(4)] == [16384 * 4096, 16384, 4096 * 16384, 4096]
    assert abs(o.lr - 1e-3) < 1e-9 and abs(o.weight_decay - 0.01) < 1e-6 and abs(o.beta1 - 0.9) < 1e-6 and abs(o.beta2 - 0.999) < 1e-6
    assert abs(o.eps - 1e-8) < 1e-12 and o.standard == 0
    want_in = [t.cls for t in params] + [t.cls for t in grads] + ([t.cls for t in m] + [t.cls for t in v] if step > 1 else [])
    assert list(mt.inputs[:mt.n_inputs]) == want_in
    want_out = [c for trio in zip(new_p, new_m, new_v) for c in (trio[0].cls, trio[1].cls, trio[2].cls)]
    assert list(mt.outputs[:mt.n_outputs]) == want_out


def test_what_is_not_a_pattern_is_left_alone(g):
    wrong_k = T.leaf(g, L.F32, (8, 5)).reshape((8, 1, 5)).expand((8, 3, 5)) * T.leaf(g, L.F32, (3, 5)).reshape((1, 3, 5)).expand((8, 3, 5))
    d = wrong_k.sum([-1])                       # product and sum, but the right operand is not a transposed [k, n] tensor
    i = T.leaf(g, L.I32, (32, 16))
    assert g.match([d.cls, (i * i + i).cls]) == []         # nor is there an elementwise program for integers
    # a bf16 tensor cast to f32 by the user and summed: the f32 row sum reads the *cast* class, never the bf16 leaf (the 16-bit
    # kernel would round the result), and the cast it now depends on becomes a program of its own
    leaf = T.leaf(g, L.BF16, (8, 4))
    wide = leaf.cast(L.F32)
    ms = g.match([wide.sum([-1]).cls])
    assert [m.pattern for m in ms] == [b"sum", b"cast"]
    assert ms[0].desc.u.rowreduce.dtype == L.F32 and ms[0].inputs[0] == wide.cls != leaf.cls
    e = ms[1].desc.u.eltwise
    assert (e.op, e.dtype, e.dtype_out, e.numel) == (L.EW_CAST, L.BF16, L.F32, 32) and ms[1].inputs[0] == leaf.cls and ms[1].outputs[0] == wide.cls


def test_constructor_arguments_are_validated(g):
    x = g.leaf(L.F32, (4, 5))
    with pytest.raises(ValueError):
        g.reshape(x, (3, 7))
    with pytest.raises(ValueError):
        g.expand(x, (4, 6))
    with pytest.raises(ValueError):
        g.permute(x, (0, 0))
    with pytest.raises(ValueError):
        g.binary(x, g.leaf(L.F32, (5, 4)), 0)
    with pytest.raises(ValueError):
        g.reduce(x, 0, (2,))


def test_mask_free_attention_core_is_one_fused_program(g):
    """q, k, v [b, t, h*128] -> head split, scores * scale, softmax, .matmul(v), heads merged: the fused attention program on
    the three stored tensors.  Outside the kernel's shapes (f32, head dimension 64) the same graph yields its separate
    batched matmuls and the softmax instead."""
    from tests.zyx_trace import attention_core
    q, k, v = (T.leaf(g, L.BF16, (2, 256, 512)) for _ in range(3))
    out = attention_core(q, k, v, heads=4)
    ms = g.match([out.cls])
    att = [m for m in ms if m.pattern == b"attention"]
    # the inner classes keep their own alternatives (the scores' matmul, the softmax, ...), as in an e-graph; the class of
    # the merged result holds the fused program, and extraction takes the cheaper cover
    assert len(att) == 1 and att[0].outputs[0] == out.cls and not any(m.outputs[0] == out.cls for m in ms if m.pattern != b"attention")
    m = att[0]
    assert m.desc.kind == L.KIND_ATTENTION
    a = m.desc.u.attention
    assert (a.dtype, a.batch, a.heads, a.seq, a.head_dim, a.causal) == (L.BF16, 2, 4, 256, 128, 0)
    assert abs(a.scale - 1.0 / math.sqrt(128)) < 1e-3
    assert list(m.inputs[:m.n_inputs]) == [q.cls, k.cls, v.cls] and list(m.outputs[:m.n_outputs]) == [out.cls]
    # head dimension 64: not the fused kernel's shape
    q2, k2, v2 = (T.leaf(g, L.BF16, (2, 256, 256)) for _ in range(3))
    out2 = attention_core(q2, k2, v2, heads=4)
    pats = sorted(m.pattern for m in g.match([out2.cls]))
    assert b"attention" not in pats and b"softmax" in pats and sum(p.startswith(b"matmul") for p in pats) >= 2


def test_mse_loss_is_the_two_stage_loss_program(g):
    y, t = T.leaf(g, L.F32, (96, 40)), T.leaf(g, L.F32, (96, 40))
    loss = y.mse_loss(t)
    m = by_pattern(g.match([loss.cls]))["mse_loss"]
    assert_same_row(m.desc, B.rowreduce_desc(L.RR_MSE, L.F32, 96, 40))
    assert list(m.inputs[:m.n_inputs]) == [y.cls, t.cls] and list(m.outputs[:m.n_outputs]) == [loss.cls]
    # 16-bit tensors: the reference's loss is a scalar of the tensor's dtype, the program's an f32 one - left to the generic path
    yb, tb = T.leaf(g, L.BF16, (96, 40)), T.leaf(g, L.BF16, (96, 40))
    assert "mse_loss" not in by_pattern(g.match([yb.mse_loss(tb).cls]))


@pytest.mark.parametrize("nesterov", [False, True])
@pytest.mark.parametrize("weight_decay", [0.0, 0.01])
def test_sgd_with_momentum_is_one_program_that_reads_and_writes_the_buffers(g, nesterov, weight_decay):
    """SGD::update with weight decay, momentum, dampening and Nesterov (sgd.rs:58-80) after the first step: one multi-tensor
    program over (p, g, buf) that writes p' and buf'; the match says which step it is, so that the program reads the buffers."""
    shapes = [(64, 32), (64,)]
    params = [T.leaf(g, L.F32, s) for s in shapes]
    grads = [T.leaf(g, L.F32, s) for s in shapes]
    bufs = [T.leaf(g, L.F32, s) for s in shapes]
    new_p, new_b = sgd_update(params, grads, 0.05, weight_decay=weight_decay, momentum=0.9, dampening=0.1, nesterov=nesterov, bufs=bufs)
    ms = g.match([t.cls for t in new_p] + [t.cls for t in new_b])
    assert [m.pattern for m in ms] == [b"sgd_nesterov" if nesterov else b"sgd_momentum"]
    m = ms[0]
    o = m.desc.u.optim
    assert (o.algo, o.dtype, o.n_tensors, o.nesterov) == (L.OPT_SGD, L.F32, 2, int(nesterov))
    for got, want in ((o.lr, 0.05), (o.momentum, 0.9), (o.dampening, 0.1), (o.weight_decay, weight_decay)):
        assert abs(got - want) < 1e-6
    assert [o.numel[i] for i in range(2)] == [64 * 32, 64]
    assert m.optim_step == 2
    assert list(m.inputs[:m.n_inputs]) == [t.cls for t in params] + [t.cls for t in grads] + [t.cls for t in bufs]
    assert list(m.outputs[:m.n_outputs]) == [new_p[0].cls, new_b[0].cls, new_p[1].cls, new_b[1].cls]


def test_first_sgd_step_with_momentum_is_the_plain_update(g):
    """On the first step the reference keeps the gradient itself as the momentum buffer: no node is added, the update is the
    plain one (with its weight decay) and the buffer's class is the decayed gradient's."""
    p, gr = T.leaf(g, L.F32, (30, 20)), T.leaf(g, L.F32, (30, 20))
    new_p, new_b = sgd_update([p], [gr], 0.1, weight_decay=0.02, momentum=0.9, bufs=None)
    ms = [m for m in g.match([new_p[0].cls]) if m.pattern.startswith(b"sgd")]
    assert [m.pattern for m in ms] == [b"sgd"]
    o = ms[0].desc.u.optim
    assert abs(o.weight_decay - 0.02) < 1e-7 and o.momentum == 0.0 and ms[0].optim_step == 1
    assert list(ms[0].inputs[:2]) == [p.cls, gr.cls]


def test_adamw_match_names_its_step(g):
    shapes = [(16, 8)]
    for step in (1, 2, 7, 40):
        params = [T.leaf(g, L.F32, s) for s in shapes]
        grads = [T.leaf(g, L.F32, s) for s in shapes]
        m = [T.leaf(g, L.F32, s) for s in shapes] if step > 1 else None
        v = [T.leaf(g, L.F32, s) for s in shapes] if step > 1 else None
        new_p, new_m, new_v = adamw_update(params, grads, m, v, step)
        ms = g.match([t.cls for t in new_p + new_m + new_v])
        assert [x.optim_step for x in ms if x.pattern.startswith(b"adamw")] == [step]


@pytest.mark.parametrize("step,weight_decay", [(1, 0.0), (5, 0.0), (5, 0.02)])
def test_adam_update_is_one_multi_tensor_program(g, step, weight_decay):
    """Adam::update (adam.rs:66-101, no amsgrad): L2 weight decay inside the gradient, p' = p - lr * mh / (sqrt(vh) + eps)."""
    shapes = [(24, 16), (24,)]
    params = [T.leaf(g, L.F32, s) for s in shapes]
    grads = [T.leaf(g, L.F32, s) for s in shapes]
    m = [T.leaf(g, L.F32, s) for s in shapes] if step > 1 else None
    v = [T.leaf(g, L.F32, s) for s in shapes] if step > 1 else None
    new_p, new_m, new_v = adam_update(params, grads, m, v, step, lr=2e-3, betas=(0.9, 0.99), eps=1e-7, weight_decay=weight_decay)
    ms = g.match([t.cls for t in new_p + new_m + new_v])
    assert [x.pattern for x in ms] == [b"adam" if step > 1 else b"adam_first_step"]
    mt = ms[0]
    o = mt.desc.u.optim
    assert (o.algo, o.n_tensors, mt.optim_step) == (L.OPT_ADAM, 2, step)
    for got, want in ((o.lr, 2e-3), (o.beta1, 0.9), (o.beta2, 0.99), (o.eps, 1e-7), (o.weight_decay, weight_decay)):
        assert abs(got - want) <= 1e-6 * max(1.0, abs(want)), (got, want)
    want_in = [t.cls for t in params] + [t.cls for t in grads] + ([t.cls for t in m] + [t.cls for t in v] if step > 1 else [])
    assert list(mt.inputs[:mt.n_inputs]) == want_in
    assert list(mt.outputs[:mt.n_outputs]) == [c for trio in zip(new_p, new_m, new_v) for c in (trio[0].cls, trio[1].cls, trio[2].cls)]


@pytest.mark.parametrize("dtype", [L.F32, L.BF16])
def test_var_std_and_column_sums(g, dtype):
    """var / std over the last axis (reduce_ops.rs:111-130) with their correction, and x.sum([0]) of a matrix - the bias
    gradient of a Linear layer - as the column-sum program."""
    x = T.leaf(g, dtype, (48, 320))
    v0, v1, sd, cs = x.var([-1], correction=0), x.var([-1]), x.std([-1]), x.sum([0])
    ms = g.match([v0.cls, v1.cls, sd.cls, cs.cls])
    at = {m.outputs[0]: m for m in ms}
    for out, pattern, op, corr in ((v0, b"var", L.RR_VAR, 0), (v1, b"var", L.RR_VAR, 1), (sd, b"std", L.RR_STD, 1)):
        m = at[out.cls]
        assert m.pattern == pattern and list(m.inputs[:m.n_inputs]) == [x.cls]
        assert_same_row(m.desc, B.rowreduce_desc(op, dtype, 48, 320, correction=corr))
    m = at[cs.cls]
    assert m.pattern == b"colsum" and list(m.inputs[:m.n_inputs]) == [x.cls]
    assert_same_row(m.desc, B.rowreduce_desc(L.RR_COLSUM, dtype, 48, 320))


def test_constant_index_tensors_are_folded(g):
    """Tensor::arange is `full(step).cumsum(0) + start - step` and a cumsum is a padded, pooled sum (tensor/mod.rs:773-781,
    reduce_ops.rs:1076-1091): the mirror carries Pad nodes and folds such constant subgraphs to their values; anything that
    reads a stored tensor has no constant value."""
    assert g.const_value(T.arange(g, 0, 10, 1).cls) == [float(i) for i in range(10)]
    assert g.const_value(T.arange(g, 3, 23, 4).cls) == [3.0, 7.0, 11.0, 15.0, 19.0]
    ones = T.full(g, [2, 3], 1, L.I32)
    assert g.const_value(ones.pad_zeros([(1, 0), (0, 2)]).cls) == [0, 0, 0, 0, 0] + [1, 1, 1, 0, 0] * 2
    assert g.const_value(T.arange(g, 0, 6, 1).reshape([2, 3]).t().slice([(1, 3), (0, 2)]).cls) == [1.0, 4.0, 2.0, 5.0]
    assert g.const_value(T.arange(g, 0, 4, 1).repeat([2]).cls) == [0.0, 1.0, 2.0, 3.0] * 2
    assert g.const_value(T.arange(g, 1, 5, 1).cumsum(0).cls) == [1.0, 3.0, 6.0, 10.0]
    assert g.const_value((T.arange(g, 0, 4, 1).cast(L.F32) * 0.5).cast(L.I32).cls) == [0.0, 0.0, 1.0, 1.0]
    for r, c, diagonal in ((4, 4, 1), (3, 5, 0), (5, 3, 2), (4, 4, -1)):      # Tensor::tri, what tril / triu and a causal mask select with
        want = [float(col >= row + diagonal) for row in range(r) for col in range(c)]
        assert g.const_value(T.tri(g, r, c, diagonal, L.BOOL).cls) == want, (r, c, diagonal)
    labels = T.leaf(g, L.I32, (4,))
    assert g.const_value(labels.unsqueeze(1).one_hot_along_dim(3, 1).cls) is None
    assert g.const_value(T.arange(g, 0, 3000, 1).cls) is None          # the pooled intermediate is past the folding limit
    with pytest.raises(ValueError):
        g.pad(labels.cls, 0, -2, 0)                                    # nothing of the axis would be left


def test_cross_entropy_with_class_indices_is_the_loss_program(g):
    """logits.cross_entropy(labels, Mean) as SimpleNet's training loop calls it (zyx-examples/examples/mnist.rs:66-67;
    tensor/mod.rs:1639-1656): one program reading the logits and the i32 labels, writing the per-sample losses and their mean
    - the descriptor of the Linear-stack plan's loss launch (host/trainer.cpp).  The one-hot matrix is recognised by folding
    its arange; the log-probabilities and the per-sample sum stay matched on their own as alternatives."""
    logits, labels = T.leaf(g, L.F32, (64, 10)), T.leaf(g, L.I32, (64,))
    loss, per_sample = logits.cross_entropy(labels)
    ms = g.match([loss.cls])
    m = by_pattern(ms)["cross_entropy"]
    assert_same_row(m.desc, B.rowreduce_desc(L.RR_CROSS_ENTROPY, L.F32, 64, 10))
    assert list(m.inputs[:m.n_inputs]) == [logits.cls, labels.cls]
    assert list(m.outputs[:m.n_outputs]) == [per_sample.cls, loss.cls]
    assert g.info(loss.cls)[2] == 1 and g.info(per_sample.cls)[2] >= 1      # Node::Kernel alternatives in both output classes
    assert {"ln_softmax", "sum"} <= set(by_pattern(ms))


def test_what_only_looks_like_a_one_hot_is_not_the_loss_program(g):
    """The comparison must be against 0 .. classes-1 along the class axis with i32 labels along the rows: an arange that starts
    at 1, labels of another integer type (the program reads i32), labels laid along the class axis of a square problem, and a
    stored one-hot matrix of floats all fall back to the separate row programs."""
    def patterns(build):
        g2 = MGraph()
        try:
            return set(by_pattern(g2.match([build(g2).cls])))
        finally:
            g2.close()

    def shifted_arange(g2):
        x, y = T.leaf(g2, L.F32, (32, 8)), T.leaf(g2, L.I32, (32,))
        target = y.unsqueeze(1).equal(T.arange(g2, 1, 9, 1).cast(L.I32))
        return (x.ln_softmax([1]).neg() * target).sum([1]).mean_all()

    def wide_labels(g2):
        x, y = T.leaf(g2, L.F32, (32, 8)), T.leaf(g2, L.I64, (32,))
        return x.cross_entropy(y)[0]

    def labels_along_the_classes(g2):
        x, y = T.leaf(g2, L.F32, (8, 8)), T.leaf(g2, L.I32, (8,))
        target = y.unsqueeze(0).equal(T.arange(g2, 0, 8, 1).cast(L.I32).reshape([8, 1]))
        return (x.ln_softmax([1]).neg() * target).sum([1]).mean_all()

    def stored_one_hot(g2):
        x, t = T.leaf(g2, L.F32, (32, 8)), T.leaf(g2, L.F32, (32, 8))
        return x.cross_entropy(t)[0]

    for build in (shifted_arange, wide_labels, labels_along_the_classes, stored_one_hot):
        got = patterns(build)
        assert "cross_entropy" not in got and "ln_softmax" in got, (build.__name__, got)


def test_matched_cross_entropy_launches_through_the_abi(g):
    """From the match to a launch without a GPU: the descriptor goes to zyxb_program_create and the matched classes name the
    launch arguments (loads, then stores) - here against the host-memory stand-in of the ABI (tests/fake), whose loss is
    computed in float64; the same path on the device is tests/test_gpu_matcher.py."""
    import ctypes as C

    import numpy as np

    from tests.fake.harness import Fake

    logits, labels = T.leaf(g, L.F32, (48, 10)), T.leaf(g, L.I32, (48,))
    loss, per_sample = logits.cross_entropy(labels)
    m = by_pattern(g.match([loss.cls]))["cross_entropy"]
    rng = np.random.default_rng(5)
    values = {logits.cls: rng.standard_normal((48, 10)).astype(np.float32), labels.cls: rng.integers(0, 10, 48).astype(np.int32)}
    fake = Fake()
    prog = C.c_uint32()
    assert fake.lib.zyxb_program_create(fake.ctx, 0, C.byref(m.desc), C.byref(prog)) == L.OK, fake.last_error()
    bufs = []
    for cls in list(m.inputs[:m.n_inputs]) + list(m.outputs[:m.n_outputs]):
        nbytes = 4 * int(np.prod(g.info(cls)[1]) or 1)
        b = C.c_uint32()
        assert fake.lib.zyxb_alloc(fake.ctx, 0, nbytes, C.byref(b), None) == L.OK
        if cls in values:
            fake.upload(b.value, values[cls])
        bufs.append(b.value)
    args = (C.c_uint32 * len(bufs))(*bufs)
    assert fake.lib.zyxb_launch(fake.ctx, 0, prog.value, args, len(bufs), None, 0, None) == L.OK, fake.last_error()
    x = values[logits.cls].astype(np.float64)
    lse = np.log(np.exp(x - x.max(1, keepdims=True)).sum(1)) + x.max(1)
    want = lse - x[np.arange(48), values[labels.cls]]
    np.testing.assert_allclose(fake.download(bufs[2], (48,)), want, rtol=1e-6)
    np.testing.assert_allclose(fake.download(bufs[3], (1,)), [want.mean()], rtol=1e-6)


CONV_CASES = [
    # dtype, x [n,c,h,w], w [o,c,kh,kw], stride (h,w), dilation (h,w), padding as Tensor::conv takes it, (top,bottom,left,right), bias
    (L.BF16, (32, 256, 56, 56), (256, 256, 3, 3), (1, 1), (1, 1), (1,), (1, 1, 1, 1), True),
    (L.F32, (2, 3, 32, 32), (16, 3, 7, 7), (2, 2), (1, 1), (3,), (3, 3, 3, 3), False),
    (L.F16, (4, 8, 20, 24), (8, 8, 3, 3), (1, 1), (2, 2), (2,), (2, 2, 2, 2), True),
    (L.F32, (3, 5, 17, 19), (6, 5, 3, 2), (2, 1), (1, 2), (1, 2, 0, 3), (0, 3, 1, 2), True),      # (left, right, top, bottom)
    (L.BF16, (8, 64, 14, 14), (128, 64, 1, 1), (1, 1), (1, 1), (0,), (0, 0, 0, 0), False),
    (L.F32, (2, 3, 32, 32), (24, 3, 4, 4), (4, 4), (1, 1), (0,), (0, 0, 0, 0), True),              # stride = filter size
    (L.I32, (1, 2, 5, 9), (3, 2, 5, 3), (1, 2), (1, 1), (0,), (0, 0, 0, 0), False),               # one output row
    (L.F32, (2, 4, 9, 9), (4, 4, 3, 3), (2, 2), (1, 1), (0,), (0, 0, 0, 0), False),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "x".join(map(str, c[1])) + "_k" + "x".join(map(str, c[2][2:])))
def test_conv_is_recognised_by_what_its_view_reads(g, case):
    """Tensor::conv (tensor/mod.rs:2583-2680): the padded input goes through Tensor::pool's dozen movement ops, whose shapes
    change with every stride and dilation.  The matcher reads the padding off the Pad nodes, measures stride and dilation on the
    view and holds the whole view against `x[b, c, oy*stride + r*dil - pad, ..]`; the descriptor is the one a caller of the
    convolution program writes by hand (zyx_b200.backend.conv_desc)."""
    dtype, xs, ws, stride, dilation, padding, pads, has_bias = case
    x, w = T.leaf(g, dtype, xs), T.leaf(g, dtype, ws)
    b = T.leaf(g, dtype, (ws[0],)) if has_bias else None
    y = x.conv(w, b, stride=stride, dilation=dilation, padding=padding)
    assert tuple(y.shape) == tuple(B.conv_out_shape(xs, ws, stride, dilation, pads))
    ms = [m for m in g.match([y.cls]) if m.outputs[0] == y.cls]
    assert [m.pattern for m in ms] == [b"conv_bias" if has_bias else b"conv"]
    m = ms[0]
    got, want = fields(m.desc.u.conv), fields(B.conv_desc(dtype, xs, ws, stride, dilation, pads, has_bias=has_bias).u.conv)
    assert m.desc.kind == L.KIND_CONV and got == want, (got, want)
    assert list(m.inputs[:m.n_inputs]) == [x.cls, w.cls] + ([b.cls] if has_bias else [])


def test_views_that_are_not_the_convolution_window_are_left_alone(g):
    """Same shapes, same node kinds, different elements read: a filter applied to the transposed window, an image read
    transposed, two groups."""
    def conv_patterns(y):
        return [m.pattern for m in g.match([y.cls]) if m.pattern.startswith(b"conv")]

    x, w = T.leaf(g, L.F32, (2, 4, 12, 12)), T.leaf(g, L.F32, (6, 4, 3, 3))
    assert conv_patterns(x.conv(w, padding=(1,))) == [b"conv"]
    wt = w.t()
    m = next(m for m in g.match([x.conv(wt, padding=(1,)).cls]) if m.pattern == b"conv")
    assert list(m.inputs[:m.n_inputs]) == [x.cls, wt.cls]                            # a transposed filter is another filter class
    assert conv_patterns(x.t().conv(w, padding=(1,))) == []                          # the view reads x[.., col, row]: no program does
    # the window's taps exchanged under the filter: reads x[.., ox + r, oy + s] where the convolution reads x[.., oy + r, ox + s]
    pooled = x.rpad_zeros([(1, 1), (1, 1)]).pool([3, 3], 1, 1)                       # [2, 4, 12, 12, 3, 3]
    swapped = pooled.permute([0, 1, 3, 2, 5, 4])
    view = swapped.reshape([2, 1, 4, 1, 12, 12, 3, 3]).expand([2, 1, 4, 6, 12, 12, 3, 3]).permute([0, 1, 3, 4, 5, 2, 6, 7])
    y = (view * w.reshape([1, 1, 6, 1, 1, 4, 3, 3])).sum([-1, -2, -3], keepdim=True).reshape([2, 6, 12, 12])
    assert conv_patterns(y) == []
    xg, wg = T.leaf(g, L.F32, (2, 4, 12, 12)), T.leaf(g, L.F32, (6, 2, 3, 3))
    assert conv_patterns(xg.conv(wg, groups=2, padding=(1,))) == []


@pytest.mark.parametrize("dtype", [L.BF16, L.F32])
def test_unfused_attention_reads_and_writes_the_per_head_views_in_place(g, dtype):
    """Outside the fused kernel's shapes (head dimension 64, f32) attention stays three programs, and none of them needs a
    [b, h, t, d] copy: q, k, v are read as per-head views of the stored [b, t, h*d] tensors (row pitch h*d, heads d apart, a
    two-level batch), and the product with v is written straight into the merged [b, t, h*d] tensor - the descriptors of the
    transformer-block plan's unfused path (host/block.cpp: head_view_a / _b / _c, score_view_a / _c)."""
    nb, t, h, d = 2, 256, 4, 64
    e = h * d
    q, k, v = (T.leaf(g, dtype, (nb, t, e)) for _ in range(3))
    split = lambda x: x.reshape([nb, t, h, d]).permute([0, 2, 1, 3])
    scale = 1.0 / math.sqrt(d)
    scores = split(q).dot(split(k).t()) * scale
    probs = scores.softmax()
    merged = probs.dot(split(v)).permute([0, 2, 1, 3]).reshape([nb, t, e])
    at = {m.outputs[0]: m for m in g.match([merged.cls])}
    ms = at[scores.cls]
    assert ms.pattern == b"matmul_nt_batched_heads" and list(ms.inputs[:ms.n_inputs]) == [q.cls, k.cls]
    want = B.gemm_desc(dtype, t, t, d, batch=nb, batch_inner=h, trans_b=True, lda=e, stride_a=t * e, stride_a_inner=d,
                       ldb=e, stride_b=t * e, stride_b_inner=d, stride_c=h * t * t, stride_c_inner=t * t)
    got_f, want_f = fields(ms.desc.u.gemm), fields(want.u.gemm)
    assert abs(got_f.pop("alpha") - scale) <= 1e-2 * scale and want_f.pop("alpha") == 0.0 and got_f == want_f, (got_f, want_f)
    mp = at[probs.cls]
    assert mp.pattern == b"softmax" and list(mp.inputs[:mp.n_inputs]) == [scores.cls]
    assert_same_row(mp.desc, B.rowreduce_desc(L.RR_SOFTMAX, dtype, nb * h * t, t))
    mv = at[merged.cls]
    assert mv.pattern == b"matmul_nn_batched_heads" and list(mv.inputs[:mv.n_inputs]) == [probs.cls, v.cls]
    assert_same_gemm(mv.desc, B.gemm_desc(dtype, t, d, t, batch=nb, batch_inner=h, stride_a=h * t * t, stride_a_inner=t * t,
                                          ldb=e, stride_b=t * e, stride_b_inner=d, ldc=e, stride_c=t * e, stride_c_inner=d))


def test_elementwise_programs_are_matched_on_demand(g):
    """No larger pattern ends at these classes, and somebody needs them - they are outputs of the graph or inputs of a matched
    program - so each becomes one elementwise program (the descriptors of zyx_b200.backend.eltwise_desc) and its operands are
    looked at in turn.  Sub-expressions nobody asks for (the inside of a gelu, the terms of an optimizer update) are not offered."""
    a, b = T.leaf(g, L.F32, (32, 16)), T.leaf(g, L.F32, (32, 16))
    ab = a * b
    s1 = ab + a
    c = s1.exp()
    ms = g.match([c.cls])
    assert [(m.pattern, list(m.inputs[:m.n_inputs]), m.outputs[0]) for m in ms] == [
        (b"exp", [s1.cls], c.cls), (b"add", [ab.cls, a.cls], s1.cls), (b"mul", [a.cls, b.cls], ab.cls)]
    for m, op in zip(ms, (L.EW_EXP, L.EW_ADD, L.EW_MUL)):
        assert m.desc.kind == L.KIND_ELTWISE and fields(m.desc.u.eltwise) == fields(B.eltwise_desc(op, L.F32, 512).u.eltwise)
    assert g.match([c.cls]) == []                                   # every class on the way now holds its program
    x = T.leaf(g, L.BF16, (64, 48))
    bias = T.leaf(g, L.BF16, (48,))
    outs = {"gelu": x.gelu(), "relu": x.relu(), "tanh": x.tanh(), "sigmoid": x.exp() / (x.exp() + 1), "scale": x * 0.25,
            "sub": x - x.relu(), "bias_add": x + bias, "cast": x.cast(L.F32)}
    at = {m.outputs[0]: m for m in g.match([t.cls for t in outs.values()])}
    ops = {"gelu": L.EW_GELU, "relu": L.EW_RELU, "tanh": L.EW_TANH, "sigmoid": L.EW_SIGMOID, "scale": L.EW_SCALE, "sub": L.EW_SUB,
           "bias_add": L.EW_BIAS_ADD, "cast": L.EW_CAST}
    for name, t in outs.items():
        m = at[t.cls]
        assert m.pattern == name.encode(), (name, m.pattern)
        want = B.eltwise_desc(ops[name], L.BF16, 64 * 48, p0=0.25 if name == "scale" else 0.0, cols=48 if name == "bias_add" else 0,
                              dtype_out=L.F32 if name == "cast" else None)
        assert fields(m.desc.u.eltwise) == fields(want.u.eltwise), name
        want_in = {"sub": [x.cls, outs["relu"].cls], "bias_add": [x.cls, bias.cls]}.get(name, [x.cls])
        assert list(m.inputs[:m.n_inputs]) == want_in, name
    assert len(at) == len(outs)                                     # x.relu() under the subtraction is the relu already matched
    # a bias laid along the rows is not the bias form; an optimizer update offers none of its terms
    col = T.leaf(g, L.BF16, (64,))
    assert g.match([(x + col.reshape([64, 1])).cls]) == []
    from tests.zyx_trace import sgd_update as sgd
    p, gr = T.leaf(g, L.F32, (50, 30)), T.leaf(g, L.F32, (50, 30))
    assert [m.pattern for m in g.match([sgd([p], [gr], 0.01, weight_decay=0.1)[0].cls])] == [b"sgd"]


def test_causal_self_attention_reads_its_fused_projection_in_place(g):
    """CausalSelfAttention::forward (zyx-nn/src/causal_self_attention.rs:36-71): q, k, v are slices of ONE [b, t, 3c] projection.
    The per-head products read them there - row pitch 3c, heads d apart, the slice's start as the argument's offset into the
    projection's buffer - and the dropout that is a division by one outside training is looked through."""
    from tests.zyx_trace import causal_self_attention
    nb, t, c, h = 2, 128, 256, 4
    d = c // h
    x = T.leaf(g, L.BF16, (nb, t, c))
    c_attn, c_proj = Linear(g, L.BF16, c, 3 * c), Linear(g, L.BF16, c, c)
    y, scores, att, merged, qkv = causal_self_attention(x, c_attn, c_proj, h)
    at = {m.outputs[0]: m for m in g.match([y.cls])}
    m = at[qkv.cls]                                       # the fused projection: one matmul over all b * t rows
    assert m.pattern == b"matmul_nt_bias" and list(m.inputs[:3]) == [x.cls, c_attn.weight.cls, c_attn.bias.cls]
    assert_same_gemm(m.desc, B.gemm_desc(L.BF16, nb * t, 3 * c, c, trans_b=True, epilogue=L.EPI_BIAS))
    ms = at[scores.cls]
    assert ms.pattern == b"matmul_nt_batched_heads" and list(ms.inputs[:2]) == [qkv.cls, qkv.cls]
    assert list(ms.input_offsets[:2]) == [0, c]           # q starts at feature 0, k at feature c of every row
    want = B.gemm_desc(L.BF16, t, t, d, batch=nb, batch_inner=h, trans_b=True, lda=3 * c, stride_a=t * 3 * c, stride_a_inner=d,
                       ldb=3 * c, stride_b=t * 3 * c, stride_b_inner=d, stride_c=h * t * t, stride_c_inner=t * t)
    got_f, want_f = fields(ms.desc.u.gemm), fields(want.u.gemm)
    assert abs(got_f.pop("alpha") - 1.0 / math.sqrt(d)) <= 1e-2 / math.sqrt(d) and want_f.pop("alpha") == 0.0 and got_f == want_f, (got_f, want_f)
    soft = next(m for m in at.values() if m.pattern == b"softmax")
    mv = at[merged.cls]
    assert mv.pattern == b"matmul_nn_batched_heads"
    assert list(mv.inputs[:2]) == [soft.outputs[0], qkv.cls] and list(mv.input_offsets[:2]) == [0, 2 * c]
    assert g.info(att.cls)[1] == (nb, h, t, t) and att.cls != soft.outputs[0]          # the division by 1 - p sits between them
    assert_same_gemm(mv.desc, B.gemm_desc(L.BF16, t, d, t, batch=nb, batch_inner=h, stride_a=h * t * t, stride_a_inner=t * t,
                                          ldb=3 * c, stride_b=t * 3 * c, stride_b_inner=d, ldc=c, stride_c=t * c, stride_c_inner=d))
    mo = at[y.cls]
    assert mo.pattern == b"matmul_nt_bias" and list(mo.inputs[:3]) == [merged.cls, c_proj.weight.cls, c_proj.bias.cls]
    # a slice that does not start on a 256-byte boundary of its buffer cannot be handed over as a view (zyxb_buffer_view): left alone
    x3 = T.leaf(g, L.BF16, (2, 32, 96))
    odd = causal_self_attention(x3, Linear(g, L.BF16, 96, 288), Linear(g, L.BF16, 96, 96), 4)
    at3 = {m.outputs[0]: m for m in g.match([odd[0].cls])}
    assert odd[1].cls not in at3 or list(at3[odd[1].cls].input_offsets[:2]) == [0, 0]
    # head dimension 128 would fit the fused program's tiles, but its q, k, v share one row pitch with its output: slices of a
    # wider tensor stay three programs
    x2 = T.leaf(g, L.BF16, (2, 256, 512))
    y2 = causal_self_attention(x2, Linear(g, L.BF16, 512, 1536), Linear(g, L.BF16, 512, 512), 4)[0]
    assert b"attention" not in {m.pattern for m in g.match([y2.cls])}


def cover(matches, outputs, leaves):
    """The programs a walk down from `outputs` uses (at each class the match found last, the largest pattern), in the order the
    walk meets them; every class on the way must be stored or produced."""
    producer = {}
    for m in matches:
        for o in m.outputs[:m.n_outputs]:
            producer[o] = m
    used, seen, need = [], set(), list(reversed(outputs))
    while need:
        c = need.pop()
        if c in seen or c in leaves:
            continue
        seen.add(c)
        assert c in producer, "class %d is needed and nothing produces it" % c
        m = producer[c]
        if not any(m is u for u in used):
            used.append(m)
        need.extend(reversed(m.inputs[:m.n_inputs]))
    return used


@pytest.mark.parametrize("norm_first", [True, False])
def test_a_whole_transformer_encoder_layer_is_covered(g, norm_first):
    """TransformerEncoderLayer::forward (zyx-nn/src/transformer_encoder_layer.rs:84-172; MultiheadAttention, two LayerNorms, the
    feed-forward pair with GELU, two residual additions, dropouts that are divisions by one outside training) traced as the
    reference builds it: the matched programs cover the graph - nothing is left for another device - and the cover is the eleven
    launches a hand-written plan would make."""
    from tests.zyx_trace import TransformerEncoderLayer
    layer = TransformerEncoderLayer(g, L.BF16, 512, 4, 2048, norm_first=norm_first)
    x = T.leaf(g, L.BF16, (2, 256, 512))
    y = layer.forward(x)
    ms = g.match([y.cls])
    assert g.uncovered([y.cls]) == []
    leaves = {x.cls}
    for lin in (layer.self_attn.q_proj, layer.self_attn.k_proj, layer.self_attn.v_proj, layer.self_attn.out_proj, layer.linear1, layer.linear2):
        leaves |= {lin.weight.cls, lin.bias.cls}
    for ln in (layer.norm1, layer.norm2):
        leaves |= {ln.weight.cls, ln.bias.cls}
    used = sorted(m.pattern.decode() for m in cover(ms, [y.cls], leaves))
    assert used == sorted(["layernorm"] * 2 + ["matmul_nt_bias"] * 5 + ["attention", "matmul_nt_bias_gelu"] + ["add"] * 2)
    # without the programs (a fresh mirror of the same graph, nothing matched yet) the output itself is what is missing
    g2 = MGraph()
    try:
        y2 = TransformerEncoderLayer(g2, L.BF16, 512, 4, 2048, norm_first=norm_first).forward(T.leaf(g2, L.BF16, (2, 256, 512)))
        assert g2.uncovered([y2.cls]) == [y2.cls]
    finally:
        g2.close()
    # a dropout probability other than zero leaves real divisions by 1 - p: scale programs (x * 1/(1 - p), the reciprocal the
    # reference's C backend forms under -ffast-math), and the attention stays three programs around the scaled probabilities
    g3 = MGraph()
    try:
        y3 = TransformerEncoderLayer(g3, L.BF16, 512, 4, 2048, dropout=0.125, norm_first=norm_first).forward(T.leaf(g3, L.BF16, (2, 256, 512)))
        ms3 = g3.match([y3.cls])
        assert g3.uncovered([y3.cls]) == []
        scales = [m for m in ms3 if m.pattern == b"scale"]
        assert len(scales) == 4 and all(abs(m.desc.u.eltwise.p0 - 1.0 / 0.875) < 1e-6 for m in scales)
        assert b"attention" not in {m.pattern for m in ms3}
    finally:
        g3.close()


def test_the_mnist_example_forward_loss_and_update_are_covered(g):
    """zyx-examples/examples/mnist.rs: `x.reshape([0, 784])`, Linear + relu, Linear, cross_entropy with class indices, and the
    SGD update with momentum of a later step.  Four programs cover it (the two layers, the loss, the update); the reshape of
    the stored batch is the batch's own buffer, so the first matmul reads the batch itself."""
    batch = T.leaf(g, L.F32, (128, 784))
    labels = T.leaf(g, L.I32, (128,))
    l1, l2 = Linear(g, L.F32, 784, 128), Linear(g, L.F32, 128, 10)
    logits = l2.forward(l1.forward(batch.reshape([128, 784])).relu())
    loss, _ = logits.cross_entropy(labels)
    params = [l1.weight, l1.bias, l2.weight, l2.bias]
    grads = [T.leaf(g, L.F32, p.shape) for p in params]          # what Tape::gradient hands to the optimizer
    bufs = [T.leaf(g, L.F32, p.shape) for p in params]
    new_p, new_b = sgd_update(params, grads, 0.01, momentum=0.9, bufs=bufs)
    outs = [loss.cls] + [t.cls for t in new_p + new_b]
    ms = g.match(outs)
    assert g.uncovered(outs) == []
    leaves = {t.cls for t in [batch, labels] + params + grads + bufs}
    used = cover(ms, outs, leaves)
    assert [m.pattern for m in used] == [b"cross_entropy", b"matmul_nt_bias", b"matmul_nt_bias_relu", b"sgd_momentum"]
    first = used[2]
    assert list(first.inputs[:3]) == [batch.cls, l1.weight.cls, l1.bias.cls]
    assert_same_gemm(first.desc, B.gemm_desc(L.F32, 128, 128, 784, trans_b=True, epilogue=L.EPI_BIAS_RELU))


def test_the_encoder_layer_at_the_transformer_configuration_size(g):
    """Batch 8, sequence 2048, d_model 2048, 16 heads of 128, feed-forward 8192 (the transformer-block configuration): covered,
    with the fused attention program at exactly that shape and the feed-forward matmuls at theirs."""
    from tests.zyx_trace import TransformerEncoderLayer
    layer = TransformerEncoderLayer(g, L.BF16, 2048, 16, 8192, norm_first=True)
    y = layer.forward(T.leaf(g, L.BF16, (8, 2048, 2048)))
    ms = g.match([y.cls])
    assert g.uncovered([y.cls]) == []
    a = next(m for m in ms if m.pattern == b"attention").desc.u.attention
    assert (a.dtype, a.batch, a.heads, a.seq, a.head_dim, a.causal) == (L.BF16, 8, 16, 2048, 128, 0) and abs(a.scale - 128 ** -0.5) < 1e-3
    up = next(m for m in ms if m.pattern == b"matmul_nt_bias_gelu")         # the batch folded into the rows: the plan's own launch
    assert_same_gemm(up.desc, B.gemm_desc(L.BF16, 8 * 2048, 8192, 2048, trans_b=True, epilogue=L.EPI_BIAS_GELU))


def test_a_small_convolutional_classifier_is_covered(g):
    """Conv2d::forward is Tensor::conv (zyx-nn/src/conv2d.rs:58-68): two strided convolutions with relu, the features flattened
    (a reshape: the same buffer) into a Linear, cross-entropy on top - six programs, nothing left over."""
    x, labels = T.leaf(g, L.F32, (16, 3, 32, 32)), T.leaf(g, L.I32, (16,))
    w1, b1 = T.leaf(g, L.F32, (8, 3, 3, 3)), T.leaf(g, L.F32, (8,))
    w2, b2 = T.leaf(g, L.F32, (16, 8, 3, 3)), T.leaf(g, L.F32, (16,))
    fc = Linear(g, L.F32, 16 * 8 * 8, 10)
    h1 = x.conv(w1, b1, stride=(2,), padding=(1,)).relu()                   # [16, 8, 16, 16]
    h2 = h1.conv(w2, b2, stride=(2,), padding=(1,)).relu()                  # [16, 16, 8, 8]
    loss, _ = fc.forward(h2.reshape([16, 16 * 8 * 8])).cross_entropy(labels)
    ms = g.match([loss.cls])
    assert g.uncovered([loss.cls]) == []
    leaves = {t.cls for t in (x, labels, w1, b1, w2, b2, fc.weight, fc.bias)}
    used = cover(ms, [loss.cls], leaves)
    assert [m.pattern for m in used] == [b"cross_entropy", b"matmul_nt_bias", b"relu", b"conv_bias", b"relu", b"conv_bias"]
    assert list(used[1].inputs[:1]) == [h2.cls]                              # the Linear reads the second relu's buffer through the reshape


def test_the_mnist_example_runs_from_its_graph_through_the_abi(g):
    """What B200Device::match_graph and ::launch do (shim/b200.rs), in Python against the host-memory stand-in of the ABI: match
    the traced graph, create one program per match of the cover, give every class a buffer, launch in dependency order with
    args = the matched inputs' buffers followed by the outputs' - an optimizer program on copies of the parameters, as the shim's
    launch does - and read the loss and the new parameters back.  They are the float64 values of the same step."""
    import ctypes as C

    import numpy as np

    from tests.fake.harness import Fake

    rng = np.random.default_rng(9)
    n = 32
    batch, labels = T.leaf(g, L.F32, (n, 784)), T.leaf(g, L.I32, (n,))
    l1, l2 = Linear(g, L.F32, 784, 128), Linear(g, L.F32, 128, 10)
    loss, _ = l2.forward(l1.forward(batch.reshape([n, 784])).relu()).cross_entropy(labels)
    params = [l1.weight, l1.bias, l2.weight, l2.bias]
    grads = [T.leaf(g, L.F32, p.shape) for p in params]
    new_p = sgd_update(params, grads, 0.05)
    outs = [loss.cls] + [t.cls for t in new_p]
    ms = g.match(outs)
    assert g.uncovered(outs) == []
    values = {batch.cls: rng.standard_normal((n, 784)).astype(np.float32), labels.cls: rng.integers(0, 10, n).astype(np.int32)}
    for p, gr in zip(params, grads):
        values[p.cls] = (0.05 * rng.standard_normal(p.shape)).astype(np.float32)
        values[gr.cls] = rng.standard_normal(gr.shape).astype(np.float32)
    fake = Fake()
    buffers = {}

    def buffer_of(cls):
        if cls not in buffers:
            nbytes = 4 * int(np.prod(g.info(cls)[1]) or 1)
            b = C.c_uint32()
            assert fake.lib.zyxb_alloc(fake.ctx, 0, nbytes, C.byref(b), None) == L.OK
            buffers[cls] = b.value
            if cls in values:
                fake.upload(b.value, values[cls])
        return buffers[cls]

    order, done = [], set()

    def schedule(m):                                    # operands before users
        if id(m) in done:
            return
        done.add(id(m))
        for c in m.inputs[:m.n_inputs]:
            if c not in values:
                schedule(producer[c])
        order.append(m)

    producer = {o: m for m in ms for o in m.outputs[:m.n_outputs]}
    for o in outs:
        schedule(producer[o])
    assert [m.pattern for m in order] == [b"matmul_nt_bias_relu", b"matmul_nt_bias", b"cross_entropy", b"sgd"]
    for m in order:
        prog = C.c_uint32()
        assert fake.lib.zyxb_program_create(fake.ctx, 0, C.byref(m.desc), C.byref(prog)) == L.OK, fake.last_error()
        ins = [buffer_of(c) for c in m.inputs[:m.n_inputs]]
        stores = [buffer_of(c) for c in m.outputs[:m.n_outputs]]
        if m.desc.kind == L.KIND_OPTIM:
            assert fake.lib.zyxb_program_set_step(fake.ctx, 0, prog.value, m.optim_step - 1) == L.OK
            t = m.desc.u.optim.n_tensors
            for i in range(t):                          # p -> p', then the program updates p' where it lies
                nbytes = 4 * int(np.prod(g.info(m.inputs[i])[1]))
                assert fake.lib.zyxb_d2d(fake.ctx, 0, ins[i], 0, 0, stores[i], 0, nbytes, None, 0, None) == L.OK
            ids = stores + ins[t:2 * t]
        else:
            ids = ins + stores
        args = (C.c_uint32 * len(ids))(*ids)
        assert fake.lib.zyxb_launch(fake.ctx, 0, prog.value, args, len(ids), None, 0, None) == L.OK, (m.pattern, fake.last_error())
    x = values[batch.cls].astype(np.float64)
    w1, b1, w2, b2 = (values[p.cls].astype(np.float64) for p in params)
    logits = np.maximum(x @ w1.T + b1, 0.0) @ w2.T + b2
    lse = np.log(np.exp(logits - logits.max(1, keepdims=True)).sum(1)) + logits.max(1)
    want_loss = (lse - logits[np.arange(n), values[labels.cls]]).mean()
    np.testing.assert_allclose(fake.download(buffers[loss.cls], (1,))[0], want_loss, rtol=1e-5)
    for p, gr, q in zip(params, grads, new_p):
        np.testing.assert_allclose(fake.download(buffers[q.cls], p.shape), values[p.cls] - 0.05 * values[gr.cls], rtol=1e-6, atol=1e-7)
        np.testing.assert_array_equal(fake.download(buffers[p.cls], p.shape), values[p.cls])      # the old parameters are untouched


def test_the_mlp_configuration_forward_loss_and_update_are_covered(g):
    """The Linear stack of the headline configuration (4096 -> 16384 -> 4096 -> 16384 -> 4096, GELU between, bf16, batch 8192, MSE
    in f32 on the cast output, AdamW at a later step): the forward is the plan's four matmuls with their epilogues, the update one
    multi-tensor program over the eight parameter tensors and their moments."""
    dims = [4096, 16384, 4096, 16384, 4096]
    x, target = T.leaf(g, L.BF16, (8192, dims[0])), T.leaf(g, L.F32, (8192, dims[-1]))
    layers = [Linear(g, L.BF16, a, b) for a, b in zip(dims, dims[1:])]
    h = x
    for i, lin in enumerate(layers):
        h = lin.forward(h)
        if i + 1 < len(layers):
            h = h.gelu()
    loss = h.cast(L.F32).mse_loss(target)
    params = [t for lin in layers for t in (lin.weight, lin.bias)]
    grads, m, v = ([T.leaf(g, L.BF16, p.shape) for p in params] for _ in range(3))
    new_p, new_m, new_v = adamw_update(params, grads, m, v, 7)
    outs = [loss.cls] + [t.cls for t in new_p + new_m + new_v]
    ms = g.match(outs)
    assert g.uncovered(outs) == []
    leaves = {t.cls for t in [x, target] + params + grads + m + v}
    used = cover(ms, outs, leaves)
    assert sorted(u.pattern.decode() for u in used) == sorted(["matmul_nt_bias_gelu"] * 3 + ["matmul_nt_bias", "cast", "mse_loss", "adamw"])
    upd = next(u for u in used if u.pattern == b"adamw")
    assert upd.desc.u.optim.n_tensors == 8 and upd.optim_step == 7 and upd.n_inputs == 32 and upd.n_outputs == 24
    first = next(u for u in used if u.inputs[0] == x.cls)
    assert_same_gemm(first.desc, B.gemm_desc(L.BF16, 8192, 16384, 4096, trans_b=True, epilogue=L.EPI_BIAS_GELU))


def test_a_residual_added_to_a_product_without_bias_is_the_add_epilogue(g):
    """`r + x.dot(w.t())` with no bias in between: the matmul adds the residual as it stores (the epilogue the block plan's
    backward uses for `dx1 + dz1.W1`); with a bias the addition stays an elementwise program after the biased matmul."""
    x, r = T.leaf(g, L.BF16, (256, 512)), T.leaf(g, L.BF16, (256, 384))
    lin = Linear(g, L.BF16, 512, 384, bias=False)
    y = r + lin.forward(x)
    m = next(m for m in g.match([y.cls]) if m.outputs[0] == y.cls)
    assert m.pattern == b"matmul_nt_add" and list(m.inputs[:m.n_inputs]) == [x.cls, lin.weight.cls, r.cls]
    assert_same_gemm(m.desc, B.gemm_desc(L.BF16, 256, 384, 512, trans_b=True, epilogue=L.EPI_ADD))
    biased = Linear(g, L.BF16, 512, 384)
    y2 = r + biased.forward(x)
    at = {m.outputs[0]: m.pattern for m in g.match([y2.cls])}
    assert at[y2.cls] == b"add"
