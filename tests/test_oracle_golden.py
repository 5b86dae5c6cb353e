"""Pins the CPU oracle to the reference's own known-answer tests (tests/golden)."""
import numpy as np

from oracle import oracle as zo
from tests.parity import ref_is_equal


def f32(x):
    return np.asarray(x, np.float32)


def test_softmax(golden):
    for case in golden["softmax"]:
        y = zo.softmax(zo.F32, f32(case["x"]))
        assert ref_is_equal(y, f32(case["y"])), case["src"]


def test_layernorm(golden):
    for case in golden["layernorm"]:
        y = zo.layernorm(zo.F32, f32(case["x"]), w=f32(case["weight"]), eps=case["eps"])
        assert ref_is_equal(y, f32(case["y"])), case["src"]


def test_cross_entropy(golden):
    for case in golden["cross_entropy"]:
        logits, labels = f32(case["logits"]), np.asarray(case["labels"], np.int32)
        want = f32(case["neg_ln_softmax_times_onehot"])
        ls = zo.ln_softmax(zo.F32, logits)
        onehot = (labels[:, None] == np.arange(logits.shape[1])[None, :]).astype(np.float32)
        assert ref_is_equal(-ls * onehot, want), case["src"]
        per, mean = zo.cross_entropy(logits, labels)
        assert ref_is_equal(per, want.sum(1)), case["src"]
        assert ref_is_equal(mean, [want.sum() / len(labels)])


def test_reduce_f32(golden):
    ops = {"sum": zo.RR_SUM, "max": zo.RR_MAX, "mean": zo.RR_MEAN, "var": zo.RR_VAR}
    for case in golden["reduce_f32"]:
        y = zo.row_reduce(ops[case["op"]], zo.F32, f32(case["x"]), correction=case["correction"])
        assert ref_is_equal(y, f32(case["y"])), case["src"]


def _int_input(case):
    rows, cols = case["rows"], case["cols"]
    if "x_fill" in case:
        return np.full((rows, cols), case["x_fill"], np.int32)
    return (np.arange(rows * cols, dtype=np.int32) + case["x_arange_from"]).reshape(rows, cols)


def test_reduce_i32(golden):
    ops = {"sum": zo.RR_SUM, "max": zo.RR_MAX}
    for case in golden["reduce_i32"]:
        y = zo.row_reduce(ops[case["op"]], zo.I32, _int_input(case))
        assert y.tolist() == case["y"], case["src"]


def test_matmul_small(golden):
    for case in golden["matmul_i32"]:
        c = zo.gemm(zo.I32, np.asarray(case["a"], np.int32), np.asarray(case["b"], np.int32))
        assert c.tolist() == case["c"], case["src"]
    for case in golden["matmul_f32"]:
        c = zo.gemm(zo.F32, f32(case["a"]), f32(case["b"]))
        assert ref_is_equal(c, f32(case["c"])), case["src"]


def test_matmul_i32_procedural(golden):
    g = golden["matmul_i32_procedural"]
    for m in g["m"]:
        for k in g["k"]:
            for n in g["n"]:
                x = (np.arange(m)[:, None] + np.arange(k)[None, :]).astype(np.int32)
                y = (np.arange(k)[:, None] - np.arange(n)[None, :]).astype(np.int32)
                want = (x.astype(np.int64) @ y.astype(np.int64)).astype(np.int32)
                assert np.array_equal(zo.gemm(zo.I32, x, y), want), (m, k, n)


def test_batched_matmul_i32_procedural(golden):
    g = golden["batched_matmul_i32_procedural"]
    for b in g["b"]:
        for m in g["m"]:
            for k in g["k"]:
                for n in g["n"]:
                    bb = np.arange(b)[:, None, None]
                    x = (bb + np.arange(m)[None, :, None] + np.arange(k)[None, None, :]).astype(np.int32)
                    y = (bb + np.arange(k)[None, :, None] - np.arange(n)[None, None, :]).astype(np.int32)
                    want = np.einsum("bmk,bkn->bmn", x.astype(np.int64), y.astype(np.int64)).astype(np.int32)
                    assert np.array_equal(zo.gemm(zo.I32, x, y), want), (b, m, k, n)


def test_bf16_matmul_procedural(golden):
    g = golden["bf16_matmul_procedural"]
    m, k, n = g["m"], g["k"], g["n"]
    xf = np.fmod(np.arange(m)[:, None] + np.arange(k)[None, :], 10).astype(np.float32)
    yf = np.fmod((np.arange(k)[:, None] - np.arange(n)[None, :]).astype(np.float32), 10).astype(np.float32)
    x, y = zo.to_bits(xf, zo.BF16), zo.to_bits(yf, zo.BF16)
    # expected as the reference test builds it: running sum rounded to bf16 after every add
    want = np.zeros((m, n), np.float32)
    for kk in range(k):
        want = zo.to_f32(zo.to_bits(want + xf[:, kk:kk + 1] * yf[kk:kk + 1, :], zo.BF16), zo.BF16)
    got = zo.to_f32(zo.gemm(zo.BF16, x, y), zo.BF16)
    assert ref_is_equal(got, want, rel=0.01, abs_tol=0.001)


def test_relu(golden):
    for case in golden["relu"]:
        y = zo.eltwise(zo.EW_RELU, zo.F32, f32(case["x"]))
        assert ref_is_equal(y, f32(case["y"])), case["src"]


def test_mlp_fwd_bwd_known_answer(golden):
    """2-layer ReLU MLP forward + backward built from oracle pieces, exact in f32 (small ints)."""
    g = golden["mlp_fwd_bwd_i32"]
    x, y = f32([g["x"]]), f32([g["y"]])
    w1, b1, w2, b2 = f32(g["w1"]), f32(g["b1"]), f32(g["w2"]), f32(g["b2"])
    h, z1 = zo.gemm(zo.F32, x, w1, bias=b1, epi=zo.EPI_BIAS_RELU, want_preact=True)
    o = zo.gemm(zo.F32, h, w2, bias=b2, epi=zo.EPI_BIAS)
    do = zo.eltwise(zo.EW_MSE_BWD, zo.F32, o, y, p0=1.0)          # d sum((o-y)^2) = 2 (o-y)
    dw2 = zo.gemm(zo.F32, h, do, ta=True)
    db2 = zo.colsum(zo.F32, do)
    dh = zo.gemm(zo.F32, do, w2, tb=True)
    dz1 = zo.eltwise(zo.EW_RELU_BWD, zo.F32, dh, z1)
    dw1 = zo.gemm(zo.F32, x, dz1, ta=True)
    db1 = zo.colsum(zo.F32, dz1)
    assert dw1.astype(np.int64).tolist() == g["w1_grad"]
    assert db1.astype(np.int64).tolist() == g["b1_grad"]
    assert dw2.astype(np.int64).tolist() == g["w2_grad"]
    assert db2.astype(np.int64).tolist() == g["b2_grad"]


def test_self_attention_known_answer(golden):
    g = golden["self_attention_f32"]
    w = f32(g["c_attn_weight_before_t"])          # [4, 12]; the test multiplies x by this matrix
    x = f32(g["x"])                                # [T=4, C=4]
    qkv = zo.gemm(zo.F32, x, w)                    # [4, 12]
    q, k, v = qkv[:, 0:4], qkv[:, 4:8], qkv[:, 8:12]
    # 4 heads of width 1: per head h, q/k/v are [T,1]
    out = np.zeros((4, 4), np.float32)
    for h in range(4):
        qh, kh, vh = (np.ascontiguousarray(t[:, h:h + 1]) for t in (q, k, v))
        att = zo.gemm(zo.F32, qh, kh, tb=True, alpha=1.0)
        att = zo.softmax(zo.F32, att)
        out[:, h:h + 1] = zo.gemm(zo.F32, att, vh)
    assert ref_is_equal(out, f32(g["y"]))


def test_rng_is_deterministic_and_in_range():
    r1, r2 = zo.Rng(42069), zo.Rng(42069)
    a, b = r1.rand(1000), r2.rand(1000)
    assert np.array_equal(a, b) and a.min() >= 0.0 and a.max() <= 1.0
    # splitmix64 seeding of xoshiro256++ (zyx/src/rng.rs:15-57): published first outputs of
    # splitmix64 for state 0 are the xoshiro state words for seed 0
    r0 = zo.Rng(0)
    assert [int(v) for v in r0.state] == [0xe220a8397b1dcdaf, 0x6e789e6aa1b965f4, 0x06c45d188009454f, 0xf88bb8a8724c81ec]
    n = zo.Rng(1).randn(20000)
    assert abs(float(n.mean())) < 0.05 and abs(float(n.std()) - 1.0) < 0.05


def test_bf16_store_truncates():
    x = f32([1.0, 1.00390625, 1.0078124, 0.9, 0.999, 1e-3, 0.99999])
    got = zo.to_f32(zo.to_bits(x, zo.BF16), zo.BF16)
    # bf16::from_f32 = bits >> 16 (zyx/src/scalar.rs:43-45): 0.9 -> 0.8984375, 0.999 -> 0.99609375
    assert got.tolist()[:5] == [1.0, 1.0, 1.0, 0.8984375, 0.99609375]
    assert got[6] == 0.99609375


def _tr(x, dtype=zo.BF16):
    """store-then-load in `dtype`: what the reference does to a value that passes through a bf16 buffer"""
    return zo.to_f32(zo.to_bits(np.asarray(x, np.float32), dtype), dtype)


def test_scalar_operands_are_cast():
    """The compiled oracle honours its own source: rank-0 scalars are truncated to the tensor dtype
    (an independent float32 numpy restatement of SGD / AdamW / layernorm agrees bit for bit)."""
    F = np.float32
    assert zo.const_cast(zo.BF16, 0.05) == 0.0498046875 and zo.const_cast(zo.BF16, 0.9) == 0.8984375
    p, g = zo.to_bits(F([-0.1240234375]), zo.BF16), zo.to_bits(F([0.2734375]), zo.BF16)
    zo.sgd(zo.BF16, p, g, None, lr=0.05)
    assert zo.to_f32(p, zo.BF16)[0] == F(-0.13671875)        # trunc(p - g * bf16(0.05)), not bf16(p - g * 0.05)

    rng = np.random.default_rng(3)
    n = 2000
    c = lambda v: F(zo.const_cast(zo.BF16, float(F(v))))
    # SGD with momentum and dampening, two steps
    p0, buf = _tr(rng.standard_normal(n)), np.zeros(n, F)
    pb, bb = zo.to_bits(p0, zo.BF16), np.zeros(n, np.uint16)
    pe = p0.copy()
    for step in (1, 2):
        g = _tr(rng.standard_normal(n) * 0.1)
        zo.sgd(zo.BF16, pb, zo.to_bits(g, zo.BF16), bb, lr=0.05, momentum=0.9, dampening=0.1, first=(step == 1))
        buf = _tr(g if step == 1 else (buf * c(0.9) + g * c(F(1.0) - F(0.1))).astype(F))
        pe = _tr((pe - buf * c(0.05)).astype(F))
        assert np.array_equal(zo.to_f32(pb, zo.BF16), pe) and np.array_equal(zo.to_f32(bb, zo.BF16), buf)
    # AdamW as the reference writes it, two steps
    pe, m, v = p0.copy(), np.zeros(n, F), np.zeros(n, F)
    pb, mb, vb = zo.to_bits(p0, zo.BF16), np.zeros(n, np.uint16), np.zeros(n, np.uint16)
    lr, wd, b1, b2, eps = F(1e-3), F(0.01), F(0.9), F(0.999), F(1e-8)
    for t in (1, 2):
        g = _tr(rng.standard_normal(n) * 0.1)
        zo.adam(zo.BF16, pb, zo.to_bits(g, zo.BF16), mb, vb, t, lr=1e-3, wd=0.01, mode=1)
        m = _tr(g * c(F(1) - b1) if t == 1 else (m * c(b1) + g * c(F(1) - b1)).astype(F))
        v = _tr(g * g * c(F(1) - b2) if t == 1 else (v * c(b2) + g * g * c(F(1) - b2)).astype(F))
        mh, vh = m / c(F(1) - F(b1 ** F(t))), v / c(F(1) - F(b2 ** F(t)))
        pe = _tr(((pe - mh / ((np.sqrt(vh) + c(eps)) * c(lr))) * c(F(1) - lr * wd)).astype(F))
        assert np.array_equal(zo.to_f32(mb, zo.BF16), m) and np.array_equal(zo.to_f32(vb, zo.BF16), v)
        got = zo.to_f32(pb, zo.BF16)
        assert np.max(np.abs(got - pe) / np.maximum(np.abs(pe), 1e-6)) <= 2 ** -7     # at most one bf16 ulp (FMA contraction)
    # layernorm with a column count that bf16 cannot hold: n -> bf16(1000) = 1000, n-1 = 999 -> 996
    x = _tr(rng.standard_normal((4, 1000)) * 2)
    mean = (x.sum(1, dtype=np.float64) / float(c(1000.0)))[:, None]
    var = (((x - mean) ** 2).sum(1) / float(c(999.0)))[:, None]
    want = (x - mean) / np.sqrt(var + float(c(1e-5)))
    got = zo.to_f32(zo.layernorm(zo.BF16, zo.to_bits(x, zo.BF16)), zo.BF16)
    assert float(c(999.0)) == 996.0
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-2)) <= 2 ** -7


def test_conv_golden_and_float64():
    """zyx/tests/05_misc.rs:880-888 (conv1) is the reference's conv vector; strides, dilations and paddings are then held
    against a float64 convolution of the same values (f32 sums of 30 products: 1e-5 relative to the largest output)."""
    import torch
    t = np.arange(9, dtype=np.float32).reshape(1, 1, 3, 3)
    assert zo.conv(zo.F32, t, np.ones((1, 1, 2, 2), np.float32)).tolist() == [[[[8.0, 12.0], [20.0, 24.0]]]]
    rng = np.random.default_rng(0)
    x = rng.standard_normal((2, 5, 9, 11)).astype(np.float32)
    w = rng.standard_normal((7, 5, 3, 2)).astype(np.float32)
    b = rng.standard_normal(7).astype(np.float32)
    for stride, dilation, pad in [(1, 1, (0, 0, 0, 0)), (2, 1, (1, 1, 1, 1)), ((2, 1), (1, 2), (1, 1, 2, 2)), (1, 2, (0, 2, 1, 3))]:
        y = zo.conv(zo.F32, x, w, b, stride, dilation, pad)
        xt = torch.nn.functional.pad(torch.from_numpy(x).double(), (pad[2], pad[3], pad[0], pad[1]))
        want = torch.nn.functional.conv2d(xt, torch.from_numpy(w).double(), torch.from_numpy(b).double(), stride=stride, dilation=dilation).numpy()
        assert y.shape == want.shape
        assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
    xi = rng.integers(-50, 50, (1, 3, 6, 7)).astype(np.int32)
    wi = rng.integers(-9, 9, (2, 3, 3, 3)).astype(np.int32)
    yi = zo.conv(zo.I32, xi, wi, None, 1, 1, 1)
    want = torch.nn.functional.conv2d(torch.from_numpy(xi).double(), torch.from_numpy(wi).double(), padding=1).numpy()
    assert np.array_equal(yi, want.astype(np.int64))
    # bf16: products exact in f32, one truncating store
    xb, wb = zo.to_bits(x, zo.BF16), zo.to_bits(w, zo.BF16)
    yb = zo.conv(zo.BF16, xb, wb, None, 1, 1, 1)
    exact = torch.nn.functional.conv2d(torch.from_numpy(zo.to_f32(xb, zo.BF16)).double(), torch.from_numpy(zo.to_f32(wb, zo.BF16)).double(), padding=1).numpy()
    got = zo.to_f32(yb, zo.BF16).astype(np.float64)
    assert np.all(np.abs(got) <= np.abs(exact) + 1e-4) and np.abs(got - exact).max() <= 2.0 ** -7 * np.abs(exact).max()


def test_conv_weight_gradient_against_float64_autograd():
    import torch
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 5, 11, 7)).astype(np.float32)
    dy = rng.standard_normal((2, 6, 5, 8)).astype(np.float32)
    got = zo.conv_weight_grad(zo.F32, x, dy, (6, 5, 3, 2), (2, 1), (1, 2), (1, 0, 2, 1))
    w = torch.zeros((6, 5, 3, 2), dtype=torch.float64, requires_grad=True)
    xt = torch.nn.functional.pad(torch.from_numpy(x).double(), (2, 1, 1, 0))
    torch.nn.functional.conv2d(xt, w, stride=(2, 1), dilation=(1, 2)).backward(torch.from_numpy(dy).double())
    assert np.abs(got - w.grad.numpy()).max() <= 1e-5 * np.abs(w.grad.numpy()).max()


def causal_self_attention(x, w_attn, w_proj, n_head, gemm, softmax):
    """CausalSelfAttention::forward (zyx-nn/src/causal_self_attention.rs:36-71) on one sequence x [T, C], composed from a
    matmul and a row softmax (the oracle's or the GPU's): c_attn, split into q, k, v, per head q.k^T * (1/sqrt(d)) -> softmax
    (no mask: lines 60-61) -> . v, heads merged, c_proj."""
    t, c = x.shape
    d = c // n_head
    qkv = gemm(x, w_attn, tb=True)
    q, k, v = qkv[:, :c], qkv[:, c:2 * c], qkv[:, 2 * c:]
    scale = float(np.float32(1.0 / np.sqrt(float(d))))
    y = np.zeros((t, c), np.float32)
    for h in range(n_head):
        qh, kh, vh = (np.ascontiguousarray(a[:, h * d:(h + 1) * d]) for a in (q, k, v))
        att = softmax(gemm(qh, kh, tb=True, alpha=scale))
        y[:, h * d:(h + 1) * d] = gemm(att, vh)
    return gemm(y, w_proj, tb=True)


def test_causal_self_attention_five_iterations_known_answer(golden):
    """The only reference vector that pins projection -> attention -> projection end to end."""
    g = golden["causal_self_attention_5_iterations_f32"]
    x = f32(g["x"])
    for _ in range(g["iterations"]):
        x = causal_self_attention(x, f32(g["c_attn_weight"]), f32(g["c_proj_weight"]), g["n_head"],
                                  lambda a, b, **kw: zo.gemm(zo.F32, a, b, **kw), lambda s: zo.softmax(zo.F32, s))
    assert ref_is_equal(x, f32(g["y"]))


def test_grad_dot_and_grad_sum_known_answers(golden):
    """The adjoints the plans use for a matmul (dX = dZ . Y^T, dY = X^T . dZ) and a full sum (ones), on the reference's vectors."""
    g = golden["grad_dot_i32"]
    x, y = np.asarray(g["x"], np.int32).reshape(1, 3), np.asarray(g["y"], np.int32)
    dz = np.ones((1, 1), np.int32)
    assert zo.gemm(zo.I32, dz, y, tb=True).ravel().tolist() == g["x_grad"]
    assert zo.gemm(zo.I32, x, dz, ta=True).tolist() == g["y_grad"]
    s = golden["grad_sum_f32"]
    xs = f32(s["x"]).reshape(1, -1)
    base = float(zo.row_reduce(0, zo.F32, xs)[0])
    fd = [float(zo.row_reduce(0, zo.F32, xs + np.eye(1, xs.size, i, dtype=np.float32))[0]) - base for i in range(xs.size)]
    assert fd == s["x_grad"]


def scalar_loop_softmax(x):
    """The loop of zyx/tests/07_realize.rs:277-293 in f32: row maximum, exp, a running sum in index order, divide."""
    m = x.max(1, keepdims=True)
    e = np.exp((x - m).astype(np.float32)).astype(np.float32)
    s = np.cumsum(e, axis=1, dtype=np.float32)[:, -1:]
    return (e / s).astype(np.float32)


def test_softmax_against_the_scalar_loop(golden):
    g = golden["softmax_scalar_loop_procedural"]
    x = zo.Rng().rand(g["rows"] * g["cols"]).reshape(g["rows"], g["cols"])
    assert ref_is_equal(zo.softmax(zo.F32, x), scalar_loop_softmax(x))
