"""Training-step parity: the C++ plan replayed through the C ABI against the same step composed
from the CPU oracle — the README SimpleNet configuration (784 -> 128 ReLU -> 10, f32, batch 64,
cross-entropy, SGD lr 0.01, Linear::new weights) and the bf16 GELU / AdamW MLP."""
import numpy as np
import pytest

from oracle import oracle as zo
from oracle import models as om
from tests.parity import TOL_BF16, TOL_F32, assert_parity, max_rel_err
from zyx_b200 import _lib as L
from zyx_b200 import host as H

pytestmark = pytest.mark.gpu


def f(x, dtype):
    return zo.to_f32(x, dtype)


def load_params(mlp, layers):
    for i, t in enumerate(om.flat(layers)):
        mlp.set_tensor(H.PARAM, i, t)


def simplenet_exact(layers, x, labels):
    """Float64 forward / backward of the two-layer ReLU network with mean cross-entropy, from the stored f32 parameters:
    the third party for error attribution (the first matmul's 784-term sums are added in another order on the GPU)."""
    (w1, b1), (w2, b2) = [(np.asarray(w, np.float64), np.asarray(b, np.float64)) for w, b in layers]
    x = np.asarray(x, np.float64)
    z1 = x @ w1.T + b1
    a1 = np.maximum(z1, 0.0)
    z2 = a1 @ w2.T + b2
    e = np.exp(z2 - z2.max(1, keepdims=True))
    sm = e / e.sum(1, keepdims=True)
    dz2 = sm.copy()
    dz2[np.arange(len(labels)), labels] -= 1.0
    dz2 /= len(labels)
    dz1 = (dz2 @ w2) * (z1 > 0)
    return z2, [dz1.T @ x, dz1.sum(0), dz2.T @ a1, dz2.sum(0)]


def test_simplenet_five_sgd_steps(sess):
    """Config 1: weights from Linear::new (zyx RNG, seed 42069), inputs N(0,1) by the reference's Box-Muller,
    labels uniform in [0,10).  Loss, gradients and parameters agree with the oracle to 1e-5 over 5 steps."""
    dims, batch = [784, 128, 10], 64
    rng = zo.Rng(42069)
    layers = om.init_linears(rng, zo.F32, dims)
    mlp = H.Mlp(sess, L.F32, batch, dims, activation=H.ACT_RELU, loss=H.LOSS_CROSS_ENTROPY, algo=L.OPT_SGD, lr=0.01)
    try:
        load_params(mlp, layers)
        opt = om.Optim("sgd", zo.F32, om.flat(layers), lr=0.01)
        nprng = np.random.default_rng(5)
        assert mlp.plan_size()[0] == 10          # 2 matmuls, 2 loss kernels, 2x(dW, db), dX fused with relu', SGD
        for step in range(5):
            x = rng.randn(batch * dims[0]).reshape(batch, dims[0])
            labels = nprng.integers(0, 10, size=batch).astype(np.int32)
            sess.pool.sync_events(mlp.set_batch(x, labels))
            mlp.forward_backward()
            want_loss, grads, want_y = om.forward_backward(zo.F32, layers, x, labels, om.ACT_RELU, om.LOSS_CE)
            assert abs(mlp.read_loss() - want_loss) <= TOL_F32 * abs(want_loss)
            exact_y, exact_g = simplenet_exact(layers, x, labels)
            assert_parity(mlp.read_output(), want_y, exact_y, TOL_F32, floor=0.1, what="logits")
            for i, g in enumerate(om.flat(grads)):
                assert_parity(mlp.get_tensor(H.GRAD, i), g, exact_g[i].reshape(g.shape), TOL_F32, floor=0.1, what="grad %d step %d" % (i, step))
            mlp.update()
            opt.update(om.flat(layers), om.flat(grads))
            for i, p in enumerate(om.flat(layers)):
                assert max_rel_err(mlp.get_tensor(H.PARAM, i), p, floor=0.1) <= TOL_F32, ("param", step, i)
    finally:
        mlp.close()


@pytest.mark.parametrize("standard", [False, True])
def test_bf16_gelu_mlp_adamw_steps(sess, standard):
    """A small instance of config 4 (4 Linear layers, GELU, bf16, MSE, AdamW lr 1e-3 wd 0.01), 3 steps.
    With the reference's AdamW (step divided by lr) an entry whose gradient is ~0 takes a step of
    +-1/lr whose sign is rounding noise, so entries with |g| below 1% of the tensor's largest are
    left out of the parameter comparison after the first update."""
    dims, batch, dt = [64, 128, 64, 128, 64], 96, L.BF16
    rng = zo.Rng(7)
    layers = om.init_linears(rng, zo.BF16, dims)
    kw = dict(lr=1e-3, weight_decay=0.01, standard=standard)
    mlp = H.Mlp(sess, dt, batch, dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, **kw)
    try:
        load_params(mlp, layers)
        opt = om.Optim("adamw", zo.BF16, om.flat(layers), **kw)
        for step in range(3 if standard else 1):
            x = zo.to_bits(rng.randn(batch * dims[0]).reshape(batch, dims[0]), zo.BF16)
            t = zo.to_bits(rng.randn(batch * dims[-1]).reshape(batch, dims[-1]), zo.BF16)
            sess.pool.sync_events(mlp.set_batch(x, t))
            mlp.forward_backward()
            want_loss, grads, want_y = om.forward_backward(zo.BF16, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
            assert abs(mlp.read_loss() - want_loss) <= TOL_BF16 * abs(want_loss)
            assert max_rel_err(f(mlp.read_output(), dt), f(want_y, dt), floor=0.1) <= TOL_BF16
            gflat = om.flat(grads)
            for i, g in enumerate(gflat):
                assert max_rel_err(f(mlp.get_tensor(H.GRAD, i), dt), f(g, dt), row_axis=None, floor=0.1) <= TOL_BF16 * 2, ("grad", step, i)
            mlp.update()
            opt.update(om.flat(layers), gflat)
            for i, p in enumerate(om.flat(layers)):
                got, want, g = f(mlp.get_tensor(H.PARAM, i), dt), f(p, dt), np.abs(f(gflat[i], dt))
                keep = g >= 1e-2 * g.max()
                assert keep.mean() > 0.9
                err = np.abs(got - want) / np.maximum(np.abs(want), 0.1 * np.abs(want).max())
                assert err[keep].max() <= TOL_BF16 * 2, ("param", step, i, float(err[keep].max()))
                for which, st in ((H.STATE0, opt.s0[i]), (H.STATE1, opt.s1[i])):
                    e = np.abs(f(mlp.get_tensor(which, i), dt) - f(st, dt)) / np.maximum(np.abs(f(st, dt)), 0.1 * np.abs(f(st, dt)).max())
                    assert e[keep].max() <= TOL_BF16 * 3, ("state", which, step, i)
    finally:
        mlp.close()


def test_config4_layer_shapes_one_step_gradients(sess):
    """The real layer sizes of config 4 (4096 <-> 16384) at batch 128: loss and gradients of one step against the oracle
    (sampled rows of the large gradients), exercising the tensor-core kernel in all three layouts."""
    dims, batch, dt = [4096, 16384, 4096, 16384, 4096], 128, L.BF16
    rng = np.random.default_rng(4)
    layers = []
    for i in range(4):
        bound = 1.0 / np.sqrt(dims[i])
        layers.append((zo.to_bits(rng.uniform(-bound, bound, (dims[i + 1], dims[i])).astype(np.float32), zo.BF16),
                       zo.to_bits(rng.uniform(-bound, bound, (dims[i + 1],)).astype(np.float32), zo.BF16)))
    x = zo.to_bits(rng.standard_normal((batch, dims[0])).astype(np.float32), zo.BF16)
    t = zo.to_bits(rng.standard_normal((batch, dims[-1])).astype(np.float32), zo.BF16)
    mlp = H.Mlp(sess, dt, batch, dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, lr=1e-3, weight_decay=0.01)
    try:
        load_params(mlp, layers)
        sess.pool.sync_events(mlp.set_batch(x, t))
        mlp.forward_backward()
        assert sess.device.status() == 0
        want_loss, grads, want_y = om.forward_backward(zo.BF16, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
        assert abs(mlp.read_loss() - want_loss) <= TOL_BF16 * abs(want_loss)
        # Four chained bf16 layers: one-ulp (0.4-0.8 %) truncation differences in a layer's output become a
        # ~0.2 % perturbation of every sum over 16384 of them in the next, so entries much smaller than the
        # row's largest are measured against half of it (each single layer is held to floor 0.1 in
        # tests/test_gpu_gemm_tc.py, where both sides see identical inputs).
        e_y = max_rel_err(f(mlp.read_output(), dt), f(want_y, dt), floor=0.5)
        assert e_y <= TOL_BF16, e_y
        for i, g in enumerate(om.flat(grads)):
            got, want = f(mlp.get_tensor(H.GRAD, i), dt), f(g, dt)
            e_g = max_rel_err(got, want, row_axis=None, floor=0.25)
            assert e_g <= TOL_BF16, ("grad", i, e_g)
    finally:
        mlp.close()


def test_simplenet_step_replayed_from_a_captured_graph(sess):
    """The same SimpleNet step recorded once (capture_begin / capture_end) and replayed, the way FrozenTape::replay re-runs a
    realised plan: three replays on three batches give the oracle's parameters."""
    dims, batch = [784, 128, 10], 64
    rng = zo.Rng(42069)
    layers = om.init_linears(rng, zo.F32, dims)
    mlp = H.Mlp(sess, L.F32, batch, dims, activation=H.ACT_RELU, loss=H.LOSS_CROSS_ENTROPY, algo=L.OPT_SGD, lr=0.01)
    graph = None
    try:
        load_params(mlp, layers)
        opt = om.Optim("sgd", zo.F32, om.flat(layers), lr=0.01)
        nprng = np.random.default_rng(9)
        sess.device.sync()
        sess.device.capture_begin()
        mlp.step()
        graph = sess.device.capture_end()
        before = sess.device.launch_count()
        for step in range(3):
            x = rng.randn(batch * dims[0]).reshape(batch, dims[0])
            labels = nprng.integers(0, 10, size=batch).astype(np.int32)
            sess.pool.sync_events(mlp.set_batch(x, labels))
            sess.device.graph_launch(graph)
            want_loss, grads, _ = om.forward_backward(zo.F32, layers, x, labels, om.ACT_RELU, om.LOSS_CE)
            opt.update(om.flat(layers), om.flat(grads))
            assert abs(mlp.read_loss() - want_loss) <= TOL_F32 * abs(want_loss)
            for i, p in enumerate(om.flat(layers)):
                assert max_rel_err(mlp.get_tensor(H.PARAM, i), p, floor=0.1) <= TOL_F32, ("param", step, i)
        assert sess.device.launch_count() - before == 3 * 14      # 10 programs, four of them two kernels each (split-k first matmul)
    finally:
        if graph:
            sess.device.graph_release(graph)
        mlp.close()


def test_sharded_optimizer_plan_equals_the_replicated_plan(sess):
    """ZeRO stage 1 on a one-rank communicator: parameters in one bucket, reduce-scatter / shard update / all-gather.  The
    kernels and their arithmetic are those of the replicated plan (an elementwise update does not care where tensors begin),
    so after three steps parameters and loss are bit-identical."""
    dims, batch, dt = [64, 128, 64, 128, 64], 96, L.BF16
    rng = zo.Rng(7)
    layers = om.init_linears(rng, zo.BF16, dims)
    kw = dict(lr=1e-3, weight_decay=0.01, standard=True)
    batches = [(zo.to_bits(rng.randn(batch * dims[0]).reshape(batch, dims[0]), zo.BF16),
                zo.to_bits(rng.randn(batch * dims[-1]).reshape(batch, dims[-1]), zo.BF16)) for _ in range(3)]

    def train(shard):
        mlp = H.Mlp(sess, dt, batch, dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, world=1, shard_optimizer=shard, **kw)
        try:
            load_params(mlp, layers)
            losses = []
            for x, t in batches:
                mlp.step(mlp.set_batch(x, t))
                losses.append(mlp.read_loss())
            assert sess.device.status() == 0
            if shard:
                assert mlp.plan_size()[1] == 8                      # four reduce-scatters, four all-gathers
                with pytest.raises(Exception):
                    mlp.tensor(H.STATE0, 0)                         # the state has no per-tensor buffers
            return losses, [mlp.get_tensor(H.PARAM, i) for i in range(mlp.n_params())]
        finally:
            mlp.close()

    want_losses, want = train(False)
    sess.device.comm_init(0, 1, sess.device.comm_unique_id())
    try:
        assert sess.device.comm_rank() == (0, 1)
        got_losses, got = train(True)
    finally:
        sess.device.comm_destroy()
    assert got_losses == want_losses
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
