"""Transformer block parity (config 5's structure at sizes the oracle finishes in seconds): the C++ plan replayed through
the C ABI against the same block composed from the CPU oracle, whose gradients are themselves checked against
finite differences on the CPU (tests/test_oracle_block.py)."""
import numpy as np
import pytest

from oracle import models as om
from oracle import oracle as zo
from tests.parity import TOL_BF16, max_rel_err
from zyx_b200 import _lib as L
from zyx_b200 import host as H

pytestmark = pytest.mark.gpu


def f(x, dtype):
    return zo.to_f32(x, dtype)


@pytest.mark.parametrize("dtype,B,T,E,heads,F,causal,tol,floor,fused", [
    (L.F32, 2, 32, 64, 4, 128, True, 2e-5, 0.1, False),
    (L.F32, 1, 40, 48, 3, 80, False, 2e-5, 0.1, False),
    (L.BF16, 2, 128, 256, 4, 512, True, TOL_BF16, 0.25, False),
    (L.BF16, 1, 256, 512, 4, 1024, True, TOL_BF16, 0.25, False),      # head_dim 128, tensor-core path for every matmul
    (L.BF16, 1, 256, 512, 4, 1024, True, TOL_BF16, 0.25, True),       # the same with the fused attention programs
    (L.BF16, 2, 128, 256, 2, 512, False, TOL_BF16, 0.25, True),
])
def test_block_forward_backward_and_update(sess, dtype, B, T, E, heads, F, causal, tol, floor, fused):
    rng = np.random.default_rng(3)
    std = 0.3 if dtype == L.F32 else 0.05
    p = om.block_init(rng, dtype, E, F, std=std)
    for k in ("g1", "g2"):       # exercise the affine part with non-trivial values
        p[k] = zo.to_bits((1 + 0.1 * rng.standard_normal(E)).astype(np.float32), dtype)
    for k in ("be1", "be2"):
        p[k] = zo.to_bits((0.1 * rng.standard_normal(E)).astype(np.float32), dtype)
    x = zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dtype)
    t = zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dtype)
    kw = dict(lr=1e-3, weight_decay=0.01, standard=True)
    blk = H.Block(sess, dtype, B, T, E, heads, F, causal=causal, algo=L.OPT_ADAMW, fused_attention=fused, **kw)
    try:
        for i, name in enumerate(om.BLOCK_PARAMS):
            blk.set_tensor(H.PARAM, i, p[name])
        sess.pool.sync_events(blk.set_batch(x, t))
        blk.forward_backward()
        assert sess.device.status() == 0
        want_loss, grads, want_y, mid = om.block_forward_backward(dtype, p, x, t, heads, causal)
        if fused:
            with pytest.raises(Exception):
                blk.activation(0, (B * heads, T, T))          # the probabilities are never materialised
        else:
            pr = f(blk.activation(0, (B * heads, T, T)), dtype)
            if causal:
                assert np.all(pr[:, np.triu_indices(T, 1)[0], np.triu_indices(T, 1)[1]] == 0.0)   # masked keys: exactly zero
            assert max_rel_err(pr, f(mid["p"], dtype), floor=0.05) <= tol * 2
        # fused attention keeps scores and probabilities in f32 where the reference composition truncates them to the
        # 16-bit type, which moves the composition itself by a few percent of the row scale: compare on that scale
        assert max_rel_err(f(blk.activation(1, (B * T, E)), dtype), f(mid["attn"], dtype), floor=1.0 if fused else floor) <= tol * 2
        assert max_rel_err(f(blk.activation(2, (B * T, E)), dtype), f(mid["x1"], dtype), floor=floor) <= tol * 2
        assert abs(blk.read_loss() - want_loss) <= 10 * tol * abs(want_loss)
        assert max_rel_err(f(blk.read_output(), dtype), f(want_y, dtype), floor=floor) <= tol * 2
        for i, name in enumerate(om.BLOCK_PARAMS):
            got = f(blk.get_tensor(H.GRAD, i), dtype)
            if name == "bk":
                # softmax does not change when every key's score moves by the same amount, so the key bias has an exactly
                # zero gradient: both sides hold rounding noise only, which must be small beside the query bias gradient
                ref_scale = np.abs(f(grads["bq"], dtype)).max()
                assert np.abs(got).max() <= (1e-3 if dtype == L.F32 else 0.1) * ref_scale
                continue
            e = max_rel_err(got, f(grads[name], dtype), row_axis=None, floor=floor)
            assert e <= tol * 5, (name, e)
        blk.update()
        flat = [p[n] for n in om.BLOCK_PARAMS]
        opt = om.Optim("adamw", dtype, flat, **kw)
        opt.update(flat, [grads[n] for n in om.BLOCK_PARAMS])
        for i, name in enumerate(om.BLOCK_PARAMS):
            if name == "bk":
                continue          # Adam normalises a pure-noise gradient to a full-size step of arbitrary sign
            e = max_rel_err(f(blk.get_tensor(H.PARAM, i), dtype), f(flat[i], dtype), row_axis=None, floor=0.1)
            assert e <= max(tol * 5, 2e-3 if dtype == L.F32 else tol), (name, e)
    finally:
        blk.close()


def block_case(seed, dtype, B, T, E, F, steps):
    """Seeded parameters and batches of a block (also used by the two-rank test)."""
    rng = np.random.default_rng(seed)
    p = om.block_init(rng, dtype, E, F, std=0.05)
    for k in ("g1", "g2"):
        p[k] = zo.to_bits((1 + 0.1 * rng.standard_normal(E)).astype(np.float32), dtype)
    batches = [(zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dtype),
                zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dtype)) for _ in range(steps)]
    return p, batches


@pytest.mark.parametrize("fused", [False, True])
def test_sharded_optimizer_block_plan_equals_the_replicated_plan(sess, tmp_path, fused):
    """ZeRO stage 1 of the block plan on a one-rank communicator: parameters in one bucket, three reduce-scatters, three
    shard updates, three all-gathers.  Kernels and arithmetic are the replicated plan's, so after three steps losses and
    parameters are bit-identical; the optimizer state has no per-tensor buffers; a checkpoint of the sharded plan restores
    into a fresh sharded plan and continues with the same bits."""
    dtype, B, T, E, heads, F = L.BF16, 2, 256, 512, 4, 1024
    p, batches = block_case(11, dtype, B, T, E, F, 4)
    kw = dict(lr=1e-3, weight_decay=0.01, standard=True)

    def train(shard, steps, resume=None, save_at=None):
        blk = H.Block(sess, dtype, B, T, E, heads, F, causal=True, algo=L.OPT_ADAMW, world=1, fused_attention=fused, shard_optimizer=shard, **kw)
        try:
            if resume:
                assert blk.load(resume) == 0
            else:
                for i, name in enumerate(om.BLOCK_PARAMS):
                    blk.set_tensor(H.PARAM, i, p[name])
            losses = []
            for n, (x, t) in enumerate(steps):
                blk.step(blk.set_batch(x, t))
                losses.append(blk.read_loss())
                if save_at == n:
                    blk.save(save_at_path)
            assert sess.device.status() == 0
            if shard:
                assert blk.plan_size()[1] == 6
                with pytest.raises(Exception):
                    blk.tensor(H.STATE0, 0)
            return losses, [blk.get_tensor(H.PARAM, i) for i in range(len(om.BLOCK_PARAMS))]
        finally:
            blk.close()

    save_at_path = str(tmp_path / "blk.safetensors")
    want_losses, want = train(False, batches)
    sess.device.comm_init(0, 1, sess.device.comm_unique_id())
    try:
        got_losses, got = train(True, batches, save_at=1)
        tail_losses, tail = train(True, batches[2:], resume=save_at_path)
    finally:
        sess.device.comm_destroy()
    assert got_losses == want_losses
    for g, w in zip(got, want):
        assert np.array_equal(g, w)
    assert tail_losses == want_losses[2:]
    for g, w in zip(tail, want):
        assert np.array_equal(g, w)
