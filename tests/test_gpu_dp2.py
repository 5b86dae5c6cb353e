"""Two ranks on two GPUs (skipped with fewer): the sharded-optimizer plan (reduce-scatter, shard update, all-gather) and the
replicated plan (allreduce, full update) give bit-identical parameters on both ranks, and both follow the single-process
oracle step on the concatenated batch."""
import os
import time

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

DIMS, BATCH, STEPS = [64, 128, 64, 128, 64], 48, 3


def _data(rank):
    from oracle import models as om
    from oracle import oracle as zo
    rng = zo.Rng(7)
    layers = om.init_linears(rng, zo.BF16, DIMS)
    batches = []
    for _ in range(STEPS):
        x = zo.to_bits(rng.randn(2 * BATCH * DIMS[0]).reshape(2 * BATCH, DIMS[0]), zo.BF16)
        t = zo.to_bits(rng.randn(2 * BATCH * DIMS[-1]).reshape(2 * BATCH, DIMS[-1]), zo.BF16)
        batches.append((x, t))
    return layers, batches


def _rank(rank, world, tmp):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from oracle import models as om
    from zyx_b200 import _lib as L
    from zyx_b200 import host as H
    from zyx_b200.ops import Session
    sess = Session(device_ids=[rank])
    try:
        uid_path = os.path.join(tmp, "uid")
        if rank == 0:
            with open(uid_path + ".tmp", "wb") as f:
                f.write(sess.device.comm_unique_id())
            os.rename(uid_path + ".tmp", uid_path)
        t0 = time.time()
        while not os.path.exists(uid_path):
            assert time.time() - t0 < 60, "no unique id from rank 0"
            time.sleep(0.05)
        sess.device.comm_init(rank, world, open(uid_path, "rb").read())
        layers, batches = _data(rank)
        out = {}
        for shard in (False, True):
            mlp = H.Mlp(sess, L.BF16, BATCH, DIMS, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, world=world,
                        shard_optimizer=shard, lr=1e-3, weight_decay=0.01, standard=True)
            try:
                for i, t in enumerate(om.flat(layers)):
                    mlp.set_tensor(H.PARAM, i, t)
                for x, t in batches:
                    lo = rank * BATCH
                    mlp.step(mlp.set_batch(np.ascontiguousarray(x[lo:lo + BATCH]), np.ascontiguousarray(t[lo:lo + BATCH])))
                out[shard] = [mlp.get_tensor(H.PARAM, i) for i in range(mlp.n_params())]
                assert sess.device.status() == 0
            finally:
                mlp.close()
        np.savez(os.path.join(tmp, "rank%d.npz" % rank), *(out[False] + out[True]))
        sess.device.comm_destroy()
    finally:
        sess.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_and_replicated_plans_agree_on_two_ranks(tmp_path):
    from oracle import models as om
    from oracle import oracle as zo
    from tests.parity import TOL_BF16
    mp.spawn(_rank, args=(2, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (np.load(str(tmp_path / ("rank%d.npz" % r))) for r in range(2))
    n = 2 * (len(DIMS) - 1)
    for i in range(n):
        rep0, shd0 = r0["arr_%d" % i], r0["arr_%d" % (n + i)]
        assert np.array_equal(rep0, r1["arr_%d" % i]) and np.array_equal(shd0, r1["arr_%d" % (n + i)])    # ranks hold the same parameters
        assert np.array_equal(rep0, shd0)                                                                # and the two plans the same bits
    # one oracle step sequence on the concatenated batch (mean over 2 x BATCH rows = mean of the two ranks' means)
    layers, batches = _data(0)
    opt = om.Optim("adamw", zo.BF16, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=True)
    for x, t in batches:
        _, grads, _ = om.forward_backward(zo.BF16, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
        opt.update(om.flat(layers), om.flat(grads))
    for i, want in enumerate(om.flat(layers)):
        got, w = zo.to_f32(r0["arr_%d" % (n + i)], zo.BF16), zo.to_f32(want, zo.BF16)
        err = np.abs(got - w) / np.maximum(np.abs(w), 0.1 * np.abs(w).max())
        assert np.quantile(err, 0.999) <= 2 * TOL_BF16, (i, float(err.max()))
