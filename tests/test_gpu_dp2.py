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

CONFIGS = {"small": ([64, 128, 64, 128, 64], 48, 3),
           # a first layer large enough for the plan to produce its weight gradient in two halves, each with its own allreduce
           "split_first_layer": ([4096, 4096, 64], 32, 2)}


def _data(config):
    DIMS, BATCH, STEPS = CONFIGS[config]
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


def _rank(rank, world, tmp, config):
    DIMS, BATCH, STEPS = CONFIGS[config]
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
        layers, batches = _data(config)
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
@pytest.mark.parametrize("config", sorted(CONFIGS))
def test_sharded_and_replicated_plans_agree_on_two_ranks(tmp_path, config):
    from oracle import models as om
    from oracle import oracle as zo
    from tests.parity import TOL_BF16
    DIMS, BATCH, STEPS = CONFIGS[config]
    mp.spawn(_rank, args=(2, str(tmp_path), config), nprocs=2, join=True)
    r0, r1 = (np.load(str(tmp_path / ("rank%d.npz" % r))) for r in range(2))
    n = 2 * (len(DIMS) - 1)
    for i in range(n):
        rep0, shd0 = r0["arr_%d" % i], r0["arr_%d" % (n + i)]
        assert np.array_equal(rep0, r1["arr_%d" % i]) and np.array_equal(shd0, r1["arr_%d" % (n + i)])    # ranks hold the same parameters
        assert np.array_equal(rep0, shd0)                                                                # and the two plans the same bits
    # one oracle step sequence on the concatenated batch (mean over 2 x BATCH rows = mean of the two ranks' means)
    layers, batches = _data(config)
    opt = om.Optim("adamw", zo.BF16, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=True)
    for x, t in batches:
        _, grads, _ = om.forward_backward(zo.BF16, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
        opt.update(om.flat(layers), om.flat(grads))
    for i, want in enumerate(om.flat(layers)):
        got, w = zo.to_f32(r0["arr_%d" % (n + i)], zo.BF16), zo.to_f32(want, zo.BF16)
        err = np.abs(got - w) / np.maximum(np.abs(w), 0.1 * np.abs(w).max())
        # Adam moves every element by about lr per step whatever the size of its gradient, so an element whose (tiny) gradient
        # rounds to the other sign on the two sides ends 2 * lr apart: with weights of 1/64 (the large layer) that is a few
        # percent of an element for a fraction of a percent of them
        assert np.quantile(err, 0.999 if config == "small" else 0.99) <= 2 * TOL_BF16, (i, float(err.max()))


def _rank_allreduce(rank, world, tmp, mode):
    """Every rank allreduces the same sequence of ranges (several dtypes, sizes that do not divide into shards, offsets into a
    larger buffer, a view, repeated calls on one buffer) and checks the sum it can compute by itself from the seeds."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["ZYXB_ALLREDUCE"] = "nccl" if mode == "nccl" else "peer"
    if mode == "peer_direct":
        os.environ["ZYXB_PEER_DIRECT"] = "1"       # the reduce kernel reads the peers' buffers itself instead of staged copies
    os.environ["ZYXB_PEER_WAIT_MS"] = "10000"
    from oracle import oracle as zo
    from zyx_b200 import _lib as L
    from zyx_b200.ops import Session
    sess = Session(device_ids=[rank])
    try:
        uid_path = os.path.join(tmp, "uid_" + mode)
        if rank == 0:
            with open(uid_path + ".tmp", "wb") as f:
                f.write(sess.device.comm_unique_id())
            os.rename(uid_path + ".tmp", uid_path)
        t0 = time.time()
        while not os.path.exists(uid_path):
            assert time.time() - t0 < 60, "no unique id from rank 0"
            time.sleep(0.05)
        sess.device.comm_init(rank, world, open(uid_path, "rb").read())
        p, d = sess.pool, sess.device
        if mode == "peer_latency":                  # the option a plan sets around its last collective: the communicator's own allreduce
            d.comm_option(L.COMM_OPT_LATENCY, 1)
        data = lambda r, n, seed: np.random.default_rng(1000 * seed + r).standard_normal(n).astype(np.float32)
        cases = [(L.F32, 1 << 20, 0, 1 << 20), (L.F32, 100003, 256, 99000), (L.BF16, 5_000_000, 128, 4_999_000), (L.F16, 777, 0, 777),
                 (L.BF16, 64, 0, 7), (L.I32, 4099, 3, 4000), (L.BF16, 1 << 24, 0, 1 << 24)]
        for seed, (dt, n, off, count) in enumerate(cases):
            conv = (lambda a: a) if dt == L.F32 else (lambda a: (a * 100).astype(np.int32)) if dt == L.I32 else (lambda a: zo.to_bits(a, dt))
            back = (lambda a: a.astype(np.float64)) if dt in (L.F32, L.I32) else (lambda a: zo.to_f32(a, dt).astype(np.float64))
            parts = [conv(data(r, n, seed)) for r in range(world)]
            buf = p.upload(parts[rank])
            for rep in range(2):                       # the second call sums the first call's sums: W * W * x
                ev = d.allreduce_sum(buf, count, dt, offset_elems=off, want_event=True)
                p.sync_events([ev])
            got = p.download(buf, (n,), parts[rank].dtype)
            want = sum(back(a) for a in parts)
            lo, hi = off, off + count
            assert np.array_equal(got[:lo], parts[rank][:lo]) and np.array_equal(got[hi:], parts[rank][hi:]), (mode, seed, "outside the range")
            w2 = want[lo:hi] * world
            err = np.abs(back(got[lo:hi]) - w2) / np.maximum(np.abs(w2), 0.05 * np.abs(w2).max())
            tol = 0 if dt == L.I32 else 1e-6 if dt == L.F32 else 2e-2
            assert err.max() <= tol, (mode, seed, float(err.max()))
            p.deallocate(buf)
        # a view of a bucket, as the plans use it
        bucket, _ = p.allocate(4 << 20)
        sess.backend._check(sess.backend.lib.zyxb_memset(sess.backend.ctx, d.dev, bucket, 0, 0, 4 << 20))
        import ctypes as C
        view = C.c_uint32()
        sess.backend._check(sess.backend.lib.zyxb_buffer_view(sess.backend.ctx, d.dev, bucket, 1 << 20, 1 << 20, C.byref(view)))
        x = data(rank, 1 << 18, 99)
        p.sync_events([p.host_to_pool(x, view.value)])
        d.allreduce_sum(view.value, 1 << 18, L.F32)
        d.sync()
        want = sum(data(r, 1 << 18, 99).astype(np.float64) for r in range(world))
        got = p.download(view.value, (1 << 18,), np.float32)
        assert np.max(np.abs(got - want)) <= 1e-5, mode
        assert d.status() == 0
        p.deallocate(view.value)
        p.deallocate(bucket)
        open(os.path.join(tmp, "ok_%s_%d" % (mode, rank)), "w").close()
        sess.device.comm_destroy()
    finally:
        sess.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["peer", "peer_direct", "peer_latency", "nccl"])
def test_allreduce_over_peer_memory_and_over_nccl(tmp_path, mode):
    """zyxb_allreduce_sum on two ranks: the copy-engine path over IPC-mapped peer memory (the default) and the NCCL path
    (ZYXB_ALLREDUCE=nccl) give the sum of the ranks' data, leave everything outside the range alone, and keep working call
    after call (the sequence numbers of the peer path only grow)."""
    mp.spawn(_rank_allreduce, args=(2, str(tmp_path), mode), nprocs=2, join=True)
    assert all(os.path.exists(str(tmp_path / ("ok_%s_%d" % (mode, r)))) for r in range(2))


def _rank_block(rank, world, tmp):
    """The transformer-block plan on two ranks, replicated (three allreduces) and with the sharded optimizer (three
    reduce-scatters, shard updates, all-gathers), each rank on its half of the batch."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from oracle import models as om
    from tests.test_gpu_block import block_case
    from zyx_b200 import _lib as L
    from zyx_b200 import host as H
    from zyx_b200.ops import Session
    B, T, E, heads, F, STEPS = 1, 256, 512, 4, 1024, 3
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
        p, batches = block_case(5, L.BF16, world * B, T, E, F, STEPS)
        out, losses = {}, {}
        for shard in (False, True):
            blk = H.Block(sess, L.BF16, B, T, E, heads, F, causal=True, algo=L.OPT_ADAMW, world=world, fused_attention=True,
                          shard_optimizer=shard, lr=1e-3, weight_decay=0.01, standard=True)
            try:
                for i, name in enumerate(om.BLOCK_PARAMS):
                    blk.set_tensor(H.PARAM, i, p[name])
                losses[shard] = []
                for x, t in batches:
                    blk.step(blk.set_batch(x[rank * B:(rank + 1) * B], t[rank * B:(rank + 1) * B]))
                    losses[shard].append(blk.read_loss())
                out[shard] = [blk.get_tensor(H.PARAM, i) for i in range(len(om.BLOCK_PARAMS))]
                assert blk.plan_size()[1] == (6 if shard else 3)
                assert sess.device.status() == 0
            finally:
                blk.close()
        assert losses[False] == losses[True]
        np.savez(os.path.join(tmp, "rank%d.npz" % rank), *(out[False] + out[True]), losses=np.array(losses[True]))
        sess.device.comm_destroy()
    finally:
        sess.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_block_plans_agree_on_two_ranks(tmp_path):
    """Both ranks end with the same parameter bits, the sharded plan with the replicated plan's bits, and the first step's
    loss (taken with identical parameters) is the oracle's on the concatenated batch: the mean over 2 x B samples equals the
    mean of the two ranks' means."""
    from oracle import models as om
    from oracle import oracle as zo
    from tests.test_gpu_block import block_case
    mp.spawn(_rank_block, args=(2, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (np.load(str(tmp_path / ("rank%d.npz" % r))) for r in range(2))
    n = len(om.BLOCK_PARAMS)
    for i in range(n):
        rep0, shd0 = r0["arr_%d" % i], r0["arr_%d" % (n + i)]
        assert np.array_equal(rep0, r1["arr_%d" % i]) and np.array_equal(shd0, r1["arr_%d" % (n + i)]), om.BLOCK_PARAMS[i]
        assert np.array_equal(rep0, shd0), om.BLOCK_PARAMS[i]
    p, batches = block_case(5, zo.BF16, 2, 256, 512, 1024, 3)
    assert any(not np.array_equal(r0["arr_%d" % i], p[name]) for i, name in enumerate(om.BLOCK_PARAMS))     # the steps did move them
    want_loss, _, _, _ = om.block_forward_backward(zo.BF16, p, batches[0][0], batches[0][1], 4, True)
    got = 0.5 * (float(r0["losses"][0]) + float(r1["losses"][0]))
    assert abs(got - want_loss) <= 0.02 * abs(want_loss)
