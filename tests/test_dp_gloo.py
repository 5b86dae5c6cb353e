"""Data-parallel formulation on CPU ranks (gloo, world_size 2): each rank runs the oracle's forward/backward
on its half of the batch, gradients are summed with an all-reduce and scaled by 1/world inside the optimizer
(what libzyxb_host does with NCCL and grad_scale) — and the result equals the single-process step on the
concatenated batch."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import models as om
from oracle import oracle as zo

DIMS, BATCH = [24, 40, 16], 32


def _data():
    rng = zo.Rng(11)
    layers = om.init_linears(rng, zo.F32, DIMS)
    x = rng.randn(BATCH * DIMS[0]).reshape(BATCH, DIMS[0])
    t = rng.randn(BATCH * DIMS[-1]).reshape(BATCH, DIMS[-1])
    return layers, x, t


def _rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layers, x, t = _data()
    lo, hi = rank * BATCH // world, (rank + 1) * BATCH // world
    _, grads, _ = om.forward_backward(zo.F32, layers, np.ascontiguousarray(x[lo:hi]), np.ascontiguousarray(t[lo:hi]), om.ACT_GELU, om.LOSS_MSE)
    flat = om.flat(grads)
    bucket = torch.from_numpy(np.concatenate([g.ravel() for g in flat]))     # one contiguous gradient bucket
    dist.all_reduce(bucket, op=dist.ReduceOp.SUM)
    off, reduced = 0, []
    for g in flat:
        reduced.append(bucket[off:off + g.size].numpy().reshape(g.shape).copy())
        off += g.size
    opt = om.Optim("adamw", zo.F32, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=True)
    opt.update(om.flat(layers), reduced, grad_scale=1.0 / world)
    if rank == 0:
        np.savez(out, *om.flat(layers))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_step_equals_single_process_step(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "params.npz")
    mp.spawn(_rank, args=(2, port, out), nprocs=2, join=True)
    layers, x, t = _data()
    _, grads, _ = om.forward_backward(zo.F32, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
    opt = om.Optim("adamw", zo.F32, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=True)
    opt.update(om.flat(layers), om.flat(grads))
    got = np.load(out)
    for i, want in enumerate(om.flat(layers)):
        g = got["arr_%d" % i]
        # mean over the whole batch == mean of the two half-batch means; only f32 summation order differs
        assert np.max(np.abs(g - want)) <= 2e-5 * max(1.0, float(np.max(np.abs(want)))), i


def _rank_sharded(rank, world, port, out):
    """ZeRO stage 1 as libzyxb_host lays it out: parameters and gradients in flat buckets padded to a multiple of `world`,
    each rank keeps the summed gradients of its own shard (gloo has no reduce-scatter: an all-reduce of which the rank reads
    only its shard), updates that shard with optimizer state of shard size, and the shards are all-gathered."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    layers, x, t = _data()
    lo, hi = rank * BATCH // world, (rank + 1) * BATCH // world
    _, grads, _ = om.forward_backward(zo.F32, layers, np.ascontiguousarray(x[lo:hi]), np.ascontiguousarray(t[lo:hi]), om.ACT_GELU, om.LOSS_MSE)
    flat_p, flat_g = om.flat(layers), om.flat(grads)
    n = sum(p.size for p in flat_p)
    padded = (n + world - 1) // world * world
    shard = padded // world
    pbucket, gbucket = np.zeros(padded, np.float32), np.zeros(padded, np.float32)
    pbucket[:n] = np.concatenate([p.ravel() for p in flat_p])
    gbucket[:n] = np.concatenate([g.ravel() for g in flat_g])
    gt = torch.from_numpy(gbucket)
    dist.all_reduce(gt, op=dist.ReduceOp.SUM)
    mine = slice(rank * shard, (rank + 1) * shard)
    p_shard, g_shard = pbucket[mine].copy(), gbucket[mine].copy()
    m, v = np.zeros(shard, np.float32), np.zeros(shard, np.float32)      # state of shard size only
    zo.adam(zo.F32, p_shard, g_shard, m, v, 1, lr=1e-3, wd=0.01, mode=2, grad_scale=1.0 / world)
    gathered = [torch.zeros(shard) for _ in range(world)]
    dist.all_gather(gathered, torch.from_numpy(p_shard))
    if rank == 0:
        np.save(out, torch.cat(gathered).numpy()[:n])
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_optimizer_step_equals_single_process_step(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "params.npy")
    mp.spawn(_rank_sharded, args=(2, port, out), nprocs=2, join=True)
    layers, x, t = _data()
    _, grads, _ = om.forward_backward(zo.F32, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
    opt = om.Optim("adamw", zo.F32, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=True)
    opt.update(om.flat(layers), om.flat(grads))
    want = np.concatenate([p.ravel() for p in om.flat(layers)])
    got = np.load(out)
    assert np.max(np.abs(got - want)) <= 2e-5 * max(1.0, float(np.max(np.abs(want))))
