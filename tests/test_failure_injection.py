"""Failure detection on the host side of the boundary, without a GPU (CPU ranks, gloo): the real plan code of libzyxb_host
runs over a host-memory fake of the C ABI (tests/fake/zyxb_fake.cpp - the counterpart of the reference's dummy backend,
zyx/src/backend/dummy.rs:36-74) that can fail the n-th allocation, launch or collective the way a device error surfaces
through the ABI (status + context string, zyx/src/error.rs:107-153).  Nothing here faults, traps or hangs anything: failures
are injected return codes, a rank leaves only between steps, and the survivor's next collective ends with an error."""
import datetime
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import models as om
from oracle import oracle as zo
from tests.fake import harness as FH
from zyx_b200 import _lib as L
from zyx_b200 import host as H

DIMS, BATCH, STEPS = [24, 40, 16], 32, 3
KW = dict(lr=1e-3, weight_decay=0.01, standard=True)


def _data(step=0):
    rng = zo.Rng(11 + step)
    x = rng.randn(BATCH * DIMS[0]).reshape(BATCH, DIMS[0])
    t = rng.randn(BATCH * DIMS[-1]).reshape(BATCH, DIMS[-1])
    return x, t


def _layers():
    return om.init_linears(zo.Rng(5), zo.F32, DIMS)


def _load(fake, mlp, layers):
    for i, p in enumerate(om.flat(layers)):
        fake.upload(mlp.tensor(H.PARAM, i), p)


def _oracle_params(steps):
    layers = _layers()
    opt = om.Optim("adamw", zo.F32, om.flat(layers), **KW)
    for s in range(steps):
        x, t = _data(s)
        _, grads, _ = om.forward_backward(zo.F32, layers, x, t, om.ACT_GELU, om.LOSS_MSE)
        opt.update(om.flat(layers), om.flat(grads))
    return om.flat(layers)


def _close(got, want):
    return np.max(np.abs(got - want)) <= 5e-5 * max(1.0, float(np.max(np.abs(want))))


def test_the_plan_runs_over_the_fake_and_matches_the_oracle():
    fake = FH.Fake()
    mlp = FH.FakeMlp(fake, BATCH, DIMS, **KW)
    assert mlp.status == L.OK
    _load(fake, mlp, _layers())
    for s in range(STEPS):
        x, t = _data(s)
        fake.upload(mlp.x, x)
        fake.upload(mlp.target, t)
        assert mlp.step() == L.OK, mlp.error()
    for i, want in enumerate(_oracle_params(STEPS)):
        assert _close(fake.download(mlp.tensor(H.PARAM, i), want.shape), want), i
    mlp.close()


def test_a_failing_allocation_fails_plan_creation_with_its_status_and_text():
    fake = FH.Fake()
    before = fake.calls(FH.ALLOC)                          # the counters belong to the loaded library, not to one context
    probe = FH.FakeMlp(fake, BATCH, DIMS, **KW)            # how many allocations a plan makes
    n_allocs = fake.calls(FH.ALLOC) - before
    probe.close()
    for nth in (0, 3, n_allocs - 1):
        fake.fail(FH.ALLOC, nth)
        mlp = FH.FakeMlp(fake, BATCH, DIMS, **KW)
        assert mlp.status == L.ERR_NAMES_INV["MemoryAllocation"] and not mlp.h
        assert "out of memory (injected)" in fake.last_error()
    ok = FH.FakeMlp(fake, BATCH, DIMS, **KW)               # and the context is still usable
    assert ok.status == L.OK
    ok.close()


def test_a_failing_launch_surfaces_from_the_step_and_the_next_step_runs():
    fake = FH.Fake()
    mlp = FH.FakeMlp(fake, BATCH, DIMS, **KW)
    _load(fake, mlp, _layers())
    x, t = _data(0)
    fake.upload(mlp.x, x)
    fake.upload(mlp.target, t)
    fake.fail(FH.LAUNCH, 4)                                # the fifth launch of the step
    st = mlp.step()
    assert st == L.ERR_NAMES_INV["KernelLaunch"]
    assert "zyxb_launch" in mlp.error() and "injected" in mlp.error()
    assert mlp.step() == L.OK, mlp.error()                 # nothing is left half-consumed: the plan replays
    mlp.close()


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out, leave_after):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    fake = FH.Fake()
    assert fake.lib.zyxb_comm_init(fake.ctx, 0, rank, world, None) == L.OK

    def collective(arr, op):
        t = torch.from_numpy(arr)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)          # raises when a peer has gone or the timeout runs out
        return 0
    fake.set_collective(collective)
    mlp = FH.FakeMlp(fake, BATCH // world, DIMS, world=world, **KW)
    assert mlp.status == L.OK, fake.last_error()
    _load(fake, mlp, _layers())
    lo, hi = rank * BATCH // world, (rank + 1) * BATCH // world
    statuses = []
    for s in range(STEPS):
        if leave_after is not None and rank == 1 and s == leave_after:
            # leaves between steps: none of its launches or collectives is in flight
            return
        x, t = _data(s)
        fake.upload(mlp.x, np.ascontiguousarray(x[lo:hi]))
        fake.upload(mlp.target, np.ascontiguousarray(t[lo:hi]))
        statuses.append((mlp.step(), mlp.error()))
        if statuses[-1][0] != L.OK:
            break
    if rank == 0:
        np.savez(out, status=np.array([s for s, _ in statuses]), text=np.array([e for _, e in statuses]),
                 **{"p%d" % i: fake.download(mlp.tensor(H.PARAM, i), mlp.shape(i)) for i in range(2 * (len(DIMS) - 1))})
    if leave_after is None:
        dist.barrier()
        dist.destroy_process_group()


def test_two_ranks_through_the_plan_equal_the_single_process_oracle(tmp_path):
    """The data-parallel plan itself (per-layer gradient buckets, one allreduce per layer as its gradients are queued, 1/world
    folded into the optimizer launch) on two gloo ranks: three steps equal three oracle steps on the whole batch."""
    out = str(tmp_path / "r0.npz")
    mp.spawn(_rank, args=(2, _port(), out, None), nprocs=2, join=True)
    got = np.load(out)
    assert got["status"].tolist() == [L.OK] * STEPS
    for i, want in enumerate(_oracle_params(STEPS)):
        assert _close(got["p%d" % i], want), i


def test_a_rank_that_leaves_between_steps_ends_the_survivors_next_collective_with_an_error(tmp_path):
    out = str(tmp_path / "r0.npz")
    mp.spawn(_rank, args=(2, _port(), out, 1), nprocs=2, join=True)
    got = np.load(out)
    assert got["status"].tolist() == [L.OK, L.ERR_NAMES_INV["KernelLaunch"]]
    assert "zyxb_allreduce_sum" in str(got["text"][1]) and "peer left or timed out" in str(got["text"][1])
    for i, want in enumerate(_oracle_params(1)):          # the completed step is intact
        assert got["p%d" % i].shape == want.shape


def test_an_injected_collective_error_is_reported_not_raised():
    fake = FH.Fake()
    assert fake.lib.zyxb_comm_init(fake.ctx, 0, 0, 1, None) == L.OK
    fake.set_collective(lambda arr, op: 0)
    mlp = FH.FakeMlp(fake, BATCH, DIMS, world=2, **KW)     # a two-rank plan whose peer is the identity callback
    _load(fake, mlp, _layers())
    x, t = _data(0)
    fake.upload(mlp.x, x)
    fake.upload(mlp.target, t)
    fake.fail(FH.COLLECTIVE, 1)
    assert mlp.step() == L.ERR_NAMES_INV["KernelLaunch"]
    assert "ncclSystemError (injected)" in mlp.error()
    mlp.close()
