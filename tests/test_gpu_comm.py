"""The collective entry points of the C ABI on one GPU: error behaviour without a communicator, and the identities that
hold on a one-rank communicator (sum over one rank, one slice scattered and gathered)."""
import numpy as np
import pytest

from zyx_b200 import _lib as L
from zyx_b200 import backend as B

pytestmark = pytest.mark.gpu


def test_collectives_without_a_communicator_are_errors(sess):
    buf = sess.pool.upload(np.arange(64, dtype=np.float32))
    try:
        for call in (lambda: sess.device.allreduce_sum(buf, 64, L.F32), lambda: sess.device.reduce_scatter_sum(buf, 64, L.F32),
                     lambda: sess.device.allgather(buf, 64, L.F32), lambda: sess.device.comm_rank()):
            with pytest.raises(B.BackendError) as e:
                call()
            assert "no communicator" in e.value.context
    finally:
        sess.pool.deallocate(buf)


def test_one_rank_communicator(sess):
    x = np.arange(256, dtype=np.float32)
    buf = sess.pool.upload(x)
    sess.device.comm_init(0, 1, sess.device.comm_unique_id())
    try:
        assert sess.device.comm_rank() == (0, 1)
        with pytest.raises(B.BackendError):
            sess.device.comm_init(0, 1, sess.device.comm_unique_id())          # one communicator per device
        ev = sess.device.allreduce_sum(buf, 256, L.F32, want_event=True)
        sess.pool.sync_events([ev])
        sess.device.reduce_scatter_sum(buf, 128, L.F32, offset_elems=64)
        sess.device.allgather(buf, 128, L.F32, offset_elems=64)
        sess.device.sync()
        assert np.array_equal(sess.pool.download(buf, x.shape, np.float32), x)
        for call in (lambda: sess.device.allreduce_sum(buf, 257, L.F32), lambda: sess.device.reduce_scatter_sum(buf, 200, L.F32, offset_elems=64),
                     lambda: sess.device.allgather(buf, 1, L.F32, offset_elems=256)):
            with pytest.raises(B.BackendError) as e:
                call()
            assert e.value.status_name == "IncorrectKernelArg"
    finally:
        sess.device.comm_destroy()
        sess.pool.deallocate(buf)
