"""The allocation-free column-sum entry point (zyxb_colsum_static), called through the C ABI.

Some callers of this library may not allocate while they run — a plan replayed in a serving loop with a
fixed memory budget, or a host whose own pool already owns all device memory — so this entry point keeps
its partial sums in a fixed array inside the library instead of the context's scratch buffer.  The test
checks it against the ordinary ZYXB_RR_COLSUM program and against the CPU oracle on two calls in a row (the
second call finds the first call's partials still in the array), that the pool's free bytes do not move
across a call once the array's address has been looked up, and that a shape beyond the fixed capacity is
refused.
It is collected last so that a run which stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, TOL_F32
from zyx_b200 import _lib as L
from zyx_b200 import backend as B

pytestmark = pytest.mark.gpu


def _bf16(x):
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


def _f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _colsum_static(sess, dtype, x_buf, y_buf, rows, cols):
    lib, be = sess.backend.lib, sess.backend
    st = lib.zyxb_colsum_static(be.ctx, sess.device.dev, dtype, x_buf, y_buf, rows, cols)
    if st != L.OK:
        raise B.BackendError(st, lib.zyxb_last_error(be.ctx).decode())


@pytest.mark.parametrize("dtype,tol", [(L.F32, TOL_F32), (L.BF16, TOL_BF16), (L.F16, TOL_BF16)])
@pytest.mark.parametrize("shapes", [[(777, 1032), (300, 4096)],      # vector path; the second call reuses dirty scratch
                                    [(129, 1031), (64, 1031)],       # a width no 128-bit vector divides: the scalar path
                                    [(3, 1 << 20), (2, 1 << 20)]])   # the widest shape the array takes: one partial row per column
def test_two_calls_match_the_colsum_program(sess, dtype, tol, shapes):
    rng = np.random.default_rng(21)
    pool, dev = sess.pool, sess.device
    for call, (rows, cols) in enumerate(shapes):
        xf = rng.standard_normal((rows, cols)).astype(np.float32)
        x = xf if dtype == L.F32 else zo.to_bits(xf, dtype)
        es = x.dtype.itemsize
        bx = pool.upload(x)
        by_ref, _ = pool.allocate(cols * es)
        by_new, _ = pool.allocate(cols * es)
        prog = dev.create_program(B.rowreduce_desc(L.RR_COLSUM, dtype, rows, cols))
        try:
            dev.launch(prog, [bx, by_ref])
            if call == 1:
                dev.sync()
                free_before = pool.free_bytes()
            _colsum_static(sess, dtype, bx, by_new, rows, cols)
            if call == 1:                                                    # the array's address is known by now: nothing is allocated
                dev.sync()
                assert pool.free_bytes() == free_before
            ref, new = pool.download(by_ref, (cols,), x.dtype), pool.download(by_new, (cols,), x.dtype)
            want = zo.to_f32(zo.colsum(dtype, x), dtype).astype(np.float64)
            ref, new = zo.to_f32(ref, dtype), zo.to_f32(new, dtype)
            scale = np.sqrt((zo.to_f32(x, dtype).astype(np.float64) ** 2).sum(0))    # a sum that cancels is measured against |x|_2 / 10
            err = np.abs(new.astype(np.float64) - ref) / np.maximum(np.abs(ref), 0.1 * scale)
            assert float(err.max()) <= tol, (call, float(err.max()))
            # the oracle adds the rows one after the other in f32, the kernel adds partial sums: within the tolerance of the oracle,
            # or of the float64 column sums where the two f32 orders themselves are farther apart than that
            exact = zo.to_f32(x, dtype).astype(np.float64).sum(0)
            err = np.abs(new.astype(np.float64) - want) / np.maximum(np.abs(want), 0.1 * scale)
            err64 = np.abs(new.astype(np.float64) - exact) / np.maximum(np.abs(exact), 0.1 * scale)
            assert float(err.max()) <= tol or float(err64.max()) <= tol, ("oracle", call, float(err.max()), float(err64.max()))
        finally:
            dev.release(prog)
            for b in (bx, by_ref, by_new):
                pool.deallocate(b)


def test_capacity_is_enforced_with_a_clear_error(sess):
    cap = C.c_uint64()
    assert sess.backend.lib.zyxb_colsum_static_capacity(C.byref(cap)) == L.OK and cap.value == 1 << 20
    cols = cap.value + 8
    bx, _ = sess.pool.allocate(cols * 4)
    by, _ = sess.pool.allocate(cols * 4)
    try:
        with pytest.raises(B.BackendError) as e:
            _colsum_static(sess, L.F32, bx, by, 1, cols)
        assert e.value.status_name == "IncorrectKernelArg" and "exceed the fixed scratch" in e.value.context
        with pytest.raises(B.BackendError):
            _colsum_static(sess, L.F32, bx, by, 4, cap.value)                 # x would need 4 rows: buffer too small
    finally:
        sess.pool.deallocate(bx)
        sess.pool.deallocate(by)
