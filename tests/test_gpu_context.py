"""Context-level behaviour of the C ABI: what a capture accepts, stream ordering of a recycled block, overflowing ranges,
and one context driving two GPUs."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import TOL_BF16, max_rel_err
from zyx_b200 import _lib as L
from zyx_b200 import backend as B

pytestmark = pytest.mark.gpu


def test_a_capture_refuses_what_it_cannot_record(sess):
    """Inside zyxb_capture_begin .. zyxb_capture_end only launches without wait lists are recorded.  Allocation, copies,
    blocking calls and optimizer programs whose update depends on the step counter (a captured launch would replay the
    captured step for ever: SGD with momentum re-initialising its buffer, Adam with frozen bias corrections) answer with
    an error text instead of invalidating the capture; plain SGD is recorded and does not advance the counter."""
    d, p = sess.device, sess.pool
    n = 4096
    rng = np.random.default_rng(3)
    pv, gv = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    bp, bg, bm, bv = p.upload(pv), p.upload(gv), p.upload(np.zeros(n, np.float32)), p.upload(np.zeros(n, np.float32))
    plain = d.create_program(B.optim_desc(L.OPT_SGD, L.F32, [n], lr=0.1))
    momentum = d.create_program(B.optim_desc(L.OPT_SGD, L.F32, [n], lr=0.1, momentum=0.9))
    adamw = d.create_program(B.optim_desc(L.OPT_ADAMW, L.F32, [n], lr=1e-3, weight_decay=0.01))
    host = np.empty(n, np.float32)
    d.sync()
    d.capture_begin()
    graph = None
    try:
        for call, text in ((lambda: d.launch(momentum, [bp, bg, bm]), "depends on the step counter"),
                           (lambda: d.launch(adamw, [bp, bg, bm, bv]), "depends on the step counter"),
                           (lambda: p.allocate(1024), "zyxb_alloc"), (lambda: p.pool_to_host(bp, host), "zyxb_d2h"),
                           (lambda: p.host_to_pool(pv, bp), "zyxb_h2d"), (lambda: d.sync(), "zyxb_device_sync"),
                           (lambda: p.deallocate(bv), "zyxb_free")):
            with pytest.raises(B.BackendError) as e:
                call()
            assert text in e.value.context, e.value.context
        d.launch(plain, [bp, bg])
        assert d.get_step(plain) == 0                  # recorded, not run
    finally:
        graph = d.capture_end()
    try:
        for _ in range(3):
            d.graph_launch(graph)
        want = pv.copy()
        for _ in range(3):
            zo.sgd(zo.F32, want, gv, None, lr=0.1)
        assert max_rel_err(p.download(bp, (n,), np.float32), want) <= 1e-5       # FMA contraction differs by an ulp of the larger operand
        # outside a capture the step-dependent programs run and count
        d.launch(momentum, [bp, bg, bm])
        d.launch(momentum, [bp, bg, bm])
        assert d.get_step(momentum) == 2 and d.status() == 0
    finally:
        d.graph_release(graph)
        for prog in (plain, momentum, adamw):
            d.release(prog)
        for b in (bp, bg, bm, bv):
            p.deallocate(b)


def test_an_upload_into_a_recycled_block_waits_for_its_previous_owner(sess):
    """zyx allocates, then uploads waiting on the event the allocation returned (a null event here).  When the block comes
    from the cache, kernels queued before its previous owner was freed may still write it: the upload on the copy stream has
    to go behind them."""
    d, p, lib, be = sess.device, sess.pool, sess.backend.lib, sess.backend
    n = 8192
    rng = np.random.default_rng(5)
    a = zo.to_bits(rng.uniform(-1, 1, (n, n)).astype(np.float32), zo.BF16)
    ba, bb = p.upload(a), p.upload(a)
    prog = d.create_program(B.gemm_desc(L.BF16, n, n, n))
    pattern = np.full(n * n, 0x3C00, np.uint16)
    be.host_register(pattern)
    got = np.empty_like(pattern)
    try:
        for _ in range(3):
            bc, _ = p.allocate(n * n * 2)
            d.launch(prog, [ba, bb, bc])                   # ~0.75 ms of writes into bc
            p.deallocate(bc)                               # back to the cache while the matmul is still queued or running
            buf, ev = C.c_uint32(), L.Event()
            assert lib.zyxb_alloc(be.ctx, d.dev, n * n * 2, C.byref(buf), C.byref(ev)) == L.OK     # the same block again
            wait = (L.Event * 1)(ev)                       # the null event, passed on as zyx would
            out = L.Event()
            assert lib.zyxb_h2d(be.ctx, d.dev, pattern.ctypes.data_as(C.c_void_p), pattern.nbytes, buf.value, 0, wait, 1, C.byref(out)) == L.OK
            p.sync_events([out])
            d.sync()
            p.pool_to_host(buf.value, got)
            assert np.array_equal(got, pattern)
            p.deallocate(buf.value)
    finally:
        be.host_unregister(pattern)
        d.release(prog)
        p.deallocate(ba)
        p.deallocate(bb)


def test_ranges_that_wrap_around_are_refused(sess):
    d, p = sess.device, sess.pool
    buf, _ = p.allocate(4096)
    host = np.zeros(16, np.uint8)
    big = (1 << 64) - 8
    try:
        with pytest.raises(B.BackendError):
            p.host_to_pool(host, buf, dst_offset=big)
        with pytest.raises(B.BackendError):
            p.pool_to_host(buf, host, src_offset=big)
        with pytest.raises(B.BackendError):
            sess.backend._check(sess.backend.lib.zyxb_memset(sess.backend.ctx, d.dev, buf, big, 0, 16))
        # a matmul whose pitch would wrap the span computation
        desc = B.gemm_desc(L.F32, 4, 4, 4, lda=(1 << 62) + 1)
        prog = d.create_program(desc)
        try:
            with pytest.raises(B.BackendError) as e:
                d.launch(prog, [buf, buf, buf])
            assert e.value.status_name == "IncorrectKernelArg"
        finally:
            d.release(prog)
    finally:
        p.deallocate(buf)


def test_communicator_options_are_validated(sess):
    d = sess.device
    d.comm_option(L.COMM_OPT_LATENCY, 1)          # a per-device setting: accepted with or without a communicator
    d.comm_option(L.COMM_OPT_LATENCY, 0)
    with pytest.raises(B.BackendError) as e:
        d.comm_option(99, 1)
    assert e.value.status_name == "IncorrectKernelArg"


def test_one_context_drives_two_gpus():
    """`zyxb_init` without device ids opens every GPU in one context.  The shared-memory limit of the tensor-core kernels is a
    per-device attribute: the second device must get it too (a bf16 matmul, the fused attention and a convolution on device 1
    after device 0).  Plain kernels only, no peer operands."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from oracle import models as zm
    from zyx_b200.ops import Session
    s = Session(device_ids=[0, 1])
    rng = np.random.default_rng(8)
    try:
        a = zo.to_bits(rng.uniform(-1, 1, (512, 384)).astype(np.float32), zo.BF16)
        b = zo.to_bits(rng.uniform(-1, 1, (384, 640)).astype(np.float32), zo.BF16)
        want = zo.to_f32(zo.gemm(zo.BF16, a, b), zo.BF16)
        q, k, v = (zo.to_bits(rng.standard_normal((1, 256, 128)).astype(np.float32), zo.BF16) for _ in range(3))
        want_o, _, exact = zm.attention(zo.BF16, q, k, v, 1, True)
        xc = zo.to_bits(rng.standard_normal((1, 64, 16, 16)).astype(np.float32), zo.BF16)
        wc = zo.to_bits((rng.standard_normal((64, 64, 3, 3)) / 24.0).astype(np.float32), zo.BF16)
        want_c = zo.to_f32(zo.conv(zo.BF16, xc, wc, None, 1, 1, 1), zo.BF16).reshape(64, -1)
        x32 = rng.standard_normal((4096, 32768)).astype(np.float32)[:512]
        for dev in (0, 1):
            sd = s.on_device(dev)
            assert max_rel_err(zo.to_f32(sd.gemm(L.BF16, a, b), zo.BF16), want, floor=0.1) <= TOL_BF16, dev
            o, _ = sd.attention(L.BF16, q, k, v, 1, causal=True)
            assert max_rel_err(zo.to_f32(o, zo.BF16), zo.to_f32(want_o, zo.BF16), floor=1.0) <= 2 * TOL_BF16, dev
            got_c = zo.to_f32(sd.conv(L.BF16, xc, wc, None, 1, 1, 1), zo.BF16).reshape(64, -1)
            assert max_rel_err(got_c, want_c, floor=0.1) <= TOL_BF16, dev
            assert max_rel_err(sd.softmax(L.F32, x32), zo.softmax(zo.F32, x32)) <= 1e-5, dev      # the staged row kernel (128 KB rows)
            assert sd.device.status() == 0
    finally:
        s.close()


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(sess):
    """The bounded wait every tensor-core kernel spins in, made to run out on purpose: a barrier nothing arrives on, a limit of
    one millisecond.  The kernel returns by itself, the status word carries the code, zyxb_device_status turns it into
    KernelSync once and clears it, and an ordinary tensor-core matmul afterwards is clean.  Nothing faults or hangs."""
    import time
    lib, be, d = sess.backend.lib, sess.backend, sess.device
    assert d.status() == 0
    gave_up = C.c_uint32(7)
    t0 = time.perf_counter()
    assert lib.zyxb_selftest_bounded_wait(be.ctx, d.dev, 1_000_000, C.byref(gave_up)) == L.OK
    assert time.perf_counter() - t0 < 1.0                # a millisecond plus launch overhead, nowhere near the 2 s production bound
    assert gave_up.value == 1
    with pytest.raises(B.BackendError) as e:
        d.status()
    assert e.value.status_name == "KernelSync" and "bounded wait" in e.value.context
    assert d.status() == 0                               # reading cleared it
    rng = np.random.default_rng(2)
    a = zo.to_bits(rng.uniform(-1, 1, (256, 512)).astype(np.float32), zo.BF16)
    b = zo.to_bits(rng.uniform(-1, 1, (512, 384)).astype(np.float32), zo.BF16)
    got = zo.to_f32(sess.gemm(L.BF16, a, b), zo.BF16)
    assert max_rel_err(got, zo.to_f32(zo.gemm(zo.BF16, a, b), zo.BF16), floor=0.1) <= TOL_BF16
    assert d.status() == 0
    with pytest.raises(B.BackendError):                  # the limit is itself bounded
        be._check(lib.zyxb_selftest_bounded_wait(be.ctx, d.dev, 10_000_000_000, C.byref(gave_up)))
