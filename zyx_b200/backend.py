"""Host-side mirror of zyx's backend interface over the C ABI.

`MemoryPool` and `Device` carry the same method names, argument meaning and error behaviour
as the enums in zyx/src/backend/mod.rs (542-803 and 806-1028); `BackendError` mirrors
zyx/src/error.rs:107-153.  Everything goes through libzyxb.so; nothing here computes.
"""
import ctypes as C

import numpy as np

from . import _lib as L


class BackendError(RuntimeError):
    """BackendError{status, context} (zyx/src/error.rs:107-111)."""

    def __init__(self, status, context):
        self.status = status
        self.status_name = L.ERR_NAMES.get(status, str(status))
        self.context = context
        super().__init__("%s: %s" % (self.status_name, context))


def _evs(events):
    events = [e for e in (events or []) if e is not None and e.id != 0]
    if not events:
        return None, 0
    arr = (L.Event * len(events))(*events)
    return arr, len(events)


class Backend:
    """One libzyxb context: what initialize_device (zyx/src/backend/cuda.rs:321-326) sets up."""

    def __init__(self, device_ids=None, debug=0, round_nearest=False):
        self.lib = L.load()
        cfg = L.Config()
        ids = list(device_ids or [])
        cfg.n_device_ids = len(ids)
        for i, d in enumerate(ids):
            cfg.device_ids[i] = d
        cfg.debug = debug
        cfg.round_nearest = int(round_nearest)
        self.ctx = C.c_void_p()
        st = self.lib.zyxb_init(C.byref(cfg), C.byref(self.ctx))
        if st != L.OK:
            raise BackendError(st, self.lib.zyxb_last_error(None).decode())
        n = C.c_int32()
        self._check(self.lib.zyxb_device_count(self.ctx, C.byref(n)))
        self.pools = [MemoryPool(self, i) for i in range(n.value)]
        self.devices = [Device(self, i, self.pools[i]) for i in range(n.value)]

    def _check(self, st):
        if st != L.OK:
            raise BackendError(st, self.lib.zyxb_last_error(self.ctx).decode())

    def deinitialize(self):
        if self.ctx:
            self.lib.zyxb_shutdown(self.ctx)
            self.ctx = None

    def host_register(self, arr):
        self._check(self.lib.zyxb_host_register(self.ctx, arr.ctypes.data_as(C.c_void_p), arr.nbytes))

    def host_unregister(self, arr):
        self._check(self.lib.zyxb_host_unregister(self.ctx, arr.ctypes.data_as(C.c_void_p)))

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.deinitialize()


class MemoryPool:
    """MemoryPool (zyx/src/backend/mod.rs:542-803)."""

    def __init__(self, backend, dev):
        self.be, self.dev = backend, dev

    def free_bytes(self):
        v = C.c_uint64()
        self.be._check(self.be.lib.zyxb_free_bytes(self.be.ctx, self.dev, C.byref(v)))
        return v.value

    def allocate(self, nbytes):
        """-> (PoolBufferId, Event)"""
        buf, ev = C.c_uint32(), L.Event()
        self.be._check(self.be.lib.zyxb_alloc(self.be.ctx, self.dev, int(nbytes), C.byref(buf), C.byref(ev)))
        return buf.value, ev

    def deallocate(self, buffer_id, event_wait_list=None):
        arr, n = _evs(event_wait_list)
        self.be._check(self.be.lib.zyxb_free(self.be.ctx, self.dev, buffer_id, arr, n))

    def host_to_pool(self, src, dst, event_wait_list=None, dst_offset=0, want_event=True):
        """Asynchronous; `src` (a contiguous numpy array) must stay alive until the event is synced."""
        assert src.flags["C_CONTIGUOUS"]
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_h2d(self.be.ctx, self.dev, src.ctypes.data_as(C.c_void_p), src.nbytes, dst, dst_offset,
                                            arr, n, C.byref(ev) if want_event else None))
        return ev

    def pool_to_host(self, src, dst, event_wait_list=None, src_offset=0):
        """Blocking."""
        assert dst.flags["C_CONTIGUOUS"]
        arr, n = _evs(event_wait_list)
        self.be._check(self.be.lib.zyxb_d2h(self.be.ctx, self.dev, src, src_offset, dst.ctypes.data_as(C.c_void_p), dst.nbytes, arr, n))

    def pool_to_pool(self, src_pool, src, dst, nbytes, event_wait_list=None, src_offset=0, dst_offset=0):
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_d2d(self.be.ctx, src_pool.dev, src, src_offset, self.dev, dst, dst_offset, int(nbytes),
                                            arr, n, C.byref(ev)))
        return ev

    def memset(self, buf, byte_value, nbytes, offset=0):
        self.be._check(self.be.lib.zyxb_memset(self.be.ctx, self.dev, buf, offset, byte_value, int(nbytes)))

    def sync_events(self, events):
        arr, n = _evs(events)
        if n:
            self.be._check(self.be.lib.zyxb_sync(self.be.ctx, self.dev, arr, n))

    def release_events(self, events):
        arr, n = _evs(events)
        if n:
            self.be._check(self.be.lib.zyxb_release_events(self.be.ctx, self.dev, arr, n))

    def store_variable(self, dtype, value_bytes):
        buf = C.c_uint32()
        raw = (C.c_uint8 * 8)(*bytes(value_bytes).ljust(8, b"\0"))
        self.be._check(self.be.lib.zyxb_store_variable(self.be.ctx, self.dev, dtype, raw, C.byref(buf)))
        return buf.value

    def get_variable(self, buffer_id):
        dt = C.c_int32()
        raw = (C.c_uint8 * 8)()
        st = self.be.lib.zyxb_get_variable(self.be.ctx, self.dev, buffer_id, C.byref(dt), raw)
        if st != L.OK:
            return None
        return dt.value, bytes(raw)[:L.DTYPE_SIZE[dt.value]]

    def view(self, parent, offset, nbytes):
        buf = C.c_uint32()
        self.be._check(self.be.lib.zyxb_buffer_view(self.be.ctx, self.dev, parent, int(offset), int(nbytes), C.byref(buf)))
        return buf.value

    def buffer_bytes(self, buffer_id):
        v = C.c_uint64()
        self.be._check(self.be.lib.zyxb_buffer_bytes(self.be.ctx, self.dev, buffer_id, C.byref(v)))
        return v.value

    # convenience used by tests and the bench
    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        buf, _ = self.allocate(max(arr.nbytes, 1))
        if arr.nbytes:
            self.sync_events([self.host_to_pool(arr, buf)])
        return buf

    def download(self, buf, shape, dtype):
        out = np.empty(shape, dtype)
        if out.nbytes:
            self.pool_to_host(buf, out)
        return out


class Device:
    """Device (zyx/src/backend/mod.rs:806-1028).  `aot_only`: programs are created from kernel
    descriptors (what the shim's match_graph recognises), never from zyx IR."""

    def __init__(self, backend, dev, pool):
        self.be, self.dev, self.pool = backend, dev, pool

    def info(self):
        o = L.DevInfo()
        self.be._check(self.be.lib.zyxb_device_info(self.be.ctx, self.dev, C.byref(o)))
        return o

    def memory_pool_id(self):
        return self.dev

    def free_compute(self):
        v = C.c_uint64()
        self.be._check(self.be.lib.zyxb_free_compute(self.be.ctx, self.dev, C.byref(v)))
        return v.value

    def aot_only(self):
        return True

    def compile(self, kernel, debug_asm=False):
        """Generic IR is not accepted (as CblasDevice::compile, zyx/src/backend/cblas.rs:203-208)."""
        raise BackendError(11, "b200 backend is AOT only")

    def create_program(self, desc):
        prog = C.c_uint32()
        self.be._check(self.be.lib.zyxb_program_create(self.be.ctx, self.dev, C.byref(desc), C.byref(prog)))
        return prog.value

    def launch(self, program_id, args, event_wait_list=None, want_event=False):
        """args = loads then stores (zyx/src/runtime.rs:2285-2291)."""
        arr, n = _evs(event_wait_list)
        a = (C.c_uint32 * len(args))(*args)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_launch(self.be.ctx, self.dev, program_id, a, len(args), arr, n,
                                               C.byref(ev) if want_event else None))
        return ev

    def release(self, program_id):
        self.be._check(self.be.lib.zyxb_program_release(self.be.ctx, self.dev, program_id))

    def set_step(self, program_id, t):
        self.be._check(self.be.lib.zyxb_program_set_step(self.be.ctx, self.dev, program_id, int(t)))

    def check_guards(self):
        """With Backend(debug=2): raises BackendError naming the buffer a kernel wrote past the end of; returns None when all are intact."""
        bad = C.c_uint32()
        self.be._check(self.be.lib.zyxb_check_guards(self.be.ctx, self.dev, C.byref(bad)))

    def get_step(self, program_id):
        t = C.c_uint64()
        self.be._check(self.be.lib.zyxb_program_get_step(self.be.ctx, self.dev, program_id, C.byref(t)))
        return t.value

    def sync(self):
        self.be._check(self.be.lib.zyxb_device_sync(self.be.ctx, self.dev))

    def status(self):
        w = C.c_uint32()
        self.be._check(self.be.lib.zyxb_device_status(self.be.ctx, self.dev, C.byref(w)))
        return w.value

    def launch_count(self):
        v = C.c_uint64()
        self.be._check(self.be.lib.zyxb_launch_count(self.be.ctx, self.dev, C.byref(v)))
        return v.value

    def event_record(self):
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_event_record(self.be.ctx, self.dev, C.byref(ev)))
        return ev

    def elapsed_ms(self, start, stop):
        ms = C.c_float()
        self.be._check(self.be.lib.zyxb_event_elapsed_ms(self.be.ctx, self.dev, start, stop, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        self.be._check(self.be.lib.zyxb_flush_l2(self.be.ctx, self.dev))

    # ---- captured launch sequences (FrozenTape::replay) ---------------------------------------------
    def capture_begin(self):
        self.be._check(self.be.lib.zyxb_capture_begin(self.be.ctx, self.dev))

    def capture_end(self):
        g = C.c_uint32()
        self.be._check(self.be.lib.zyxb_capture_end(self.be.ctx, self.dev, C.byref(g)))
        return g.value

    def graph_launch(self, graph, event_wait_list=None, want_event=False):
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_graph_launch(self.be.ctx, self.dev, graph, arr, n, C.byref(ev) if want_event else None))
        return ev

    def graph_release(self, graph):
        self.be._check(self.be.lib.zyxb_graph_release(self.be.ctx, self.dev, graph))

    # ---- data-parallel exchange -------------------------------------------------------------
    def comm_unique_id(self):
        raw = (C.c_uint8 * 128)()
        self.be._check(self.be.lib.zyxb_comm_unique_id(self.be.ctx, raw))
        return bytes(raw)

    def comm_init(self, rank, world, unique_id):
        raw = (C.c_uint8 * 128)(*unique_id)
        self.be._check(self.be.lib.zyxb_comm_init(self.be.ctx, self.dev, rank, world, raw))

    def allreduce_sum(self, buf, count, dtype, offset_elems=0, event_wait_list=None, want_event=False):
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_allreduce_sum(self.be.ctx, self.dev, buf, offset_elems, count, dtype, arr, n,
                                                      C.byref(ev) if want_event else None))
        return ev

    def reduce_scatter_sum(self, buf, count_per_rank, dtype, offset_elems=0, event_wait_list=None, want_event=False):
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_reduce_scatter_sum(self.be.ctx, self.dev, buf, offset_elems, count_per_rank, dtype, arr, n,
                                                           C.byref(ev) if want_event else None))
        return ev

    def allgather(self, buf, count_per_rank, dtype, offset_elems=0, event_wait_list=None, want_event=False):
        arr, n = _evs(event_wait_list)
        ev = L.Event()
        self.be._check(self.be.lib.zyxb_allgather(self.be.ctx, self.dev, buf, offset_elems, count_per_rank, dtype, arr, n,
                                                  C.byref(ev) if want_event else None))
        return ev

    def comm_option(self, option, value):
        self.be._check(self.be.lib.zyxb_comm_option(self.be.ctx, self.dev, option, value))

    def comm_rank(self):
        r, w = C.c_int32(), C.c_int32()
        self.be._check(self.be.lib.zyxb_comm_rank(self.be.ctx, self.dev, C.byref(r), C.byref(w)))
        return r.value, w.value

    def comm_destroy(self):
        self.be._check(self.be.lib.zyxb_comm_destroy(self.be.ctx, self.dev))


# ---- descriptor builders (what the shim's matcher would fill in) --------------------------------
def rowreduce_desc(op, dtype, rows, cols, eps=0.0, correction=1, has_weight=False, has_bias=False, scale=0.0, causal=False,
                   period=0):
    d = L.KernelDesc()
    d.kind = L.KIND_ROWREDUCE
    r = d.u.rowreduce
    r.op, r.dtype, r.rows, r.cols, r.eps, r.correction = op, dtype, rows, cols, eps, correction
    r.has_weight, r.has_bias, r.scale, r.causal, r.period = int(has_weight), int(has_bias), scale, int(causal), period
    return d


def attention_desc(dtype, batch, heads, seq, head_dim, ld=0, scale=0.0, causal=False, backward=False):
    d = L.KernelDesc()
    d.kind = L.KIND_ATTENTION_BWD if backward else L.KIND_ATTENTION
    a = d.u.attention
    a.dtype, a.batch, a.heads, a.seq, a.head_dim, a.ld, a.scale, a.causal = dtype, batch, heads, seq, head_dim, ld, scale, int(causal)
    return d


def _pads(padding):
    """(top, bottom, left, right) from an int, (pad_h, pad_w) or the four values."""
    if isinstance(padding, int):
        return (padding,) * 4
    if len(padding) == 2:
        return (padding[0], padding[0], padding[1], padding[1])
    return tuple(padding)


def conv_out_shape(x_shape, w_shape, stride=1, dilation=1, padding=0):
    """[n, o, oh, ow] of Tensor::conv (zyx/src/tensor/mod.rs:2583-2680) for x [n,c,h,w], w [o,c,kh,kw]."""
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    dh, dw = (dilation, dilation) if isinstance(dilation, int) else dilation
    pt, pb, pl, pr = _pads(padding)
    n, _, h, w = x_shape
    o, _, kh, kw = w_shape
    return (n, o, (h + pt + pb - dh * (kh - 1) - 1) // sh + 1, (w + pl + pr - dw * (kw - 1) - 1) // sw + 1)


def conv_desc(dtype, x_shape, w_shape, stride=1, dilation=1, padding=0, has_bias=False, channels_last=False, flip_filter=False):
    """x_shape is always given as (n, c, h, w), whatever the memory layout; w_shape as (o, c, kh, kw) of THIS convolution
    (with flip_filter the buffer itself is laid out [c, o, kh, kw]: the forward convolution's filter)."""
    d = L.KernelDesc()
    d.kind = L.KIND_CONV
    c = d.u.conv
    c.dtype = dtype
    c.n, c.c, c.h, c.w = x_shape
    c.o, _, c.kh, c.kw = w_shape
    c.stride_h, c.stride_w = (stride, stride) if isinstance(stride, int) else stride
    c.dil_h, c.dil_w = (dilation, dilation) if isinstance(dilation, int) else dilation
    c.pad_top, c.pad_bottom, c.pad_left, c.pad_right = _pads(padding)
    c.has_bias, c.channels_last, c.flip_filter = int(has_bias), int(channels_last), int(flip_filter)
    return d


def gemm_desc(dtype, m, n, k, batch=1, trans_a=False, trans_b=False, stride_a=None, stride_b=None, stride_c=None,
              epilogue=L.EPI_NONE, store_preact=False, alpha=0.0, lda=0, ldb=0, ldc=0, batch_inner=0, stride_a_inner=0,
              stride_b_inner=0, stride_c_inner=0, tri=0):
    d = L.KernelDesc()
    d.kind = L.KIND_GEMM
    g = d.u.gemm
    g.dtype, g.m, g.n, g.k, g.batch = dtype, m, n, k, batch
    g.trans_a, g.trans_b = int(trans_a), int(trans_b)
    g.stride_a = m * k if stride_a is None else stride_a
    g.stride_b = k * n if stride_b is None else stride_b
    g.stride_c = m * n if stride_c is None else stride_c
    g.epilogue, g.store_preact, g.alpha = epilogue, int(store_preact), alpha
    g.lda, g.ldb, g.ldc, g.batch_inner = lda, ldb, ldc, batch_inner
    g.stride_a_inner, g.stride_b_inner, g.stride_c_inner = stride_a_inner, stride_b_inner, stride_c_inner
    g.tri = tri
    return d


def eltwise_desc(op, dtype, numel, p0=0.0, dtype_out=None, cols=0):
    d = L.KernelDesc()
    d.kind = L.KIND_ELTWISE
    e = d.u.eltwise
    e.op, e.dtype, e.dtype_out, e.numel, e.cols, e.p0 = op, dtype, dtype if dtype_out is None else dtype_out, numel, cols, p0
    return d


def optim_desc(algo, dtype, numels, lr, weight_decay=0.0, momentum=0.0, dampening=0.0, nesterov=False, maximize=False,
               beta1=0.9, beta2=0.999, eps=1e-8, grad_scale=0.0, standard=False):
    d = L.KernelDesc()
    d.kind = L.KIND_OPTIM
    o = d.u.optim
    arr = (C.c_uint64 * len(numels))(*numels)
    d._numel_keepalive = arr
    o.algo, o.dtype, o.n_tensors, o.numel = algo, dtype, len(numels), arr
    o.lr, o.weight_decay, o.momentum, o.dampening, o.nesterov, o.maximize = lr, weight_decay, momentum, dampening, int(nesterov), int(maximize)
    o.beta1, o.beta2, o.eps, o.grad_scale, o.standard = beta1, beta2, eps, grad_scale, int(standard)
    return d
