"""ctypes binding of libzyxb_host.so (include/zyxb_host.h): the C++ training plan for a stack of
zyx_nn::Linear layers, replayed through the C ABI.  Python only moves host arrays in and out."""
import ctypes as C
import os

import numpy as np

from . import _lib as L
from .backend import BackendError

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(_HERE, "libzyxb_host.so")

ACT_NONE, ACT_RELU, ACT_GELU = range(3)
LOSS_MSE, LOSS_CROSS_ENTROPY = range(2)


class MlpConfig(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint64), ("n_layers", C.c_int32), ("dims", C.c_uint64 * 9), ("activation", C.c_int32),
                ("loss", C.c_int32), ("optim", L.OptimDesc), ("world", C.c_int32), ("bucket_per_layer", C.c_int32), ("shard_optimizer", C.c_int32)]


_P = C.c_void_p
HOST_SIGNATURES = {
    "zyxb_mlp_create": (C.c_int32, [_P, C.c_int32, C.POINTER(MlpConfig), C.POINTER(_P)]),
    "zyxb_mlp_destroy": (C.c_int32, [_P]),
    "zyxb_mlp_last_error": (C.c_char_p, [_P]),
    "zyxb_mlp_tensor": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "zyxb_mlp_io": (C.c_int32, [_P] + [C.POINTER(C.c_uint32)] * 4),
    "zyxb_mlp_activation": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "zyxb_mlp_forward_backward": (C.c_int32, [_P]),
    "zyxb_mlp_update": (C.c_int32, [_P]),
    "zyxb_mlp_step": (C.c_int32, [_P, C.POINTER(L.Event), C.c_int32]),
    "zyxb_mlp_step_event": (C.c_int32, [_P, C.POINTER(L.Event), C.c_int32, C.POINTER(L.Event)]),
    "zyxb_mlp_bind_inputs": (C.c_int32, [_P, C.c_uint32, C.c_uint32]),
    "zyxb_mlp_plan_size": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "zyxb_mlp_profile": (C.c_int32, [_P, C.c_int32]),
    "zyxb_mlp_profile_read": (C.c_int32, [_P, C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
}

_lib = None


def load():
    global _lib
    if _lib is None:
        L.load()   # libzyxb.so first: the host library resolves the C ABI from it
        if not os.path.exists(HOST_LIB_PATH):
            raise ImportError("zyx_b200: %s is missing — build it with `python -m zyx_b200.build`" % HOST_LIB_PATH)
        lib = C.CDLL(HOST_LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in HOST_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


PARAM, GRAD, STATE0, STATE1 = range(4)
ACT_OUT, ACT_PRE, ACT_GRAD = range(3)


class Mlp:
    """A stack of Linear layers with its training plan (forward, loss, backward, optimizer)."""

    def __init__(self, session, dtype, batch, dims, activation=ACT_GELU, loss=LOSS_MSE, algo=L.OPT_ADAMW, world=1,
                 bucket_per_layer=True, shard_optimizer=False, **optim_kw):
        self.lib, self.sess = load(), session
        cfg = MlpConfig()
        cfg.dtype, cfg.batch, cfg.n_layers, cfg.activation, cfg.loss = dtype, batch, len(dims) - 1, activation, loss
        for i, d in enumerate(dims):
            cfg.dims[i] = d
        o = cfg.optim
        o.algo = algo
        o.lr, o.weight_decay = optim_kw.get("lr", 1e-3), optim_kw.get("weight_decay", 0.0)
        o.momentum, o.dampening = optim_kw.get("momentum", 0.0), optim_kw.get("dampening", 0.0)
        o.nesterov, o.maximize = int(optim_kw.get("nesterov", False)), int(optim_kw.get("maximize", False))
        o.beta1, o.beta2, o.eps = optim_kw.get("beta1", 0.9), optim_kw.get("beta2", 0.999), optim_kw.get("eps", 1e-8)
        o.standard = int(optim_kw.get("standard", False))
        cfg.world, cfg.bucket_per_layer, cfg.shard_optimizer = world, int(bucket_per_layer), int(shard_optimizer)
        self.cfg, self.dims, self.dtype, self.batch = cfg, list(dims), dtype, batch
        self.h = _P()
        st = self.lib.zyxb_mlp_create(session.backend.ctx, session.device.dev, C.byref(cfg), C.byref(self.h))
        if st != L.OK:
            raise BackendError(st, session.backend.lib.zyxb_last_error(session.backend.ctx).decode())
        bufs = [C.c_uint32() for _ in range(4)]
        self._check(self.lib.zyxb_mlp_io(self.h, *[C.byref(b) for b in bufs]))
        self.x, self.target, self.loss, self.y = (b.value for b in bufs)
        self.np_dtype = np.float32 if dtype == L.F32 else np.uint16

    def _check(self, st):
        if st != L.OK:
            raise BackendError(st, self.lib.zyxb_mlp_last_error(self.h).decode())

    def n_params(self):
        return 2 * self.cfg.n_layers

    def tensor(self, which, i):
        buf, n = C.c_uint32(), C.c_uint64()
        self._check(self.lib.zyxb_mlp_tensor(self.h, which, i, C.byref(buf), C.byref(n)))
        return buf.value, n.value

    def shape(self, i):
        layer = i // 2
        return (self.dims[layer + 1], self.dims[layer]) if i % 2 == 0 else (self.dims[layer + 1],)

    def set_tensor(self, which, i, arr):
        buf, n = self.tensor(which, i)
        arr = np.ascontiguousarray(arr)
        assert arr.size == n and arr.dtype == self.np_dtype
        self.sess.pool.sync_events([self.sess.pool.host_to_pool(arr, buf)])

    def get_tensor(self, which, i):
        buf, _ = self.tensor(which, i)
        return self.sess.pool.download(buf, self.shape(i), self.np_dtype)

    def set_batch(self, x, target):
        p = self.sess.pool
        return [p.host_to_pool(np.ascontiguousarray(x), self.x), p.host_to_pool(np.ascontiguousarray(target), self.target)]

    def activation(self, which, layer, rows=None):
        """A tensor the plan keeps between forward and backward: which = ACT_OUT (the layer's output), ACT_PRE (its
        pre-activation) or ACT_GRAD (the loss gradient w.r.t. the pre-activation), [batch, dims[layer+1]]; `rows` selects rows."""
        buf, n = C.c_uint32(), C.c_uint64()
        self._check(self.lib.zyxb_mlp_activation(self.h, which, layer, C.byref(buf), C.byref(n)))
        cols = self.dims[layer + 1]
        if rows is None:
            return self.sess.pool.download(buf.value, (self.batch, cols), self.np_dtype)
        out = np.empty((len(rows), cols), self.np_dtype)
        for i, r in enumerate(rows):
            self.sess.pool.pool_to_host(buf.value, out[i], src_offset=int(r) * cols * out.itemsize)
        return out

    def forward_backward(self):
        self._check(self.lib.zyxb_mlp_forward_backward(self.h))

    def update(self):
        self._check(self.lib.zyxb_mlp_update(self.h))

    def save(self, path):
        """Parameters, optimizer state and step counter into a safetensors file (Module::save)."""
        self._check(self.lib.zyxb_mlp_save(self.h, os.fsencode(path)))

    def load(self, path):
        """-> number of the plan's tensors the file did not hold."""
        missing = C.c_int32()
        self._check(self.lib.zyxb_mlp_load(self.h, os.fsencode(path), C.byref(missing)))
        return missing.value

    def step(self, events=None, want_event=False):
        events = [e for e in (events or []) if e.id != 0]
        arr = (L.Event * len(events))(*events) if events else None
        if not want_event:
            self._check(self.lib.zyxb_mlp_step(self.h, arr, len(events)))
            return None
        ev = L.Event()
        self._check(self.lib.zyxb_mlp_step_event(self.h, arr, len(events), C.byref(ev)))
        return ev

    def bind_inputs(self, x_buf, target_buf):
        self._check(self.lib.zyxb_mlp_bind_inputs(self.h, x_buf, target_buf))
        self.x, self.target = x_buf, target_buf

    def read_loss(self):
        return float(self.sess.pool.download(self.loss, (1,), np.float32)[0])

    def read_output(self):
        return self.sess.pool.download(self.y, (self.batch, self.dims[-1]), self.np_dtype)

    def plan_size(self):
        a, b = C.c_int32(), C.c_int32()
        self._check(self.lib.zyxb_mlp_plan_size(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def profile(self, enable):
        self._check(self.lib.zyxb_mlp_profile(self.h, int(enable)))

    def profile_read(self):
        """-> (ms per instruction summed over the recorded steps, kind per instruction, steps)"""
        n, steps = C.c_int32(), C.c_int32()
        self._check(self.lib.zyxb_mlp_profile_read(self.h, None, None, 0, C.byref(n), C.byref(steps)))
        ms, kind = (C.c_float * n.value)(), (C.c_int32 * n.value)()
        self._check(self.lib.zyxb_mlp_profile_read(self.h, ms, kind, n.value, C.byref(n), C.byref(steps)))
        return list(ms), list(kind), steps.value

    def close(self):
        if self.h:
            self.lib.zyxb_mlp_destroy(self.h)
            self.h = None


# ---- transformer block ---------------------------------------------------------------------------------
class BlockConfig(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("batch", C.c_uint64), ("seq", C.c_uint64), ("dim", C.c_uint64), ("heads", C.c_uint64),
                ("ffn", C.c_uint64), ("causal", C.c_int32), ("eps", C.c_float), ("optim", L.OptimDesc), ("world", C.c_int32),
                ("fused_attention", C.c_int32), ("shard_optimizer", C.c_int32)]


BLOCK_SIGNATURES = {
    "zyxb_block_create": (C.c_int32, [_P, C.c_int32, C.POINTER(BlockConfig), C.POINTER(_P)]),
    "zyxb_block_destroy": (C.c_int32, [_P]),
    "zyxb_block_last_error": (C.c_char_p, [_P]),
    "zyxb_block_tensor": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "zyxb_block_io": (C.c_int32, [_P] + [C.POINTER(C.c_uint32)] * 4),
    "zyxb_block_forward_backward": (C.c_int32, [_P]),
    "zyxb_block_update": (C.c_int32, [_P]),
    "zyxb_block_step": (C.c_int32, [_P, C.POINTER(L.Event), C.c_int32]),
    "zyxb_block_plan_size": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "zyxb_block_activation": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_uint32)]),
}
HOST_SIGNATURES.update(BLOCK_SIGNATURES)


class StTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.POINTER(C.c_uint64)), ("data", C.c_void_p)]


ST_SIGNATURES = {
    "zyxb_st_save": (C.c_int32, [C.c_char_p, C.POINTER(StTensor), C.c_int32]),
    "zyxb_st_open": (C.c_int32, [C.c_char_p, C.POINTER(_P)]),
    "zyxb_st_count": (C.c_int32, [_P]),
    "zyxb_st_info": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_char_p), C.POINTER(C.c_int32), C.POINTER(C.c_int32),
                                 C.POINTER(C.POINTER(C.c_uint64)), C.POINTER(C.c_uint64)]),
    "zyxb_st_find": (C.c_int32, [_P, C.c_char_p]),
    "zyxb_st_read": (C.c_int32, [_P, C.c_int32, C.c_void_p, C.c_uint64]),
    "zyxb_st_close": (C.c_int32, [_P]),
    "zyxb_st_last_error": (C.c_char_p, []),
    "zyxb_mlp_save": (C.c_int32, [_P, C.c_char_p]),
    "zyxb_mlp_load": (C.c_int32, [_P, C.c_char_p, C.POINTER(C.c_int32)]),
    "zyxb_block_save": (C.c_int32, [_P, C.c_char_p]),
    "zyxb_block_load": (C.c_int32, [_P, C.c_char_p, C.POINTER(C.c_int32)]),
}
HOST_SIGNATURES.update(ST_SIGNATURES)
BLOCK_ACTIVATIONS = {name: i for i, name in enumerate(["p", "attn", "x1", "q", "k", "v", "o", "s1", "z1", "h", "m", "s2", "dy", "ds2", "dz1", "dx1",
                                                        "ds1", "dattn", "dq", "dk", "dv"])}
BLOCK_PARAM_NAMES = ["wq", "bq", "wk", "bk", "wv", "bv", "wo", "bo", "w1", "b1", "w2", "b2", "g1", "be1", "g2", "be2"]


class Block:
    """One transformer block (attention + feed-forward, post-norm) with its training plan."""

    def __init__(self, session, dtype, batch, seq, dim, heads, ffn, causal=True, eps=1e-5, algo=L.OPT_ADAMW, world=1, fused_attention=False, shard_optimizer=False,
                 **optim_kw):
        self.lib, self.sess = load(), session
        cfg = BlockConfig()
        cfg.dtype, cfg.batch, cfg.seq, cfg.dim, cfg.heads, cfg.ffn, cfg.causal, cfg.eps, cfg.world = dtype, batch, seq, dim, heads, ffn, int(causal), eps, world
        cfg.fused_attention, cfg.shard_optimizer = int(fused_attention), int(shard_optimizer)
        o = cfg.optim
        o.algo = algo
        o.lr, o.weight_decay = optim_kw.get("lr", 1e-3), optim_kw.get("weight_decay", 0.0)
        o.momentum, o.beta1, o.beta2, o.eps = optim_kw.get("momentum", 0.0), optim_kw.get("beta1", 0.9), optim_kw.get("beta2", 0.999), optim_kw.get("eps", 1e-8)
        o.standard = int(optim_kw.get("standard", False))
        self.cfg, self.dtype = cfg, dtype
        self.shape_in = (batch, seq, dim)
        self.h = _P()
        st = self.lib.zyxb_block_create(session.backend.ctx, session.device.dev, C.byref(cfg), C.byref(self.h))
        if st != L.OK:
            raise BackendError(st, session.backend.lib.zyxb_last_error(session.backend.ctx).decode())
        bufs = [C.c_uint32() for _ in range(4)]
        self._check(self.lib.zyxb_block_io(self.h, *[C.byref(b) for b in bufs]))
        self.x, self.target, self.loss, self.y = (b.value for b in bufs)
        self.np_dtype = np.float32 if dtype == L.F32 else np.uint16
        E, F = dim, ffn
        self.shapes = [(E, E), (E,)] * 4 + [(F, E), (F,), (E, F), (E,)] + [(E,)] * 4

    def _check(self, st):
        if st != L.OK:
            raise BackendError(st, self.lib.zyxb_block_last_error(self.h).decode())

    def tensor(self, which, i):
        buf, n = C.c_uint32(), C.c_uint64()
        self._check(self.lib.zyxb_block_tensor(self.h, which, i, C.byref(buf), C.byref(n)))
        return buf.value, n.value

    def set_tensor(self, which, i, arr):
        buf, n = self.tensor(which, i)
        arr = np.ascontiguousarray(arr)
        assert arr.size == n and arr.dtype == self.np_dtype
        self.sess.pool.sync_events([self.sess.pool.host_to_pool(arr, buf)])

    def get_tensor(self, which, i):
        buf, _ = self.tensor(which, i)
        return self.sess.pool.download(buf, self.shapes[i], self.np_dtype)

    def set_batch(self, x, target):
        p = self.sess.pool
        return [p.host_to_pool(np.ascontiguousarray(x), self.x), p.host_to_pool(np.ascontiguousarray(target), self.target)]

    def activation(self, which, shape):
        """which: an index or a name of BLOCK_ACTIVATIONS."""
        buf = C.c_uint32()
        self._check(self.lib.zyxb_block_activation(self.h, BLOCK_ACTIVATIONS.get(which, which), C.byref(buf)))
        return self.sess.pool.download(buf.value, shape, self.np_dtype)

    def forward_backward(self):
        self._check(self.lib.zyxb_block_forward_backward(self.h))

    def update(self):
        self._check(self.lib.zyxb_block_update(self.h))

    def save(self, path):
        self._check(self.lib.zyxb_block_save(self.h, os.fsencode(path)))

    def load(self, path):
        missing = C.c_int32()
        self._check(self.lib.zyxb_block_load(self.h, os.fsencode(path), C.byref(missing)))
        return missing.value

    def step(self, events=None):
        events = [e for e in (events or []) if e.id != 0]
        arr = (L.Event * len(events))(*events) if events else None
        self._check(self.lib.zyxb_block_step(self.h, arr, len(events)))

    def read_loss(self):
        return float(self.sess.pool.download(self.loss, (1,), np.float32)[0])

    def read_output(self):
        return self.sess.pool.download(self.y, self.shape_in, self.np_dtype)

    def plan_size(self):
        a, b = C.c_int32(), C.c_int32()
        self._check(self.lib.zyxb_block_plan_size(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def close(self):
        if self.h:
            self.lib.zyxb_block_destroy(self.h)
            self.h = None
