"""Builds and loads the host-memory fake of libzyxb (tests/fake/zyxb_fake.cpp) together with a copy of libzyxb_host linked
against it, so that the real plan code (zyx_b200/csrc/host/*.cpp) runs on CPU ranks.  TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import glob
import os
import subprocess

import numpy as np

from zyx_b200 import _lib as L
from zyx_b200 import host as H

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "_build")
FAKE, HOST = os.path.join(OUT, "libzyxb_fake.so"), os.path.join(OUT, "libzyxb_host_fake.so")
COLLECTIVE_CB = C.CFUNCTYPE(C.c_int32, C.c_void_p, C.c_uint64, C.c_int32, C.c_int32)
ALLOC, LAUNCH, COLLECTIVE = range(3)


def build():
    os.makedirs(OUT, exist_ok=True)
    host_srcs = sorted(glob.glob(os.path.join(ROOT, "zyx_b200", "csrc", "host", "*.cpp")))
    deps = host_srcs + glob.glob(os.path.join(ROOT, "zyx_b200", "csrc", "host", "*.hpp")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    fake_src = os.path.join(HERE, "zyxb_fake.cpp")
    flags = ["-O1", "-std=c++17", "-fPIC", "-fvisibility=hidden"]
    if not os.path.exists(FAKE) or os.path.getmtime(FAKE) < max(os.path.getmtime(p) for p in [fake_src] + deps):
        subprocess.check_call(["g++", "-shared", "-o", FAKE] + flags + [fake_src])
    if not os.path.exists(HOST) or os.path.getmtime(HOST) < max(os.path.getmtime(p) for p in deps + [FAKE]):
        subprocess.check_call(["g++", "-shared", "-o", HOST] + flags + host_srcs + ["-L", OUT, "-lzyxb_fake", "-Wl,-rpath,$ORIGIN"])
    return FAKE, HOST


class Fake:
    """One fake context plus the plan library bound to it."""

    def __init__(self):
        build()
        # The real libzyxb may already be loaded in this process with global visibility (zyx_b200.host does that so that
        # libzyxb_host finds it).  RTLD_DEEPBIND makes the plan library built here look in its own dependency - the fake - first.
        self.lib = C.CDLL(FAKE)
        self.host = C.CDLL(HOST, mode=os.RTLD_NOW | os.RTLD_DEEPBIND)
        for name, (res, args) in L.SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args
        for name, (res, args) in H.HOST_SIGNATURES.items():
            if name.startswith("zyxb_mlp_"):
                fn = getattr(self.host, name)
                fn.restype, fn.argtypes = res, args
        self.lib.zyxb_fake_fail.argtypes = [C.c_int32, C.c_int64]
        self.lib.zyxb_fake_calls.restype, self.lib.zyxb_fake_calls.argtypes = C.c_uint64, [C.c_int32]
        self.lib.zyxb_fake_set_collective.argtypes = [COLLECTIVE_CB]
        self.ctx = C.c_void_p()
        assert self.lib.zyxb_init(None, C.byref(self.ctx)) == L.OK
        self._cb = None

    def set_collective(self, fn):
        """fn(np.ndarray float32 view of the range, op) -> 0 on success; op 0 allreduce, 1 reduce-scatter, 2 allgather."""
        def cb(ptr, count, dtype, op):
            try:
                arr = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_float)), shape=(count,))
                return int(fn(arr, op) or 0)
            except Exception:       # a peer that left or a timeout: the ABI reports it as a status, it never raises
                return 1
        self._cb = COLLECTIVE_CB(cb)
        self.lib.zyxb_fake_set_collective(self._cb)

    def fail(self, kind, after_n_calls):
        self.lib.zyxb_fake_fail(kind, after_n_calls)

    def calls(self, kind):
        return self.lib.zyxb_fake_calls(kind)

    def last_error(self):
        return self.lib.zyxb_last_error(self.ctx).decode()

    def upload(self, buf, arr):
        arr = np.ascontiguousarray(arr)
        assert self.lib.zyxb_h2d(self.ctx, 0, arr.ctypes.data_as(C.c_void_p), arr.nbytes, buf, 0, None, 0, None) == L.OK

    def download(self, buf, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        assert self.lib.zyxb_d2h(self.ctx, 0, buf, 0, out.ctypes.data_as(C.c_void_p), out.nbytes, None, 0) == L.OK
        return out


class FakeMlp:
    """zyxb_mlp_* of the plan library over the fake context (the subset of zyx_b200.host.Mlp the tests need)."""

    def __init__(self, fake, batch, dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, world=1, **kw):
        self.fake, self.dims, self.batch = fake, list(dims), batch
        cfg = H.MlpConfig()
        cfg.dtype, cfg.batch, cfg.n_layers, cfg.activation, cfg.loss = L.F32, batch, len(dims) - 1, activation, loss
        for i, d in enumerate(dims):
            cfg.dims[i] = d
        o = cfg.optim
        o.algo, o.lr, o.weight_decay = algo, kw.get("lr", 1e-3), kw.get("weight_decay", 0.0)
        o.beta1, o.beta2, o.eps, o.standard = 0.9, 0.999, 1e-8, int(kw.get("standard", True))
        cfg.world, cfg.bucket_per_layer = world, 1
        self.h = C.c_void_p()
        self.status = fake.host.zyxb_mlp_create(fake.ctx, 0, C.byref(cfg), C.byref(self.h))
        if self.status == L.OK:
            bufs = [C.c_uint32() for _ in range(4)]
            assert fake.host.zyxb_mlp_io(self.h, *[C.byref(b) for b in bufs]) == L.OK
            self.x, self.target, self.loss, self.y = (b.value for b in bufs)

    def tensor(self, which, i):
        buf, n = C.c_uint32(), C.c_uint64()
        assert self.fake.host.zyxb_mlp_tensor(self.h, which, i, C.byref(buf), C.byref(n)) == L.OK
        return buf.value

    def shape(self, i):
        return (self.dims[i // 2 + 1], self.dims[i // 2]) if i % 2 == 0 else (self.dims[i // 2 + 1],)

    def step(self):
        return self.fake.host.zyxb_mlp_step(self.h, None, 0)

    def error(self):
        return self.fake.host.zyxb_mlp_last_error(self.h).decode()

    def close(self):
        if self.h:
            self.fake.host.zyxb_mlp_destroy(self.h)
            self.h = None
