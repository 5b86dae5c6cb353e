"""Host-array convenience layer: numpy in, numpy out, every call through the C ABI
(allocate -> host_to_pool -> launch -> pool_to_host -> deallocate), the call sequence
Runtime::materialize_kernel makes (zyx/src/runtime.rs:2075-2308).

bf16 / f16 tensors are carried as numpy uint16 bit patterns.
"""
import numpy as np

from . import _lib as L
from . import backend as B

NP_DTYPE = {L.BF16: np.uint16, L.F16: np.uint16, L.F32: np.float32, L.I32: np.int32}


class Session:
    """A device plus its pool; programs are cached per descriptor like the reference's kernel cache."""

    def __init__(self, backend=None, dev=0, **kw):
        self.backend = backend or B.Backend(**kw)
        self.device = self.backend.devices[dev]
        self.pool = self.backend.pools[dev]
        self.check_guards = bool(kw.get("debug", 0) & 2)

    def close(self):
        self.backend.deinitialize()

    def on_device(self, dev):
        """The same context's device `dev` (a context opened with several device ids drives them all)."""
        return Session(backend=self.backend, dev=dev)

    def run(self, desc, inputs, out_specs, out_init=None):
        """inputs: host arrays; out_specs: [(shape, np dtype)] -> list of host arrays.  out_init: host array the first
        output buffer holds before the launch (for kernels that leave part of their output untouched)."""
        prog = self.device.create_program(desc)
        in_bufs = [self.pool.upload(a) for a in inputs]
        out_bufs = [self.pool.allocate(max(int(np.prod(s)) * np.dtype(t).itemsize, 1))[0] for s, t in out_specs]
        try:
            if out_init is not None:
                self.pool.sync_events([self.pool.host_to_pool(np.ascontiguousarray(out_init), out_bufs[0])])
            self.device.launch(prog, in_bufs + out_bufs)
            if self.check_guards:          # a context opened with debug=2: no kernel may have written past the end of a buffer
                self.device.check_guards()
            return [self.pool.download(b, s, t) for b, (s, t) in zip(out_bufs, out_specs)]
        finally:
            for b in in_bufs + out_bufs:
                self.pool.deallocate(b)
            self.device.release(prog)

    # ---- row kernels ---------------------------------------------------------------------------
    def row_reduce(self, op, dtype, x, correction=1):
        rows, cols = x.shape
        return self.run(B.rowreduce_desc(op, dtype, rows, cols, correction=correction), [x], [((rows,), NP_DTYPE[dtype])])[0]

    def softmax(self, dtype, x, scale=0.0, causal=False, period=0, log=False):
        rows, cols = x.shape
        op = L.RR_LN_SOFTMAX if log else L.RR_SOFTMAX
        return self.run(B.rowreduce_desc(op, dtype, rows, cols, scale=scale, causal=causal, period=period), [x], [(x.shape, x.dtype)])[0]

    def layernorm(self, dtype, x, w=None, b=None, eps=1e-5):
        rows, cols = x.shape
        ins = [x] + ([w] if w is not None else []) + ([b] if b is not None else [])
        d = B.rowreduce_desc(L.RR_LAYERNORM, dtype, rows, cols, eps=eps, has_weight=w is not None, has_bias=b is not None)
        return self.run(d, ins, [(x.shape, x.dtype)])[0]

    def layernorm_bwd(self, dtype, x, dy, w=None, eps=1e-5):
        rows, cols = x.shape
        ins = [x, dy] + ([w] if w is not None else [])
        d = B.rowreduce_desc(L.RR_LAYERNORM_BWD, dtype, rows, cols, eps=eps, has_weight=w is not None)
        return self.run(d, ins, [(x.shape, x.dtype)])[0]

    def layernorm_dyxhat(self, dtype, x, dy, eps=1e-5):
        rows, cols = x.shape
        return self.run(B.rowreduce_desc(L.RR_LAYERNORM_DYXHAT, dtype, rows, cols, eps=eps), [x, dy], [(x.shape, x.dtype)])[0]

    def softmax_bwd(self, dtype, p, dp, causal=False, period=0):
        rows, cols = p.shape
        return self.run(B.rowreduce_desc(L.RR_SOFTMAX_BWD, dtype, rows, cols, causal=causal, period=period), [p, dp],
                        [(p.shape, p.dtype)])[0]

    def cross_entropy(self, logits, labels):
        rows, cols = logits.shape
        per, mean = self.run(B.rowreduce_desc(L.RR_CROSS_ENTROPY, L.F32, rows, cols), [logits, labels],
                             [((rows,), np.float32), ((1,), np.float32)])
        return per, mean

    def cross_entropy_bwd(self, logits, labels):
        rows, cols = logits.shape
        return self.run(B.rowreduce_desc(L.RR_CROSS_ENTROPY_BWD, L.F32, rows, cols), [logits, labels], [(logits.shape, np.float32)])[0]

    def colsum(self, dtype, x):
        rows, cols = x.shape
        return self.run(B.rowreduce_desc(L.RR_COLSUM, dtype, rows, cols), [x], [((cols,), x.dtype)])[0]

    def mse(self, dtype, y, t):
        rows, cols = y.shape
        return float(self.run(B.rowreduce_desc(L.RR_MSE, dtype, rows, cols), [y, t], [((1,), np.float32)])[0][0])

    # ---- elementwise ---------------------------------------------------------------------------
    def eltwise(self, op, dtype, a, b=None, p0=0.0, dtype_out=None, cols=0):
        od = NP_DTYPE[dtype_out] if (op == L.EW_CAST and dtype_out is not None) else a.dtype
        ins = [a] + ([b] if b is not None else [])
        return self.run(B.eltwise_desc(op, dtype, a.size, p0=p0, dtype_out=dtype_out, cols=cols), ins, [(a.shape, od)])[0]

    # ---- matmul --------------------------------------------------------------------------------
    def gemm(self, dtype, a, b, ta=False, tb=False, bias=None, epi=L.EPI_NONE, alpha=0.0, want_preact=False, tri=0, out_init=None):
        batch = a.shape[0] if a.ndim == 3 else 1
        m, k = (a.shape[-1], a.shape[-2]) if ta else (a.shape[-2], a.shape[-1])
        n = b.shape[-2] if tb else b.shape[-1]
        shape = (batch, m, n) if a.ndim == 3 else (m, n)
        d = B.gemm_desc(dtype, m, n, k, batch=batch, trans_a=ta, trans_b=tb, stride_b=(0 if b.ndim == 2 else k * n),
                        epilogue=epi, store_preact=want_preact, alpha=alpha, tri=tri)
        ins = [a, b] + ([bias] if bias is not None else [])      # bias [n], or z shaped like the result for MUL_*_GRAD
        outs = [(shape, a.dtype)] * (2 if want_preact else 1)
        r = self.run(d, ins, outs, out_init=out_init)
        return (r[0], r[1]) if want_preact else r[0]

    def attention(self, dtype, q, k, v, heads, scale=0.0, causal=False):
        """q, k, v: [batch, seq, heads*head_dim] -> (o like q, lse [batch*heads, seq] f32)."""
        batch, seq, e = q.shape
        d = B.attention_desc(dtype, batch, heads, seq, e // heads, scale=scale, causal=causal)
        o, lse = self.run(d, [q, k, v], [(q.shape, q.dtype), ((batch * heads, seq), np.float32)])
        return o, lse

    def attention_bwd(self, dtype, q, k, v, o, do, lse, heads, scale=0.0, causal=False):
        """-> (dq, dk, dv), each like q."""
        batch, seq, e = q.shape
        d = B.attention_desc(dtype, batch, heads, seq, e // heads, scale=scale, causal=causal, backward=True)
        return tuple(self.run(d, [q, k, v, o, do, np.ascontiguousarray(lse, np.float32)], [(q.shape, q.dtype)] * 3))

    def conv(self, dtype, x, w, bias=None, stride=1, dilation=1, padding=0, channels_last=False):
        """x [n,c,h,w], w [o,c,kh,kw], bias [o] -> y [n,o,oh,ow]  (Tensor::conv, groups = 1);
        channels_last: x [n,h,w,c] -> y [n,oh,ow,o]."""
        xs = (x.shape[0], x.shape[3], x.shape[1], x.shape[2]) if channels_last else x.shape
        assert xs[1] == w.shape[1], "conv: channel counts differ"
        d = B.conv_desc(dtype, xs, w.shape, stride, dilation, padding, has_bias=bias is not None, channels_last=channels_last)
        shape = B.conv_out_shape(xs, w.shape, stride, dilation, padding)
        if channels_last:
            shape = (shape[0], shape[2], shape[3], shape[1])
        return self.run(d, [x, w] + ([bias] if bias is not None else []), [(shape, x.dtype)])[0]

    def conv_weight_grad(self, dtype, x, dy, w_shape, stride=1, dilation=1, padding=0, channels_last=False):
        """dw of y = conv(x, w, ...): x [n,c,h,w], dy [n,o,oh,ow] -> dw [o,c,kh,kw] (channels_last: x [n,h,w,c], dy [n,oh,ow,o])."""
        xs = (x.shape[0], x.shape[3], x.shape[1], x.shape[2]) if channels_last else x.shape
        d = B.conv_desc(dtype, xs, w_shape, stride, dilation, padding, channels_last=channels_last)
        d.kind = L.KIND_CONV_WGRAD
        return self.run(d, [x, dy], [(tuple(w_shape), x.dtype)])[0]

    def conv_input_grad(self, dtype, dy, w, x_hw, stride=1, dilation=1, padding=0, channels_last=False):
        """dx of y = conv(x, w, stride, dilation, padding): dy [n,o,oh,ow], w [o,c,kh,kw] (the forward filter, unchanged)
        -> dx [n,c,h,w] (channels_last: dy [n,oh,ow,o] -> dx [n,h,w,c]).  The descriptor is the forward convolution's."""
        o, c, kh, kw = w.shape
        n = dy.shape[0]
        xs = (n, c, x_hw[0], x_hw[1])
        d = B.conv_desc(dtype, xs, w.shape, stride, dilation, padding, channels_last=channels_last)
        d.kind = L.KIND_CONV_DGRAD
        want = B.conv_out_shape(xs, w.shape, stride, dilation, padding)
        got = (n, dy.shape[3], dy.shape[1], dy.shape[2]) if channels_last else dy.shape
        assert tuple(got) == tuple(want), (got, want)
        out = (n, x_hw[0], x_hw[1], c) if channels_last else xs
        return self.run(d, [dy, w], [(out, dy.dtype)])[0]

    # ---- optimizers (in place on the host arrays, like the oracle's) ------------------------------
    def optim_step(self, desc_kw, dtype, algo, tensors, t=None):
        """tensors: list of groups [p, g (, m, v | , buf)] of host arrays per parameter; updated in place."""
        n = len(tensors)
        groups = len(tensors[0])
        numels = [int(tt[0].size) for tt in tensors]
        prog = self.device.create_program(B.optim_desc(algo, dtype, numels, **desc_kw))
        if t is not None:
            self.device.set_step(prog, t - 1)
        bufs = [[self.pool.upload(tt[g]) for tt in tensors] for g in range(groups)]
        try:
            self.device.launch(prog, [b for grp in bufs for b in grp])
            if self.check_guards:
                self.device.check_guards()
            for g in range(groups):
                if g == 1:
                    continue
                for i in range(n):
                    tensors[i][g][...] = self.pool.download(bufs[g][i], tensors[i][g].shape, tensors[i][g].dtype)
        finally:
            for grp in bufs:
                for b in grp:
                    self.pool.deallocate(b)
            self.device.release(prog)
