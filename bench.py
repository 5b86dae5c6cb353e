#!/usr/bin/env python
"""Benchmark of the zyx_b200 hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  Workloads (synthetic, seeded, shapes of the reference's configurations):
  mlp         4 x Linear 4096<->16384, GELU, bf16, batch 8192 per GPU, MSE, AdamW; data parallel   (samples/s)  [default]
  block       transformer block d=2048, 16 heads, FFN 8192, seq 2048, batch 8 over the GPUs, bf16, causal; fwd+bwd+AdamW   (samples/s)
  simplenet   README SimpleNet 784->128->10, f32, batch 64, CE, SGD; step replayed from a captured graph   (samples/s)
  rowreduce   row softmax + row layernorm on f32 [8192, 32768]         (fused-reduce GB/s)
  gemm_bf16   C = A.B, M=N=K=8192 bf16, f32 accumulate                  (GEMM TFLOP/s)
  gemm_f32    C = A.B, M=N=K=4096 f32                                   (GEMM TFLOP/s)
Under torchrun every rank drives its own GPU through its own libzyxb context.
`--impl reference` times the CPU oracle (the restatement of the reference's C backend; the
reference itself is Rust and cannot be built here) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---- clocks ----------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU every 200 ms (read-only)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.thread, self.gpu = [], None, None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---- workloads ---------------------------------------------------------------------------------------
class RowReduce:
    """Row softmax and row layernorm (gamma=1, beta=0, eps=1e-5, unbiased variance) on f32 [8192, 32768], N(0,1) seeded."""
    name = "rowreduce_softmax_layernorm_f32_8192x32768"
    metric, unit, dtype, bound = "fused-reduce GB/s (row softmax + row layernorm)", "GB/s", "f32", "hbm"
    rows, cols = 8192, 32768
    # ncu capture of the softmax launch at [2048, 32768] (268.44 MB in, 268.44 MB out): 268.50 MB read, 209.61 MB written
    # before the kernel ended - the last 58.8 MB of output were still dirty in the 126 MB L2.  That residue does not grow
    # with the rows, so a larger launch moves its algorithmic bytes plus the read overhead, minus the residue once.
    traffic_rows, traffic_read, traffic_written = 2048, 268.50e6, 209.61e6

    def __init__(self, rows=None):
        if rows:
            self.rows = rows
            self.name = "rowreduce_softmax_layernorm_f32_%dx%d" % (rows, self.cols)
        self.alg_bytes_softmax = self.rows * self.cols * 8                       # read once + write once
        self.alg_read_softmax = self.rows * self.cols * 4
        self.alg_bytes_layernorm = self.rows * self.cols * 8 + 2 * self.cols * 4
        self.units_per_step = (self.alg_bytes_softmax + self.alg_bytes_layernorm) / 1e9   # GB of algorithmic traffic
        self.h2d_bytes = self.rows * self.cols * 4
        self.d2h_bytes = 2 * self.rows * self.cols * 4

    def host_inputs(self, seed=1):
        rng = np.random.default_rng(seed)
        self.x = rng.standard_normal((self.rows, self.cols), dtype=np.float32)
        self.gamma, self.beta = np.ones(self.cols, np.float32), np.zeros(self.cols, np.float32)

    def setup(self, sess):
        from zyx_b200 import _lib as L, backend as B
        self.sess, self.L = sess, L
        self.host_inputs()
        p, d = sess.pool, sess.device
        self.bx, self.bg, self.bb = p.upload(self.x), p.upload(self.gamma), p.upload(self.beta)
        self.by1, _ = p.allocate(self.x.nbytes)
        self.by2, _ = p.allocate(self.x.nbytes)
        self.p_sm = d.create_program(B.rowreduce_desc(L.RR_SOFTMAX, L.F32, self.rows, self.cols))
        self.p_ln = d.create_program(B.rowreduce_desc(L.RR_LAYERNORM, L.F32, self.rows, self.cols, eps=1e-5, has_weight=True, has_bias=True))
        self.config = {"workload": self.name, "l2": "inputs (1 GiB) larger than L2 (126 MB)", "ops": "softmax, layernorm"}
        self.kernel_events = []

    def step(self, timed=False):
        d = self.sess.device
        if timed:
            e0 = d.event_record()
        d.launch(self.p_sm, [self.bx, self.by1])
        if timed:
            e1 = d.event_record()
        d.launch(self.p_ln, [self.bx, self.bg, self.bb, self.by2])
        if timed:
            e2 = d.event_record()
            self.kernel_events.append((e0, e1, e2))

    def roofline(self, peaks, clocks=None):
        d = self.sess.device
        sm = [d.elapsed_ms(a, b) for a, b, _ in self.kernel_events]
        ln = [d.elapsed_ms(b, c) for _, b, c in self.kernel_events]
        t_sm, t_ln = float(np.mean(sm)), float(np.mean(ln))
        ach = self.alg_bytes_softmax / (t_sm * 1e-3) / 1e9
        ach_ln = self.alg_bytes_layernorm / (t_ln * 1e-3) / 1e9
        # DRAM bytes of one softmax launch from the ncu capture of a smaller case of the same kernel: reads scale with the rows,
        # writes are the output bytes minus the constant part still dirty in L2 when the kernel ends
        rd, wr = self.alg_read_softmax, self.alg_bytes_softmax - self.alg_read_softmax
        k = self.traffic_rows / float(self.rows)
        traffic = rd * (self.traffic_read / (rd * k)) + wr - (wr * k - self.traffic_written) if self.rows >= self.traffic_rows else None
        return ({"bound": "hbm", "kernel": "row_staged_kernel<f32, softmax>", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                 "frac": ach / peaks["hbm_gbs"], "traffic": traffic,
                 "traffic_source": "ncu capture at %d rows: reads scaled by rows, writes = output bytes minus the L2-resident residue of that capture (a constant)" % self.traffic_rows,
                 "peak_source": peaks["source"], "ms_per_launch": t_sm},
                {"softmax": {"ms": t_sm, "GB/s": ach, "frac": ach / peaks["hbm_gbs"]},
                 "layernorm": {"ms": t_ln, "GB/s": ach_ln, "frac": ach_ln / peaks["hbm_gbs"]}})

    def e2e_setup(self):
        self.hy1, self.hy2 = np.empty_like(self.x), np.empty_like(self.x)
        for a in (self.x, self.hy1, self.hy2):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p, d = self.sess.pool, self.sess.device
        ev = p.host_to_pool(self.x, self.bx)
        d.launch(self.p_sm, [self.bx, self.by1], [ev])
        d.launch(self.p_ln, [self.bx, self.bg, self.bb, self.by2])
        p.pool_to_host(self.by1, self.hy1)
        p.pool_to_host(self.by2, self.hy2)

    def check(self):
        """One small invocation against the oracle (sampled rows)."""
        from oracle import oracle as zo
        pick = np.array([0, 1, self.rows // 2, self.rows - 1])
        y = np.empty((len(pick), self.cols), np.float32)
        for i, r in enumerate(pick):
            self.sess.pool.pool_to_host(self.by1, y[i], src_offset=int(r) * self.cols * 4)
        want = zo.softmax(zo.F32, self.x[pick])
        return float(np.max(np.abs(y - want) / np.maximum(np.abs(want), 1e-2 * want.max(1, keepdims=True))))

    def check_layernorm(self):
        from oracle import oracle as zo
        pick = np.array([0, 1, self.rows // 2, self.rows - 1])
        y = np.empty((len(pick), self.cols), np.float32)
        for i, r in enumerate(pick):
            self.sess.pool.pool_to_host(self.by2, y[i], src_offset=int(r) * self.cols * 4)
        want = zo.layernorm(zo.F32, self.x[pick], self.gamma, self.beta, 1e-5)
        return float(np.max(np.abs(y - want) / np.maximum(np.abs(want), 1e-2 * np.abs(want).max(1, keepdims=True))))

    def release(self):
        for b in (self.bx, self.bg, self.bb, self.by1, self.by2):
            self.sess.pool.deallocate(b)
        self.x = None

    # CPU leg: the oracle on a bounded sample of the same rows
    def cpu_run(self, rows):
        from oracle import oracle as zo
        x = self.x[:rows]
        t0 = time.perf_counter()
        zo.softmax(zo.F32, x)
        zo.layernorm(zo.F32, x, self.gamma, self.beta, 1e-5)
        dt = time.perf_counter() - t0
        return rows * self.cols * 16 / 1e9 / dt, dt

    def cpu_baseline(self, budget_s=12.0):
        self.host_inputs() if not hasattr(self, "x") else None
        v, dt = self.cpu_run(64)
        rows = int(min(self.rows, max(64, 64 * budget_s / max(dt, 1e-6))))
        v, dt = self.cpu_run(rows)
        return v, "%d of %d rows of [%d, %d] f32, softmax + layernorm, %.1f s" % (rows, self.rows, self.rows, self.cols, dt)


class Gemm:
    """C = A.B, row-major, A and B uniform(-1, 1) seeded; bf16 inputs are rounded the way bf16::from_f32 does (truncation)."""
    bound = "tensor"

    def __init__(self, dtype_name="bf16", n=None):
        from zyx_b200 import _lib as L
        self.dtype = dtype_name
        self.dt = {"bf16": L.BF16, "f32": L.F32}[dtype_name]
        self.n = n or (8192 if dtype_name == "bf16" else 4096)
        self.es = 2 if dtype_name == "bf16" else 4
        self.name = "gemm_%s_%d^3" % (dtype_name, self.n)
        self.metric, self.unit = "GEMM TFLOP/s (%s, M=N=K=%d, f32 accumulate)" % (dtype_name, self.n), "TFLOP/s"
        self.flops = 2.0 * self.n ** 3
        self.units_per_step = self.flops / 1e12
        self.h2d_bytes = 2 * self.n * self.n * self.es
        self.d2h_bytes = self.n * self.n * self.es

    def host_inputs(self):
        from oracle import oracle as zo
        rng = np.random.default_rng(2)
        a = rng.uniform(-1, 1, (self.n, self.n)).astype(np.float32)
        rng = np.random.default_rng(3)
        b = rng.uniform(-1, 1, (self.n, self.n)).astype(np.float32)
        if self.dtype == "bf16":
            a, b = zo.to_bits(a, zo.BF16), zo.to_bits(b, zo.BF16)
        self.a, self.b = a, b

    def setup(self, sess):
        from zyx_b200 import backend as B
        self.sess = sess
        self.host_inputs()
        p, d = sess.pool, sess.device
        self.ba, self.bb = p.upload(self.a), p.upload(self.b)
        self.bc, _ = p.allocate(self.a.nbytes)
        self.prog = d.create_program(B.gemm_desc(self.dt, self.n, self.n, self.n))
        self.config = {"workload": self.name, "l2": "L2 flushed between timed iterations (256 MB memset)", "layout": "NN row-major"}
        self.kernel_events = []

    def step(self, timed=False):
        d = self.sess.device
        d.flush_l2()
        if timed:
            e0 = d.event_record()
        d.launch(self.prog, [self.ba, self.bb, self.bc])
        if timed:
            self.kernel_events.append((e0, d.event_record()))

    def roofline(self, peaks, clocks=None):
        d = self.sess.device
        ms = [d.elapsed_ms(a, b) for a, b in self.kernel_events]
        t = float(np.mean(ms))
        ach = self.flops / (t * 1e-3) / 1e12
        extra = {}
        if self.dtype == "bf16":
            peak, kern, src = peaks["bf16_tflops"], "gemm_tc_kernel (tcgen05)", peaks["source"]
        else:
            # f32 at f32 accuracy on the tensor cores: three TF32 products per k-step.  TF32 runs at half the bf16 rate, so the
            # ceiling of the scheme is a sixth of the measured bf16 peak; the FP32 FMA roofline is given beside it.
            mhz = (clocks or {}).get("sm_mhz") or 1965.0
            fma = 148 * 128 * 2 * mhz * 1e6 / 1e12
            peak, kern = peaks["bf16_tflops"] / 6.0, "gemm_tf32x3_kernel (tcgen05, 3 x TF32; the launch also runs two operand-split kernels)"
            src = peaks["source"] + " bf16 matmul peak / 6 (TF32 at half rate, three products)"
            extra = {"fp32_fma_peak": fma, "frac_of_fp32_fma_peak": ach / fma,
                     "fp32_fma_peak_source": "computed: 148 SM x 128 FMA x 2 x %.0f MHz (median sampled SM clock)" % mhz}
        self.t_kernel_ms = t
        main = {"bound": "tensor", "kernel": kern, "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                "peak_source": src, "ms_per_launch": t, "ms_best": float(np.min(ms))}
        main.update(extra)
        return (main, {"gemm": {"ms": t, "TFLOP/s": ach}})

    def e2e_setup(self):
        self.hc = np.empty_like(self.a)
        for a in (self.a, self.b, self.hc):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p, d = self.sess.pool, self.sess.device
        e1, e2 = p.host_to_pool(self.a, self.ba), p.host_to_pool(self.b, self.bb)
        d.launch(self.prog, [self.ba, self.bb, self.bc], [e1, e2])
        p.pool_to_host(self.bc, self.hc)

    def check(self):
        from oracle import oracle as zo
        rows = np.array([0, 129, self.n // 2 + 1, self.n - 1])
        got = np.empty((len(rows), self.n), self.a.dtype)
        for i, r in enumerate(rows):
            self.sess.pool.pool_to_host(self.bc, got[i], src_offset=int(r) * self.n * self.es)
        af = zo.to_f32(self.a[rows], zo.BF16) if self.dtype == "bf16" else self.a[rows]
        bf = zo.to_f32(self.b, zo.BF16) if self.dtype == "bf16" else self.b
        want = af.astype(np.float64) @ bf.astype(np.float64)
        gf = zo.to_f32(got, zo.BF16) if self.dtype == "bf16" else got
        return float(np.max(np.abs(gf - want) / np.maximum(np.abs(want), 0.1 * np.abs(want).max(1, keepdims=True))))

    def release(self):
        for b in (self.ba, self.bb, self.bc):
            self.sess.pool.deallocate(b)
        self.a = self.b = None

    def cpu_run(self, n):
        from oracle import oracle as zo
        a, b = np.ascontiguousarray(self.a[:n, :n]), np.ascontiguousarray(self.b[:n, :n])
        t0 = time.perf_counter()
        zo.gemm(zo.BF16 if self.dtype == "bf16" else zo.F32, a, b)
        dt = time.perf_counter() - t0
        return 2.0 * n ** 3 / 1e12 / dt, dt

    def cpu_baseline(self, budget_s=12.0):
        if not hasattr(self, "a"):
            self.host_inputs()
        v, dt = self.cpu_run(512)
        n = int(min(self.n, max(512, 512 * (budget_s / max(dt, 1e-6)) ** (1.0 / 3.0)))) // 64 * 64
        v, dt = self.cpu_run(n)
        return v, "%d^3 corner of the %d^3 problem (%s), %.1f s" % (n, self.n, self.dtype, dt)


def f32_to_bf16_bits(x):
    """bf16 storage of an f32 array, truncating like the reference's bf16::from_f32."""
    return (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)


class AttnRows(RowReduce):
    """The two row kernels of the transformer block's attention on its score matrix: causal softmax over keys and the
    softmax backward, bf16 [batch*heads*T, T] with T = 2048 (rows restart their causal position every T rows)."""
    name = "attn_rows_causal_softmax_fwd_bwd_bf16_262144x2048"
    metric, unit, dtype, bound = "fused-reduce GB/s (causal softmax + softmax backward)", "GB/s", "bf16", "hbm"
    rows, cols = 8 * 16 * 2048, 2048
    traffic_rows, traffic_read, traffic_written = 65536, 138.48e6, 210.46e6      # causal softmax launch at [65536, 2048]

    def __init__(self, rows=None):
        if rows:
            self.rows = rows
            self.name = "attn_rows_causal_softmax_fwd_bwd_bf16_%dx%d" % (rows, self.cols)
        self.alg_bytes_softmax = self.rows * (self.cols + 1) + self.rows * self.cols * 2     # bf16: lower triangle read, all written
        self.alg_read_softmax = self.rows * (self.cols + 1)
        self.alg_bytes_layernorm = self.rows * (self.cols + 1) * 2 + self.rows * self.cols * 2  # backward: triangles of p and dp read
        self.units_per_step = (self.alg_bytes_softmax + self.alg_bytes_layernorm) / 1e9
        self.h2d_bytes = self.rows * self.cols * 2
        self.d2h_bytes = 2 * self.rows * self.cols * 2

    def host_inputs(self, seed=1):
        rng = np.random.default_rng(seed)
        self.x = f32_to_bf16_bits(rng.standard_normal((self.rows, self.cols), dtype=np.float32))

    def setup(self, sess):
        from zyx_b200 import _lib as L, backend as B
        self.sess, self.L = sess, L
        self.host_inputs()
        p, d = sess.pool, sess.device
        self.bx = p.upload(self.x)
        self.by1, _ = p.allocate(self.x.nbytes)
        self.by2, _ = p.allocate(self.x.nbytes)
        self.p_sm = d.create_program(B.rowreduce_desc(L.RR_SOFTMAX, L.BF16, self.rows, self.cols, causal=True, period=self.cols))
        self.p_bw = d.create_program(B.rowreduce_desc(L.RR_SOFTMAX_BWD, L.BF16, self.rows, self.cols, causal=True, period=self.cols))
        self.config = {"workload": self.name, "l2": "inputs (%d MiB) larger than L2 (126 MB)" % (self.x.nbytes >> 20),
                       "ops": "causal softmax, softmax backward (upstream gradient = the scores)"}
        self.kernel_events = []

    def step(self, timed=False):
        d = self.sess.device
        if timed:
            e0 = d.event_record()
        d.launch(self.p_sm, [self.bx, self.by1])
        if timed:
            e1 = d.event_record()
        d.launch(self.p_bw, [self.by1, self.bx, self.by2])
        if timed:
            e2 = d.event_record()
            self.kernel_events.append((e0, e1, e2))

    def roofline(self, peaks, clocks=None):
        main, both = RowReduce.roofline(self, peaks, clocks)
        main["kernel"] = "row kernel <bf16, causal softmax>"
        both["softmax_bwd"] = both.pop("layernorm")
        return main, both

    def e2e_setup(self):
        self.hy1, self.hy2 = np.empty_like(self.x), np.empty_like(self.x)
        for a in (self.x, self.hy1, self.hy2):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p, d = self.sess.pool, self.sess.device
        ev = p.host_to_pool(self.x, self.bx)
        d.launch(self.p_sm, [self.bx, self.by1], [ev])
        d.launch(self.p_bw, [self.by1, self.bx, self.by2])
        p.pool_to_host(self.by1, self.hy1)
        p.pool_to_host(self.by2, self.hy2)

    def check(self):
        from oracle import oracle as zo
        T = self.cols
        first = min(self.rows - T, (self.rows // T // 2) * T)                    # one whole causal period
        pick = first + np.array([0, 1, T // 2, T - 1])
        y = np.empty((len(pick), self.cols), np.uint16)
        g = np.empty((len(pick), self.cols), np.uint16)
        for i, r in enumerate(pick):
            self.sess.pool.pool_to_host(self.by1, y[i], src_offset=int(r) * self.cols * 2)
            self.sess.pool.pool_to_host(self.by2, g[i], src_offset=int(r) * self.cols * 2)
        want = zo.softmax(zo.BF16, self.x[first:first + T], causal=True, period=T)[pick - first]
        want_g = zo.softmax_bwd(zo.BF16, want, self.x[pick])
        f = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
        e1 = np.max(np.abs(f(y) - f(want)) / np.maximum(np.abs(f(want)), 1e-2 * f(want).max(1, keepdims=True)))
        e2 = np.max(np.abs(f(g) - f(want_g)) / np.maximum(np.maximum(np.abs(f(want_g)), 1e-2 * np.abs(f(want_g)).max(1, keepdims=True)), 1e-30))
        return float(max(e1, e2))

    def cpu_run(self, rows):
        from oracle import oracle as zo
        x = self.x[:rows]
        t0 = time.perf_counter()
        p = zo.softmax(zo.BF16, x, causal=True, period=self.cols)
        zo.softmax_bwd(zo.BF16, p, x)
        dt = time.perf_counter() - t0
        return rows * self.cols * 10 / 1e9 / dt, dt

    def cpu_baseline(self, budget_s=12.0):
        self.host_inputs() if not hasattr(self, "x") else None
        v, dt = self.cpu_run(2048)
        rows = int(min(self.rows, max(2048, 2048 * int(budget_s / max(dt, 1e-6)))))
        v, dt = self.cpu_run(rows)
        return v, "%d of %d rows of [%d, %d] bf16, causal softmax + backward, %.1f s" % (rows, self.rows, self.rows, self.cols, dt)


class AttentionFwd:
    """Fused causal self-attention forward at config 5's shape: q, k, v bf16 [8, 2048, 16*128], N(0,1) seeded."""
    metric, unit, dtype, bound = "fused attention forward TFLOP/s (causal, executed FLOPs)", "TFLOP/s", "bf16", "tensor"
    B, T, H, D = 8, 2048, 16, 128

    def __init__(self, size=0):
        if size:
            self.B = size
        self.name = "attention_fwd_causal_bf16_b%d_h%d_t%d_d%d" % (self.B, self.H, self.T, self.D)
        n_t = self.T // 128
        self.flops = 4.0 * 128 * 128 * self.D * (n_t * (n_t + 1) // 2) * self.B * self.H     # the tiles on and below the diagonal
        self.flops_dense = 4.0 * self.T * self.T * self.D * self.B * self.H
        self.units_per_step = self.flops / 1e12
        self.h2d_bytes = 3 * self.B * self.T * self.H * self.D * 2
        self.d2h_bytes = self.B * self.T * self.H * self.D * 2

    def host_inputs(self):
        rng = np.random.default_rng(5)
        shape = (self.B, self.T, self.H * self.D)
        self.q, self.k, self.v = (f32_to_bf16_bits(rng.standard_normal(shape, dtype=np.float32)) for _ in range(3))

    def setup(self, sess):
        from zyx_b200 import _lib as L, backend as B
        self.sess = sess
        self.host_inputs()
        p, d = sess.pool, sess.device
        self.bq, self.bk, self.bv = p.upload(self.q), p.upload(self.k), p.upload(self.v)
        self.bo, _ = p.allocate(self.q.nbytes)
        self.blse, _ = p.allocate(self.B * self.H * self.T * 4)
        self.prog = d.create_program(B.attention_desc(L.BF16, self.B, self.H, self.T, self.D, causal=True))
        self.prog_bwd = d.create_program(B.attention_desc(L.BF16, self.B, self.H, self.T, self.D, causal=True, backward=True))
        self.bdo = p.upload(self.q[::-1].copy())              # any N(0,1) tensor serves as the upstream gradient
        self.bdq, self.bdk, self.bdv = (p.allocate(self.q.nbytes)[0] for _ in range(3))
        self.bwd_events = []
        self.config = {"workload": self.name, "l2": "L2 flushed (256 MB memset) before every timed launch",
                       "flops": "executed: 128 x 128 tiles on and below the diagonal; dense equivalent %.0f GFLOP" % (self.flops_dense / 1e9)}
        self.kernel_events = []

    def step(self, timed=False):
        d = self.sess.device
        d.flush_l2()
        e0 = d.event_record() if timed else None
        d.launch(self.prog, [self.bq, self.bk, self.bv, self.bo, self.blse])
        if timed:
            self.kernel_events.append((e0, d.event_record()))
        d.flush_l2()
        e1 = d.event_record() if timed else None
        d.launch(self.prog_bwd, [self.bq, self.bk, self.bv, self.bo, self.bdo, self.blse, self.bdq, self.bdk, self.bdv])
        if timed:
            self.bwd_events.append((e1, d.event_record()))

    def roofline(self, peaks, clocks=None):
        d = self.sess.device
        ms = [d.elapsed_ms(a, b) for a, b in self.kernel_events]
        t = float(np.mean(ms))
        ach = self.flops / (t * 1e-3) / 1e12
        return ({"bound": "tensor", "kernel": "attn_fwd2_kernel (tcgen05; two query tiles per CTA, P as a TMEM operand)", "achieved": ach, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                 "frac": ach / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"], "ms_per_launch": t,
                 "tflops_dense_equivalent": self.flops_dense / (t * 1e-3) / 1e12},
                {"attention": {"ms": t, "TFLOP/s": ach},
                 "attention_backward": (lambda tb: {"ms": tb, "TFLOP/s": 3.5 * self.flops / (tb * 1e-3) / 1e12,
                                                    "note": "7 tensor-core products per tile pair (S and dP are computed by both backward kernels)"})(
                     float(np.mean([d.elapsed_ms(a, b) for a, b in self.bwd_events])))})

    def e2e_setup(self):
        self.ho = np.empty_like(self.q)
        for a in (self.q, self.k, self.v, self.ho):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p, d = self.sess.pool, self.sess.device
        evs = [p.host_to_pool(a, b) for a, b in ((self.q, self.bq), (self.k, self.bk), (self.v, self.bv))]
        d.launch(self.prog, [self.bq, self.bk, self.bv, self.bo, self.blse], evs)
        p.pool_to_host(self.bo, self.ho)

    def check(self):
        from oracle import models as zm, oracle as zo
        rows = 256                                            # the first 256 queries of one head of one batch: causal, so self-contained
        o = np.empty((rows, self.D), np.uint16)
        for r in range(rows):
            self.sess.pool.pool_to_host(self.bo, o[r], src_offset=(r * self.H * self.D) * 2)
        sl = lambda a: np.ascontiguousarray(a[:1, :rows, :self.D])
        want, _, _ = zm.attention(zo.BF16, sl(self.q), sl(self.k), sl(self.v), 1, True)
        f = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
        w = f(want.reshape(rows, self.D))
        return float(np.max(np.abs(f(o) - w) / np.maximum(np.abs(w), np.abs(w).max(1, keepdims=True))))

    def cpu_baseline(self, budget_s=12.0):
        from oracle import models as zm, oracle as zo
        self.host_inputs() if not hasattr(self, "q") else None
        heads = 2
        sl = lambda a: np.ascontiguousarray(a[:1, :, :heads * self.D])
        t0 = time.perf_counter()
        zm.attention(zo.BF16, sl(self.q), sl(self.k), sl(self.v), heads, True)
        dt = time.perf_counter() - t0
        n_t = self.T // 128
        fl = 4.0 * 128 * 128 * self.D * (n_t * (n_t + 1) // 2) * heads
        return fl / dt / 1e12, "%d of %d (batch, head) pairs, composed scores -> softmax -> P.V (plus a float64 check), %.1f s" % (heads, self.B * self.H, dt)


class Conv:
    """A ResNet-style 3x3 convolution layer, bf16: x [32, 256, 56, 56] N(0,1), w [256, 256, 3, 3] U(+-1/sqrt(c*9)) as
    Conv2d::new draws it (zyx-nn/src/conv2d.rs:38-47), bias, stride 1, padding 1; channels-first in and out."""
    metric, unit, dtype, bound = "convolution forward + input gradient + weight gradient TFLOP/s (implicit GEMM, 3x3, 256 -> 256 channels; L2 flushes inside the step)", "TFLOP/s", "bf16", "tensor"
    N, C, H, W, O, K = 32, 256, 56, 56, 256, 3

    def __init__(self, size=0, channels_last=False):
        if size:
            self.N = size
        self.channels_last = channels_last
        self.name = "conv3x3_bf16_n%d_c%d_%dx%d_o%d%s" % (self.N, self.C, self.H, self.W, self.O, "_channels_last" if channels_last else "")
        self.flops = 2.0 * self.N * self.H * self.W * self.O * self.C * self.K * self.K
        self.units_per_step = 3 * self.flops / 1e12            # forward and the two gradients: the same product count each
        self.h2d_bytes = self.N * self.C * self.H * self.W * 2
        self.d2h_bytes = self.N * self.O * self.H * self.W * 2

    def host_inputs(self):
        rng = np.random.default_rng(6)
        bound = 1.0 / np.sqrt(self.C * self.K * self.K)
        self.x = f32_to_bf16_bits(rng.standard_normal((self.N, self.C, self.H, self.W), dtype=np.float32))
        self.w = f32_to_bf16_bits(rng.uniform(-bound, bound, (self.O, self.C, self.K, self.K)).astype(np.float32))
        self.b = f32_to_bf16_bits(rng.uniform(-bound, bound, self.O).astype(np.float32))

    def setup(self, sess):
        from zyx_b200 import _lib as L, backend as B
        self.sess = sess
        self.host_inputs()
        p, d = sess.pool, sess.device
        self.xdev = np.ascontiguousarray(self.x.transpose(0, 2, 3, 1)) if self.channels_last else self.x
        self.bx, self.bw, self.bb = p.upload(self.xdev), p.upload(self.w), p.upload(self.b)
        self.by, _ = p.allocate(self.d2h_bytes)
        self.prog = d.create_program(B.conv_desc(L.BF16, self.x.shape, self.w.shape, 1, 1, 1, has_bias=True, channels_last=self.channels_last))
        # the two gradients of the same layer (timed beside the forward, reported under "kernels"): dy stands in as an
        # N(0,1) tensor of y's shape; the input gradient is the flipped-filter convolution of dy (3x3, padding 1: same shape)
        dgrad = B.conv_desc(L.BF16, (self.N, self.O, self.H, self.W), (self.C, self.O, self.K, self.K), 1, 1, 1, channels_last=self.channels_last, flip_filter=True)
        wgrad = B.conv_desc(L.BF16, self.x.shape, self.w.shape, 1, 1, 1, channels_last=self.channels_last)
        wgrad.kind = L.KIND_CONV_WGRAD
        self.prog_dgrad, self.prog_wgrad = d.create_program(dgrad), d.create_program(wgrad)
        rng = np.random.default_rng(7)
        self.bdy = p.upload(f32_to_bf16_bits(rng.standard_normal((self.N * self.O * self.H * self.W,), dtype=np.float32)))
        self.bdx, _ = p.allocate(self.h2d_bytes)
        self.bdw, _ = p.allocate(self.w.nbytes)
        self.grad_events = {"input_gradient": [], "weight_gradient": []}
        self.config = {"workload": self.name, "l2": "L2 flushed (256 MB memset) before every timed launch",
                       "launch": "two kernels: filters to [o, tap, c], implicit GEMM reading x in place" if self.channels_last else
                                 "three kernels: activations to channels-last, filters to [o, tap, c], implicit GEMM"}
        self.kernel_events = []

    def step(self, timed=False):
        d = self.sess.device
        d.flush_l2()
        e0 = d.event_record() if timed else None
        d.launch(self.prog, [self.bx, self.bw, self.bb, self.by])
        if timed:
            self.kernel_events.append((e0, d.event_record()))
        for name, prog, args in (("input_gradient", self.prog_dgrad, [self.bdy, self.bw, self.bdx]),
                                 ("weight_gradient", self.prog_wgrad, [self.bx, self.bdy, self.bdw])):
            d.flush_l2()
            e1 = d.event_record() if timed else None
            d.launch(prog, args)
            if timed:
                self.grad_events[name].append((e1, d.event_record()))

    def roofline(self, peaks, clocks=None):
        d = self.sess.device
        t = float(np.mean([d.elapsed_ms(a, b) for a, b in self.kernel_events]))
        ach = self.flops / (t * 1e-3) / 1e12
        grads = {}
        for name, evs in self.grad_events.items():
            tg = float(np.mean([d.elapsed_ms(a, b) for a, b in evs]))
            grads[name] = {"ms": tg, "TFLOP/s": self.flops / (tg * 1e-3) / 1e12}
        return ({"bound": "tensor", "kernel": "conv_tc_kernel (tcgen05) with its two layout kernels", "achieved": ach, "peak": peaks["bf16_tflops"],
                 "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"], "ms_per_launch": t},
                dict({"conv": {"ms": t, "TFLOP/s": ach}}, **grads))

    def e2e_setup(self):
        self.hy = np.empty((self.N, self.O, self.H, self.W), np.uint16)
        for a in (self.xdev, self.hy):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p, d = self.sess.pool, self.sess.device
        ev = p.host_to_pool(self.xdev, self.bx)
        d.launch(self.prog, [self.bx, self.bw, self.bb, self.by], [ev])
        p.pool_to_host(self.by, self.hy)

    def check(self):
        from oracle import oracle as zo
        y = np.empty((1, self.H, self.W, self.O) if self.channels_last else (1, self.O, self.H, self.W), np.uint16)   # the first image, every filter
        self.sess.pool.pool_to_host(self.by, y)
        if self.channels_last:
            y = y.transpose(0, 3, 1, 2)
        o = 8
        want = zo.conv(zo.BF16, self.x[:1], self.w[:o], self.b[:o], 1, 1, 1)
        f = lambda b: (b.astype(np.uint32) << 16).view(np.float32)
        g, w = f(y[:, :o]), f(want)
        return float(np.max(np.abs(g - w) / np.maximum(np.abs(w), 0.1 * np.abs(w).max())))

    def cpu_baseline(self, budget_s=12.0):
        from oracle import oracle as zo
        self.host_inputs() if not hasattr(self, "x") else None
        n, o = 1, 32
        dy = np.ascontiguousarray(self.x[:n, :o])                      # any tensor of y's shape [n, o, 56, 56] serves as dy
        flipped = np.ascontiguousarray(self.w[:o].transpose(1, 0, 2, 3)[:, :, ::-1, ::-1])
        t0 = time.perf_counter()
        zo.conv(zo.BF16, self.x[:n], self.w[:o], self.b[:o], 1, 1, 1)
        zo.conv(zo.BF16, dy, flipped, None, 1, 1, 1)                   # input gradient: dy with the transposed, reversed filter
        zo.conv_weight_grad(zo.BF16, self.x[:n], dy, (o, self.C, self.K, self.K), 1, 1, 1)
        dt = time.perf_counter() - t0
        fl = 3 * 2.0 * n * self.H * self.W * o * self.C * self.K * self.K
        return fl / dt / 1e12, "forward, input gradient and filter gradient of %d image(s) x %d of %d filters, %.1f s" % (n, o, self.O, dt)


class MlpTrain:
    """Config 4: 4 x Linear 4096 -> 16384 -> 4096 -> 16384 -> 4096, GELU between, bf16, batch 8192 per GPU, MSE against
    N(0,1) targets, AdamW lr 1e-3 wd 0.01; data parallel over the ranks with an NCCL gradient allreduce."""
    dims = [4096, 16384, 4096, 16384, 4096]
    batch = 8192
    unit, dtype, bound = "samples/s", "bf16", "tensor"

    def __init__(self, size=0, standard=False, rank=0, world=1, shard_optimizer=False):
        self.full_size = not size
        if size:
            self.batch = size
        self.standard, self.rank, self.world, self.shard = standard, rank, world, shard_optimizer
        self.name = "mlp_4xlinear_4096_16384_gelu_bf16_adamw_batch%d_per_gpu" % self.batch
        self.metric = "MLP train samples/s (4x Linear 4096<->16384, GELU, bf16, AdamW, batch %d per GPU)" % self.batch
        self.units_per_step = float(self.batch)
        self.h2d_bytes = self.batch * (self.dims[0] + self.dims[-1]) * 2
        self.d2h_bytes = 4
        n = len(self.dims) - 1
        # matmul FLOPs of one step: forward, weight gradient and (all but the first layer) input gradient
        self.gemm_flops = sum(2.0 * self.batch * self.dims[i] * self.dims[i + 1] * (3 if i > 0 else 2) for i in range(n))
        self.n_params = sum(self.dims[i] * self.dims[i + 1] + self.dims[i + 1] for i in range(n))

    def host_inputs(self):
        rng = np.random.default_rng(100 + self.rank)
        self.hx = f32_to_bf16_bits(rng.standard_normal((self.batch, self.dims[0]), dtype=np.float32))
        self.ht = f32_to_bf16_bits(rng.standard_normal((self.batch, self.dims[-1]), dtype=np.float32))

    def setup(self, sess):
        from zyx_b200 import _lib as L, host as H
        self.sess, self.H = sess, H
        self.host_inputs()
        self.mlp = H.Mlp(sess, L.BF16, self.batch, self.dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, world=self.world,
                         bucket_per_layer=True, shard_optimizer=self.shard, lr=1e-3, weight_decay=0.01, standard=self.standard)
        rng = np.random.default_rng(0)            # the same random-init weights on every rank (Linear::new's distribution)
        for i in range(self.mlp.n_params()):
            layer = i // 2
            bound = 1.0 / np.sqrt(self.dims[layer])
            self.mlp.set_tensor(H.PARAM, i, f32_to_bf16_bits(rng.uniform(-bound, bound, self.mlp.shape(i)).astype(np.float32)))
        sess.pool.sync_events(self.mlp.set_batch(self.hx, self.ht))
        # Pristine copies of the parameters.  Every step starts by copying them back (device to device, inside the
        # timed step): the reference's AdamW divides its update by lr, so after one step every weight is about
        # -+1/lr and from the second step on all values are NaN; timing GEMMs on NaNs draws less power and
        # flatters the clock.  With the reset every timed step is the configuration's step on finite N(0,1)-scale data.
        self.params = [self.mlp.tensor(H.PARAM, i) for i in range(self.mlp.n_params())]
        self.pristine = []
        for buf, numel in self.params:
            copy, _ = sess.pool.allocate(numel * 2)
            sess.pool.release_events([sess.pool.pool_to_pool(sess.pool, buf, copy, numel * 2)])
            self.pristine.append(copy)
        self.reset_bytes = sum(n for _, n in self.params) * 2
        launches, colls = self.mlp.plan_size()
        self.config = {"workload": self.name, "global_batch": self.batch * self.world, "parallelism": "dp%d" % self.world,
                       "optimizer": "AdamW lr=1e-3 wd=0.01, " + ("textbook update" if self.standard else
                                    "update as the reference writes it (step divided by lr)"),
                       "l2": "working set (params 0.5 GB, activations 2.7 GB) larger than L2", "launches_per_step": launches,
                       "collectives_per_step": colls, "optimizer_state": "sharded over the ranks (reduce-scatter, shard update, all-gather)" if self.shard else "replicated",
                       "param_reset": "parameters copied back from a pristine device copy at the start of every step "
                                      "(%d bytes d2d inside the timed step) so all values stay finite" % self.reset_bytes}
        self.x0, self.t0 = self.mlp.x, self.mlp.target
        self.mlp.profile(True)
        self.losses = []

    def reset_params(self):
        p = self.sess.pool
        if self.shard:
            self.mlp.tensor(self.H.PARAM, 0)      # blocks until the previous step's parameter all-gathers have landed: the reset must not race them
        for (buf, numel), copy in zip(self.params, self.pristine):
            p.release_events([p.pool_to_pool(p, copy, buf, numel * 2)])

    def step(self, timed=False):
        self.reset_params()
        self.mlp.step()

    def warm_reset(self):
        self.mlp.profile_read()    # drop what the warm-up steps recorded

    def roofline(self, peaks, clocks=None):
        ms, kind, steps = self.mlp.profile_read()
        gemm_ms = sum(m for m, k in zip(ms, kind) if k // 100 == 2) / max(steps, 1)
        groups = {}
        names = {2: "matmul", 1: "row", 3: "eltwise", 4: "optimizer"}
        for m, k in zip(ms, kind):
            key = "allreduce(+wait)" if k < 0 else names.get(k // 100, "?") + (":" + ["NN", "NT", "TN", "TT"][k % 100] if k // 100 == 2 else "")
            groups[key] = groups.get(key, 0.0) + m / max(steps, 1)
        ach = self.gemm_flops / (gemm_ms * 1e-3) / 1e12
        n_gemm = sum(1 for k in kind if k // 100 == 2)
        return ({"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05), %d launches per step" % n_gemm, "achieved": ach,
                 "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops_sustained"],
                 # dram__bytes_read + write of the step's eleven matmul launches (one-pass ncu capture at full size), mean per launch
                 "traffic": 1.2508e9 if self.full_size else None,
                 "peak_source": peaks["source"] + " (sustained: the kernel runs inside a long step)", "ms_per_launch": gemm_ms / n_gemm,
                 "flops_per_step": self.gemm_flops},
                {"ms_per_step_by_kind": {k: round(v, 4) for k, v in groups.items()},
                 "ms_per_instruction": [[int(k), round(m / max(steps, 1), 4)] for m, k in zip(ms, kind)]})

    def e2e_setup(self):
        """Two device input sets: the upload of the next batch (pinned host memory, copy stream) overlaps this step."""
        self.mlp.profile(False)
        p = self.sess.pool
        for a in (self.hx, self.ht):
            self.sess.backend.host_register(a)
        self.sets = [(self.mlp.x, self.mlp.target), (p.allocate(self.hx.nbytes)[0], p.allocate(self.ht.nbytes)[0])]
        self.cur = 0
        self.ready = [p.host_to_pool(self.hx, self.sets[0][0]), p.host_to_pool(self.ht, self.sets[0][1])]
        self.done = [None, None]      # event of the last step that read each set

    def e2e_step(self):
        p, cur, nxt = self.sess.pool, self.cur, 1 - self.cur
        # upload the next batch into the other set as soon as the step that last read it has finished
        dep = [self.done[nxt]] if self.done[nxt] is not None else []
        nx = p.host_to_pool(self.hx, self.sets[nxt][0], dep)
        nt = p.host_to_pool(self.ht, self.sets[nxt][1])          # no wait list: ordered after everything queued, hence after dep too
        self.mlp.bind_inputs(*self.sets[cur])
        self.reset_params()
        self.done[cur] = self.mlp.step(self.ready, want_event=True)
        self.losses.append(self.mlp.read_loss())                 # 4-byte device-to-host read; blocks until the step is done
        self.ready, self.cur = [nx, nt], nxt

    def check(self):
        """One forward + backward of the timed configuration (pristine parameters, this rank's batch), then every stage of it
        against the oracle on sampled rows, each stage fed with the tensor the GPU stored (oracle/sampled_checks.py).  With
        more than one rank the gradients hold sums over ranks, so only the forward stages are compared."""
        from oracle import oracle as zo, sampled_checks as sc
        self.mlp.profile(False)
        self.reset_params()
        self.mlp.bind_inputs(self.x0, self.t0)
        self.sess.pool.sync_events(self.mlp.set_batch(self.hx, self.ht))
        self.mlp.forward_backward()              # every rank: the plan's collectives need all of them
        if self.rank != 0 or self.shard:
            return None
        layers = [(self.mlp.get_tensor(self.H.PARAM, 2 * i), self.mlp.get_tensor(self.H.PARAM, 2 * i + 1)) for i in range(len(self.dims) - 1)]
        errs = sc.mlp_stage_errors(self.mlp, zo.BF16, layers, self.hx, self.ht, backward=self.world == 1)
        self.parity = {k: float("%.3g" % v) for k, v in errs.items()}
        self.parity["what"] = ("every stage of one step at batch %d against the CPU oracle on sampled rows, stage inputs = the GPU's stored tensors; "
                               "error relative to max(|want|, 0.1 x row max)" % self.batch)
        return float(max(v for k, v in errs.items() if not k.endswith("float64")))

    def cpu_baseline(self, budget_s=12.0):
        from oracle import models as om, oracle as zo
        if not hasattr(self, "cpu_layers"):
            rng = np.random.default_rng(0)
            self.cpu_layers = []
            for i in range(len(self.dims) - 1):
                b = 1.0 / np.sqrt(self.dims[i])
                self.cpu_layers.append((f32_to_bf16_bits(rng.uniform(-b, b, (self.dims[i + 1], self.dims[i])).astype(np.float32)),
                                        f32_to_bf16_bits(rng.uniform(-b, b, (self.dims[i + 1],)).astype(np.float32))))
        layers = [(w.copy(), b.copy()) for w, b in self.cpu_layers]       # the optimizer updates in place
        if not hasattr(self, "hx"):
            self.host_inputs()
        # batch of the measured sample: 8 on the first call, then what fits the time budget at the measured cost per sample
        bs = 8 if not hasattr(self, "cpu_s_per_sample") else int(min(32, max(4, budget_s / self.cpu_s_per_sample)))
        opt = om.Optim("adamw", zo.BF16, om.flat(layers), lr=1e-3, weight_decay=0.01, standard=self.standard)
        t0 = time.perf_counter()
        _, grads, _ = om.forward_backward(zo.BF16, layers, self.hx[:bs], self.ht[:bs], om.ACT_GELU, om.LOSS_MSE)
        t_fb = time.perf_counter() - t0
        self.cpu_s_per_sample = t_fb / bs
        t0 = time.perf_counter()
        opt.update(om.flat(layers), om.flat(grads))
        t_opt = time.perf_counter() - t0
        # Composed for the configuration's batch: forward + backward cost grows with the batch (every matmul of the step has the
        # batch as one of its extents), the AdamW pass over all parameters is paid once per step whatever the batch.
        step_s = t_fb / bs * self.batch + t_opt
        self.cpu_ms_per_step = step_s * 1e3
        return self.batch / step_s, ("composed: forward + MSE + backward measured at batch %d (%.2f s, %.4f s per sample) scaled to batch %d, plus one "
                                     "measured AdamW pass over all %d parameters (%.2f s); a whole step at batch %d would take %.0f s") % (
            bs, t_fb, t_fb / bs, self.batch, self.n_params, t_opt, self.batch, step_s)


class SimpleNet:
    """Config 1: README SimpleNet 784 -> 128 (ReLU) -> 10, f32, batch 64, cross-entropy, SGD lr 0.01 (the MNIST shapes of the
    reference's own benchmark; inputs N(0,1), labels uniform in [0,10)).  Launch-latency bound: the step is replayed from a
    captured graph (FrozenTape::replay's analogue); the eager figure is reported beside it."""
    dims, batch = [784, 128, 10], 64
    unit, dtype, bound = "samples/s", "f32", "launch"

    def __init__(self, size=0, rank=0, world=1):
        if size:
            self.batch = size
        self.rank, self.world = rank, world
        self.name = "simplenet_784_128_10_f32_batch%d_ce_sgd" % self.batch
        self.metric = "SimpleNet train samples/s (784->128->10, f32, batch %d, CE, SGD)" % self.batch
        self.units_per_step = float(self.batch)
        self.h2d_bytes, self.d2h_bytes = self.batch * 784 * 4 + self.batch * 4, 4

    def host_inputs(self):
        rng = np.random.default_rng(200 + self.rank)
        self.hx = rng.standard_normal((self.batch, 784), dtype=np.float32)
        self.ht = rng.integers(0, 10, size=self.batch).astype(np.int32)

    def setup(self, sess):
        from zyx_b200 import _lib as L, host as H
        self.sess, self.H = sess, H
        self.host_inputs()
        self.mlp = H.Mlp(sess, L.F32, self.batch, self.dims, activation=H.ACT_RELU, loss=H.LOSS_CROSS_ENTROPY, algo=L.OPT_SGD, lr=0.01)
        rng = np.random.default_rng(0)
        for i in range(self.mlp.n_params()):
            bound = 1.0 / np.sqrt(self.dims[i // 2])
            self.mlp.set_tensor(H.PARAM, i, rng.uniform(-bound, bound, self.mlp.shape(i)).astype(np.float32))
        sess.pool.sync_events(self.mlp.set_batch(self.hx, self.ht))
        d = sess.device
        d.sync()
        t0 = time.perf_counter()
        for _ in range(200):
            self.mlp.step()
        d.sync()
        self.eager_us = (time.perf_counter() - t0) / 200 * 1e6
        d.capture_begin()
        self.mlp.step()
        self.graph = d.capture_end()
        self.inner = 100       # replays per timed "step" so that a step is long enough for event timing
        self.units_per_step = float(self.batch * self.inner)
        self.config = {"workload": self.name, "l2": "working set (0.8 MB) is L2-resident by nature: the step is launch-latency bound",
                       "replay": "captured graph, %d replays per timed step" % self.inner, "launches_per_train_step": self.mlp.plan_size()[0]}
        self.losses = []

    def step(self, timed=False):
        for _ in range(self.inner):
            self.sess.device.graph_launch(self.graph)

    def roofline(self, peaks, clocks=None):
        return ({"bound": "launch-latency", "kernel": "14 kernels per training step (39 MFLOP)", "achieved": None, "peak": None, "unit": "us/step",
                 "frac": None, "traffic": None}, {"eager_us_per_train_step": self.eager_us})

    def e2e_setup(self):
        for a in (self.hx, self.ht):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        p = self.sess.pool
        for _ in range(self.inner):
            evs = self.mlp.set_batch(self.hx, self.ht)        # upload this step's batch, replay the step, read the loss
            self.sess.device.graph_launch(self.graph, evs)
            loss = self.mlp.read_loss()
        self.losses.append(loss)

    def check(self):
        return None

    def cpu_baseline(self, budget_s=12.0):
        from oracle import models as om, oracle as zo
        rng = np.random.default_rng(0)
        layers = [(rng.uniform(-1, 1, (self.dims[i + 1], self.dims[i])).astype(np.float32) / np.float32(np.sqrt(self.dims[i])),
                   rng.uniform(-1, 1, (self.dims[i + 1],)).astype(np.float32) / np.float32(np.sqrt(self.dims[i]))) for i in range(2)]
        if not hasattr(self, "hx"):
            self.host_inputs()
        opt = om.Optim("sgd", zo.F32, om.flat(layers), lr=0.01)
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < min(budget_s, 5.0):
            _, grads, _ = om.forward_backward(zo.F32, layers, self.hx, self.ht, om.ACT_RELU, om.LOSS_CE)
            opt.update(om.flat(layers), om.flat(grads))
            n += 1
        dt = time.perf_counter() - t0
        return n * self.batch / dt, "%d full training steps at batch %d, %.1f s" % (n, self.batch, dt)


class BlockTrain:
    """Config 5: one transformer block (MultiheadAttention + MLP, post-norm), d_model 2048, 16 heads x 128, FFN 8192, seq 2048,
    batch 8 split across the GPUs, bf16, causal, weights N(0, 0.02), inputs and targets N(0,1): forward + backward (+ AdamW)."""
    E, H, F, T, GLOBAL_B = 2048, 16, 8192, 2048, 8
    scaling = "strong"      # the global batch of 8 is divided over the ranks (one sample per GPU at 8 GPUs)
    unit, dtype, bound = "samples/s", "bf16", "tensor"

    def __init__(self, size=0, rank=0, world=1, fused=False, shard_optimizer=False):
        self.rank, self.world, self.fused, self.shard = rank, world, fused, shard_optimizer
        self.B = size if size else max(1, self.GLOBAL_B // world)
        self.name = "transformer_block_d2048_h16_ffn8192_seq2048_bf16_causal_batch%d_per_gpu" % self.B
        self.metric = "transformer block train samples/s (d=2048, 16x128 heads, FFN 8192, seq 2048, bf16, causal, fwd+bwd+AdamW)"
        self.units_per_step = float(self.B)
        R, E, F, T, H, D = self.B * self.T, self.E, self.F, self.T, self.H, self.E // self.H
        proj = 4 * 2.0 * R * E * E            # q, k, v, out
        attn = 2 * 2.0 * self.B * H * T * T * D
        ffn = 2 * 2.0 * R * E * F
        self.gemm_flops_dense = 3.0 * (proj + attn + ffn) - 3 * 2.0 * R * E * E      # no input gradient for the q/k/v projections
        # causal attention: the six score-shaped matmuls skip the tiles / k-blocks above the diagonal (128-row tiles, 256-wide
        # score tiles, 64-deep k-blocks at T = 2048): 72 of 128 output tiles, 17/32 of the k range
        n_t = T // 128
        out_frac = sum(min(T // 256, t // 2 + 1) for t in range(n_t)) / float(n_t * (T // 256)) if T % 256 == 0 else 1.0
        k_frac = sum((t + 1) * 2 for t in range(n_t)) / float(n_t * (T // 64)) if T % 128 == 0 else 1.0
        attn_exec = (attn / 2) * (2 * out_frac + 4 * k_frac)
        if self.fused:   # 128 x 128 tiles on and below the diagonal; 2 products forward, 7 backward (both backward kernels recompute S and dP)
            attn_exec = (attn / 2) * 9 * (n_t * (n_t + 1) / 2.0) / float(n_t * n_t) if T % 128 == 0 else 9 * attn / 2
        self.gemm_flops = self.gemm_flops_dense - 3.0 * attn + attn_exec             # FLOPs the kernels execute
        self.h2d_bytes, self.d2h_bytes = 2 * R * E * 2, 4

    def host_inputs(self):
        rng = np.random.default_rng(300 + self.rank)
        self.hx = f32_to_bf16_bits(rng.standard_normal((self.B, self.T, self.E), dtype=np.float32))
        self.ht = f32_to_bf16_bits(rng.standard_normal((self.B, self.T, self.E), dtype=np.float32))

    def setup(self, sess):
        from zyx_b200 import _lib as L, host as H
        self.sess, self.Hm = sess, H
        self.host_inputs()
        self.blk = H.Block(sess, L.BF16, self.B, self.T, self.E, self.H, self.F, causal=True, algo=L.OPT_ADAMW, world=self.world,
                           fused_attention=self.fused, shard_optimizer=self.shard, lr=1e-3, weight_decay=0.01, standard=True)
        self.init_params()
        sess.pool.sync_events(self.blk.set_batch(self.hx, self.ht))
        launches, colls = self.blk.plan_size()
        self.config = {"workload": self.name, "global_batch": self.B * self.world, "parallelism": "dp%d" % self.world,
                       "optimizer": "AdamW lr=1e-3 wd=0.01 (textbook update: the reference's literal form overflows after one step)",
                       "attention": ("fused (scores and probabilities stay on chip, recomputed in the backward)" if self.fused else
                                     "scores materialised ([B*H, T, T] bf16) as in the reference; causal mask as a select"),
                       "l2": "working set (activations %d MiB) larger than L2" % (30 * self.B * self.T * self.E * 2 >> 20),
                       "launches_per_step": launches, "collectives_per_step": colls,
                       "optimizer_state": "sharded over the ranks (reduce-scatter, shard update, all-gather)" if self.shard else "replicated"}
        self.losses = []
        self.step_events = []

    def init_params(self):
        """The configuration's parameters: weights N(0, 0.02), LayerNorm weight 1 and bias 0."""
        rng = np.random.default_rng(0)
        for i, shape in enumerate(self.blk.shapes):
            if i >= 12:
                w = np.ones(shape, np.float32) if i % 2 == 0 else np.zeros(shape, np.float32)
            else:
                w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
            self.blk.set_tensor(self.Hm.PARAM, i, f32_to_bf16_bits(w))

    def step(self, timed=False):
        self.blk.step()

    def roofline(self, peaks, clocks=None):
        # the whole step against the matmul FLOPs it contains (the step is one plan; per-kernel shares are in profiles/)
        t = self.ms_per_step_hint
        ach = self.gemm_flops / (t * 1e-3) / 1e12
        return ({"bound": "tensor", "kernel": "whole step (gemm_tc_kernel dominant; executed FLOPs: causal attention matmuls skip the masked tiles)", "achieved": ach, "peak": peaks["bf16_tflops_sustained"],
                 "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops_sustained"], "traffic": None, "peak_source": peaks["source"] + " (sustained)",
                 "ms_per_launch": t, "flops_per_step": self.gemm_flops, "flops_per_step_dense": self.gemm_flops_dense,
                 "tflops_dense_equivalent": self.gemm_flops_dense / (t * 1e-3) / 1e12}, {})

    def e2e_setup(self):
        for a in (self.hx, self.ht):
            self.sess.backend.host_register(a)

    def e2e_step(self):
        self.blk.step(self.blk.set_batch(self.hx, self.ht))
        self.losses.append(self.blk.read_loss())

    def check(self):
        """One forward + backward at the timed size with the configuration's parameters, every stage against the oracle on
        sampled rows and sampled (batch, head) pairs (oracle/sampled_checks.py).  More than one rank: forward stages only."""
        from oracle import models as om, oracle as zo, sampled_checks as sc
        # with the configuration's parameters again: a few dozen AdamW steps towards random targets drive the attention into a
        # regime where the query / key gradients are ill-conditioned in 16-bit arithmetic on both sides (the oracle's own
        # distance from the float64 value of the same formula grows from 0.025 to 0.3 - 0.6 after four steps)
        self.init_params()
        self.sess.pool.sync_events(self.blk.set_batch(self.hx, self.ht))
        self.blk.forward_backward()
        if self.rank != 0:
            return None
        p = {name: self.blk.get_tensor(self.Hm.PARAM, i) for i, name in enumerate(om.BLOCK_PARAMS)}
        errs, att = sc.block_stage_errors(self.blk, zo.BF16, p, self.hx, self.ht, self.H, True, backward=self.world == 1)
        self.parity = {k: float("%.3g" % v) for k, v in errs.items()}
        self.parity.update({k: {a: (float("%.3g" % b) if a != "ok" else b) for a, b in v.items()} for k, v in att.items()})
        self.parity["what"] = ("every stage of one step at the timed size, parameters re-drawn as the configuration states them, against the CPU "
                               "oracle on sampled rows (attention: sampled heads, whole sequence), stage inputs = the GPU's stored tensors; attention entries give gpu-vs-oracle / gpu-vs-float64 / oracle-vs-float64")
        return float(max([v for k, v in errs.items() if not k.endswith("float64")] + [v["gpu_vs_oracle"] for v in att.values() if not v["ok"]]))

    def cpu_baseline(self, budget_s=12.0):
        from oracle import models as om, oracle as zo
        E, F, H, T = 256, 1024, 2, 256        # one sample of a 1/8-width block: the full-size scalar step would take hours
        rng = np.random.default_rng(0)
        p = om.block_init(rng, zo.BF16, E, F, std=0.02)
        x = zo.to_bits(rng.standard_normal((1, T, E)).astype(np.float32), zo.BF16)
        t0 = time.perf_counter()
        om.block_forward_backward(zo.BF16, p, x, x, H, True)
        dt = time.perf_counter() - t0
        flops = 3.0 * (4 * 2.0 * T * E * E + 2 * 2.0 * H * T * T * (E // H) + 2 * 2.0 * T * E * F)
        full = self.gemm_flops / self.B
        return (flops / dt) / full, ("forward + backward of a reduced block (d=%d, ffn=%d, %d heads, seq %d, 1 sample: %.2f GFLOP in %.1f s); "
                                      "samples/s extrapolated to the full block by matmul FLOPs (%.1f GFLOP per sample)") % (E, F, H, T, flops / 1e9, dt, full / 1e9)


WORKLOADS = {"block": BlockTrain, "simplenet": SimpleNet, "mlp": MlpTrain, "rowreduce": RowReduce, "attn_rows": AttnRows, "attention": AttentionFwd, "conv": Conv, "conv_nhwc": lambda: Conv(channels_last=True), "gemm_bf16": lambda: Gemm("bf16"), "gemm_f32": lambda: Gemm("f32")}


def make_workload(args, rank=0, world=1):
    if args.workload == "mlp":
        return MlpTrain(size=args.size, standard=args.standard_adamw, rank=rank, world=world, shard_optimizer=args.shard_optimizer)
    if args.workload == "simplenet":
        return SimpleNet(size=args.size, rank=rank, world=world)
    if args.workload == "block":
        return BlockTrain(size=args.size, rank=rank, world=world, fused=not args.unfused_attention, shard_optimizer=args.shard_optimizer)
    if args.size:
        return {"rowreduce": lambda: RowReduce(rows=args.size), "attn_rows": lambda: AttnRows(rows=args.size), "attention": lambda: AttentionFwd(args.size), "conv": lambda: Conv(args.size), "conv_nhwc": lambda: Conv(args.size, True), "gemm_bf16": lambda: Gemm("bf16", args.size),
                "gemm_f32": lambda: Gemm("f32", args.size)}[args.workload]()
    return WORKLOADS[args.workload]()


def run_secondary(sess, peaks, gpu_index, launches=10, warmup=3):
    """The other two thirds of the metric in the same run: the bf16 8192^3 and f32 4096^3 matmuls and the two fused-reduce row
    kernels on f32 [8192, 32768], each `launches` launches timed one by one with CUDA events after `warmup` (L2 flushed before
    every matmul launch; the row inputs exceed L2), checked on sampled rows, with the clocks sampled meanwhile."""
    out = {}
    for key, make in (("gemm_bf16", lambda: Gemm("bf16")), ("gemm_f32", lambda: Gemm("f32")), ("rowreduce", RowReduce)):
        w = make()
        w.setup(sess)
        dev = sess.device
        for _ in range(warmup):
            w.step()
        dev.sync()
        sampler = ClockSampler(gpu_index)
        sampler.start()
        time.sleep(0.3)                    # let the sampler take its first reading before the short timed burst
        n0 = dev.launch_count()
        e0 = dev.event_record()
        for _ in range(launches):
            w.step(timed=True)
        e1 = dev.event_record()
        dev.sync()
        n_launch = dev.launch_count() - n0
        clocks = sampler.stop()
        main, kern = w.roofline(peaks, clocks)
        err = w.check()
        if key == "rowreduce":
            for name in ("softmax", "layernorm"):
                k = kern[name]
                out[name] = {"metric": "fused-reduce GB/s (row %s, f32 [8192, 32768])" % name, "value": k["GB/s"], "unit": "GB/s",
                             "roofline": {"bound": "hbm", "achieved": k["GB/s"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": k["frac"],
                                          "traffic": main["traffic"] if name == "softmax" else None, "ms_per_launch": k["ms"],
                                          "peak_source": peaks["source"]},
                             "max_rel_err_sampled": err if name == "softmax" else w.check_layernorm(), "launches": launches, "clocks": clocks,
                             "config": w.config}
        else:
            out[key] = {"metric": w.metric, "value": main["achieved"], "unit": w.unit, "roofline": main, "max_rel_err_sampled": err,
                        "launches": launches, "gpu_launches": int(n_launch), "ms_total_incl_l2_flush": dev.elapsed_ms(e0, e1), "clocks": clocks,
                        "config": w.config}
        w.release()
    return out


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, rank, world):
    """The reference arm: the CPU oracle (port of the reference C backend) on all host threads."""
    if rank != 0:
        return None
    os.environ["OMP_NUM_THREADS"] = str(host_threads())     # torchrun sets it to 1
    w = make_workload(args)
    if hasattr(w, "host_inputs"):
        w.host_inputs()
    vals = []
    sample = ""
    budget = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    for i in range(args.warmup + args.steps):
        v, sample = w.cpu_baseline(budget_s=budget)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals))
    ms = 1e3 * w.units_per_step / value      # time the CPU would need for one step of the configuration (composed or extrapolated from the sample)
    line = {"impl": "reference", "metric": w.metric, "value": value, "unit": w.unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": w.dtype, "data": "synthetic", "config": {"workload": w.name},
            "ms_per_step_note": "derived from the bounded sample (see cpu_baseline.sample), not a wall-clock step of this run",
            "cpu_baseline": {"value": value, "unit": w.unit, "cores": host_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": w.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    return json.dumps(line)


def main():
    # stdout carries exactly one JSON line: anything a library prints there (NCCL's version banner) goes to stderr
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        line = run()
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
    if line is not None:
        print(line, flush=True)


def run():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="mlp", choices=sorted(WORKLOADS))
    ap.add_argument("--unfused-attention", action="store_true",
                    help="block: materialise scores and probabilities as the reference does instead of the fused attention programs")
    ap.add_argument("--standard-adamw", action="store_true", help="mlp: textbook AdamW instead of the reference's literal update")
    ap.add_argument("--impl", default="zyx_b200", choices=["zyx_b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end leg; 0 = max(steps, 20)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the GEMM and fused-reduce legs the default 1-GPU run appends")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-check", action="store_true", help="skip the sampled parity check against the oracle (quick comparisons)")
    ap.add_argument("--shard-optimizer", action="store_true", help="mlp and block workloads: ZeRO stage 1 (reduce-scatter, sharded AdamW, all-gather) instead of allreduce + replicated AdamW")
    ap.add_argument("--size", type=int, default=0, help="reduced problem size for profiler captures: rows (rowreduce) or N (gemm)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.e2e_steps <= 0:
        args.e2e_steps = max(args.steps, 20)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    out_line = None

    import torch
    import torch.distributed as dist
    if world > 1:
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    from zyx_b200 import build
    from zyx_b200.ops import Session
    if rank == 0 or not os.path.exists(os.path.join(ROOT, "zyx_b200", "libzyxb.so")):
        build.build()
    if world > 1:
        dist.barrier()
    sess = Session(device_ids=[local_rank])
    dev = sess.device
    peaks = load_peaks()
    w = make_workload(args, rank, world)
    if world > 1:
        # one NCCL communicator for the library: rank 0 creates the id, torch.distributed carries it
        uid = torch.zeros(128, dtype=torch.uint8, device="cuda")
        if rank == 0:
            uid = torch.tensor(list(dev.comm_unique_id()), dtype=torch.uint8, device="cuda")
        dist.broadcast(uid, 0)
        dev.comm_init(rank, world, bytes(uid.cpu().tolist()))
    w.setup(sess)

    def barrier():
        if world > 1:
            dist.barrier()
        dev.sync()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        w.step()
    barrier()
    if hasattr(w, "warm_reset"):
        w.warm_reset()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = dev.launch_count()
    barrier()
    e_start = dev.event_record()
    for _ in range(args.steps):
        w.step(timed=True)
    e_stop = dev.event_record()
    barrier()
    ms_total = dev.elapsed_ms(e_start, e_stop)
    launches = dev.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * w.units_per_step / (ms_step * 1e-3)
    w.ms_per_step_hint = ms_step
    roofline, kernels = w.roofline(peaks, clocks)

    # end to end through the public API: host buffers in, host buffers out, copies inside the timed region.  It follows the
    # device-timed region directly (the checker and the CPU legs come later), so both see the GPU in the same power state.
    e2e = None
    if not args.no_e2e:
        w.e2e_setup()
        for _ in range(2):
            w.e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            w.e2e_step()
        dev.sync()
        e2e_s = (time.perf_counter() - t0) / args.e2e_steps
        if world > 1:
            t = torch.tensor([e2e_s], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_s = float(t.item())
        e2e = {"value": world * w.units_per_step / e2e_s, "unit": w.unit, "h2d_bytes_per_step": w.h2d_bytes, "d2h_bytes_per_step": w.d2h_bytes,
               "steps": args.e2e_steps, "ms_per_step": e2e_s * 1e3}
    err = None if args.no_check else w.check()
    secondary = None
    if world == 1 and args.workload == "mlp" and not args.size and not args.no_secondary:
        secondary = run_secondary(sess, peaks, local_rank)

    if rank == 0:
        line = {"metric": w.metric, "value": value, "unit": w.unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": getattr(w, "scaling", "weak"), "vs_baseline": None, "dtype": w.dtype,
                "data": "synthetic", "config": w.config, "roofline": roofline, "kernels": kernels, "e2e": e2e,
                "gpu_launches": int(launches), "clocks": clocks, "max_rel_err_sampled": err}
        if getattr(w, "parity", None):
            line["parity"] = w.parity
        if secondary:
            line["secondary"] = secondary
        if getattr(w, "losses", None):
            line["loss_e2e_steps"] = w.losses[:8]
        if world == 1 and not args.no_cpu_baseline:
            os.environ.setdefault("OMP_NUM_THREADS", str(host_threads()))
            v, sample = w.cpu_baseline()
            line["cpu_baseline"] = {"value": v, "unit": w.unit, "cores": host_threads(), "kind": "port", "sample": sample}
        out_line = json.dumps(line)
    sess.close()
    if world > 1:
        dist.destroy_process_group()
    return out_line


if __name__ == "__main__":
    main()
