"""The oracle's transformer-block backward pass against central finite differences (CPU, f32): pins the adjoints the GPU
plan is compared with, since the reference's own autograd for reshape/expand/reduce is unimplemented at this snapshot."""
import numpy as np

from oracle import models as om
from oracle import oracle as zo


def test_block_gradients_match_finite_differences():
    rng = np.random.default_rng(0)
    B, T, E, H, F = 2, 8, 16, 4, 32
    p = om.block_init(rng, zo.F32, E, F, std=0.3)
    p["g1"] = (1 + 0.1 * rng.standard_normal(E)).astype(np.float32)
    p["be1"] = (0.1 * rng.standard_normal(E)).astype(np.float32)
    x = rng.standard_normal((B, T, E)).astype(np.float32)
    t = rng.standard_normal((B, T, E)).astype(np.float32)
    for causal in (True, False):
        _, g, _, _ = om.block_forward_backward(zo.F32, p, x, t, H, causal)
        for name, idx in [("wq", (1, 2)), ("bq", (3,)), ("wk", (3, 3)), ("wv", (0, 0)), ("wo", (2, 5)), ("bo", (2,)), ("w1", (3, 4)),
                          ("b1", (7,)), ("w2", (4, 9)), ("b2", (1,)), ("g1", (5,)), ("be1", (6,)), ("g2", (1,)), ("be2", (1,))]:
            eps = 1e-2
            pp = {k: v.copy() for k, v in p.items()}
            pp[name][idx] += eps
            lp = om.block_forward_backward(zo.F32, pp, x, t, H, causal)[0]
            pp[name][idx] -= 2 * eps
            lm = om.block_forward_backward(zo.F32, pp, x, t, H, causal)[0]
            fd = (lp - lm) / (2 * eps)
            assert abs(fd - g[name][idx]) <= 2e-3 * max(abs(fd), 1e-2), (causal, name, fd, float(g[name][idx]))
