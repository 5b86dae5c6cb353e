"""The sampled-row stage checker (oracle/sampled_checks.py) against plans faked from the oracle's own full runs (CPU): on
the oracle's own intermediates every stage error must be exactly zero, and a corrupted tensor must be reported."""
import numpy as np

from oracle import models as om
from oracle import oracle as zo
from oracle import sampled_checks as sc


class FakeMlp:
    def __init__(self, dtype, layers, x, t):
        self.keep = {}
        self.loss, self.grads, self.y = om.forward_backward(dtype, layers, x, t, om.ACT_GELU, om.LOSS_MSE, keep=self.keep)

    def activation(self, which, layer, rows=None):
        a = self.keep[["act", "pre", "dz"][which]][layer]
        return a.copy() if rows is None else np.ascontiguousarray(a[rows])

    def get_tensor(self, which, i):
        assert which == sc.GRAD
        return self.grads[i // 2][i % 2]

    def read_loss(self):
        return self.loss


class FakeBlock:
    def __init__(self, dtype, p, x, t, heads, causal):
        self.loss, self.g, self.y, self.mid = om.block_forward_backward(dtype, p, x, t, heads, causal)

    def activation(self, name, shape):
        return self.mid[name].reshape(shape).copy()

    def get_tensor(self, which, i):
        return self.g[om.BLOCK_PARAMS[i]]

    def read_output(self):
        return self.y

    def read_loss(self):
        return self.loss


def test_mlp_checker_is_exact_on_the_oracle_and_sees_corruption():
    dims, batch, dt = [32, 64, 48, 64, 32], 40, zo.BF16
    rng = zo.Rng(5)
    layers = om.init_linears(rng, dt, dims)
    x = zo.to_bits(rng.randn(batch * dims[0]).reshape(batch, dims[0]), dt)
    t = zo.to_bits(rng.randn(batch * dims[-1]).reshape(batch, dims[-1]), dt)
    fake = FakeMlp(dt, layers, x, t)
    errs = sc.mlp_stage_errors(fake, dt, layers, x, t)
    stage = {k: v for k, v in errs.items() if not k.endswith("float64")}
    assert len(stage) == 4 + 3 + 1 + 1 + 4 + 4 + 3 and max(stage.values()) == 0.0, stage
    assert errs["loss_vs_float64"] <= 1e-5
    fake.keep["dz"][2][:, 1] ^= np.uint16(0x0040)          # a wrong mantissa bit in one column of one stored gradient
    bad = sc.mlp_stage_errors(fake, dt, layers, x, t)
    assert bad["weight_gradient_layer2"] > 0 and bad["bias_gradient_layer2"] > 0 and bad["input_gradient_layer2"] > 0
    assert bad["forward_layer0"] == 0.0


def test_block_checker_is_exact_on_the_oracle_and_sees_corruption():
    dt, B, T, E, H, F = zo.BF16, 2, 24, 32, 4, 64
    rng = np.random.default_rng(1)
    p = om.block_init(rng, dt, E, F, std=0.2)
    x = zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dt)
    t = zo.to_bits(rng.standard_normal((B, T, E)).astype(np.float32), dt)
    for causal in (True, False):
        fake = FakeBlock(dt, p, x, t, H, causal)
        e, att = sc.block_stage_errors(fake, dt, p, x, t, H, causal)
        stage = {k: v for k, v in e.items() if not k.endswith("float64")}
        assert max(stage.values()) == 0.0, stage
        assert all(a["ok"] and a["gpu_vs_oracle"] == 0.0 for a in att.values()), att
        assert len(att) == 4 * 3 and len(stage) == 11 + 6 + 15
    fake.mid["h"][3, 5] ^= np.uint16(0x0100)
    e, _ = sc.block_stage_errors(fake, dt, p, x, t, H, False, rows=[0, 3, 5])
    assert e["h"] > 0 and e["q"] == 0.0
