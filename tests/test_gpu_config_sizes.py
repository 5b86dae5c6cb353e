"""Parity at the stated size of the training configurations: config 4 (4 x Linear 4096 <-> 16384, GELU, bf16) at batch 8192 and
config 5 (transformer block d = 2048, 16 heads x 128, FFN 8192, seq 2048, causal, bf16) at one sample.  The scalar oracle
cannot run those steps whole, so every stage of the GPU plan is checked against the oracle on sampled rows, each stage fed
with the tensor the GPU itself stored (oracle/sampled_checks.py; the checker is held to exactly zero on the oracle's own
runs by tests/test_sampled_checks.py).  Tolerance: 2e-2 (bf16), relative to max(|want|, 0.1 x the row's largest |want|)."""
import numpy as np
import pytest

from oracle import models as om
from oracle import oracle as zo
from oracle import sampled_checks as sc
from tests.parity import TOL_BF16, record_fallback
from zyx_b200 import _lib as L
from zyx_b200 import host as H

pytestmark = pytest.mark.gpu


def test_config4_batch_8192_every_stage_against_the_oracle(sess, record_property):
    dims, batch, dt = [4096, 16384, 4096, 16384, 4096], 8192, L.BF16
    rng = np.random.default_rng(4)
    layers = []
    for i in range(4):
        bound = 1.0 / np.sqrt(dims[i])
        layers.append((zo.to_bits(rng.uniform(-bound, bound, (dims[i + 1], dims[i])).astype(np.float32), zo.BF16),
                       zo.to_bits(rng.uniform(-bound, bound, (dims[i + 1],)).astype(np.float32), zo.BF16)))
    x = zo.to_bits(rng.standard_normal((batch, dims[0]), dtype=np.float32), zo.BF16)
    t = zo.to_bits(rng.standard_normal((batch, dims[-1]), dtype=np.float32), zo.BF16)
    mlp = H.Mlp(sess, dt, batch, dims, activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, lr=1e-3, weight_decay=0.01)
    try:
        for i, (w, b) in enumerate(layers):
            mlp.set_tensor(H.PARAM, 2 * i, w)
            mlp.set_tensor(H.PARAM, 2 * i + 1, b)
        sess.pool.sync_events(mlp.set_batch(x, t))
        mlp.forward_backward()
        assert sess.device.status() == 0
        errs = sc.mlp_stage_errors(mlp, zo.BF16, layers, x, t)
    finally:
        mlp.close()
    for k, v in errs.items():
        record_property(k, v)
    bad = {k: v for k, v in errs.items() if not k.endswith("float64") and not (v <= TOL_BF16)}
    assert not bad, (bad, errs)
    assert errs["loss_vs_float64"] <= 1e-4, errs
    assert len(errs) == 22


@pytest.mark.parametrize("fused", [False, True])
def test_config5_seq_2048_every_stage_against_the_oracle(sess, record_property, fused):
    B, T, E, heads, F, dt = 1, 2048, 2048, 16, 8192, L.BF16
    rng = np.random.default_rng(5)
    p = om.block_init(rng, dt, E, F, std=0.02)
    x = zo.to_bits(rng.standard_normal((B, T, E), dtype=np.float32), dt)
    t = zo.to_bits(rng.standard_normal((B, T, E), dtype=np.float32), dt)
    blk = H.Block(sess, dt, B, T, E, heads, F, causal=True, algo=L.OPT_ADAMW, fused_attention=fused, lr=1e-3, weight_decay=0.01, standard=True)
    try:
        for i, name in enumerate(om.BLOCK_PARAMS):
            blk.set_tensor(H.PARAM, i, p[name])
        sess.pool.sync_events(blk.set_batch(x, t))
        blk.forward_backward()
        assert sess.device.status() == 0
        errs, att = sc.block_stage_errors(blk, dt, p, x, t, heads, True, head_samples=[(0, 0), (0, 7), (0, 15)])
    finally:
        blk.close()
    for k, v in errs.items():
        record_property(k, v)
    for k, v in att.items():
        record_property(k, "%.3g / %.3g / %.3g" % (v["gpu_vs_oracle"], v["gpu_vs_float64"], v["oracle_vs_float64"]))
        if v["gpu_vs_oracle"] > TOL_BF16:
            record_fallback("config 5 " + k, TOL_BF16, 1.0, v["gpu_vs_oracle"], v["gpu_vs_float64"], v["oracle_vs_float64"])
    bad = {k: v for k, v in errs.items() if not k.endswith("float64") and not (v <= TOL_BF16)}
    assert not bad, (bad, errs, att)
    assert errs["loss_vs_float64"] <= 1e-4, errs
    bad_att = {k: v for k, v in att.items() if not v["ok"]}
    assert not bad_att, (bad_att, att)
    assert len(errs) == 34 and len(att) == 12
