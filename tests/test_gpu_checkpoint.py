"""Checkpoints of the plans (parameters + optimizer state + step counter in a safetensors file) and the reference's
`matmul_disk` test (zyx/tests/05_misc.rs:638-660) with the matmul on the GPU."""
import os

import numpy as np
import pytest

from oracle import oracle as zo
from zyx_b200 import _lib as L
from zyx_b200 import host as H
from zyx_b200 import safetensors as st

pytestmark = pytest.mark.gpu
CROP = os.path.join(os.path.dirname(__file__), "golden", "xyz2_crop.safetensors")


def test_matmul_disk_on_the_gpu(sess):
    """x, y, z loaded from the reference's file (cropped): z == x.matmul(y) exactly.  The integers are small (entries
    below 10, sums below 2^31), so the exact i32 matmul serves the I64 tensors."""
    t = st.load(CROP)
    x, y = t["x"].astype(np.int32), t["y"].astype(np.int32)
    got = sess.gemm(L.I32, x, y)
    assert np.array_equal(got.astype(np.int64), t["z"])


def _mlp(sess):
    return H.Mlp(sess, L.BF16, 64, [96, 160, 48], activation=H.ACT_GELU, loss=H.LOSS_MSE, algo=L.OPT_ADAMW, lr=1e-3, weight_decay=0.01,
                 standard=True)


def test_mlp_checkpoint_resumes_bit_exactly(sess, tmp_path):
    rng = np.random.default_rng(11)
    batches = [(zo.to_bits(rng.standard_normal((64, 96)).astype(np.float32), zo.BF16),
                zo.to_bits(rng.standard_normal((64, 48)).astype(np.float32), zo.BF16)) for _ in range(4)]
    init = [zo.to_bits((0.1 * rng.standard_normal(s)).astype(np.float32), zo.BF16) for s in ((160, 96), (160,), (48, 160), (48,))]
    path = str(tmp_path / "mlp.safetensors")

    def run(mlp, which):
        for i in which:
            sess.pool.sync_events(mlp.set_batch(*batches[i]))
            mlp.step()
        return [mlp.get_tensor(w, i) for w in (H.PARAM, H.STATE0, H.STATE1) for i in range(4)]

    a = _mlp(sess)
    try:
        for i, w in enumerate(init):
            a.set_tensor(H.PARAM, i, w)
        run(a, [0, 1])
        a.save(path)
        want = run(a, [2, 3])
    finally:
        a.close()
    names = list(st.load(path))
    assert names[:4] == ["layers.0.weight", "layers.0.bias", "layers.1.weight", "layers.1.bias"]
    assert "optim.m.layers.1.weight" in names and "optim.v.layers.0.bias" in names and names[-1] == "optim.t"
    assert st.load(path)["optim.t"].tolist() == [2]
    b = _mlp(sess)
    try:
        assert b.load(path) == 0
        got = run(b, [2, 3])            # resumes at step 3: the bias corrections depend on the restored counter
    finally:
        b.close()
    for g, w in zip(got, want):
        assert np.array_equal(g, w)


def test_block_checkpoint_round_trip_and_partial_files(sess, tmp_path):
    kw = dict(lr=1e-3, weight_decay=0.01, standard=True)
    rng = np.random.default_rng(12)
    x = zo.to_bits(rng.standard_normal((1, 128, 256)).astype(np.float32), zo.BF16)
    path, part = str(tmp_path / "blk.safetensors"), str(tmp_path / "part.safetensors")
    a = H.Block(sess, L.BF16, 1, 128, 256, 2, 512, causal=True, algo=L.OPT_ADAMW, **kw)
    try:
        for i, shape in enumerate(a.shapes):
            a.set_tensor(H.PARAM, i, zo.to_bits((0.05 * rng.standard_normal(shape)).astype(np.float32), zo.BF16))
        sess.pool.sync_events(a.set_batch(x, x))
        a.step()
        a.save(path)
        want = [a.get_tensor(w, i) for w in (H.PARAM, H.STATE0, H.STATE1) for i in range(16)]
    finally:
        a.close()
    t = st.load(path, with_dtypes=True)
    assert list(t)[:2] == ["attn.q_proj.weight", "attn.q_proj.bias"] and t["mlp.weight"][0].shape == (512, 256) and t["mlp.weight"][1] == L.BF16
    b = H.Block(sess, L.BF16, 1, 128, 256, 2, 512, causal=True, algo=L.OPT_ADAMW, **kw)
    try:
        assert b.load(path) == 0
        got = [b.get_tensor(w, i) for w in (H.PARAM, H.STATE0, H.STATE1) for i in range(16)]
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
        # a file that holds only some parameters (as one written by another program might): the rest stay, and are counted
        st.save(part, {"norm1.weight": t["norm1.weight"], "mlp2.bias": t["mlp2.bias"]})
        assert b.load(part) == 3 * 16 - 2
        # a tensor of the wrong size is refused
        st.save(part, {"norm1.weight": (np.zeros(7, np.uint16), L.BF16)})
        with pytest.raises(Exception, match="another dtype or element count"):
            b.load(part)
    finally:
        b.close()
