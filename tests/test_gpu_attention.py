"""Parity of the fused attention kernel (tcgen05) with the oracle's composition of the reference's attention:
scores matmul -> masked softmax -> probabilities matmul, each stored in the tensor dtype."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import models as zm
from oracle import oracle as zo
from tests.parity import TOL_BF16, assert_parity, max_rel_err, record_fallback
from zyx_b200 import _lib as L
from zyx_b200 import backend as B

pytestmark = pytest.mark.gpu
RNG = np.random.default_rng(23)


def rand(shape, dtype, scale=1.0):
    return zo.to_bits((RNG.standard_normal(size=shape) * scale).astype(np.float32), dtype)


def check(o, want, exact, dtype):
    """An attention output is a weighted mean of value rows, so errors scale with the row's largest magnitude, not with
    the entry: tolerance 2e-2 relative to max(|want|, the row's largest |want|).  The reference composition truncates
    the scores and the probabilities to the 16-bit type, which moves its own result by 1e-2 .. 6e-2 on that scale away
    from the unrounded attention of the same inputs (probabilities that no longer sum to one); the fused kernel keeps
    both in f32.  So: within tolerance of the oracle, or within tolerance of the unrounded (float64) attention with the
    remaining gap to the oracle no larger than the tolerance plus the oracle's own distance from it."""
    got, ref = zo.to_f32(o, dtype).astype(np.float64), zo.to_f32(want, dtype).astype(np.float64)
    assert_parity(got, ref, exact, TOL_BF16, floor=1.0, what="attention")


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("batch,heads,seq", [(1, 1, 128), (2, 3, 256), (1, 2, 640)])
def test_fused_attention_matches_the_composed_reference(sess, dtype, causal, batch, heads, seq):
    D = 128
    q, k, v = (rand((batch, seq, heads * D), dtype) for _ in range(3))
    o, lse = sess.attention(dtype, q, k, v, heads, causal=causal)
    assert sess.device.status() == 0
    want, want_lse, exact = zm.attention(dtype, q, k, v, heads, causal)
    check(o, want, exact, dtype)
    assert np.max(np.abs(lse - want_lse)) <= 1e-3 * max(1.0, float(np.max(np.abs(want_lse))))


_CHILD = """
import sys, numpy as np
from zyx_b200 import ops
d = np.load(sys.argv[1])
s = ops.Session(device_ids=[0])
o, lse = s.attention(int(d['dtype']), d['q'], d['k'], d['v'], int(d['heads']), causal=bool(d['causal']))
assert s.device.status() == 0
out = dict(o=o, lse=lse)
if 'do' in d:
    dq, dk, dv = s.attention_bwd(int(d['dtype']), d['q'], d['k'], d['v'], o, d['do'], lse, int(d['heads']), causal=bool(d['causal']))
    assert s.device.status() == 0
    out.update(dq=dq, dk=dk, dv=dv)
np.savez(sys.argv[2], **out)
s.close()
"""


@pytest.mark.parametrize("causal", [True, False])
def test_two_tile_and_one_tile_forward_agree(sess, tmp_path, causal):
    """Lengths that are multiples of 256 take the kernel with two query tiles per CTA (P as a TMEM operand); a child
    process with ZYXB_ATTENTION_ONE_TILE set runs the same inputs through the one-tile kernel.  Both keep scores and sums
    in f32 and round P to the 16-bit type once, so outputs differ by at most one rounding step of the output type."""
    dtype, batch, heads, seq, D = L.BF16, 2, 2, 1024, 128
    q, k, v = (rand((batch, seq, heads * D), dtype) for _ in range(3))
    o2, lse2 = sess.attention(dtype, q, k, v, heads, causal=causal)
    assert sess.device.status() == 0
    want, want_lse, exact = zm.attention(dtype, q, k, v, heads, causal)
    check(o2, want, exact, dtype)
    src, dst = tmp_path / "in.npz", tmp_path / "out.npz"
    np.savez(src, q=q, k=k, v=v, dtype=dtype, heads=heads, causal=causal)
    env = dict(os.environ, ZYXB_ATTENTION_ONE_TILE="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run([sys.executable, "-c", _CHILD, str(src), str(dst)], check=True, env=env, cwd=root, timeout=600)
    one = np.load(dst)
    a, b = zo.to_f32(o2, dtype).astype(np.float64), zo.to_f32(one["o"], dtype).astype(np.float64)
    scale = np.maximum(np.abs(b), np.max(np.abs(b), axis=-1, keepdims=True))
    assert np.max(np.abs(a - b) / scale) <= 2.0 ** -7          # two bf16 roundings of nearly equal f32 values
    assert np.max(np.abs(lse2 - one["lse"])) <= 1e-4 * max(1.0, float(np.max(np.abs(want_lse))))


@pytest.mark.parametrize("causal", [True, False])
def test_persistent_forward_equals_one_cta_per_item(sess, tmp_path, causal):
    """More work items than SMs (320 of 256 query rows each): one CTA per SM walks several items, loading the next item's
    tiles and issuing its first products under the previous item's output stores, with every barrier phase counted across
    items.  The arithmetic per item does not change, so the result must equal, bit for bit, the same kernel launched with one
    CTA per item (ZYXB_ATTENTION_CTA_PER_ITEM in a child process) - the form the other tests hold against the oracle."""
    dtype, batch, heads, seq, D = L.BF16, 10, 16, 512, 128
    q, k, v = (rand((batch, seq, heads * D), dtype) for _ in range(3))
    o, lse = sess.attention(dtype, q, k, v, heads, causal=causal)
    do = rand((batch, seq, heads * D), dtype)
    dq, dk, dv = sess.attention_bwd(dtype, q, k, v, o, do, lse, heads, causal=causal)      # the dQ kernel walks 640 items the same way
    assert sess.device.status() == 0
    src, dst = tmp_path / "in.npz", tmp_path / "out.npz"
    np.savez(src, q=q, k=k, v=v, do=do, dtype=dtype, heads=heads, causal=causal)
    env = dict(os.environ, ZYXB_ATTENTION_CTA_PER_ITEM="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    subprocess.run([sys.executable, "-c", _CHILD, str(src), str(dst)], check=True, env=env, cwd=root, timeout=600)
    one = np.load(dst)
    assert np.array_equal(o, one["o"]) and np.array_equal(lse, one["lse"])
    assert np.array_equal(dq, one["dq"]) and np.array_equal(dk, one["dk"]) and np.array_equal(dv, one["dv"])
    # and one sampled head against the oracle
    b, h = 7, 11
    sl = slice(h * D, (h + 1) * D)
    want, want_lse, exact = zm.attention(dtype, q[b:b + 1, :, sl], k[b:b + 1, :, sl], v[b:b + 1, :, sl], 1, causal)
    check(np.ascontiguousarray(o[b:b + 1, :, sl]), want, exact, dtype)


def test_fused_attention_large_scores_and_custom_scale(sess):
    """Peaked softmax rows (scores of order 30) exercise the running-maximum rescale of the output tile."""
    dtype, batch, heads, seq, D = L.BF16, 1, 2, 512, 128
    q, k, v = rand((batch, seq, heads * D), dtype, 1.5), rand((batch, seq, heads * D), dtype, 1.5), rand((batch, seq, heads * D), dtype)
    o, _ = sess.attention(dtype, q, k, v, heads, scale=0.25, causal=True)
    want, _, exact = zm.attention(dtype, q, k, v, heads, True, scale=0.25)
    assert sess.device.status() == 0
    check(o, want, exact, dtype)


@pytest.mark.parametrize("dtype", [L.BF16, L.F16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("batch,heads,seq", [(1, 1, 128), (2, 2, 256), (1, 2, 640)])
def test_fused_attention_backward(sess, dtype, causal, batch, heads, seq):
    D = 128
    q, k, v, do = (rand((batch, seq, heads * D), dtype) for _ in range(4))
    o, lse = sess.attention(dtype, q, k, v, heads, causal=causal)
    dq, dk, dv = sess.attention_bwd(dtype, q, k, v, o, do, lse, heads, causal=causal)
    assert sess.device.status() == 0
    wq, wk, wv, exact = zm.attention_bwd(dtype, q, k, v, do, heads, causal)
    for name, got, want, ex in (("dq", dq, wq, exact[0]), ("dk", dk, wk, exact[1]), ("dv", dv, wv, exact[2])):
        g, w = zo.to_f32(got, dtype).astype(np.float64), zo.to_f32(want, dtype).astype(np.float64)
        # The adjoint is ill-conditioned in 16-bit storage on both sides: dS = P*(dP - delta) subtracts numbers of size
        # sqrt(head_dim) to get one of size 1, the reference from a dP stored in the 16-bit type, the fused kernel from a
        # delta computed from the stored o.  Both land a few percent (of the row scale) from the unrounded adjoint, and
        # the first rows of a causal dq are exactly zero mathematically (one key), so the scale is also bounded below by
        # 5 % of the tensor's largest magnitude.  Required: as close to the unrounded adjoint as the reference
        # composition is (within a quarter), and no farther from the reference than tolerance plus its own distance.
        kw = dict(floor=1.0, abs_floor=0.05 * float(np.abs(ex).max()))
        e_go, e_ge, e_oe = max_rel_err(g, w, **kw), max_rel_err(g, ex, **kw), max_rel_err(w, ex, **kw)
        if e_go > TOL_BF16:
            record_fallback("attention backward " + name, TOL_BF16, 1.0, e_go, e_ge, e_oe)
        assert e_go <= TOL_BF16 or (e_ge <= max(TOL_BF16, 1.25 * e_oe) and e_go <= TOL_BF16 + e_oe), (name, e_go, e_ge, e_oe)


def test_attention_descriptor_is_validated(sess):
    for kw in (dict(head_dim=64, seq=128), dict(head_dim=128, seq=100), dict(head_dim=128, seq=128, dtype=L.F32)):
        args = dict(dtype=L.BF16, batch=1, heads=1)
        args.update(kw)
        with pytest.raises(B.BackendError):
            sess.device.create_program(B.attention_desc(args["dtype"], args["batch"], args["heads"], args["seq"], args["head_dim"]))
