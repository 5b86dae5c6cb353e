"""Known answers of the reference's own tests that span more than one kernel, on the GPU path through the C ABI: the five
iterations of CausalSelfAttention (zyx-nn/src/causal_self_attention.rs:74-158), the matmul adjoints of grad_dot
(zyx/tests/11_autograd.rs:355-367) and the softmax of a [2048, 320] tensor against the scalar loop of
zyx/tests/07_realize.rs:264-301."""
import numpy as np
import pytest

from oracle import oracle as zo
from tests.parity import ref_is_equal
from tests.test_oracle_golden import causal_self_attention, f32, scalar_loop_softmax
from zyx_b200 import _lib as L

pytestmark = pytest.mark.gpu


def test_causal_self_attention_five_iterations_known_answer(sess, golden):
    g = golden["causal_self_attention_5_iterations_f32"]
    x = f32(g["x"])
    for _ in range(g["iterations"]):
        x = causal_self_attention(x, f32(g["c_attn_weight"]), f32(g["c_proj_weight"]), g["n_head"],
                                  lambda a, b, **kw: sess.gemm(L.F32, np.ascontiguousarray(a), np.ascontiguousarray(b), **kw),
                                  lambda s: sess.softmax(L.F32, s))
    assert ref_is_equal(x, f32(g["y"]))


def test_grad_dot_known_answer(sess, golden):
    g = golden["grad_dot_i32"]
    x, y = np.asarray(g["x"], np.int32).reshape(1, 3), np.asarray(g["y"], np.int32)
    dz = np.ones((1, 1), np.int32)
    assert sess.gemm(L.I32, dz, y, tb=True).ravel().tolist() == g["x_grad"]
    assert sess.gemm(L.I32, x, dz, ta=True).tolist() == g["y_grad"]


def test_softmax_against_the_scalar_loop(sess, golden):
    g = golden["softmax_scalar_loop_procedural"]
    x = zo.Rng().rand(g["rows"] * g["cols"]).reshape(g["rows"], g["cols"])
    assert ref_is_equal(sess.softmax(L.F32, x), scalar_loop_softmax(x))
