"""ctypes binding of the e-graph matcher in libzyxb_host.so (include/zyxb_host.h, "e-graph matcher"): a mirror of zyx's graph
(zyx/src/graph/mod.rs:100-182) is built node by node and `match` plays the device's match_graph over it
(zyx/src/backend/mod.rs:952-961), returning kernel descriptors with their launch arguments."""
import ctypes as C

from . import _lib as L
from . import host as H

# zyx's enum orders (zyx/src/kernel/ops.rs:187-214, 222-262)
(U_NEG, U_BITNOT, U_EXP, U_EXP2, U_LN, U_LOG2, U_RECIPROCAL, U_SQRT, U_SIN, U_COS, U_FLOOR, U_TRUNC, U_ABS) = range(13)
(B_ADD, B_SUB, B_MUL, B_DIV, B_POW, B_MOD, B_CMPLT, B_CMPGT, B_CMPGE, B_MAX, B_OR, B_AND, B_BITXOR, B_BITOR, B_BITAND, B_SHL, B_SHR,
 B_NOTEQ, B_EQ) = range(19)
NONE = 0xFFFFFFFF


class Match(C.Structure):
    _fields_ = [("pattern", C.c_char * 32), ("n_inputs", C.c_int32), ("n_outputs", C.c_int32), ("inputs", C.c_uint32 * 128),
                ("outputs", C.c_uint32 * 96), ("desc", L.KernelDesc), ("optim_step", C.c_uint64), ("input_offsets", C.c_uint64 * 128)]


_P = C.c_void_p
_U64_P = C.POINTER(C.c_uint64)
_I32_P = C.POINTER(C.c_int32)
MATCHER_SIGNATURES = {
    "zyxb_mgraph_create": (C.c_int32, [C.POINTER(_P)]),
    "zyxb_mgraph_destroy": (C.c_int32, [_P]),
    "zyxb_mgraph_const": (C.c_uint32, [_P, C.c_int32, C.c_double]),
    "zyxb_mgraph_leaf": (C.c_uint32, [_P, C.c_int32, C.c_uint32, _U64_P, C.c_int32]),
    "zyxb_mgraph_expand": (C.c_uint32, [_P, C.c_uint32, _U64_P, C.c_int32]),
    "zyxb_mgraph_reshape": (C.c_uint32, [_P, C.c_uint32, _U64_P, C.c_int32]),
    "zyxb_mgraph_permute": (C.c_uint32, [_P, C.c_uint32, _I32_P, C.c_int32]),
    "zyxb_mgraph_reduce": (C.c_uint32, [_P, C.c_uint32, C.c_int32, _I32_P, C.c_int32]),
    "zyxb_mgraph_pad": (C.c_uint32, [_P, C.c_uint32, C.c_int32, C.c_int64, C.c_uint64]),
    "zyxb_mgraph_cast": (C.c_uint32, [_P, C.c_uint32, C.c_int32]),
    "zyxb_mgraph_unary": (C.c_uint32, [_P, C.c_uint32, C.c_int32]),
    "zyxb_mgraph_binary": (C.c_uint32, [_P, C.c_uint32, C.c_uint32, C.c_int32]),
    "zyxb_mgraph_class_info": (C.c_int32, [_P, C.c_uint32, _I32_P, _I32_P, _U64_P, _I32_P]),
    "zyxb_mgraph_const_value": (C.c_int32, [_P, C.c_uint32, C.POINTER(C.c_double), C.c_uint64, _U64_P]),
    "zyxb_mgraph_uncovered": (C.c_int32, [_P, C.POINTER(C.c_uint32), C.c_int32, C.POINTER(C.c_uint32), C.c_int32, _I32_P]),
    "zyxb_mgraph_match": (C.c_int32, [_P, C.POINTER(C.c_uint32), C.c_int32, C.POINTER(Match), C.c_int32, _I32_P]),
}
H.HOST_SIGNATURES.update(MATCHER_SIGNATURES)


class MGraph:
    """A mirror of one zyx graph.  Node constructors return class ids; `match(outputs)` returns the recognised subgraphs."""

    def __init__(self):
        self.lib = H.load()
        self.h = _P()
        assert self.lib.zyxb_mgraph_create(C.byref(self.h)) == L.OK
        self.n_leaves = 0

    def close(self):
        if self.h:
            self.lib.zyxb_mgraph_destroy(self.h)
            self.h = None

    def _ok(self, c, what):
        if c == NONE:
            raise ValueError("bad %s node" % what)
        return c

    @staticmethod
    def _dims(shape):
        return (C.c_uint64 * max(len(shape), 1))(*shape), len(shape)

    def const(self, dtype, value):
        return self._ok(self.lib.zyxb_mgraph_const(self.h, dtype, float(value)), "const")

    def leaf(self, dtype, shape):
        arr, n = self._dims(shape)
        self.n_leaves += 1
        return self._ok(self.lib.zyxb_mgraph_leaf(self.h, dtype, self.n_leaves, arr, n), "leaf")

    def expand(self, x, shape):
        arr, n = self._dims(shape)
        return self._ok(self.lib.zyxb_mgraph_expand(self.h, x, arr, n), "expand")

    def reshape(self, x, shape):
        arr, n = self._dims(shape)
        return self._ok(self.lib.zyxb_mgraph_reshape(self.h, x, arr, n), "reshape")

    def permute(self, x, axes):
        arr = (C.c_int32 * len(axes))(*axes)
        return self._ok(self.lib.zyxb_mgraph_permute(self.h, x, arr, len(axes)), "permute")

    def reduce(self, x, rop, axes):
        arr = (C.c_int32 * len(axes))(*axes)
        return self._ok(self.lib.zyxb_mgraph_reduce(self.h, x, rop, arr, len(axes)), "reduce")

    def pad(self, x, axis, lp, length):
        return self._ok(self.lib.zyxb_mgraph_pad(self.h, x, axis, lp, length), "pad")

    def cast(self, x, dtype):
        return self._ok(self.lib.zyxb_mgraph_cast(self.h, x, dtype), "cast")

    def unary(self, x, uop):
        return self._ok(self.lib.zyxb_mgraph_unary(self.h, x, uop), "unary")

    def binary(self, x, y, bop):
        return self._ok(self.lib.zyxb_mgraph_binary(self.h, x, y, bop), "binary")

    def info(self, cls):
        """-> (dtype, shape, number of Node::Kernel alternatives in the class)"""
        dt, rank, k = C.c_int32(), C.c_int32(), C.c_int32()
        shape = (C.c_uint64 * 8)()
        assert self.lib.zyxb_mgraph_class_info(self.h, cls, C.byref(dt), C.byref(rank), shape, C.byref(k)) == L.OK
        return dt.value, tuple(shape[:rank.value]), k.value

    def const_value(self, cls):
        """The values of a class built from constants only (row-major list), or None when it is not one."""
        n = C.c_uint64()
        if self.lib.zyxb_mgraph_const_value(self.h, cls, None, 0, C.byref(n)) != L.OK:
            return None
        buf = (C.c_double * max(n.value, 1))()
        assert self.lib.zyxb_mgraph_const_value(self.h, cls, buf, n.value, C.byref(n)) == L.OK
        return list(buf[:n.value])

    def match(self, outputs):
        outs = (C.c_uint32 * len(outputs))(*outputs)
        n = C.c_int32()
        cap = 64
        buf = (Match * cap)()
        st = self.lib.zyxb_mgraph_match(self.h, outs, len(outputs), buf, cap, C.byref(n))
        if st != L.OK:
            raise ValueError("zyxb_mgraph_match failed: %d" % st)
        return [buf[i] for i in range(min(n.value, cap))]

    def uncovered(self, outputs):
        """Classes the matched programs need but nothing produces (not stored, no program): empty when the graph is covered."""
        outs = (C.c_uint32 * len(outputs))(*outputs)
        n = C.c_int32()
        buf = (C.c_uint32 * 256)()
        assert self.lib.zyxb_mgraph_uncovered(self.h, outs, len(outputs), buf, 256, C.byref(n)) == L.OK
        return list(buf[:min(n.value, 256)])
