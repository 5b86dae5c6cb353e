"""safetensors files through the host library (zyxb_st_*): the layout Module::save writes (zyx/src/module.rs:36-63)
and Tensor::load_safetensors reads (module.rs:436-529).  Tensors are numpy arrays; bf16 / f16 travel as uint16 bit
patterns with their dtype stated explicitly."""
import ctypes as C
import os

import numpy as np

from . import _lib as L
from . import host as H

_NP_OF = {L.F32: np.float32, L.F64: np.float64, L.U8: np.uint8, L.U16: np.uint16, L.U32: np.uint32, L.U64: np.uint64,
          L.I8: np.int8, L.I16: np.int16, L.I32: np.int32, L.I64: np.int64, L.BOOL: np.bool_, L.BF16: np.uint16, L.F16: np.uint16}
_DT_OF = {np.dtype(v): k for k, v in _NP_OF.items() if k not in (L.BF16, L.F16)}


class SafetensorsError(RuntimeError):
    pass


def _check(lib, st):
    if st != L.OK:
        raise SafetensorsError(lib.zyxb_st_last_error().decode())


def save(path, tensors):
    """tensors: {name: array} or {name: (array, zyxb dtype)} (the explicit form for bf16 / f16 bit patterns); written in
    the mapping's order."""
    lib = H.load()
    items, keep = (H.StTensor * len(tensors))(), []
    for i, (name, val) in enumerate(tensors.items()):
        arr, dtype = val if isinstance(val, tuple) else (val, None)
        arr = np.asarray(arr)
        if not arr.flags.c_contiguous:
            arr = arr.copy()                      # (np.ascontiguousarray would turn a rank-0 array into rank 1)
        if dtype is None:
            if arr.dtype not in _DT_OF:
                raise SafetensorsError("no safetensors dtype for numpy %s" % arr.dtype)
            dtype = _DT_OF[arr.dtype]
        if np.dtype(_NP_OF[dtype]).itemsize != arr.dtype.itemsize:
            raise SafetensorsError("'%s': array of %s cannot hold dtype %d" % (name, arr.dtype, dtype))
        shape = (C.c_uint64 * max(arr.ndim, 1))(*arr.shape)
        keep += [arr, shape]
        items[i].name, items[i].dtype, items[i].rank, items[i].shape = name.encode(), dtype, arr.ndim, shape
        items[i].data = arr.ctypes.data
    _check(lib, lib.zyxb_st_save(os.fsencode(path), items, len(tensors)))


def load(path, with_dtypes=False):
    """-> {name: array} in header order (bf16 / f16 as uint16 bit patterns); with_dtypes: {name: (array, zyxb dtype)}."""
    lib = H.load()
    f = C.c_void_p()
    _check(lib, lib.zyxb_st_open(os.fsencode(path), C.byref(f)))
    out = {}
    try:
        for i in range(lib.zyxb_st_count(f)):
            name, dtype, rank, shape, nbytes = C.c_char_p(), C.c_int32(), C.c_int32(), C.POINTER(C.c_uint64)(), C.c_uint64()
            _check(lib, lib.zyxb_st_info(f, i, C.byref(name), C.byref(dtype), C.byref(rank), C.byref(shape), C.byref(nbytes)))
            arr = np.empty(tuple(shape[k] for k in range(rank.value)), _NP_OF[dtype.value])
            assert arr.nbytes == nbytes.value
            _check(lib, lib.zyxb_st_read(f, i, arr.ctypes.data, arr.nbytes))
            out[name.value.decode()] = (arr, dtype.value) if with_dtypes else arr
    finally:
        lib.zyxb_st_close(f)
    return out
