"""safetensors reader / writer of the host library against the reference's own fixture and format
(Module::save, zyx/src/module.rs:36-63; Tensor::load_safetensors, module.rs:436-529; test matmul_disk,
zyx/tests/05_misc.rs:638-660)."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

from zyx_b200 import _lib as L
from zyx_b200 import safetensors as st

HERE = os.path.dirname(__file__)
CROP = os.path.join(HERE, "golden", "xyz2_crop.safetensors")
REF = json.load(open(os.path.join(HERE, "golden", "safetensors_reference.json")))


def test_reads_the_reference_layout_and_reproduces_matmul_disk():
    t = st.load(CROP)
    assert list(t) == ["x", "y", "z"] and all(a.dtype == np.int64 for a in t.values())
    assert t["x"].shape == (16, 512) and t["y"].shape == (512, 16) and t["z"].shape == (16, 16)
    for k, a in t.items():
        assert hashlib.sha256(a.tobytes()).hexdigest() == REF["crop_sha256"][k]
    assert np.array_equal(t["x"] @ t["y"], t["z"])                 # the reference test's assertion
    assert t["z"][0, :8].tolist() == REF["z_first_row"]


def test_writer_emits_the_reference_header_byte_for_byte(tmp_path):
    """Same names, dtypes and shapes as the reference's file must give the same header bytes: Tensor::load_safetensors
    scans the header positionally, so key order and the absence of whitespace are part of the format."""
    shapes = {"x": (256, 512), "y": (512, 368), "z": (256, 368)}
    p = tmp_path / "w.safetensors"
    st.save(p, {k: np.zeros(s, np.int64) for k, s in shapes.items()})
    raw = open(p, "rb").read()
    n = struct.unpack("<Q", raw[:8])[0]
    assert raw[8:8 + n].decode() == REF["header"]
    assert len(raw) == REF["file_bytes"]


REF_CHECKOUT = os.environ.get("ZYX_REFERENCE", "")       # path of a zyx checkout, when one is at hand


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_CHECKOUT, "zyx/tests/xyz2.safetensors")), reason="ZYX_REFERENCE does not point at a zyx checkout")
def test_reads_the_reference_file_itself():
    t = st.load(os.path.join(REF_CHECKOUT, "zyx/tests/xyz2.safetensors"))
    for k, a in t.items():
        assert hashlib.sha256(a.tobytes()).hexdigest() == REF["sha256"][k]


def test_round_trip_every_dtype_and_rank(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {
        "w.bf16": (rng.integers(0, 65536, (3, 5), dtype=np.uint16), L.BF16), "w.f16": (rng.integers(0, 65536, (7,), dtype=np.uint16), L.F16),
        "f32": rng.standard_normal((2, 3, 4)).astype(np.float32), "f64": rng.standard_normal((5,)), "u8": rng.integers(0, 255, (9,), dtype=np.uint8),
        "i32": rng.integers(-9, 9, (4, 4), dtype=np.int32), "i64": rng.integers(-9, 9, (2, 2), dtype=np.int64), "flag": np.array([True, False, True]),
        "scalar": np.float32(3.5).reshape(()), "empty": np.zeros((0, 4), np.float32), 'quo"te\\name': np.arange(3, dtype=np.uint32),
    }
    p = tmp_path / "rt.safetensors"
    st.save(p, tensors)
    got = st.load(p, with_dtypes=True)
    assert list(got) == list(tensors)
    for k, v in tensors.items():
        arr, dt = v if isinstance(v, tuple) else (v, None)
        g, gdt = got[k]
        assert g.shape == np.asarray(arr).shape and np.array_equal(g, arr)
        if dt is not None:
            assert gdt == dt


def _file(tmp_path, header, data=b""):
    p = tmp_path / "h.safetensors"
    h = header.encode()
    open(p, "wb").write(struct.pack("<Q", len(h)) + h + data)
    return p


def test_accepts_any_valid_safetensors_header(tmp_path):
    """Files from other writers: a __metadata__ object, whitespace, keys and data in any order."""
    a, b = np.arange(6, dtype=np.float32), np.arange(4, dtype=np.int16)
    header = ('{ "__metadata__": {"format": "pt", "note": "{[\\"]}"},\n "b": {"data_offsets": [24, 32], "shape": [2, 2], "dtype": "I16"},'
              ' "a": {"shape": [6], "dtype": "F32", "data_offsets": [0, 24], "extra": [1, {"k": null}]} }')
    t = st.load(_file(tmp_path, header, a.tobytes() + b.tobytes()))
    assert list(t) == ["b", "a"] and np.array_equal(t["a"], a) and np.array_equal(t["b"], b.reshape(2, 2))


@pytest.mark.parametrize("header,data,what", [
    ('{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,12]}}', b"\0" * 16, "disagree"),          # the reference's own check
    ('{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}}', b"\0" * 8, "past the end"),
    ('{"a":{"dtype":"F8","shape":[4],"data_offsets":[0,4]}}', b"\0" * 4, "unsupported dtype"),
    ('{"a":{"dtype":"F32","shape":[4]}}', b"\0" * 16, "lacks"),
    ('{"a":{"dtype":"F32","shape":[4],"data_offsets":[0,16]}', b"\0" * 16, "header"),
])
def test_malformed_files_are_refused_with_a_message(tmp_path, header, data, what):
    with pytest.raises(st.SafetensorsError, match=what):
        st.load(_file(tmp_path, header, data))


def test_truncated_and_missing_files(tmp_path):
    p = tmp_path / "short.safetensors"
    open(p, "wb").write(b"\x10\0\0")
    with pytest.raises(st.SafetensorsError):
        st.load(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(st.SafetensorsError, match="exceeds"):
        st.load(p)
    with pytest.raises(st.SafetensorsError, match="cannot open"):
        st.load(tmp_path / "absent.safetensors")
    with pytest.raises(st.SafetensorsError, match="duplicate"):
        _dup(p)


def _dup(p):
    from zyx_b200 import host as H
    import ctypes as C
    lib = H.load()
    arr = np.zeros(1, np.float32)
    shape = (C.c_uint64 * 1)(1)
    items = (H.StTensor * 2)()
    for it in items:
        it.name, it.dtype, it.rank, it.shape, it.data = b"a", L.F32, 1, shape, arr.ctypes.data
    if lib.zyxb_st_save(os.fsencode(p), items, 2) != L.OK:
        raise st.SafetensorsError(lib.zyxb_st_last_error().decode())
