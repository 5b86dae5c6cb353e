"""CPU-side checks of the drop-in boundary: the shared library loads and exports every symbol
include/zyxb.h declares; no compute is attempted without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from zyx_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "zyxb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(zyxb_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from zyx_b200 import _lib
    declared = _declared_symbols()
    assert declared, "no declarations found"
    assert sorted(_lib.SIGNATURES) == declared


def test_every_declared_symbol_is_exported(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), name


def test_struct_sizes_match_the_header():
    """sizeof() of every ABI struct, compiled from the header with gcc, equals the ctypes mirror."""
    import subprocess
    import tempfile
    from zyx_b200 import _lib as L
    src = r'''
#include <stdio.h>
#include "zyxb.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\n", sizeof(zyxb_event), sizeof(zyxb_config), sizeof(zyxb_devinfo),
         sizeof(zyxb_rowreduce_desc), sizeof(zyxb_gemm_desc), sizeof(zyxb_eltwise_desc), sizeof(zyxb_optim_desc),
         sizeof(zyxb_attention_desc), sizeof(zyxb_conv_desc), sizeof(zyxb_kernel_desc));
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", os.path.join(d, "t")])
        out = subprocess.check_output([os.path.join(d, "t")]).split()
    want = [C.sizeof(t) for t in (L.Event, L.Config, L.DevInfo, L.RowReduceDesc, L.GemmDesc, L.EltwiseDesc, L.OptimDesc, L.AttentionDesc, L.ConvDesc, L.KernelDesc)]
    assert [int(v) for v in out] == want


def test_init_fails_loudly_without_a_gpu(lib):
    """No CPU fallback: with no CUDA device zyxb_init reports DeviceEnumeration and an error text."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from zyx_b200 import Backend, BackendError
    with pytest.raises(BackendError) as e:
        Backend()
    assert e.value.status_name == "DeviceEnumeration"
    assert "no CPU fallback" in e.value.context
