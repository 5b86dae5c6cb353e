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


RUST_TO_C = {"ZyxbEvent": ("zyxb_event", "Event"), "ZyxbConfig": ("zyxb_config", "Config"), "ZyxbDevinfo": ("zyxb_devinfo", "DevInfo"),
             "ZyxbRowreduceDesc": ("zyxb_rowreduce_desc", "RowReduceDesc"), "ZyxbGemmDesc": ("zyxb_gemm_desc", "GemmDesc"),
             "ZyxbEltwiseDesc": ("zyxb_eltwise_desc", "EltwiseDesc"), "ZyxbOptimDesc": ("zyxb_optim_desc", "OptimDesc"),
             "ZyxbAttentionDesc": ("zyxb_attention_desc", "AttentionDesc"), "ZyxbConvDesc": ("zyxb_conv_desc", "ConvDesc"),
             "ZyxbKernelDesc": ("zyxb_kernel_desc", "KernelDesc")}
RUST_SIZES = {"i32": 4, "u32": 4, "f32": 4, "i64": 8, "u64": 8, "f64": 8, "c_char": 1, "u8": 1, "i8": 1}


def _rust_structs():
    """name -> [(field, size, align)] of every #[repr(C)] struct in shim/b200.rs, laid out by the C rules repr(C) follows."""
    text = open(os.path.join(ROOT, "shim", "b200.rs")).read()
    out = {}
    for m in re.finditer(r"#\[repr\(C\)\][^\n]*\n\s*pub struct (\w+) \{(.*?)\}", text, flags=re.S):
        fields = []
        for f in re.finditer(r"pub (\w+): ([^,}]+?)\s*(?:,|$)", m.group(2).strip(), flags=re.S):
            name, ty = f.group(1), f.group(2).strip()
            arr = re.fullmatch(r"\[(\w+); (\d+)\]", ty)
            if arr:
                size, align = RUST_SIZES[arr.group(1)] * int(arr.group(2)), RUST_SIZES[arr.group(1)]
            elif ty.startswith("*"):
                size = align = 8
            elif ty in RUST_SIZES:
                size = align = RUST_SIZES[ty]
            else:
                size = align = None            # a nested struct / union: offset still checked, size taken from C
            fields.append((name, size, align))
        out[m.group(1)] = fields
    return out


def test_field_offsets_agree_between_the_header_the_ctypes_mirror_and_the_rust_shim():
    """offsetof() of every field of every ABI struct, compiled from include/zyxb.h with gcc, against (a) the ctypes mirror the
    tests drive the library with and (b) the #[repr(C)] structs of shim/b200.rs (field names, order and C layout)."""
    import subprocess
    import tempfile
    from zyx_b200 import _lib as L
    rust = _rust_structs()
    assert set(RUST_TO_C) <= set(rust), sorted(set(RUST_TO_C) - set(rust))
    lines = []
    for rname, (cname, _) in RUST_TO_C.items():
        for field, _, _ in rust[rname]:
            lines.append('  printf("%s.%s %%zu\\n", offsetof(%s, %s));' % (rname, field, cname, field))
        lines.append('  printf("%s.sizeof %%zu\\n", sizeof(%s));' % (rname, cname))
    src = "#include <stdio.h>\n#include <stddef.h>\n#include \"zyxb.h\"\nint main(void) {\n" + "\n".join(lines) + "\n  return 0;\n}\n"
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", os.path.join(d, "t")])
        c_off = dict(line.split() for line in subprocess.check_output([os.path.join(d, "t")], text=True).splitlines())
    for rname, (cname, pyname) in RUST_TO_C.items():
        py = getattr(L, pyname)
        assert [f for f, _, _ in rust[rname]] == [f for f, _ in py._fields_], rname          # same fields, same order
        off = 0
        for field, size, align in rust[rname]:
            want = int(c_off["%s.%s" % (rname, field)])
            assert getattr(py, field).offset == want, (pyname, field)
            if size is None:                                   # nested aggregate (the descriptor union): 8-byte aligned
                off = (off + 7) // 8 * 8
                assert off == want, (rname, field)
                off = int(c_off[rname + ".sizeof"])
                continue
            off = (off + align - 1) // align * align
            assert off == want, (rname, field, off, want)
            off += size
        assert C.sizeof(py) == int(c_off[rname + ".sizeof"]), rname


def test_host_header_and_binding_agree():
    """Every function include/zyxb_host.h declares is exported by libzyxb_host.so and bound with a prototype."""
    from zyx_b200 import host, matcher   # noqa: F401  (importing matcher registers its prototypes)
    text = open(os.path.join(ROOT, "include", "zyxb_host.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = sorted(set(re.findall(r"\b(zyxb_[a-z0-9_]+)\s*\(", text)))
    assert declared and sorted(host.HOST_SIGNATURES) == declared, sorted(set(declared) ^ set(host.HOST_SIGNATURES))
    lib = host.load()
    for name in declared:
        assert hasattr(lib, name), name
    st = subprocess_sizeof("zyxb_match")
    assert st == C.sizeof(matcher.Match)


def subprocess_sizeof(ctype):
    import subprocess
    import tempfile
    src = '#include <stdio.h>\n#include "zyxb_host.h"\nint main(void) { printf("%%zu\\n", sizeof(%s)); return 0; }\n' % ctype
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.check_call(["gcc", "-std=c11", "-I", os.path.join(ROOT, "include"), os.path.join(d, "t.c"), "-o", os.path.join(d, "t")])
        return int(subprocess.check_output([os.path.join(d, "t")]))


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
