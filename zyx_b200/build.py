"""Builds zyx_b200/libzyxb.so from zyx_b200/csrc with nvcc for sm_100a (in-tree, no JIT cache).

    python -m zyx_b200.build [--force]

Objects go to zyx_b200/_build/; a source is recompiled when it, or any header, is newer than
its object.  nvcc cross-compiles without a GPU.
"""
import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libzyxb.so")
HOST_LIB = os.path.join(HERE, "libzyxb_host.so")
ROOT = os.path.dirname(HERE)

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "-diag-suppress", "177"]
NVCC_FLAGS += os.environ.get("ZYXB_NVCC_EXTRA", "").split()      # e.g. -DZYXB_ATTN_TRACE for the attention kernel's clock trace
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-I/usr/local/cuda/include"]


def _newest_header():
    hs = glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(src, obj):
    if src.endswith(".cu"):
        cmd = [NVCC] + NVCC_FLAGS + ["-c", src, "-o", obj]
    else:
        cmd = ["g++"] + CXX_FLAGS + ["-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return src


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))
    hdr_time = _newest_header()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s) + ".o")
        objs.append(o)
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr_time):
            jobs.append((s, o))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            for done in ex.map(lambda j: _compile(*j), jobs):
                if verbose:
                    print("compiled", os.path.basename(done))
    if jobs or not os.path.exists(LIB):
        tmp = LIB + ".tmp%d" % os.getpid()           # linked beside the target and renamed: a reader never sees half a library
        cmd = [NVCC, "-shared", "-o", tmp] + objs + ["-cudart", "static", "-ldl", "-lpthread",
                                                      "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
        os.replace(tmp, LIB)
    build_host(force or bool(jobs))
    return LIB


def build_host(force=False):
    """libzyxb_host.so: the C++ host runtime (include/zyxb_host.h); it uses libzyxb.so only through its C ABI."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "host", "*.cpp")))
    newest = max([os.path.getmtime(s) for s in srcs + glob.glob(os.path.join(CSRC, "host", "*.hpp"))] + [_newest_header()])
    if force or not os.path.exists(HOST_LIB) or os.path.getmtime(HOST_LIB) < newest:
        tmp = HOST_LIB + ".tmp%d" % os.getpid()
        cmd = ["g++", "-shared", "-o", tmp] + CXX_FLAGS + srcs + ["-L", HERE, "-lzyxb", "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("host link failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
        os.replace(tmp, HOST_LIB)
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
