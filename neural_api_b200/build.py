"""Builds libcai_cuda.so in-tree with nvcc for sm_100a.

    python -m neural_api_b200.build [--force] [--verbose] [--checked | --all]

One object per .cu under csrc/, linked into neural_api_b200/libcai_cuda.so. The
library links the CUDA runtime statically and NCCL dynamically; it does not
link PyTorch. Objects are rebuilt when their source or a header is newer.
--checked builds libcai_cuda_checked.so instead (-DCAI_CHECKED: every launch is
synchronized and looked at, silent index clamps are reported; objects under
build_checked/); --all builds both.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libcai_cuda.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
          "-I", os.path.join(HERE, "..", "include")]


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths.append(os.path.join(HERE, "..", "include", "cai_cuda.h"))
    return max(os.path.getmtime(p) for p in paths)


def _compile(src, force, verbose, checked=False):
    bdir = BUILD + ("_checked" if checked else "")
    obj = os.path.join(bdir, src[:-3] + ".o")
    srcp = os.path.join(CSRC, src)
    if (not force and os.path.exists(obj)
            and os.path.getmtime(obj) >= max(os.path.getmtime(srcp), _headers_mtime())):
        return obj, ""
    cmd = [NVCC] + ARCH_FLAGS + COMMON + (["-DCAI_CHECKED=1"] if checked else []) + ["-c", srcp, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = r.stdout + r.stderr
    with open(os.path.join(bdir, src[:-3] + ".ptxas.log"), "w") as f:
        f.write(log)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s" % (src, log))
    if verbose:
        print(log)
    return obj, log


def build(force=False, verbose=False, checked=False):
    bdir = BUILD + ("_checked" if checked else "")
    lib = os.path.join(HERE, "libcai_cuda_checked.so") if checked else LIB
    os.makedirs(bdir, exist_ok=True)
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        results = list(ex.map(lambda s: _compile(s, force, verbose, checked), srcs))
    objs = [o for o, _ in results]
    newest = max(os.path.getmtime(o) for o in objs)
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < newest:
        cmd = [NVCC] + ARCH_FLAGS + ["-shared", "-o", lib] + objs + ["-cudart", "static", "-lnccl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return lib


if __name__ == "__main__":
    kinds = [False, True] if "--all" in sys.argv else [("--checked" in sys.argv)]
    for k in kinds:
        print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, checked=k))
