"""Builds libmugraph.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m attention_superoptimizer_b200.build [--force]

Sources: csrc/kernels/*.cu (CUDA), csrc/host/*.cc (host C++).  Objects go to
attention_superoptimizer_b200/build/, the library to attention_superoptimizer_b200/lib/.
A file is recompiled when it or any header is newer than its object.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIBDIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIBDIR, "libmugraph.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
INCLUDES = ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CSRC, "host"), "-I" + os.path.join(CSRC, "kernels")]


def _headers():
    pats = [os.path.join(ROOT, "include", "**", "*.h"), os.path.join(CSRC, "**", "*.h"),
            os.path.join(CSRC, "**", "*.cuh")]
    out = []
    for p in pats:
        out += glob.glob(p, recursive=True)
    return out


def _stale(src, obj, newest_header):
    if not os.path.exists(obj):
        return True
    t = os.path.getmtime(obj)
    return os.path.getmtime(src) > t or newest_header > t


def _compile(job):
    src, obj, verbose = job
    if src.endswith(".cu"):
        cmd = [NVCC, "-std=c++17", "-O3", "-lineinfo", *ARCH, "-Xcompiler", "-fPIC", *INCLUDES, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
    else:
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-Wall", *INCLUDES, "-I/usr/local/cuda/include", "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return src, r.stderr


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "kernels", "*.cu")) + glob.glob(os.path.join(CSRC, "host", "*.cc")))
    newest = max([os.path.getmtime(h) for h in _headers()] + [0.0])
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s) + ".o")
        objs.append(o)
        if force or _stale(s, o, newest):
            jobs.append((s, o, verbose))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for src, log in ex.map(_compile, jobs):
                if verbose and log:
                    sys.stderr.write("== %s\n%s" % (os.path.basename(src), log))
    if jobs or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", *ARCH, "-o", LIB, *objs, "-cudart", "static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s" % (" ".join(cmd), r.stderr))
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
