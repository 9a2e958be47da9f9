"""Builds libtsb.so (the C-ABI shared library) in-tree with nvcc for sm_100a.

    python -m turbospark_b200.build [--force] [--verbose]

Every .cu under csrc/ is compiled to an object under _build/ (only when stale)
and linked into turbospark_b200/libtsb.so.  No CPU fallback exists: if this
library is missing the package refuses to load.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
# TSB_BUILD_DIR redirects objects and the library (a scratch build that leaves the in-tree library alone)
OUT = os.path.join(os.environ["TSB_BUILD_DIR"], "obj") if os.environ.get("TSB_BUILD_DIR") else os.path.join(HERE, "_build")
LIB = os.path.join(os.environ["TSB_BUILD_DIR"], "libtsb.so") if os.environ.get("TSB_BUILD_DIR") else os.path.join(HERE, "libtsb.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "--expt-relaxed-constexpr",
    "-I", INCLUDE,
] + os.environ.get("TSB_NVCC_EXTRA", "").split()


def _sources():
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers_mtime():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "tsb.h"))
    return max(os.path.getmtime(h) for h in hs)


def _compile(src, verbose):
    obj = os.path.join(OUT, src[:-3] + ".o")
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
    return src, r.stderr


def build(force=False, verbose=False):
    os.makedirs(OUT, exist_ok=True)
    hm = _headers_mtime()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OUT, src[:-3] + ".o")
        objs.append(obj)
        stale = (force or not os.path.exists(obj)
                 or os.path.getmtime(obj) < max(os.path.getmtime(os.path.join(CSRC, src)), hm))
        if stale:
            todo.append(src)
    logs = []
    if todo:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(todo))) as ex:
            for src, log in ex.map(lambda s: _compile(s, verbose), todo):
                logs.append((src, log))
    if todo or not os.path.exists(LIB):
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    if verbose:
        for src, log in logs:
            print("==", src)
            print(log)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
