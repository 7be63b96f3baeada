"""Builds sager_b200/libsager_b200.so from sager_b200/csrc/*.cu with nvcc for
sm_100a. The library is built in-tree (next to this file) so that it travels
with the source tree; nothing is installed. Every source file is compiled to
its own object (in parallel, only when it or a header changed) and the objects
are linked into the shared library."""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libsager_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr", "--extended-lambda",
]
LINK_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static",
              "-Xcompiler", "-fPIC"]


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    """CUDA sources and the host-only C++ sources (compiled by the same nvcc as host code)."""
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.abspath(__file__)] + \
        glob.glob(os.path.join(os.path.dirname(HERE), "include", "*.h"))


def _obj(src):
    return os.path.join(OBJ, os.path.splitext(os.path.basename(src))[0] + ".o")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(p) > t for p in sources() + headers())


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = nvcc_path()
    hdr_t = max(os.path.getmtime(p) for p in headers())
    inc = ["-I", CSRC, "-I", os.path.join(os.path.dirname(HERE), "include")]

    def compile_one(src):
        obj = _obj(src)
        if not force and not ptxas_info and os.path.exists(obj) and \
                os.path.getmtime(obj) > max(hdr_t, os.path.getmtime(src)):
            return src, 0, ""
        flags = list(NVCC_FLAGS)
        if src.endswith(".cpp"):
            # host arithmetic that must reproduce the reference's bytes: hardware FMA for the fused
            # operations the source spells out, and no other contraction
            flags[flags.index("-fPIC,-fvisibility=hidden")] = "-fPIC,-fvisibility=hidden,-mfma,-ffp-contract=off"
        cmd = [nvcc] + flags + (["-Xptxas", "-v"] if ptxas_info else []) + inc + ["-c", "-o", obj, src]
        if verbose:
            print(" ".join(cmd))
        res = subprocess.run(cmd, capture_output=True, text=True)
        return src, res.returncode, res.stdout + res.stderr

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        results = list(ex.map(compile_one, sources()))
    failed = [r for r in results if r[1] != 0]
    if failed:
        for _, _, log in failed:
            sys.stderr.write(log)
        raise RuntimeError("nvcc failed: " + ", ".join(os.path.basename(r[0]) for r in failed))
    if ptxas_info or verbose:
        for _, _, log in results:
            sys.stderr.write(log)
    # objects of sources that no longer exist must not be linked
    objs = [_obj(s) for s in sources()]
    for stale in set(glob.glob(os.path.join(OBJ, "*.o"))) - set(objs):
        os.remove(stale)
    res = subprocess.run([nvcc] + LINK_FLAGS + ["-o", LIB + ".tmp"] + objs, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    os.replace(LIB + ".tmp", LIB)          # a reader never sees a half-written library
    return LIB


if __name__ == "__main__":
    build(force="--incremental" not in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(LIB)
