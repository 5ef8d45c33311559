"""In-tree build of ``libcerium_b200.so`` with nvcc for sm_100a.

``python -m cerium_b200.build`` compiles every ``csrc/*.cu`` into an object file next to it
and links ``cerium_b200/libcerium_b200.so``.  The shared object is git-ignored but travels
with the tree, so a GPU host without the sources' build step can still load it.
``bench_probe/probe.cu`` (the register-only arithmetic-rate probe that bench.py reports its
arithmetic roofline against) becomes a library of its own, ``libcerium_b200_probe.so``: it is
benchmark infrastructure and stays out of the evaluation library.  ``function_map_shim.so`` is the
per-partition plugin of the reference runtime (see ``cerium_b200/plugin.py``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcerium_b200.so")
SHIM_SRC = os.path.join(CSRC, "plugin_shim", "function_map_shim.cpp")
SHIM_LIB = os.path.join(HERE, "function_map_shim.so")
PROBE_SRC = os.path.join(HERE, "bench_probe", "probe.cu")
PROBE_LIB = os.path.join(HERE, "libcerium_b200_probe.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return exe


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "cerium_b200.h"))
    objs = []
    jobs = []
    for src in sources():
        obj = src[:-3] + ".o"
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc] + ARCH + NVCC_FLAGS + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (src, r.stderr))
        return src, r.stderr

    with ThreadPoolExecutor(max_workers=4) as ex:
        for src, log in ex.map(compile_one, jobs):
            if verbose:
                print("== ptxas %s ==\n%s" % (os.path.basename(src), log))
    if jobs or force or _stale(LIB, objs):
        cmd = [nvcc] + ARCH + ["-shared", "-Xcompiler", "-fPIC", "-o", LIB] + objs + ["-lcudart_static", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n%s" % r.stderr)
    if force or _stale(SHIM_LIB, [SHIM_SRC, LIB]):
        # the per-partition plugin of the reference runtime: links the library by absolute run path,
        # because copies of it are installed into program directories
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-o", SHIM_LIB, SHIM_SRC,
               "-L" + HERE, "-lcerium_b200", "-Wl,-rpath," + HERE, "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("g++ failed for %s:\n%s" % (SHIM_SRC, r.stderr))
    if force or _stale(PROBE_LIB, [PROBE_SRC] + headers):
        cmd = [nvcc] + ARCH + NVCC_FLAGS + ["-shared", "-o", PROBE_LIB, PROBE_SRC, "-lcudart_static"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s" % (PROBE_SRC, r.stderr))
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
