"""Builds tests/emu/libcerium_b200_emu.so: the library's own sources compiled with g++ against
the CUDA stand-ins of emu_cuda.h.  TEST INFRASTRUCTURE ONLY; the package never loads it."""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CSRC = os.path.join(ROOT, "cerium_b200", "csrc")
LIB = os.path.join(HERE, "libcerium_b200_emu.so")


def build(force: bool = False) -> str:
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps += [os.path.join(HERE, "emu_cuda.h"), os.path.join(HERE, "emu_runtime.cpp"),
             os.path.join(ROOT, "include", "cerium_b200.h")]
    if not force and os.path.exists(LIB) and all(os.path.getmtime(d) <= os.path.getmtime(LIB) for d in deps):
        return LIB
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-DCERIUM_EMU", "-I" + HERE,
           "-Wno-unused-variable", "-o", LIB, os.path.join(HERE, "emu_runtime.cpp")]
    for s in srcs:
        cmd += ["-x", "c++", s]
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
