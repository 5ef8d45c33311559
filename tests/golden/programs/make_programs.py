"""Generates the compiled-program fixtures of this directory with the REFERENCE's own compiler.

    python tests/golden/programs/make_programs.py [--ref <reference checkout>]

1. Builds the reference compiler's Python module (cerium/compiler/**, cerium/python/compiler/wrapper.cpp)
   with g++ and pybind11 into oracle/_ref/refcompiler/ (git-ignored).  Its one external dependency,
   {fmt} 9.1.0, is not in this image; the few calls it makes are served by the stand-in header of
   fmt_standin/ (this directory).
2. Runs the reference's example programs through its DSL and compiler (examples/<name>/program.py, built
   for the GPU counts below) and copies the TEXT artefacts a runtime needs - the kernel stream
   `ll.functions` as `functions<p>`, `inputs<p>`, `program_inputs`, `compile_config` - into
   tests/golden/programs/<name>_<g>gpu/ (committed).
3. Compiles the generated CUDA code of every partition (kernels_*.cu, function_map.cu) against the
   reference's kernel headers, with plugin_stubs.cu standing in for kernels/function.cu (which needs
   CUDA 13), into oracle/_ref/programs/<name>_<g>gpu/function_map_<p>.orig.so (git-ignored, travels to
   the GPU host like every built object).  The generated sources themselves are not kept.
4. The reference's bootstrapping benchmark (benchmarks/bootstrap_32K/bootstrap.py, built for 1, 2, 4 and 8 GPUs;
   one GPU: 462 records, 195 key digits, 259 plaintexts): the same three steps, the text artefacts xz-compressed
   under tests/golden/programs/bootstrap_32K_<g>gpu/; and the benchmark's own plaintext / scalar VALUES (FFT-factor
   diagonals, sine-approximation coefficients: benchmarks/bootstrap_32K/bootstrap_values.py, imported here) saved
   as oracle/_ref/programs/bootstrap_32K_<g>gpu/raw_inputs.npz (20 MB each, git-ignored like the plugins, travels with
   the tree), so that the GPU test can decrypt a bootstrapped ciphertext and report its precision.
Nothing here runs at test time: tests read the committed text files and load the built plugins.
"""
from __future__ import annotations

import argparse
import glob
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(HERE)))
OUT_REF = os.path.join(ROOT, "oracle", "_ref")
PROGRAMS = [("rotation", 1), ("relinearization", 1), ("rescale", 1), ("rotation", 2), ("relinearization", 2), ("rescale", 2),
            ("addition", 1), ("multiplication", 1), ("periodic_plaintext_matrix", 1), ("function_calling", 1)]


def build_compiler(ref: str) -> str:
    import pybind11
    work = os.path.join(OUT_REF, "refcompiler")
    obj = os.path.join(work, "obj")
    os.makedirs(obj, exist_ok=True)
    c = os.path.join(ref, "cerium", "compiler")
    srcs = (glob.glob(c + "/*.cpp") + glob.glob(c + "/util/*.cpp") + glob.glob(c + "/util/*.cc") +
            glob.glob(c + "/frontend/*.cpp") + glob.glob(c + "/backend/*.cc") +
            [os.path.join(ref, "cerium", "python", "compiler", "wrapper.cpp")])
    inc = ["-I" + ref, "-I" + os.path.join(ref, "cerium"), "-I" + os.path.join(HERE, "fmt_standin"),
           "-I" + sysconfig.get_paths()["include"], "-I" + pybind11.get_include()]

    def comp(s):
        o = os.path.join(obj, hashlib.md5(s.encode()).hexdigest()[:8] + "_" + os.path.basename(s) + ".o")
        if not os.path.exists(o) or os.path.getmtime(o) < os.path.getmtime(s):
            subprocess.check_call(["g++", "-O1", "-std=c++17", "-fPIC", '-DCERIUM_VERSION_STR="0"'] + inc + ["-c", s, "-o", o])
        return o
    with ThreadPoolExecutor(8) as ex:
        objs = list(ex.map(comp, srcs))
    pkg = os.path.join(work, "pkg", "cerium")
    os.makedirs(os.path.join(pkg, "compiler"), exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    subprocess.check_call(["g++", "-shared", "-o", os.path.join(pkg, "compiler", "_cerium_compiler" + ext)] + objs)
    py = os.path.join(ref, "cerium", "python")
    shutil.copy(os.path.join(py, "compiler", "__init__.py"), os.path.join(pkg, "compiler"))
    for sub in ("compiler", "dsl", "passes"):
        shutil.copytree(os.path.join(py, "compiler", sub), os.path.join(pkg, "compiler", sub), dirs_exist_ok=True)
    shutil.copy(os.path.join(py, "cerium", "__init__.py"), pkg)
    for sub in ("dsl", "passes"):
        shutil.copytree(os.path.join(py, "cerium", sub), os.path.join(pkg, sub), dirs_exist_ok=True)
    return os.path.dirname(pkg)


def compile_example(ref: str, pkg: str, name: str, gpus: int) -> str:
    run = os.path.join(OUT_REF, "refcompiler", "run")
    if os.path.isdir(os.path.join(run, "examples")):
        shutil.rmtree(os.path.join(run, "examples"))
    shutil.copytree(os.path.join(ref, "examples"), os.path.join(run, "examples"))   # the compiler writes beside the program
    env = dict(os.environ, PYTHONPATH=pkg + os.pathsep + run)
    subprocess.check_call([sys.executable, "-m", "examples.%s.program" % name, "--gpus", str(gpus)], cwd=run, env=env)
    return os.path.join(run, "examples", name, "outputs", name, "main_%dgpus" % gpus)


def make_bootstrap(ref: str, pkg: str, kern: str, gpus: int = 1):
    import lzma
    tag, fn = "bootstrap_32K_%dgpu" % gpus, "bootstrap_32Kslots_33levels_%dgpus" % gpus
    run = os.path.join(OUT_REF, "refcompiler", "run_bootstrap")
    if os.path.isdir(run):
        shutil.rmtree(run)
    shutil.copytree(os.path.join(ref, "benchmarks", "bootstrap_32K"), run)
    env = dict(os.environ, PYTHONPATH=pkg)
    subprocess.check_call([sys.executable, "bootstrap.py", "--gpus", str(gpus), "--prefix", os.path.join(run, "out") + "/"], cwd=run, env=env)
    src = os.path.join(run, "out", fn)
    dst = os.path.join(HERE, tag)
    os.makedirs(dst, exist_ok=True)
    plug = os.path.join(OUT_REF, "programs", tag)
    os.makedirs(plug, exist_ok=True)
    flags = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcudafe", "--diag_suppress=177",
             "-Xcompiler", "-fPIC", "-D__FNAME__=%s" % fn, "-I" + kern]
    texts = [(os.path.join(src, "program_inputs"), "program_inputs")]
    jobs = []
    for p in range(gpus):
        part = os.path.join(src, "partition_%d" % p)
        texts += [(os.path.join(part, "ll.functions"), "functions%d" % p), (os.path.join(part, "inputs%d" % p), "inputs%d" % p)]
        for c in sorted(glob.glob(os.path.join(part, "kernels_*.cu"))) + [os.path.join(part, "function_map.cu"),
                                                                           os.path.join(HERE, "plugin_stubs.cu")]:
            jobs.append((p, c, os.path.join(plug, "p%d_%s.o" % (p, os.path.basename(c)))))
    for path, name in texts:
        with open(path, "rb") as f, lzma.open(os.path.join(dst, name + ".xz"), "wb", preset=9) as g:
            g.write(f.read())

    def comp(job):       # one object per generated source, in parallel: the kernel files are large
        subprocess.check_call(["nvcc"] + flags + ["-c", job[1], "-o", job[2]])
    with ThreadPoolExecutor(8) as ex:
        list(ex.map(comp, jobs))
    for p in range(gpus):
        objs = [o for q, _, o in jobs if q == p]
        subprocess.check_call(["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o",
                               os.path.join(plug, "function_map_%d.orig.so" % p)] + objs)
        for o in objs:
            os.remove(o)
    # the benchmark's plaintext and scalar values, by input name (bootstrap_runner.py:84-87)
    config = "b33" if gpus == 1 else "b33_multi"
    code = ("import sys, numpy as np; sys.path.insert(0, %r); from bootstrap_values import get_bootstrap_runner_inputs; "
            "raw = get_bootstrap_runner_inputs(%r, 18); "
            "np.savez_compressed(%r, **{'v:' + k: np.asarray(v[0]) for k, v in raw.items()}, "
            "**{'s:' + k: np.asarray(float(v[1])) for k, v in raw.items()})") % (run, config, os.path.join(plug, "raw_inputs.npz"))
    subprocess.check_call([sys.executable, "-c", code], cwd=run)
    print("made", tag)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CERIUM_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference"))
    args = ap.parse_args()
    ref = args.ref
    kern = os.path.join(ref, "cerium", "compiler", "backend", "kernels")
    pkg = build_compiler(ref)
    for name, gpus in PROGRAMS:
        src = compile_example(ref, pkg, name, gpus)
        tag = "%s_%dgpu" % (name, gpus)
        # every function of the program (the entry function and the ones it calls); a program of one function is
        # stored flat, a program of several with one directory per function, as the compiler lays them out
        functions = sorted(d for d in os.listdir(os.path.dirname(src)) if os.path.isdir(os.path.join(os.path.dirname(src), d)))
        for fn in functions:
            fsrc = os.path.join(os.path.dirname(src), fn)
            sub = fn if len(functions) > 1 else ""
            dst = os.path.join(HERE, tag, sub)
            os.makedirs(dst, exist_ok=True)
            for f in ("program_inputs", "compile_config", "calls"):
                shutil.copy(os.path.join(fsrc, f), dst)
            plug = os.path.join(OUT_REF, "programs", tag, sub)
            os.makedirs(plug, exist_ok=True)
            for p in range(gpus):
                part = os.path.join(fsrc, "partition_%d" % p)
                shutil.copy(os.path.join(part, "ll.functions"), os.path.join(dst, "functions%d" % p))
                shutil.copy(os.path.join(part, "inputs%d" % p), dst)
                cu = sorted(glob.glob(os.path.join(part, "kernels_*.cu"))) + [os.path.join(part, "function_map.cu"),
                                                                               os.path.join(HERE, "plugin_stubs.cu")]
                subprocess.check_call(["nvcc", "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                                       "-Xcudafe", "--diag_suppress=177", "-Xcompiler", "-fPIC", "-shared",
                                       "-D__FNAME__=%s" % fn, "-I" + kern,
                                       "-o", os.path.join(plug, "function_map_%d.orig.so" % p)] + cu)
        print("made", tag, functions)
    for gpus in (1, 2, 4, 8):
        make_bootstrap(ref, pkg, kern, gpus)
    # the working copies of the reference's example and benchmark directories (the compiler writes beside the
    # program it compiles) and what it generated there are scratch: only the files copied out above are kept
    for scratch in ("run", "run_bootstrap"):
        shutil.rmtree(os.path.join(OUT_REF, "refcompiler", scratch), ignore_errors=True)


if __name__ == "__main__":
    main()
