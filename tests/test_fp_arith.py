"""The exact double-precision modular arithmetic of the transforms (primes below 2^50), checked on
the CPU against 128-bit integers: the test compiles tests/fp_arith_check.cpp, which includes the
library's own modarith.cuh, and runs it."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_fp_mulmod_reduce_and_conversions_are_exact(tmp_path):
    exe = str(tmp_path / "fp_arith_check")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-ffp-contract=off", "-DCERIUM_EMU",
                           "-I" + os.path.join(ROOT, "tests", "emu"), "-I" + os.path.join(ROOT, "cerium_b200", "csrc"),
                           "-o", exe, os.path.join(ROOT, "tests", "fp_arith_check.cpp")])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and out.stdout.startswith("OK"), out.stdout + out.stderr
    worst = float(out.stdout.split()[1])
    assert worst <= 0.5 + 4.0 / 32.0 + 1e-6   # |y| <= 4q
