"""Pins the CPU oracle (and, on a GPU, the product's 32-bit kernels) to the reference's own CUDA
kernels through the committed fixture tests/golden/ref_cuda_golden.json, which
tests/golden/make_ref_cuda_golden.py produced on a B200 from oracle/_ref/libref_cuda.so."""
import importlib.util
import json
import os

import numpy as np
import pytest

import oracle
from cerium_b200 import params

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "ref_cuda_golden.json")
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_ref_cuda_golden.py"))
G = importlib.util.module_from_spec(spec)
spec.loader.exec_module(G)

pytestmark = pytest.mark.skipif(not os.path.exists(FIXTURE), reason="golden fixture not generated yet")


@pytest.fixture(scope="module")
def golden():
    with open(FIXTURE) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def octx():
    return oracle.OracleContext(16, G.PRIMES)


def oracle_output(octx, name):
    kind, seed, d = G.CASES[name]
    inp = G.case_inputs(name)
    if kind == "ntt":
        x = inp["x"].astype(np.uint64)
        return octx.ntt_inverse(x, d["bases"]) if d["inverse"] else octx.ntt_forward(x, d["bases"])
    if kind == "bconv":
        return oracle.bconv(oracle.BCONV_LAZY, [G.PRIMES[i] for i in d["in_idx"]], inp["x"].astype(np.uint64),
                            [G.PRIMES[j] for j in d["out_idx"]])
    f = G.sud_factors(d["divide"])
    return np.stack([octx.sud(b, inp["in1"][i].astype(np.uint64), inp["in2"][i].astype(np.uint64), f[b])
                     for i, b in enumerate(d["bases"])])


@pytest.mark.parametrize("name", sorted(G.CASES))
def test_oracle_matches_reference_cuda_golden(golden, octx, name):
    got = G.digest(oracle_output(octx, name).astype(np.uint32))
    want = golden["cases"][name]
    assert got["head"] == want["head"]
    assert got["sha256"] == want["sha256"]


def test_reference_primes_are_the_example_chain():
    p = params.reference_primes_28bit(64, 16)
    assert p[0] == 204865537 and p[-1] == 268042241 and len(p) == 64
