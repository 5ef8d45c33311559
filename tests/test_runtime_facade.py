"""The reference's Python runtime surface (cerium.runtime names) over this library.

CPU tests run the façade on the emulation build (host memory) and check its key material with the
oracle's operators: a ciphertext it encrypts, rotated / multiplied by the ORACLE with keys it generated,
must decrypt to the rotated / multiplied message.  GPU tests follow the reference's own example driver
step for step (examples/common.py:83-142: context, keys, IOGenerator, FusedKernelProgram.make_program,
copy_ciphertext_inputs_to_gpu, run, get_program_outputs, decrypt_and_decode, np.allclose with its
tolerances) on the programs the reference's compiler produced for examples/rotation,
examples/relinearization and examples/rescale, and report the precision in bits."""
import os
import random
import shutil

import numpy as np
import pytest

from cerium_b200 import params, runtime

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROGS = os.path.join(ROOT, "tests", "golden", "programs")
PLUGINS = os.path.join(ROOT, "oracle", "_ref", "programs")
SLOTS, LEVEL = 32 * 1024, 12                                    # examples/common.py:26-27
PRIMES = params.reference_primes_28bit(64, 16)                   # examples/primes.py
Q_IDX = list(range(LEVEL))
P_IDX = list(range(52, 64))


def sample_vector(seed):
    return np.random.default_rng(seed).integers(0, 5, size=SLOTS).astype(float)       # examples/common.py:67-69


def _secret_key(rng, hamming_weight):                                                   # examples/common.py:72-76
    key = [0] * (2 * SLOTS)
    for position in rng.sample(range(2 * SLOTS), hamming_weight):
        key[position] = rng.choice((-1, 1))
    return key


def _keys(context):
    rng = random.Random(10)
    seed = np.random.default_rng(10).integers(0, 2 ** 32, size=8, dtype=np.uint64).tolist()
    ectx = runtime.CKKSEncryptorContext(context, _secret_key(rng, SLOTS), _secret_key(rng, 32), seed)
    return ectx, runtime.CKKSEncryptor(ectx, seed)


def _bits(actual, expected):
    return float(-np.log2(np.max(np.abs(np.asarray(actual) - np.asarray(expected))) + 2.0 ** -200))


# ---------------------------------------------------------------------------------------------------------
# CPU: the façade on the emulation build, evaluated by the oracle
# ---------------------------------------------------------------------------------------------------------

@pytest.fixture(scope="module")
def emu():
    from tests.backends import EmuBackend
    be = EmuBackend()
    context = runtime.Context(SLOTS, PRIMES, lib=be.lib, memory="host")
    assert context.coeff_count == 2 * SLOTS
    ectx, enc = _keys(context)
    return context, ectx, enc


def test_encrypt_decrypt_round_trip(emu):
    _context, _ectx, enc = emu
    x = sample_vector(1)
    for scale in (1 << 56, 1 << 84):
        ct = enc.encode_and_encrypt(x, scale, Q_IDX)
        assert ct.c0.shape == (LEVEL, 2 * SLOTS) and ct.c0.dtype == np.uint32 and ct.rns_base_ids == Q_IDX
        assert _bits(enc.decrypt_and_decode(ct, scale), x) > 40
    z = np.exp(2j * np.pi * np.arange(SLOTS) / SLOTS)                     # complex slots
    ct = enc.encode_and_encrypt(z, 1 << 56, Q_IDX[:3])
    assert _bits(enc.decrypt_and_decode(ct, 1 << 56), z) > 40
    ct = enc.encode_and_encrypt(2.5, 1 << 56, Q_IDX[:3])                  # a scalar fills every slot
    assert _bits(enc.decrypt_and_decode(ct, 1 << 56), np.full(SLOTS, 2.5)) > 40


def _key_tensor(enc, key_type, rot):
    """One-digit key in the oracle's layout [1][2][Q limbs, extension limbs ascending][n]."""
    c0, c1 = enc.generate_evalkey(key_type, LEVEL, LEVEL, rot, Q_IDX)
    ids = enc.key_rns_base_ids(LEVEL, LEVEL)
    assert ids == Q_IDX + P_IDX[::-1]                                     # extension primes from the top of the chain
    order = [ids.index(p) for p in Q_IDX + P_IDX]
    return np.stack([np.stack([c0.numpy()[order], c1.numpy()[order]])]).astype(np.uint64)


def test_generated_keys_work_under_the_oracles_operators(emu):
    import oracle
    context, _ectx, enc = emu
    orc = oracle.OracleContext(16, PRIMES)
    x, y = sample_vector(1), sample_vector(2)
    cx = enc.encode_and_encrypt(x, 1 << 84, Q_IDX)
    # rotation by one slot to the left with the key of step 1 (examples/rotation)
    evk = _key_tensor(enc, runtime.KEY_ROT, 1)
    elt = oracle.galois_elt_from_step(1, 16)
    r0, r1 = orc.hrot(oracle.BCONV_LAZY, oracle.ROUND_FLOOR, Q_IDX, P_IDX, 1, elt,
                      cx.c0.astype(np.uint64), cx.c1.astype(np.uint64), evk)
    got = enc.decrypt_and_decode(runtime.Ciphertext(r0.astype(np.uint32), r1.astype(np.uint32), Q_IDX), 1 << 84)
    assert np.allclose(got, np.roll(x, -1), rtol=1e-5, atol=1e-4), _bits(got, np.roll(x, -1))
    # conjugation key: step 0
    z = np.exp(2j * np.pi * np.arange(SLOTS) / SLOTS)
    cz = enc.encode_and_encrypt(z, 1 << 84, Q_IDX)
    evk = _key_tensor(enc, runtime.KEY_CON, 0)
    r0, r1 = orc.hrot(oracle.BCONV_LAZY, oracle.ROUND_FLOOR, Q_IDX, P_IDX, 1, 2 * context.n - 1,
                      cz.c0.astype(np.uint64), cz.c1.astype(np.uint64), evk)
    got = enc.decrypt_and_decode(runtime.Ciphertext(r0.astype(np.uint32), r1.astype(np.uint32), Q_IDX), 1 << 84)
    assert np.allclose(got, np.conj(z), rtol=1e-5, atol=1e-4)
    # multiplication + relinearisation with the key of s^2 (examples/relinearization)
    ax = enc.encode_and_encrypt(x, 1 << 56, Q_IDX)
    ay = enc.encode_and_encrypt(y, 1 << 56, Q_IDX)
    evk = _key_tensor(enc, runtime.KEY_MUL, 0)
    u = [a.astype(np.uint64) for a in (ax.c0, ax.c1, ay.c0, ay.c1)]
    r0, r1 = orc.hmult_relin(oracle.BCONV_LAZY, oracle.ROUND_FLOOR, False, Q_IDX, P_IDX, 1, *u, evk)
    got = enc.decrypt_and_decode(runtime.Ciphertext(r0.astype(np.uint32), r1.astype(np.uint32), Q_IDX), float(1 << 112))
    assert np.allclose(got, x * y, rtol=1e-5, atol=1e-4), _bits(got, x * y)


def test_generator_writes_what_program_inputs_asks_for(emu, tmp_path):
    from cerium_b200 import containers
    context, ectx, _enc = emu
    gen = runtime.IOGenerator(context)
    # evaluation keys of the compiled rotation: one entry (one digit), both polynomials on Q and extension limbs
    pin = os.path.join(PROGS, "rotation_1gpu", "program_inputs")
    streams = runtime.parse_program_inputs(pin)
    assert [t for t, _, _ in streams["Ciphertext Stream"]] == ["i2", "i1"]
    assert len(streams["Evalkey Stream"]) == 4 and streams["Plaintext Stream"] == []
    gen.generate_and_serialize_evalkeys(str(tmp_path / "evalkeys"), pin, ectx)
    c = containers.read(str(tmp_path / "evalkeys"))
    assert c.kind == "evalkeys" and list(c.entries) == ["1:12:12:1:[0,1,2,3,4,5,6,7,8,9,10,11]"]
    assert sorted(c.entries["1:12:12:1:[0,1,2,3,4,5,6,7,8,9,10,11]"].limb_ids()) == Q_IDX + P_IDX
    assert containers.evalkey_tensor(c, 1, 12, 12, 1, Q_IDX + P_IDX).shape == (1, 2, 24, 2 * SLOTS)
    # the plaintext of the compiled rescale program, and ciphertext inputs by name
    pin = os.path.join(PROGS, "rescale_1gpu", "program_inputs")
    raw = runtime.RawInputsWrapper({"x": (sample_vector(1), 1 << 56), "factor": (sample_vector(2) + 1, 1 << 28)})
    gen.generate_and_serialize_plaintexts(str(tmp_path / "plaintexts"), pin, raw)
    c = containers.read(str(tmp_path / "plaintexts"))
    assert list(c.entries) == ["factor"] and c.entries["factor"].limb_ids() == Q_IDX
    cts = gen.generate_ciphertext_inputs(pin, raw, ectx)
    assert list(cts) == ["x"] and cts["x"].rns_base_ids == Q_IDX
    gen.generate_and_serialize_ciphertexts(str(tmp_path / "ciphertexts"), pin, raw, ectx)
    back = runtime.IOGenerator.deserialize_ciphertexts(context, str(tmp_path / "ciphertexts"))
    assert list(back) == ["x"] and back["x"].c0.shape == (LEVEL, 2 * SLOTS)
    with pytest.raises(KeyError):
        gen.generate_ciphertext_inputs(pin, runtime.RawInputsWrapper({}), ectx)


# ---------------------------------------------------------------------------------------------------------
# GPU: the reference's example driver, with this module in place of cerium.runtime
# ---------------------------------------------------------------------------------------------------------

def _compiled(tmp_path, example, gpus=1):
    """<compiled>/<function>_<g>gpus/ for every function of the program, as the reference's build leaves them:
    records, input lists and the generated plugin of each partition."""
    tag = "%s_%dgpu" % (example, gpus)
    src, plug = os.path.join(PROGS, tag), os.path.join(PLUGINS, tag)
    main = "main_%dgpus" % gpus
    functions = [main] if os.path.exists(os.path.join(src, "program_inputs")) else sorted(os.listdir(src))
    for fn in functions:
        fsrc, fplug = (src, plug) if functions == [main] else (os.path.join(src, fn), os.path.join(plug, fn))
        d = tmp_path / "compiled" / fn
        d.mkdir(parents=True)
        shutil.copy(os.path.join(fsrc, "program_inputs"), d / "program_inputs")
        for p in range(gpus):
            orig = os.path.join(fplug, "function_map_%d.orig.so" % p)
            if not os.path.exists(orig):
                pytest.skip("the generated plugin of %s was not built (tests/golden/programs/make_programs.py)" % tag)
            shutil.copy(os.path.join(fsrc, "functions%d" % p), d / ("functions%d" % p))
            shutil.copy(os.path.join(fsrc, "inputs%d" % p), d / ("inputs%d" % p))
            shutil.copy(orig, d / ("function_map_%d.so" % p))
    return tmp_path / "compiled"


def run_program(tmp_path, example, raw_inputs, expected, output_scale, atol=1e-4, gpus=1, partition=0, comm=None,
                gather=None, device=0):
    """examples/common.py:83-142 with one import changed.  With gpus > 1 this process is one partition (the
    reference drives all partitions from one process): `gather` collects the output limbs of all partitions."""
    name = "main_%dgpus" % gpus
    compiled = _compiled(tmp_path, example, gpus)
    context = runtime.Context(SLOTS, PRIMES, device=device)
    encryptor_context, encryptor = _keys(context)
    inputs = runtime.RawInputsWrapper(raw_inputs)
    generator = runtime.IOGenerator(context)
    program_inputs = str(compiled / name / "program_inputs")
    for function_dir in sorted(compiled.glob("*_%dgpus" % gpus)):
        function_inputs = function_dir / "program_inputs"
        generator.generate_and_serialize_evalkeys(str(function_dir / "evalkeys"), str(function_inputs), encryptor_context)
        generator.generate_and_serialize_plaintexts(str(function_dir / "plaintexts"), str(function_inputs), inputs)
    program = runtime.FusedKernelProgram(context, str(compiled), name)
    if gpus == 1:
        functions = program.make_program(gpus, {name: {"use_cudagraph": "True"}}, inputs)
    else:
        functions = program.make_program(gpus, {name: {"use_cudagraph": "True"}}, inputs, partition=partition, comm=comm)
    encrypted_inputs = generator.generate_ciphertext_inputs(program_inputs, inputs, encryptor_context)
    functions[name].copy_ciphertext_inputs_to_gpu(str(compiled / name / "inputs"), gpus, encrypted_inputs)
    program.run()
    program.run()                                   # a program is built once and run many times
    encrypted_output = functions[name].get_program_outputs()["z"]
    if gather is not None:
        encrypted_output = gather(encrypted_output)
    actual = np.asarray(encryptor.decrypt_and_decode(encrypted_output, output_scale))
    expected = np.asarray(expected)
    bits = _bits(actual, expected)
    print("%s: maximum absolute error %.3e (%.1f bits)" % (example, float(np.max(np.abs(actual - expected))), bits))
    assert np.allclose(actual, expected, rtol=1e-5, atol=atol), "%s output differs from its expected result" % example
    return bits


@pytest.mark.gpu
def test_rotation_example(tmp_path):
    x = sample_vector(1)
    scale = 1 << 84
    assert run_program(tmp_path, "rotation", {"x": (x, scale)}, np.roll(x, -1), scale) > 13      # examples/rotation/runner.py


@pytest.mark.gpu
def test_relinearization_example(tmp_path):
    x, y = sample_vector(1), sample_vector(2)
    scale = 1 << 56
    assert run_program(tmp_path, "relinearization", {"x": (x, scale), "y": (y, scale)}, x * y, float(scale * scale)) > 13


@pytest.mark.gpu
def test_rescale_example(tmp_path):
    x, factor = sample_vector(1), sample_vector(2) + 1
    ciphertext_scale, plaintext_scale = 1 << 56, 1 << 28
    output_scale = ciphertext_scale * plaintext_scale / PRIMES[LEVEL - 1]                    # examples/rescale/runner.py
    assert run_program(tmp_path, "rescale", {"x": (x, ciphertext_scale), "factor": (factor, plaintext_scale)},
                       x * factor, output_scale) > 13


@pytest.mark.gpu
def test_addition_example(tmp_path):
    x, y = sample_vector(1), sample_vector(2)
    scale = 1 << 56
    assert run_program(tmp_path, "addition", {"x": (x, scale), "y": (y, scale)}, x + y, scale) > 13


@pytest.mark.gpu
def test_multiplication_example(tmp_path):
    x, factor = sample_vector(1), sample_vector(2) + 1
    scale = 1 << 28
    assert run_program(tmp_path, "multiplication", {"x": (x, scale), "factor": (factor, scale)}, x * factor, scale * scale) > 13


@pytest.mark.gpu
def test_periodic_plaintext_matrix_example(tmp_path):
    """Plaintexts that repeat every 2 slots (stored as 4 words per limb) and rotations by +1 and -1."""
    x = sample_vector(1)
    expected = np.empty_like(x)
    expected[0::2] = 2 * x[0::2] + x[1::2]
    expected[1::2] = x[0::2] + 3 * x[1::2]
    scale, ciphertext_scale = 1 << 28, 1 << 84
    raw = {"x": (x, ciphertext_scale), "diagonal": (np.array([2.0, 3.0]), scale),
           "left_mask": (np.array([1.0, 0.0]), scale), "right_mask": (np.array([0.0, 1.0]), scale)}
    assert run_program(tmp_path, "periodic_plaintext_matrix", raw, expected, float(ciphertext_scale * scale)) > 13


@pytest.mark.gpu
def test_function_calling_example(tmp_path):
    """The entry function is one call record; the called function's limbs are bound to the caller's."""
    x = sample_vector(1)
    scale = 1 << 56
    assert run_program(tmp_path, "function_calling", {"x": (x, scale)}, 2 * x, scale) > 13


# a function compiled for two GPUs: one process per partition, drm records on NCCL ------------------------

def _two_gpu_worker(rank, world, port, workdir, example, ret):
    import sys
    import pathlib
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from cerium_b200 import _capi, sharded
    comm = sharded.nccl_comm(_capi.load(), rank, world, rank)

    def gather(ct):
        parts = [None] * world
        dist.all_gather_object(parts, (ct.rns_base_ids, ct.c0, ct.c1))
        ids = sorted(i for p in parts for i in p[0])
        rows0 = {i: p[1][k] for p in parts for k, i in enumerate(p[0])}
        rows1 = {i: p[2][k] for p in parts for k, i in enumerate(p[0])}
        return runtime.Ciphertext(np.stack([rows0[i] for i in ids]), np.stack([rows1[i] for i in ids]), ids)

    x, y = sample_vector(1), sample_vector(2)
    cases = {"rotation": ({"x": (x, 1 << 84)}, np.roll(x, -1), float(1 << 84)),
             "relinearization": ({"x": (x, 1 << 56), "y": (y, 1 << 56)}, x * y, float(1 << 112)),
             "rescale": ({"x": (x, 1 << 56), "factor": (y + 1, 1 << 28)}, x * (y + 1), (1 << 84) / PRIMES[LEVEL - 1])}
    raw, expected, out_scale = cases[example]
    try:
        bits = run_program(pathlib.Path(workdir) / ("rank%d" % rank), example, raw, expected, out_scale, gpus=world,
                           partition=rank, comm=comm, gather=gather, device=rank)
        ret[rank] = bits
    finally:
        comm.close()
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("example", ["rotation", "relinearization", "rescale"])
def test_two_gpu_examples(tmp_path, example):
    import socket
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    if not os.path.exists(os.path.join(PLUGINS, example + "_2gpu", "function_map_1.orig.so")):
        pytest.skip("the generated plugins of %s_2gpu were not built" % example)
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_two_gpu_worker, args=(r, 2, port, str(tmp_path), example, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert all(ret.get(r, 0) > 13 for r in range(2)), dict(ret)


def test_periodic_plaintext_is_the_subsampled_transform(emu):
    """A plaintext that repeats every 1024 slots: the compact form (one word per run of 32) expands to the
    full transform, and multiplying by it through the library's periodic entry point gives the product slots."""
    import torch
    context, _ectx, enc = emu
    pe = runtime._PlainEncoder(context)
    period = 1024
    v = np.random.default_rng(3).integers(1, 5, size=period).astype(float)
    idx = Q_IDX[:3]
    compact = pe.encode(v, 1 << 28, idx, period)
    full = pe.encode(np.tile(v, SLOTS // period), 1 << 28, idx)
    assert compact.shape == (3, 2 * period)
    assert torch.equal(compact.repeat_interleave(SLOTS // period, dim=1), full)
    x = sample_vector(1)
    ct = enc.encode_and_encrypt(x, 1 << 28, idx)
    pt = compact.to(torch.int32).contiguous()
    outs = []
    for c in (ct.c0, ct.c1):
        a = torch.from_numpy(c.view(np.int32).copy())
        o = torch.empty_like(a)
        context.handle.mul_plain_periodic(o.data_ptr(), a.data_ptr(), pt.data_ptr(), 5, idx)
        outs.append(o.numpy().view(np.uint32))
    got = enc.decrypt_and_decode(runtime.Ciphertext(outs[0], outs[1], idx), float(1 << 56))
    assert np.allclose(got, x * np.tile(v, SLOTS // period), rtol=1e-5, atol=1e-4)


# the reference's bootstrapping benchmark ---------------------------------------------------------------

BOOT_TAG, BOOT_FN = "bootstrap_32K_%dgpu", "bootstrap_32Kslots_33levels_%dgpus"


def bootstrap_directory(tmp_path, gpus=1):
    """<compiled>/<function>/ of the compiled bootstrapping benchmark (benchmarks/bootstrap_32K)."""
    import lzma
    tag, fn = BOOT_TAG % gpus, BOOT_FN % gpus
    d = tmp_path / "compiled" / fn
    d.mkdir(parents=True)
    names = ["program_inputs"] + ["%s%d" % (f, p) for p in range(gpus) for f in ("functions", "inputs")]
    for f in names:
        with lzma.open(os.path.join(PROGS, tag, f + ".xz"), "rb") as src, open(d / f, "wb") as dst:
            dst.write(src.read())
    for p in range(gpus):
        shutil.copy(os.path.join(PLUGINS, tag, "function_map_%d.orig.so" % p), d / ("function_map_%d.so" % p))
    return tmp_path / "compiled"


def bootstrap_built(gpus=1):
    tag = BOOT_TAG % gpus
    return all(os.path.exists(os.path.join(PLUGINS, tag, f)) for f in
               ["raw_inputs.npz"] + ["function_map_%d.orig.so" % p for p in range(gpus)])


def bootstrap_raw_inputs(gpus=1):
    z = np.load(os.path.join(PLUGINS, BOOT_TAG % gpus, "raw_inputs.npz"))
    return {k[2:]: (z[k][()] if z[k].ndim == 0 else z[k], float(z["s:" + k[2:]])) for k in z.files if k.startswith("v:")}


def bootstrap_run(tmp_path, gpus=1, partition=0, comm=None, gather=None, device=0, barrier=None, runs=5, graph=False):
    """benchmarks/bootstrap_32K/bootstrap_runner.py:83-170 with this module in place of cerium.runtime: a level-2
    ciphertext of unit-modulus complex slots is bootstrapped to level 18 by the reference's compiled program
    (one GPU: 195 key digits, 259 plaintexts, 31 scalars, 347 launches) and decrypted.
    Returns (milliseconds per run, precision bits as the runner prints them, steps, setup seconds)."""
    import time
    import torch
    fn = BOOT_FN % gpus
    compiled = bootstrap_directory(tmp_path, gpus)
    rnd = random.Random(10)

    def generate_secret_key(hamming_weight):                       # bootstrap_runner.py:29-43
        key = [0] * (2 * SLOTS)
        for position in rnd.sample(range(2 * SLOTS), hamming_weight):
            key[position] = rnd.choice((-1, 1))
        return key
    raw_inputs = runtime.RawInputsWrapper(bootstrap_raw_inputs(gpus))
    context = runtime.Context(SLOTS, PRIMES, device=device)
    seed = np.random.default_rng(10).integers(0, 2 ** 32 - 1, size=8).tolist()
    encryptor_context = runtime.CKKSEncryptorContext(context, generate_secret_key(SLOTS), generate_secret_key(32), seed)
    encryptor = runtime.CKKSEncryptor(encryptor_context, seed)
    inp_scale = PRIMES[1] * PRIMES[0] / (1 << 5)                   # log_message_ratio = 5
    arr = np.exp(1j * np.random.default_rng(10).uniform(0, 2 * np.pi, SLOTS))
    inputs = runtime.RawInputsWrapper({"x": (arr, inp_scale)})
    program = runtime.FusedKernelProgram(context, str(compiled), fn)
    t0 = time.time()
    functions = program.make_program(gpus, {fn: {"use_cudagraph": str(graph)}}, raw_inputs, partition=partition, comm=comm,
                                     encryptor_context=encryptor_context)
    t_setup = time.time() - t0
    main = functions[fn]
    generator = runtime.IOGenerator(context)
    encrypted_inputs = generator.generate_ciphertext_inputs(str(compiled / fn / "program_inputs"), inputs, encryptor_context)
    main.copy_ciphertext_inputs_to_gpu(str(compiled / fn / "inputs"), gpus, encrypted_inputs)
    program.run()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = context.stream()
    if barrier is not None:
        barrier()
    e0.record()
    for _ in range(runs):
        main.program.run(stream)
    e1.record()
    torch.cuda.synchronize()
    out = main.get_program_outputs()["z"]
    if gather is not None:
        out = gather(out)
    z = np.asarray(encryptor.decrypt_and_decode(out, inp_scale))
    err = float(np.max(np.abs(z - arr)))
    ms = e0.elapsed_time(e1) / runs
    if gpus == 1 and not graph:
        # the same program recorded into a CUDA graph (the reference's default mode): same result, replayed
        before = {k: (v.c0.copy(), v.c1.copy()) for k, v in main.get_program_outputs().items()}
        main.program.capture()
        main.program.run(stream)
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(runs):
            main.program.run(stream)
        g1.record()
        torch.cuda.synchronize()
        after = main.get_program_outputs()
        assert all(np.array_equal(after[k].c0, before[k][0]) and np.array_equal(after[k].c1, before[k][1]) for k in before), \
            "graph replay differs from stream replay"
        print("bootstrap program as a CUDA graph: %.2f ms per run (stream mode %.2f)" % (g0.elapsed_time(g1) / runs, ms))
    return ms, float(-np.log2(err)), main.program.num_steps, t_setup


def test_bootstrap_program_records():
    """The compiled benchmark as the executor's parser sees it: 462 records, ten of them two-limb CRT
    compositions (rsv), no exchange records on one GPU."""
    import lzma
    import tempfile
    from cerium_b200 import _capi
    with tempfile.TemporaryDirectory() as t:
        path = os.path.join(t, "functions0")
        def kinds(gpus, part):
            with lzma.open(os.path.join(PROGS, BOOT_TAG % gpus, "functions%d.xz" % part), "rb") as src, open(path, "wb") as dst:
                dst.write(src.read())
            out = {}
            for r in _capi.inspect_program(_capi.load(), path):
                out[r["type"]] = out.get(r["type"], 0) + 1
            return out
        assert kinds(1, 0) == {"int": 62, "bco": 56, "ntt": 26, "generic": 137, "pmu": 19, "mov": 115, "sud": 37, "rsv": 10}
        # the builds for several GPUs exchange limbs: all-gathers, reduce-scatters and all-reduces
        k8 = kinds(8, 0)
        assert (k8["drm"], k8["ags"], k8["ard"], k8["rsv"]) == (27, 8, 6, 11)


@pytest.mark.gpu
def test_bootstrap_benchmark_program(tmp_path):
    if not bootstrap_built(1):
        pytest.skip("the benchmark's plugin and plaintext values were not built (tests/golden/programs/make_programs.py)")
    ms, bits, steps, setup = bootstrap_run(tmp_path)
    print("bootstrap program, 1 GPU: %d steps, setup %.1f s, %.2f ms per run, precision bits %.2f" % (steps, setup, ms, bits))
    assert steps == 347 and bits > 15, "the bootstrapped ciphertext does not decrypt to its input"


def _bootstrap_worker(rank, world, port, workdir, ret):
    import sys
    import pathlib
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from cerium_b200 import _capi, sharded
    comm = sharded.nccl_comm(_capi.load(), rank, world, rank)

    def gather(ct):
        parts = [None] * world
        dist.all_gather_object(parts, (ct.rns_base_ids, ct.c0, ct.c1))
        ids = sorted(i for p in parts for i in p[0])
        rows0 = {i: p[1][k] for p in parts for k, i in enumerate(p[0])}
        rows1 = {i: p[2][k] for p in parts for k, i in enumerate(p[0])}
        return runtime.Ciphertext(np.stack([rows0[i] for i in ids]), np.stack([rows1[i] for i in ids]), ids)
    try:
        ms, bits, steps, setup = bootstrap_run(pathlib.Path(workdir) / ("rank%d" % rank), world, rank, comm, gather, rank,
                                               barrier=dist.barrier)
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ret[rank] = (float(t.item()), bits, steps, setup)
    finally:
        comm.close()
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_bootstrap_benchmark_program_multi_gpu(tmp_path, world):
    """The benchmark compiled for several GPUs: one process per partition; drm, ags and ard records on NCCL."""
    import socket
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    if not bootstrap_built(world):
        pytest.skip("the benchmark's plugins and plaintext values were not built (tests/golden/programs/make_programs.py)")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    procs = [ctx.Process(target=_bootstrap_worker, args=(r, world, port, str(tmp_path), ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(900)
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    ms, bits, steps, setup = ret[0]
    print("bootstrap program, %d GPUs: %d steps on partition 0, setup %.1f s, %.2f ms per run (max over ranks), "
          "precision bits %.2f" % (world, steps, setup, ms, bits))
    assert all(ret[r][1] > 15 for r in range(world)), dict(ret)


def test_importable_under_the_references_module_name():
    """A driver that says `import cerium.runtime as runtime` finds the same classes with cerium_b200/as_cerium on
    its path."""
    import importlib
    import sys
    path = os.path.join(ROOT, "cerium_b200", "as_cerium")
    saved = {k: sys.modules.pop(k) for k in list(sys.modules) if k == "cerium" or k.startswith("cerium.")}
    sys.path.insert(0, path)
    try:
        mod = importlib.import_module("cerium.runtime")
        for name in ("Context", "Ciphertext", "CKKSEncryptor", "CKKSEncryptorContext", "IOGenerator",
                     "CeriumFunctionExecutor", "RawInputsWrapper", "FusedKernelProgram"):     # wrapper.cpp:62-235
            assert getattr(mod, name) is getattr(runtime, name)
        assert callable(mod.FusedKernelProgram.make_program) and callable(mod.FusedKernelProgram.run)
    finally:
        sys.path.remove(path)
        for k in [k for k in sys.modules if k == "cerium" or k.startswith("cerium.")]:
            del sys.modules[k]
        sys.modules.update(saved)
