"""The reference runtime's Python surface over this library.

The reference exposes its runtime to Python as ``cerium.runtime`` (pybind11,
``cerium/python/runtime/wrapper.cpp:62-235``): ``Context``, ``CKKSEncryptorContext``, ``CKKSEncryptor``,
``RawInputsWrapper``, ``IOGenerator``, ``CeriumFunctionExecutor`` and ``FusedKernelProgram``.  This module
keeps those names, argument orders and meanings, so that a driver written like
``examples/common.py:83-142`` runs with ``import cerium_b200.runtime as runtime`` in place of
``import cerium.runtime as runtime``:

* the compiled function (``functions<p>``, ``program_inputs``, the kernel plugin) is loaded by the executor
  of the C library (``cerium_program_*``) and replayed on the GPU;
* keys, plaintexts and ciphertexts are generated here - encoding and sampling in numpy on the host, every
  transform, automorphism and modular product on the GPU through the C ABI - with the semantics of the
  reference's generator: symmetric encryption ``(c0, c1) = (-(a s) + e + m, a)``
  (``cerium/runtime/io/ckks-encryptor.cpp:311-370, 427-455``), an evaluation-key digit = an encryption of
  zero over the Q and extension primes whose c0 gets ``[P]_q * s'`` on the digit's limbs (``:534-599``), the
  key kinds of ``:601-766``, the term lists of ``program_inputs`` as ``cerium/runtime/io/generator.cpp:166-300``
  parses them, and the container files of ``cerium_b200/containers.py``.

Random numbers come from numpy's generator, not from the reference's (SEAL's) one: key material is
equivalent, not byte-identical.  One process drives one GPU; a function compiled for several GPUs takes a
``comm`` and runs as this process's partition.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import _capi, containers

KEY_MUL, KEY_ROT, KEY_CON, KEY_BOOT, KEY_EPHEMERAL, KEY_BOOT2, KEY_ROT_INV = range(7)


# ---------------------------------------------------------------------------------------------------------
# context
# ---------------------------------------------------------------------------------------------------------

class Context:
    """``runtime.Context(slots, rns_moduli)`` (wrapper.cpp:68-74): ring degree 2 * slots, the prime chain.

    ``memory="host"`` with an explicit ``lib`` is for a library build that computes in host memory (the
    test-suite's emulation build); the shipped library computes on ``cuda:<device>``."""

    def __init__(self, slots: int, rns_moduli: Sequence[int], lib: Optional[_capi.Library] = None, device: int = 0,
                 memory: str = "cuda"):
        import torch
        self.torch = torch
        self.slots = int(slots)
        self.n = 2 * self.slots
        self.logn = self.n.bit_length() - 1
        if 1 << self.logn != self.n:
            raise ValueError("slots must be a power of two")
        self.moduli = [int(q) for q in rns_moduli]
        self.lib = lib if lib is not None else _capi.load()
        self.device_index = device
        if memory == "cuda":
            if not torch.cuda.is_available():
                raise RuntimeError("cerium_b200.runtime needs a CUDA device")
            self.device = torch.device("cuda", device)
        else:
            self.device = torch.device("cpu")
        self.handle = _capi.Context(self.lib, self.moduli, 32, device=device, logn=self.logn)
        self._q = torch.tensor(self.moduli, dtype=torch.int64, device=self.device)

    @property
    def coeff_count(self) -> int:
        return self.n

    # -- device arithmetic on [k][n] int64 tensors of residues ------------------------------------------
    def stream(self) -> int:
        return self.torch.cuda.current_stream(self.device).cuda_stream if self.device.type == "cuda" else 0

    def q(self, idx: Sequence[int]):
        return self._q[self.torch.tensor(list(idx), dtype=self.torch.int64, device=self.device)].view(-1, 1)

    def _sync(self):
        if self.device.type == "cuda":
            self.torch.cuda.synchronize(self.device)

    def ntt(self, x, idx: Sequence[int], inverse: bool = False):
        w = x.to(self.torch.int32).contiguous()
        f = self.handle.ntt_inverse if inverse else self.handle.ntt_forward
        f(w.data_ptr(), w.data_ptr(), list(idx), stream=self.stream())
        self._sync()
        return w.to(self.torch.int64) % self.q(idx)

    def galois_ntt(self, x, galois_elt: int):
        w = x.to(self.torch.int32).contiguous()
        o = self.torch.empty_like(w)
        self.handle.automorph(o.data_ptr(), w.data_ptr(), galois_elt, w.shape[0], stream=self.stream())
        self._sync()
        return o.to(self.torch.int64)

    def signed_to_rns(self, v: np.ndarray, idx: Sequence[int]):
        """Small signed integer coefficients [n] -> residues [len(idx)][n]."""
        t = self.torch.from_numpy(np.asarray(v, dtype=np.int64)).to(self.device)
        return t.view(1, -1) % self.q(idx)

    def float_to_rns(self, c: np.ndarray, idx: Sequence[int]):
        """Integer-valued doubles of any magnitude -> exact residues: c = M * 2^E with a 53-bit M."""
        m, e = np.frexp(np.abs(c))
        big = (m * 2.0 ** 53).astype(np.int64)
        e = e.astype(np.int64) - 53
        small = np.where(e < 0, big >> np.minimum(-e, 63), big)         # c is an integer: the shifted-out bits are zero
        up = np.maximum(e, 0)
        out = np.empty((len(idx), c.size), dtype=np.int64)
        for k, p in enumerate(idx):
            q = self.moduli[p]
            pow2 = np.array([pow(2, int(s), q) for s in range(int(up.max()) + 1)], dtype=np.int64)
            r = (small % q) * pow2[up] % q
            out[k] = np.where(c < 0, (q - r) % q, r)
        return self.torch.from_numpy(out).to(self.device)


class Ciphertext:
    """A pair of RNS polynomials in NTT form: ``c0``, ``c1`` are [len(rns_base_ids)][n] uint32 (host)."""

    def __init__(self, c0: np.ndarray, c1: np.ndarray, rns_base_ids: Sequence[int]):
        self.c0, self.c1 = c0, c1
        self.rns_base_ids = [int(i) for i in rns_base_ids]


class RawInputsWrapper:
    """Named raw inputs: ``{name: (values, scale)}`` (wrapper.cpp:205-214)."""

    def __init__(self, raw_inputs: Dict[str, Tuple[object, float]]):
        self.raw_inputs = dict(raw_inputs)


# ---------------------------------------------------------------------------------------------------------
# encoder and encryptor
# ---------------------------------------------------------------------------------------------------------

class _Encoder:
    """Canonical-embedding encoder: slot k is the evaluation at the primitive root's power 5^k."""

    def __init__(self, n: int):
        self.n = n
        m = 2 * n
        e = 1
        self.slot_pos = np.empty(n // 2, dtype=np.int64)
        self.conj_pos = np.empty(n // 2, dtype=np.int64)
        for k in range(n // 2):
            self.slot_pos[k] = (e - 1) // 2
            self.conj_pos[k] = (m - e - 1) // 2
            e = e * 5 % m
        self.twist = np.exp(-1j * np.pi * np.arange(n) / n)

    def slots_of(self, message) -> np.ndarray:
        half = self.n // 2
        z = np.atleast_1d(np.asarray(message, dtype=np.complex128))
        if z.size > half or half % z.size:
            raise ValueError("a message must have a power-of-two length of at most %d slots" % half)
        return np.tile(z, half // z.size)

    def encode(self, message, scale: float) -> np.ndarray:
        """-> the n integer coefficients of round(scale * m), as integer-valued doubles."""
        v = np.zeros(self.n, dtype=np.complex128)
        z = self.slots_of(message)
        v[self.slot_pos] = z
        v[self.conj_pos] = np.conj(z)
        coeff = np.fft.fft(v) / self.n * self.twist
        return np.rint(coeff.real * float(scale))

    def decode(self, coeff: np.ndarray, scale: float) -> np.ndarray:
        v = self.n * np.fft.ifft(coeff * np.conj(self.twist))
        return v[self.slot_pos] / float(scale)


class CKKSEncryptorContext:
    """``runtime.CKKSEncryptorContext(context, secret_key[, ephemeral_key][, prng_seed])`` (wrapper.cpp:118-148):
    keys are ternary coefficient vectors; their NTT forms over the whole chain are kept on the device."""

    def __init__(self, context: Context, secret_key: Sequence[int], ephemeral_key=None, prng_seed=None):
        if prng_seed is None and ephemeral_key is not None and len(ephemeral_key) != context.n:
            ephemeral_key, prng_seed = None, ephemeral_key        # (context, secret_key, prng_seed)
        self.context = context
        self.seed = prng_seed
        all_idx = list(range(len(context.moduli)))
        sk = np.asarray(secret_key, dtype=np.int64)
        ek = sk if ephemeral_key is None else np.asarray(ephemeral_key, dtype=np.int64)
        if sk.size != context.n or ek.size != context.n:
            raise ValueError("a key has %d coefficients" % context.n)
        self.secret_key_rns = context.ntt(context.signed_to_rns(sk, all_idx), all_idx)
        self.ephemeral_key_rns = context.ntt(context.signed_to_rns(ek, all_idx), all_idx)
        self.secret_key_squared_rns = self.secret_key_rns * self.secret_key_rns % context.q(all_idx)


def _rng(seed):
    if seed is None:
        return np.random.default_rng()
    return np.random.default_rng([int(s) & 0xFFFFFFFFFFFFFFFF for s in np.atleast_1d(seed)])


class CKKSEncryptor:
    """``runtime.CKKSEncryptor(encryptor_context[, prng_seed])`` (wrapper.cpp:78-116)."""

    def __init__(self, encryptor_context: CKKSEncryptorContext, prng_seed=None):
        self.ectx = encryptor_context
        self.context = encryptor_context.context
        self.rng = _rng(prng_seed if prng_seed is not None else encryptor_context.seed)
        self.encoder = _Encoder(self.context.n)

    # -- sampling ---------------------------------------------------------------------------------------
    def _noise(self, idx):
        """Centred binomial error, 21 coin pairs per coefficient (standard deviation 3.24), in NTT form."""
        n = self.context.n
        bits = self.rng.integers(0, 1 << 21, size=(2, n), dtype=np.int64)
        pop = np.zeros((2, n), dtype=np.int64)
        for b in range(21):
            pop += (bits >> b) & 1
        return self.context.ntt(self.context.signed_to_rns(pop[0] - pop[1], idx), idx)

    def _uniform(self, idx):
        ctx = self.context
        rows = [self.rng.integers(0, ctx.moduli[p], size=ctx.n, dtype=np.int64) for p in idx]
        return ctx.torch.from_numpy(np.stack(rows)).to(ctx.device)

    def encrypt_zero(self, key_rns, idx):
        """(c0, c1) = (-(a s) + e, a) over the primes `idx` under the key whose chain-wide NTT form is `key_rns`."""
        ctx = self.context
        q = ctx.q(idx)
        sel = ctx.torch.tensor(list(idx), dtype=ctx.torch.int64, device=ctx.device)
        c1 = self._uniform(idx)
        c0 = (q - c1 * key_rns[sel] % q + self._noise(idx)) % q
        return c0, c1

    # -- messages ---------------------------------------------------------------------------------------
    def encode(self, message, scale: float, rns_base_ids: Sequence[int]):
        """Plaintext polynomial in NTT form on the given primes ([k][n] int64 tensor of residues)."""
        ctx = self.context
        return ctx.ntt(ctx.float_to_rns(self.encoder.encode(message, scale), rns_base_ids), rns_base_ids)

    def encode_and_encrypt(self, message, scale: float, rns_base_ids: Sequence[int]) -> Ciphertext:
        ctx = self.context
        idx = list(rns_base_ids)
        c0, c1 = self.encrypt_zero(self.ectx.secret_key_rns, idx)
        c0 = (c0 + self.encode(message, scale, idx)) % ctx.q(idx)
        return Ciphertext(_words(c0), _words(c1), idx)

    def decrypt_and_decode(self, ciphertext: Ciphertext, scale: float) -> np.ndarray:
        """Complex slot values of c0 + c1 s, composed over every limb of the ciphertext."""
        ctx = self.context
        idx = ciphertext.rns_base_ids
        q = ctx.q(idx)
        sel = ctx.torch.tensor(idx, dtype=ctx.torch.int64, device=ctx.device)
        c0 = ctx.torch.from_numpy(ciphertext.c0.astype(np.int64)).to(ctx.device) % q
        c1 = ctx.torch.from_numpy(ciphertext.c1.astype(np.int64)).to(ctx.device) % q
        m = ctx.ntt((c0 + c1 * self.ectx.secret_key_rns[sel]) % q, idx, inverse=True).cpu().numpy()
        mods = [ctx.moduli[p] for p in idx]
        big_q = 1
        for p in mods:
            big_q *= p
        vals = np.zeros(ctx.n, dtype=object)
        for i, p in enumerate(mods):
            qi = big_q // p
            vals = vals + m[i].astype(object) * (qi * pow(qi, -1, p) % big_q)
        vals = vals % big_q
        centred = np.where(vals > big_q // 2, vals - big_q, vals)
        return self.encoder.decode(centred.astype(np.float64), scale)

    # -- evaluation keys --------------------------------------------------------------------------------
    def key_rns_base_ids(self, level: int, extension_size: int) -> List[int]:
        top = len(self.context.moduli)
        return list(range(level)) + [top - 1 - i for i in range(extension_size)]

    def generate_evalkey(self, key_type: int, level: int, extension_size: int, rotation: int,
                         digit_partition: Sequence[int]):
        """One digit of a key: (c0, c1) [level + extension_size][n] int64 tensors on key_rns_base_ids()."""
        ctx, e = self.context, self.ectx
        idx = self.key_rns_base_ids(level, extension_size)
        digit = list(digit_partition)
        dsel = ctx.torch.tensor(digit, dtype=ctx.torch.int64, device=ctx.device)
        qd = ctx.q(digit)
        old = e.secret_key_rns
        if key_type == KEY_MUL:
            new = e.secret_key_squared_rns[dsel]
        elif key_type in (KEY_ROT, KEY_CON):
            elt = self.galois_elt(0 if key_type == KEY_CON else rotation)      # step 0 is the conjugation
            new = ctx.galois_ntt(e.secret_key_rns[dsel], elt)
        elif key_type == KEY_ROT_INV:
            old = ctx.galois_ntt(e.secret_key_rns, self.galois_elt(rotation))
            new = e.secret_key_rns[dsel]
        elif key_type in (KEY_BOOT, KEY_BOOT2):
            src = e.secret_key_rns if key_type == KEY_BOOT else e.ephemeral_key_rns
            new = src[dsel] * (ctx.q([level - 1]).view(1, 1) % qd) % qd
        elif key_type == KEY_EPHEMERAL:
            old = e.ephemeral_key_rns
            new = e.secret_key_rns[dsel]
        else:
            raise ValueError("evaluation-key type %r" % (key_type,))
        c0, c1 = self.encrypt_zero(old, idx)
        big_p = 1
        for p in idx[level:]:
            big_p *= ctx.moduli[p]
        factor = ctx.torch.tensor([big_p % ctx.moduli[p] for p in digit], dtype=ctx.torch.int64, device=ctx.device).view(-1, 1)
        rows = ctx.torch.tensor([idx.index(p) for p in digit], dtype=ctx.torch.int64, device=ctx.device)
        c0[rows] = (c0[rows] + new * factor % qd) % qd
        return c0, c1

    def galois_elt(self, step: int) -> int:
        return int(self.context.lib.galois_elt_from_step(step, self.context.logn))


def _words(t) -> np.ndarray:
    return np.ascontiguousarray(t.cpu().numpy().astype(np.uint32))


# ---------------------------------------------------------------------------------------------------------
# program_inputs and the generator
# ---------------------------------------------------------------------------------------------------------

def _ids(text: str) -> List[int]:
    return [int(x) for x in text.strip().strip("[]").split(",") if x.strip()]


def parse_program_inputs(path: str) -> Dict[str, List[Tuple[str, str, List[int]]]]:
    """{stream name: [(term, description, rns_base_ids)]} of a ``program_inputs`` / ``inputs<p>`` file
    (``term | description | [ids]`` lines between ``<name> Stream:`` and ``;``)."""
    streams: Dict[str, List[Tuple[str, str, List[int]]]] = {}
    cur = None
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if line.endswith("Stream:"):
                cur = streams.setdefault(line[:-1].strip(), [])
            elif line == ";":
                cur = None
            elif cur is not None:
                parts = [p.strip() for p in line.replace(" ", "").split("|")]
                if len(parts) != 3:
                    raise ValueError("%s: invalid line %r" % (path, line))
                cur.append((parts[0], parts[1], _ids(parts[2])))
    return streams


def parse_evalkey_description(desc: str):
    """"K:<type>:<level>:<ext>:<rot>:c<0|1>:[digit limbs]" -> (container id, type, level, ext, rot, poly, digit)
    (cerium/runtime/io/generator.cpp:166-228)."""
    head, _, digits = desc.partition(":[")
    k, t, level, ext, rot, poly = head.split(":")
    if k != "K" or poly not in ("c0", "c1"):
        raise ValueError("invalid evaluation-key entry %r" % desc)
    digit = _ids(digits)
    ident = "%s:%s:%s:%s:[%s]" % (t, level, ext, rot, ",".join(str(d) for d in digit))
    return ident, int(t), int(level), int(ext), int(rot), int(poly[1]), digit


class IOGenerator:
    """``runtime.IOGenerator(context)`` (wrapper.cpp:150-185): prepares what ``program_inputs`` asks for."""

    def __init__(self, context: Context):
        self.context = context

    def _container(self, kind: str) -> containers.Container:
        return containers.Container(kind=kind, n=self.context.n, primes=list(self.context.moduli), entries={})

    def generate_and_serialize_evalkeys(self, outputs_file_name: str, inputs_file_name: str,
                                        encryptor_context: CKKSEncryptorContext):
        enc = CKKSEncryptor(encryptor_context)
        out = self._container("evalkeys")
        for _term, desc, _bases in parse_program_inputs(inputs_file_name).get("Evalkey Stream", []):
            ident, t, level, ext, rot, _poly, digit = parse_evalkey_description(desc)
            if ident in out.entries:
                continue
            c0, c1 = enc.generate_evalkey(t, level, ext, rot, digit)
            ids = enc.key_rns_base_ids(level, ext)
            w0, w1 = _words(c0), _words(c1)
            out.entries[ident] = containers.Entry(ident, [[(p, w0[i]) for i, p in enumerate(ids)],
                                                          [(p, w1[i]) for i, p in enumerate(ids)]])
        containers.write(outputs_file_name, out)

    def generate_and_serialize_plaintexts(self, outputs_file_name: str, inputs_file_name: str,
                                          raw_inputs_wrapper: RawInputsWrapper, stream_name: str = "Plaintext Stream"):
        enc = _PlainEncoder(self.context)
        out = self._container("plaintexts")
        for _term, desc, bases in parse_program_inputs(inputs_file_name).get(stream_name, []):
            var, kind, elt = desc.split(":")
            if kind != "p":
                raise ValueError("invalid plaintext entry %r" % desc)
            if var not in raw_inputs_wrapper.raw_inputs:
                raise KeyError("Raw Inputs key error: " + var)
            if var in out.entries:
                continue
            values, scale = raw_inputs_wrapper.raw_inputs[var]
            w = _words(enc.encode(values, scale, bases, int(elt)))
            out.entries[var] = containers.Entry(var, [[(p, w[i]) for i, p in enumerate(bases)]])
        containers.write(outputs_file_name, out)

    generate_and_serialize_remapables = generate_and_serialize_plaintexts

    def generate_ciphertext_inputs(self, inputs_file_name: str, raw_inputs_wrapper: RawInputsWrapper,
                                   encryptor_context: CKKSEncryptorContext) -> Dict[str, Ciphertext]:
        enc = CKKSEncryptor(encryptor_context)
        out: Dict[str, Ciphertext] = {}
        for _term, desc, bases in parse_program_inputs(inputs_file_name).get("Ciphertext Stream", []):
            var = desc.split(":")[0]
            if var in out:
                continue
            if var not in raw_inputs_wrapper.raw_inputs:
                raise KeyError("Raw Inputs key error: " + var)
            values, scale = raw_inputs_wrapper.raw_inputs[var]
            out[var] = enc.encode_and_encrypt(values, scale, bases)
        return out

    def generate_and_serialize_ciphertexts(self, output_file_name: str, inputs_file_name: str,
                                           raw_inputs_wrapper: RawInputsWrapper, encryptor_context: CKKSEncryptorContext):
        out = self._container("ciphertexts")
        for var, ct in self.generate_ciphertext_inputs(inputs_file_name, raw_inputs_wrapper, encryptor_context).items():
            out.entries[var] = containers.Entry(var, [[(p, ct.c0[i]) for i, p in enumerate(ct.rns_base_ids)],
                                                      [(p, ct.c1[i]) for i, p in enumerate(ct.rns_base_ids)]])
        containers.write(output_file_name, out)

    @staticmethod
    def deserialize_ciphertexts(context: Context, ciphertexts_file_name: str) -> Dict[str, Ciphertext]:
        c = containers.read(ciphertexts_file_name)
        out = {}
        for name, e in c.entries.items():
            ids = e.limb_ids()
            out[name] = Ciphertext(e.stack(0, ids), e.stack(1, ids), ids)
        return out


class _PlainEncoder:
    def __init__(self, context: Context):
        self.context = context
        self.encoder = _Encoder(context.n)

    def encode(self, message, scale, rns_base_ids, elt_size: Optional[int] = None):
        """NTT form on the given primes.  A plaintext whose slots repeat every `elt_size` < slots values is a
        polynomial in X^(slots / elt_size): its NTT values come in runs of slots / elt_size equal words, and the
        reference stores (cerium/runtime/io/ckks-encoder.h:205-372) and reads (pt[i >> log2 repeat]) one per run."""
        ctx = self.context
        elt = ctx.slots if elt_size is None else int(elt_size)
        if elt <= 0 or elt > ctx.slots or elt & (elt - 1):
            raise ValueError("elt_size must be a power of two of at most %d" % ctx.slots)
        z = np.atleast_1d(np.asarray(message))
        if z.size not in (1, elt, ctx.slots):
            raise ValueError("values_size must be equal to context slots or elt_size")
        if z.size == ctx.slots and elt < ctx.slots:
            z = z[:elt]
        full = ctx.ntt(ctx.float_to_rns(self.encoder.encode(z, scale), rns_base_ids), rns_base_ids)
        return full[:, ::ctx.slots // elt].contiguous()


# ---------------------------------------------------------------------------------------------------------
# compiled functions
# ---------------------------------------------------------------------------------------------------------

class CeriumFunctionExecutor:
    """One compiled function on this process's GPU (wrapper.cpp:187-203; ``Cerium::Runtime::CeriumFunction``)."""

    def __init__(self, context: Context, name: str = "", use_uvm: bool = False):
        if use_uvm:
            raise NotImplementedError("managed memory is not used: program memory is device memory")
        self.context = context
        self.function_name = name
        self.program: Optional[_capi.Program] = None
        self.streams: Dict[str, list] = {}

    def _scalars(self, raw_inputs: Optional[RawInputsWrapper]) -> Dict[str, int]:
        """Scalar Stream: `term | name:s | [ids]` -> {"term(id)": round(value * scale) mod q_id}, the constant
        plaintext the reference's encode_scalar produces (cerium/runtime/execution/function_io.cpp:306-381)."""
        out: Dict[str, int] = {}
        for term, desc, bases in self.streams.get("Scalar Stream", []):
            var, kind = desc.split(":")
            if kind != "s":
                raise ValueError("invalid scalar entry %r" % desc)
            if raw_inputs is None or var not in raw_inputs.raw_inputs:
                raise KeyError("Raw Inputs key error: " + var)
            value, scale = raw_inputs.raw_inputs[var]
            c = int(np.rint(float(np.real(value)) * float(scale)))
            for b in bases:
                out["%s(%d)" % (term, b)] = c % self.context.moduli[b]
        return out

    def _load(self, directory: str, partition: int, comm, raw_inputs: Optional[RawInputsWrapper] = None):
        from . import plugin
        functions = os.path.join(directory, "functions%d" % partition)
        shim = os.path.join(directory, "function_map_%d.so" % partition)
        if not os.path.exists(os.path.join(directory, "function_map_%d.orig.so" % partition)):
            plugin.install(directory)           # keeps the generated plugin as .orig.so, installs this library's launchers
        self.directory, self.partition = directory, partition
        self.streams = parse_program_inputs(os.path.join(directory, "program_inputs"))
        self.program = _capi.Program(self.context.handle, functions, shim, scalars=self._scalars(raw_inputs), comm=comm)

    def _mine(self, term: str, ids: Sequence[int]) -> List[int]:
        """The limbs of `term` that this partition's function names (a partition holds its own limbs only)."""
        out = []
        for l in ids:
            try:
                self.program.memory("%s(%d)" % (term, l))
                out.append(l)
            except _capi.CeriumError:
                pass
        return out

    def _put(self, term: str, ids: Sequence[int], rows: np.ndarray, all_ids: Sequence[int]):
        mine = self._mine(term, ids)
        if mine:
            pos = [list(all_ids).index(l) for l in mine]
            self.program.write(term, mine, np.ascontiguousarray(rows[pos], dtype=np.uint32), self.context.stream())

    def generate_inputs(self, evalkeys_file_name: str, plaintexts_file_name: str):
        """Loads evaluation keys and plaintexts from their container files into program memory."""
        keys = containers.read(evalkeys_file_name) if self.streams.get("Evalkey Stream") else None
        for term, desc, bases in self.streams.get("Evalkey Stream", []):
            ident, _t, _level, _ext, _rot, poly, _digit = parse_evalkey_description(desc)
            e = keys.entries[ident]
            self._put(term, bases, e.stack(poly, bases), bases)
        pts = containers.read(plaintexts_file_name) if self.streams.get("Plaintext Stream") else None
        for term, desc, bases in self.streams.get("Plaintext Stream", []):
            e = pts.entries[desc.split(":")[0]]
            rows = e.stack(0, bases)
            if rows.shape[1] < self.context.n:          # a periodic plaintext fills the head of its limb
                rows = np.pad(rows, ((0, 0), (0, self.context.n - rows.shape[1])))
            self._put(term, bases, rows, bases)

    def generate_inputs_direct(self, encryptor_context: Optional["CKKSEncryptorContext"],
                               raw_inputs: Optional[RawInputsWrapper]):
        """The same inputs without the container files: every key digit and plaintext is generated and written
        straight into program memory (a bootstrapping function holds gigabytes of keys)."""
        if self.streams.get("Evalkey Stream"):
            if encryptor_context is None:
                raise ValueError("the function takes evaluation keys: pass encryptor_context or write the evalkeys file")
            enc = CKKSEncryptor(encryptor_context)
            by_key: Dict[str, list] = {}
            for term, desc, bases in self.streams["Evalkey Stream"]:
                by_key.setdefault(parse_evalkey_description(desc)[0], []).append((term, desc, bases))
            for ident, lines in by_key.items():
                _id, t, level, ext, rot, _poly, digit = parse_evalkey_description(lines[0][1])
                polys = [_words(c) for c in enc.generate_evalkey(t, level, ext, rot, digit)]
                ids = enc.key_rns_base_ids(level, ext)
                for term, desc, bases in lines:
                    poly = parse_evalkey_description(desc)[5]
                    self._put(term, bases, polys[poly][[ids.index(b) for b in bases]], bases)
        if self.streams.get("Plaintext Stream"):
            if raw_inputs is None:
                raise ValueError("the function takes plaintexts: pass the raw inputs or write the plaintexts file")
            pe = _PlainEncoder(self.context)
            for term, desc, bases in self.streams["Plaintext Stream"]:
                var, kind, elt = desc.split(":")
                if var not in raw_inputs.raw_inputs:
                    raise KeyError("Raw Inputs key error: " + var)
                values, scale = raw_inputs.raw_inputs[var]
                rows = _words(pe.encode(values, scale, bases, int(elt)))
                if rows.shape[1] < self.context.n:
                    rows = np.pad(rows, ((0, 0), (0, self.context.n - rows.shape[1])))
                self._put(term, bases, rows, bases)

    # wrapper.cpp:196-200: inputs that a caller re-maps between calls of one function (the weights of a layer).
    # The executor refuses functions that read them, so these only say so.
    def generate_remapable_inputs(self, remapables_file_name, plaintexts_file_name, map_key, remapables_use_uvm=False):
        raise NotImplementedError("re-mappable inputs are not served by the executor")

    def copy_remapable_inputs_to_device(self, *args):
        raise NotImplementedError("re-mappable inputs are not served by the executor")

    def create_remapable_offsets(self, *args):
        raise NotImplementedError("re-mappable inputs are not served by the executor")

    def copy_inputs_to_device(self):
        """Inputs are written straight into device memory by generate_inputs; nothing is staged."""

    def copy_ciphertext_inputs_to_gpu(self, inputs_file_name: str, gpus: int, encrypted_inputs: Dict[str, Ciphertext]):
        del inputs_file_name, gpus              # the term list was read from program_inputs at load
        for term, desc, bases in self.streams.get("Ciphertext Stream", []):
            var, poly = desc.split(":")
            ct = encrypted_inputs[var]
            rows = ct.c0 if poly == "c0" else ct.c1
            self._put(term, bases, rows[[ct.rns_base_ids.index(l) for l in bases]], bases)

    def get_program_outputs(self) -> Dict[str, Ciphertext]:
        """{name: Ciphertext} of the Output Stream; on a partition, only the limbs it holds."""
        ctx = self.context
        got: Dict[str, Dict[str, Tuple[List[int], np.ndarray]]] = {}
        for term, desc, bases in self.streams.get("Output Stream", []):
            var, poly = desc.split(":")
            mine = self._mine(term, bases)
            rows = np.empty((len(mine), ctx.n), dtype=np.uint32)
            if mine:
                self.program.read(term, mine, rows, ctx.stream())
            q = np.array([ctx.moduli[l] for l in mine], dtype=np.uint32).reshape(-1, 1)
            got.setdefault(var, {})[poly] = (mine, rows % q if mine else rows)
        return {var: Ciphertext(p["c0"][1], p["c1"][1], p["c0"][0]) for var, p in got.items()}

    def run(self):
        self.program.run(self.context.stream())
        self.context._sync()


class FusedKernelProgram:
    """``runtime.FusedKernelProgram(context, directory_base, top_level_function)`` (wrapper.cpp:216-234).

    ``make_program(gpus, options, inputs)`` loads ``<directory_base>/<function>/`` - ``functions<p>``,
    ``program_inputs``, the kernel plugin, and the ``evalkeys`` / ``plaintexts`` containers if the function has
    such inputs - and returns ``{function name: CeriumFunctionExecutor}``.  For ``gpus > 1`` this process is
    one partition: pass ``partition`` and ``comm`` (the reference runs all partitions from one process).
    Functions the entry function calls are loaded with it by the executor, from their own directories under
    ``directory_base``; their plugins are installed here first.  With ``encryptor_context`` given and no
    ``evalkeys`` file in the function directory, keys and plaintexts are generated straight into device
    memory instead of being read from container files."""

    def __init__(self, context: Context, directory_base: str, top_level_function: str):
        self.context = context
        self.directory_base = directory_base
        self.top = top_level_function
        self.functions: Dict[str, CeriumFunctionExecutor] = {}

    def make_program(self, gpus: int = 1, options: Optional[dict] = None, inputs: Optional[RawInputsWrapper] = None,
                     partition: int = 0, comm=None, encryptor_context: Optional[CKKSEncryptorContext] = None
                     ) -> Dict[str, CeriumFunctionExecutor]:
        graph = str(((options or {}).get(self.top) or {}).get("use_cudagraph", "False")).lower() in ("true", "1", "yes")
        if gpus > 1 and comm is None:
            raise ValueError("a function compiled for %d GPUs runs as %d processes: pass partition= and comm=" % (gpus, gpus))
        from . import plugin
        d = os.path.join(self.directory_base, self.top)
        for other in sorted(os.listdir(self.directory_base)):       # called functions: the executor loads their shims
            od = os.path.join(self.directory_base, other)
            if other != self.top and os.path.isfile(os.path.join(od, "function_map_%d.so" % partition)) and \
                    not os.path.exists(os.path.join(od, "function_map_%d.orig.so" % partition)):
                plugin.install(od)
        f = CeriumFunctionExecutor(self.context, self.top)
        f._load(d, partition, comm, inputs)
        if encryptor_context is not None and not os.path.exists(os.path.join(d, "evalkeys")):
            f.generate_inputs_direct(encryptor_context, inputs)      # no container files: generate into device memory
        else:
            f.generate_inputs(os.path.join(d, "evalkeys"), os.path.join(d, "plaintexts"))
        if graph:
            f.program.run(self.context.stream())    # once eagerly (lazy set-up inside the launchers), then recorded
            self.context._sync()
            f.program.capture()
        self.functions = {self.top: f}
        return self.functions

    def run(self):
        self.functions[self.top].run()
