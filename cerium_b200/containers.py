"""On-disk containers of the reference runtime: evaluation keys, plaintexts and ciphertexts.

Reads and writes the three binary files the reference's IOGenerator produces and its runtime
loads (``cerium/runtime/io/generator.cpp:503-564`` evalkeys, ``:737-789`` plaintexts, ``:791-860``
ciphertexts; headers in ``cerium/runtime/io/generator.h:113-115``), so that keys and inputs generated
for a Cerium program can be fed to this library and results written back in the same form.

Layout (native little-endian, ``size_t`` = 8 bytes)::

    header string + NUL          "Cerium::Evalkeys\\n" | "Cerium::Plaintexts\\n" | "Cerium::Ciphertexts\\n"
    size_t n                     ring degree
    size_t n_primes; u64 primes[n_primes]
    size_t n_entries
    size_t payload_bytes         number of 32-bit words of all limbs, times 4
    per entry:
        size_t id_len (with NUL); char id[id_len]
        size_t n_limbs
        [plaintexts, ciphertexts only] size_t elt_count     words per limb
        polynomial 0: n_limbs x (u64 limb_id, u32 data[elt_count or n])
        [evalkeys, ciphertexts] polynomial 1: the same

An evaluation-key entry is ONE digit of a key; its id is ``"<type>:<level>:<ext>:<rot>:[digit limbs]"``
(``cerium/compiler/backend/compiler_keyswitch.cc:143-160``).  ``evalkey_tensor`` stacks the digits of a
key into the ``[digit][c0, c1][limb][N]`` array the key-switch entry points take.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Dict, List, Sequence, Tuple

import numpy as np

EVALKEY_HEADER = b"Cerium::Evalkeys\n\0"
PLAINTEXT_HEADER = b"Cerium::Plaintexts\n\0"
CIPHERTEXT_HEADER = b"Cerium::Ciphertexts\n\0"
_KINDS = {EVALKEY_HEADER: ("evalkeys", 2, False), PLAINTEXT_HEADER: ("plaintexts", 1, True),
          CIPHERTEXT_HEADER: ("ciphertexts", 2, True)}


@dataclass
class Entry:
    """One named object: ``polys[p]`` is a list of (limb_id, uint32 array) in file order."""
    name: str
    polys: List[List[Tuple[int, np.ndarray]]]

    def limb_ids(self) -> List[int]:
        return [lid for lid, _ in self.polys[0]]

    def stack(self, poly: int, limb_order: Sequence[int]) -> np.ndarray:
        """[len(limb_order)][words] array of polynomial `poly`, limbs in the given prime-index order."""
        by_id = dict(self.polys[poly])
        missing = [l for l in limb_order if l not in by_id]
        if missing:
            raise KeyError("%s: limbs %s are not in the container" % (self.name, missing))
        return np.stack([by_id[l] for l in limb_order])


@dataclass
class Container:
    kind: str                      # "evalkeys" | "plaintexts" | "ciphertexts"
    n: int
    primes: List[int]
    entries: Dict[str, Entry] = field(default_factory=dict)


class _Reader:
    def __init__(self, buf: bytes):
        self.buf, self.at = memoryview(buf), 0

    def take(self, n: int) -> memoryview:
        if self.at + n > len(self.buf):
            raise ValueError("container is truncated at byte %d" % self.at)
        out = self.buf[self.at:self.at + n]
        self.at += n
        return out

    def size(self) -> int:
        return struct.unpack("<Q", self.take(8))[0]


def read(path: str) -> Container:
    """Reads any of the three containers; the header says which."""
    with open(path, "rb") as f:
        r = _Reader(f.read())
    for header, (kind, n_polys, has_count) in _KINDS.items():
        if bytes(r.buf[:len(header)]) == header:
            r.take(len(header))
            break
    else:
        raise ValueError("%s: not a Cerium container (unknown header)" % path)
    n = r.size()
    n_primes = r.size()
    primes = list(struct.unpack("<%dQ" % n_primes, r.take(8 * n_primes)))
    n_entries = r.size()
    payload = r.size()
    out = Container(kind, n, primes)
    words = 0
    for _ in range(n_entries):
        id_len = r.size()
        raw = bytes(r.take(id_len))
        if not raw or raw[-1] != 0:
            raise ValueError("entry name is not NUL-terminated")
        name = raw[:-1].decode()
        n_limbs = r.size()
        count = r.size() if has_count else n
        polys = []
        for _p in range(n_polys):
            limbs = []
            for _l in range(n_limbs):
                lid = r.size()
                limbs.append((lid, np.frombuffer(r.take(4 * count), dtype="<u4").copy()))
                words += count
            polys.append(limbs)
        out.entries[name] = Entry(name, polys)
    if payload != 4 * words:
        raise ValueError("payload size in the header (%d) differs from the limbs read (%d)" % (payload, 4 * words))
    if r.at != len(r.buf):
        raise ValueError("%d trailing bytes after the last entry" % (len(r.buf) - r.at))
    return out


def write(path: str, c: Container) -> None:
    """Writes a container in the reference's layout (entries in insertion order)."""
    header = {k: h for h, (k, _, _) in _KINDS.items()}[c.kind]
    _, n_polys, has_count = _KINDS[header]
    words = sum(len(limb) for e in c.entries.values() for p in e.polys for _, limb in p)
    with open(path, "wb") as f:
        f.write(header)
        f.write(struct.pack("<QQ", c.n, len(c.primes)))
        f.write(struct.pack("<%dQ" % len(c.primes), *c.primes))
        f.write(struct.pack("<QQ", len(c.entries), 4 * words))
        for e in c.entries.values():
            if len(e.polys) != n_polys:
                raise ValueError("%s: %d polynomials, the %s container holds %d" % (e.name, len(e.polys), c.kind, n_polys))
            raw = e.name.encode() + b"\0"
            f.write(struct.pack("<Q", len(raw)))
            f.write(raw)
            n_limbs = len(e.polys[0])
            f.write(struct.pack("<Q", n_limbs))
            count = len(e.polys[0][0][1]) if n_limbs else c.n
            if has_count:
                f.write(struct.pack("<Q", count))
            elif count != c.n:
                raise ValueError("%s: evaluation-key limbs hold n words" % e.name)
            for p in e.polys:
                if len(p) != n_limbs:
                    raise ValueError("%s: polynomials with different limb counts" % e.name)
                for lid, limb in p:
                    if len(limb) != count:
                        raise ValueError("%s: limbs of different sizes" % e.name)
                    f.write(struct.pack("<Q", lid))
                    f.write(np.ascontiguousarray(limb, dtype="<u4").tobytes())


def parse_evalkey_id(name: str):
    """"<type>:<level>:<ext>:<rot>:[a,b,...]" -> (type, level, ext, rot, [digit limbs])."""
    head, _, digits = name.partition(":[")
    t, level, ext, rot = head.split(":")
    limbs = [int(x) for x in digits.rstrip("]").replace(",", " ").split()] if digits else []
    return int(t), int(level), int(ext), int(rot), limbs


def evalkey_tensor(c: Container, key_type: int, level: int, ext: int, rot: int,
                   limb_order: Sequence[int]) -> np.ndarray:
    """The key (type, level, ext, rot) as [digit][2][len(limb_order)][n] uint32, digits ordered by their
    first limb, limbs in `limb_order` (the plan's Q primes followed by its extension primes)."""
    if c.kind != "evalkeys":
        raise ValueError("not an evaluation-key container")
    digits = []
    for name, e in c.entries.items():
        t, lv, ex, ro, dl = parse_evalkey_id(name)
        if (t, lv, ex, ro) == (key_type, level, ext, rot):
            digits.append((min(dl) if dl else 0, e))
    if not digits:
        raise KeyError("no evaluation key %d:%d:%d:%d in the container" % (key_type, level, ext, rot))
    digits.sort(key=lambda d: d[0])
    return np.stack([np.stack([e.stack(0, limb_order), e.stack(1, limb_order)]) for _, e in digits])
