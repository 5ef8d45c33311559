"""Minimal CKKS encode / keygen / encrypt / decrypt in numpy, used only by tests to check that
key switching, rotation and multiplication are *cryptographically* right (decrypted slots), not
just equal between the oracle and the kernels.

Follows the reference's key material layout: evaluation key of digit d is an encryption of zero
under the secret key over the primes Q u P whose first polynomial gets [P]_{q_i} * s' added on the
limbs of digit d only (cerium/runtime/io/ckks-encryptor.cpp:534-599); ciphertext (c0, c1) with
c0 = -(c1*s) + e + m (cerium/runtime/io/ckks-encryptor.cpp:311-370); slot checks like
examples/common.py:134-142.  Transforms come from the CPU oracle.
"""
from __future__ import annotations

import numpy as np

import oracle


class CkksRef:
    def __init__(self, prm, seed=10, hamming_weight=192, sigma=3.2):
        self.prm = prm
        self.n = prm.n
        self.logn = prm.logn
        self.moduli = prm.moduli
        self.rng = np.random.default_rng(seed)
        self.sigma = sigma
        self.octx = oracle.OracleContext(prm.logn, prm.moduli)
        s = np.zeros(self.n, dtype=np.int64)
        pos = self.rng.choice(self.n, size=hamming_weight, replace=False)
        s[pos] = self.rng.choice([-1, 1], size=hamming_weight)
        self.s_coeff = s
        self.all_idx = list(prm.q_idx) + list(prm.p_idx)
        self.s_ntt = {p: self.octx.ntt_forward(self._signed_to_limb(s, p), [p])[0] for p in self.all_idx}
        # slot k of the canonical embedding sits at the odd exponent 5^k (and its conjugate at -5^k)
        m = 2 * self.n
        e = 1
        self.slot_pos = np.empty(self.n // 2, dtype=np.int64)
        self.conj_pos = np.empty(self.n // 2, dtype=np.int64)
        for k in range(self.n // 2):
            self.slot_pos[k] = (e - 1) // 2
            self.conj_pos[k] = (m - e - 1) // 2
            e = e * 5 % m

    # ---- helpers
    def _signed_to_limb(self, v, p):
        q = self.moduli[p]
        return np.mod(v.astype(object), q).astype(np.uint64) if v.dtype == object else np.mod(v, q).astype(np.uint64)

    def _uniform(self, idx):
        return np.stack([self.rng.integers(0, self.moduli[p], size=self.n, dtype=np.uint64) for p in idx])

    def _noise_ntt(self, idx):
        e = np.rint(self.rng.normal(0, self.sigma, size=self.n)).astype(np.int64)
        return np.stack([self.octx.ntt_forward(self._signed_to_limb(e, p), [p])[0] for p in idx])

    def _mul(self, a, b, idx):
        return np.stack([oracle.ew("mul", self.moduli[p], a[i], b[i]) for i, p in enumerate(idx)])

    def _add(self, a, b, idx):
        return np.stack([oracle.ew("add", self.moduli[p], a[i], b[i]) for i, p in enumerate(idx)])

    def _neg(self, a, idx):
        return np.stack([oracle.ew("neg", self.moduli[p], a[i]) for i, p in enumerate(idx)])

    # ---- encoding
    def encode(self, z, scale):
        """complex/real slots [n/2] -> integer coefficients (int64) of round(scale * m)."""
        n = self.n
        v = np.zeros(n, dtype=np.complex128)
        v[self.slot_pos] = z
        v[self.conj_pos] = np.conj(z)
        coeff = np.fft.fft(v) / n * np.exp(-1j * np.pi * np.arange(n) / n)
        v = np.rint(coeff.real * scale)
        return v.astype(np.int64) if scale < 2.0 ** 60 else np.array([int(x) for x in v], dtype=object)

    def decode(self, coeff_float, scale):
        n = self.n
        v = n * np.fft.ifft(coeff_float * np.exp(1j * np.pi * np.arange(n) / n))
        return v[self.slot_pos] / scale

    # ---- encryption
    def encrypt(self, z, scale):
        idx = list(self.prm.q_idx)
        m = self.encode(z, scale)
        m_ntt = np.stack([self.octx.ntt_forward(self._signed_to_limb(m, p), [p])[0] for p in idx])
        c1 = self._uniform(idx)
        s = np.stack([self.s_ntt[p] for p in idx])
        c0 = self._add(self._add(self._neg(self._mul(c1, s, idx), idx), self._noise_ntt(idx), idx), m_ntt, idx)
        return c0, c1

    def decrypt(self, c0, c1, scale, n_limbs=None, use=2):
        """Decrypts with the first `use` limbs (exact CRT, centred) and decodes."""
        L = c0.shape[0] if n_limbs is None else n_limbs
        idx = list(self.prm.q_idx)[:L]
        s = np.stack([self.s_ntt[p] for p in idx])
        m_ntt = self._add(c0[:L], self._mul(c1[:L], s, idx), idx)
        m = self.octx.ntt_inverse(m_ntt, idx)
        use = min(L, use)
        mods = [self.moduli[p] for p in idx[:use]]
        Q = 1
        for q in mods:
            Q *= q
        vals = np.zeros(self.n, dtype=object)
        for i, q in enumerate(mods):
            Qi = Q // q
            vals = (vals + m[i].astype(object) * (Qi * pow(Qi, -1, q))) % Q
        centred = np.where(vals > Q // 2, vals - Q, vals)
        return self.decode(centred.astype(np.float64), scale)

    # ---- evaluation keys: [dnum][2][L+K][N]
    def _evalkey(self, new_key_ntt):
        prm = self.prm
        idx = self.all_idx
        P = 1
        for p in prm.p_idx:
            P *= self.moduli[p]
        s = np.stack([self.s_ntt[p] for p in idx])
        out = []
        for d in range(prm.dnum):
            a = self._uniform(idx)
            b = self._add(self._neg(self._mul(a, s, idx), idx), self._noise_ntt(idx), idx)
            for i in range(prm.L):
                if i % prm.dnum == d:
                    q = self.moduli[idx[i]]
                    b[i] = oracle.ew("pmu", q, b[i], new_key_ntt[idx[i]], scalar=P % q)
            out.append(np.stack([b, a]))
        return np.stack(out)

    def rotation_key(self, galois_elt):
        rot = oracle.apply_galois_coeff(galois_elt, self.logn, 1 << 40, np.mod(self.s_coeff, 1 << 40).astype(np.uint64))
        signed = rot.astype(np.int64)
        signed[signed > (1 << 39)] -= (1 << 40)
        new_key = {p: self.octx.ntt_forward(self._signed_to_limb(signed, p), [p])[0] for p in self.all_idx}
        return self._evalkey(new_key)

    def relin_key(self):
        new_key = {p: oracle.ew("mul", self.moduli[p], self.s_ntt[p], self.s_ntt[p]) for p in self.all_idx}
        return self._evalkey(new_key)
