// Host-side number theory for building the device tables: modular inverse, minimal
// primitive 2N-th root, bit-reversed twiddle tables with Shoup companions, Barrett
// constants, CRT factors for base conversion.
//
// Replaces the SEAL-backed table construction of
// cerium/runtime/execution/evaluator.cpp:58-231 (EvaluatorContext::init_params /
// init_ntt_params) and cerium/runtime/math/ntt.cpp:99-149.  The reference permutes its
// tables for its own radix-4/radix-8 access pattern (evaluator.cpp:93-113,199-210); these
// tables stay in plain bit-reversed order: entry brev(i) holds psi^i.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <vector>

namespace cerium {
namespace host {

using u64 = uint64_t;
using u128 = unsigned __int128;

inline u64 mulmod(u64 a, u64 b, u64 q) { return (u64)(((u128)a * b) % q); }

inline u64 powmod(u64 a, u64 e, u64 q) {
  u64 r = 1 % q;
  a %= q;
  for (; e; e >>= 1) {
    if (e & 1) r = mulmod(r, a, q);
    a = mulmod(a, a, q);
  }
  return r;
}

// Extended Euclid; returns 0 if a is not invertible mod q.
inline u64 invmod(u64 a, u64 q) {
  __int128 t = 0, nt = 1, r = q, nr = a % q;
  while (nr != 0) {
    __int128 k = r / nr;
    __int128 tmp = t - k * nt;
    t = nt;
    nt = tmp;
    tmp = r - k * nr;
    r = nr;
    nr = tmp;
  }
  if (r != 1) return 0;
  if (t < 0) t += q;
  return (u64)t;
}

inline bool is_prime(u64 n) {
  static const u64 bases[] = {2, 3, 5, 7, 11, 13, 17, 19, 23, 29, 31, 37};
  if (n < 2) return false;
  for (u64 b : bases)
    if (n % b == 0) return n == b;
  u64 d = n - 1;
  int s = 0;
  while (!(d & 1)) {
    d >>= 1;
    s++;
  }
  for (u64 b : bases) {
    u64 x = powmod(b, d, n);
    if (x == 1 || x == n - 1) continue;
    bool composite = true;
    for (int r = 1; r < s && composite; r++) {
      x = mulmod(x, x, n);
      if (x == n - 1) composite = false;
    }
    if (composite) return false;
  }
  return true;
}

inline uint32_t brev(uint32_t x, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++) {
    r = (r << 1) | (x & 1);
    x >>= 1;
  }
  return r;
}

// Smallest primitive 2N-th root of unity mod q (the root SEAL's
// try_minimal_primitive_root yields, used at evaluator.cpp:140); 0 if none exists.
inline u64 minimal_primitive_root(u64 q, int logn) {
  const u64 two_n = (u64)2 << logn;
  if ((q - 1) % two_n) return 0;
  const u64 e = (q - 1) / two_n;
  u64 r = 0;
  for (u64 g = 2; g < q; g++) {
    u64 c = powmod(g, e, q);
    if (powmod(c, two_n >> 1, q) == q - 1) {
      r = c;
      break;
    }
  }
  if (!r) return 0;
  const u64 sq = mulmod(r, r, q);
  u64 cur = r, best = r;
  for (u64 i = 0; i < (two_n >> 1); i++) {
    if (cur < best) best = cur;
    cur = mulmod(cur, sq, q);
  }
  return best;
}

// floor(w * 2^bits / q)
inline u64 shoup(u64 w, u64 q, int bits) { return (u64)((((u128)w) << bits) / q); }

struct PrimeTables {
  u64 q = 0, psi = 0, psi_inv = 0, ninv = 0, two_inv = 0;
  u64 mu_hi = 0, mu_lo = 0;       // floor(2^(2*bits) / q)
  std::vector<u64> w, wi;         // bit-reversed powers of psi and of psi^-1
};

inline PrimeTables build_prime_tables(u64 q, int logn, int bits) {
  PrimeTables t;
  const size_t n = (size_t)1 << logn;
  t.q = q;
  t.psi = minimal_primitive_root(q, logn);
  if (!t.psi) throw std::invalid_argument("modulus is not a prime congruent to 1 mod 2N");
  t.psi_inv = invmod(t.psi, q);
  t.ninv = invmod((u64)n % q, q);
  if (bits == 64) {
    const u128 mu = (~(u128)0) / q;  // q is odd, so this is floor(2^128 / q)
    t.mu_hi = (u64)(mu >> 64);
    t.mu_lo = (u64)mu;
  } else {
    const u64 mu = ~(u64)0 / q;
    t.mu_hi = mu >> 32;
    t.mu_lo = mu & 0xffffffffu;
  }
  t.w.resize(n);
  t.wi.resize(n);
  u64 p = 1, pi = 1;
  for (size_t i = 0; i < n; i++) {
    const uint32_t r = brev((uint32_t)i, logn);
    t.w[r] = p;
    t.wi[r] = pi;
    p = mulmod(p, t.psi, q);
    pi = mulmod(pi, t.psi_inv, q);
  }
  return t;
}

// prod_{k in idx} moduli[k] mod q
inline u64 product_mod(const std::vector<u64>& moduli, const std::vector<uint32_t>& idx, u64 q) {
  u64 p = 1 % q;
  for (uint32_t k : idx) p = mulmod(p, moduli[k] % q, q);
  return p;
}

}  // namespace host
}  // namespace cerium
