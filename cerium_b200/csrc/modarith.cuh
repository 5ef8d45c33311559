// Word-generic modular arithmetic for RNS limbs (uint32_t with primes below 2^30,
// uint64_t with primes below 2^62).  Device code only uses integer multiply/add;
// there is no floating point and no tensor-core use on this path.
//
// Replaces cerium/compiler/backend/kernels/fhe_arith.cuh:28-193 (32-bit Barrett with
// k = 58, lazy products below q^2) and the Shoup butterfly helpers of
// cerium/compiler/backend/kernels/fhe_ntt.cuh:68-88,380-392.  Unlike the reference,
// every value that leaves a kernel is canonical, i.e. in [0, q).
#pragma once
#include <cstdint>

#if defined(CERIUM_EMU)
#include "emu_cuda.h"  // host stand-ins for the CUDA built-ins (kernel-logic tests on CPU)
#else
#include <cuda_runtime.h>
#endif

// Dynamic shared memory of the running CTA as a byte pointer.
#if defined(CERIUM_EMU)
#define CERIUM_DYN_SMEM(name) unsigned char* name = cerium_emu::dyn_smem()
#else
#define CERIUM_DYN_SMEM(name) extern __shared__ __align__(16) unsigned char name[]
#endif

namespace cerium {

constexpr int kLogN = 16;
constexpr int kN = 1 << kLogN;

template <typename W>
struct WordTraits;

template <>
struct WordTraits<uint32_t> {
  using Pair = uint2;  // {w, floor(w * 2^32 / q)}
  static constexpr int kBits = 32;
  static __device__ __forceinline__ uint32_t mulhi(uint32_t a, uint32_t b) { return __umulhi(a, b); }
  static __host__ __device__ __forceinline__ Pair make(uint32_t a, uint32_t b) { return make_uint2(a, b); }
};

template <>
struct WordTraits<uint64_t> {
  using Pair = ulonglong2;  // {w, floor(w * 2^64 / q)}
  static constexpr int kBits = 64;
  static __device__ __forceinline__ uint64_t mulhi(uint64_t a, uint64_t b) { return __umul64hi(a, b); }
  static __host__ __device__ __forceinline__ Pair make(uint64_t a, uint64_t b) {
    return make_ulonglong2(a, b);
  }
};

// Per-prime constants, one entry per modulus of the context, resident in global
// memory (read through the read-only path; every thread of a CTA reads the same entry).
template <typename W>
struct PrimeConst {
  W q;           // modulus
  W q2;          // 2q
  W mu_hi;       // floor(2^(2B) / q), high word
  W mu_lo;       //                    low word
  W one_shoup;   // floor(2^B / q): Shoup companion of 1
  W ninv;        // N^-1 mod q
  W ninv_shoup;  //
  W w1ninv;      // psi^-(N/2) * N^-1 mod q  (inverse twiddle of index 1 times N^-1)
  W w1ninv_shoup;
  W pad[7];
};

// x * w mod q in [0, 2q) for ANY word x, given ws = floor(w * 2^B / q) with w < q.
template <typename W>
__device__ __forceinline__ W mul_shoup_lazy(W x, W w, W ws, W q) {
  return x * w - WordTraits<W>::mulhi(x, ws) * q;
}

template <typename W>
__device__ __forceinline__ W csub(W x, W q) {
  return x >= q ? x - q : x;
}

// Any word -> [0, q) through a Shoup product with 1.
template <typename W>
__device__ __forceinline__ W reduce_word(W x, const PrimeConst<W>& pc) {
  return csub(mul_shoup_lazy<W>(x, (W)1, pc.one_shoup, pc.q), pc.q);
}

// Barrett reduction of the two-word value hi*2^B + lo (any value below 2^(2B)) to [0, q).
// qhat = hi*mu_hi + hi32(lo*mu_hi) + hi32(hi*mu_lo) underestimates floor(x/q) by at most 3,
// and only its low word matters for the low word of x - qhat*q, which is < 4q < 2^B.
template <typename W>
__device__ __forceinline__ W barrett2(W hi, W lo, const PrimeConst<W>& pc) {
  W qhat = hi * pc.mu_hi + WordTraits<W>::mulhi(lo, pc.mu_hi) + WordTraits<W>::mulhi(hi, pc.mu_lo);
  W r = lo - qhat * pc.q;
  r = csub(r, pc.q2);
  return csub(r, pc.q);
}

template <typename W>
__device__ __forceinline__ W mul_mod(W a, W b, const PrimeConst<W>& pc) {
  return barrett2<W>(WordTraits<W>::mulhi(a, b), a * b, pc);
}

template <typename W>
__device__ __forceinline__ W add_mod(W a, W b, W q) {
  return csub<W>(a + b, q);
}

template <typename W>
__device__ __forceinline__ W sub_mod(W a, W b, W q) {
  return a >= b ? a - b : a + q - b;
}

// Two-word accumulator: acc += a * b (no reduction; caller bounds the number of terms).
template <typename W>
struct Acc2 {
  W hi, lo;
  __device__ __forceinline__ void clear() { hi = 0; lo = 0; }
  __device__ __forceinline__ void mad(W a, W b) {
    W pl = a * b;
    W ph = WordTraits<W>::mulhi(a, b);
    lo += pl;
    hi += ph + (lo < pl ? (W)1 : (W)0);
  }
  __device__ __forceinline__ void add_word(W a) {
    lo += a;
    hi += (lo < a ? (W)1 : (W)0);
  }
};

// Harvey forward butterfly: a, b in [0, 4q) -> [0, 4q).
template <typename W>
__device__ __forceinline__ void butterfly_fwd(W& a, W& b, W w, W ws, W q, W q2) {
  W u = csub<W>(a, q2);
  W v = mul_shoup_lazy<W>(b, w, ws, q);
  a = u + v;
  b = u + q2 - v;
}

// Gentleman-Sande inverse butterfly: a, b in [0, 2q) -> [0, 2q).
template <typename W>
__device__ __forceinline__ void butterfly_inv(W& a, W& b, W w, W ws, W q, W q2) {
  W s = csub<W>(a + b, q2);
  W d = a + q2 - b;
  a = s;
  b = mul_shoup_lazy<W>(d, w, ws, q);
}

}  // namespace cerium
