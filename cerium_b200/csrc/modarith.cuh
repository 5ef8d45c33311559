// Word-generic modular arithmetic for RNS limbs (uint32_t with primes below 2^30,
// uint64_t with primes below 2^62).  Integer multiply/add throughout, except the transforms of
// 64-bit primes below 2^50, whose butterflies run exactly on the FP64 pipe (see "double-precision
// modular arithmetic" below); there is no tensor-core use on this path.
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

// Programmatic dependent launch: every kernel of this library is launched with stream
// serialisation relaxed, so the next kernel's CTAs are placed (and read their constant tables)
// while the last CTAs of this one drain.  grid_dependency_launch() lets the next kernel start
// being placed; grid_dependency_wait() returns once every earlier kernel of the stream has
// completed and its writes are visible.  EVERY kernel must call the wait before it touches a
// buffer another kernel may have written or may still read.
__device__ __forceinline__ void grid_dependency_launch() {
#if !defined(CERIUM_EMU)
  asm volatile("griddepcontrol.launch_dependents;");
#endif
}
__device__ __forceinline__ void grid_dependency_wait() {
#if !defined(CERIUM_EMU)
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}

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
  W lazy_ok;     // 1 when q < 2^52 (64-bit words only): butterflies may skip range corrections
  // 64-bit words, q < 2^50: constants of the double-precision butterflies, as bit patterns of doubles
  W fp_ok;        // 1 when the transforms of this prime run on the FP64 pipe
  W fp_qinv;      // RN(1 / q)
  W fp_ninv;      // N^-1 mod q, centred in (-q/2, q/2)
  W fp_ninv_q;    // RN(fp_ninv / q)
  W fp_w1ninv;    // psi^-(N/2) * N^-1 mod q, centred
  W fp_w1ninv_q;  // RN(fp_w1ninv / q)
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
  W hi_, lo_;
  __device__ __forceinline__ void clear() { hi_ = 0; lo_ = 0; }
  __device__ __forceinline__ void mad(W a, W b) {
    W pl = a * b;
    W ph = WordTraits<W>::mulhi(a, b);
    lo_ += pl;
    hi_ += ph + (lo_ < pl ? (W)1 : (W)0);
  }
  __device__ __forceinline__ W hi() const { return hi_; }
  __device__ __forceinline__ W lo() const { return lo_; }
};
// 32-bit words: the two words are one 64-bit register pair and a term is a single IMAD.WIDE.
template <>
struct Acc2<uint32_t> {
  uint64_t v;
  __device__ __forceinline__ void clear() { v = 0; }
  __device__ __forceinline__ void mad(uint32_t a, uint32_t b) { v += (uint64_t)a * b; }
  __device__ __forceinline__ uint32_t hi() const { return (uint32_t)(v >> 32); }
  __device__ __forceinline__ uint32_t lo() const { return (uint32_t)v; }
};

// ---------------------------------------------------------------------------------------
// 64-bit fast path.  On sm_100 a 32-bit IMAD / IMAD.WIDE issues at half rate (64 lanes per
// SM per clock) and a 64-bit butterfly is bound by that pipe plus the carry/compare/select
// instructions around it, so the products are spelled out in 32-bit pieces:
//   mulhi_approx64  3 wide multiplies instead of the 4 (+ carries) of mul.hi.u64; drops the
//                   low partial product, so it returns floor(a*b / 2^64) - e with e in {0,1,2}
//   lo_madd64       low 64 bits of x*w + h*nq as 2 wide multiply-adds + 4 mad.lo, no carries
// A Shoup product built from them is x*w mod q in [0, 4q) for any 64-bit x.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint64_t mulhi_approx64(uint64_t a, uint64_t b) {
#if defined(CERIUM_EMU)
  const uint64_t a0 = (uint32_t)a, a1 = a >> 32, b0 = (uint32_t)b, b1 = b >> 32;
  return a1 * b1 + ((a0 * b1) >> 32) + ((a1 * b0) >> 32);
#else
  uint32_t a0, a1, b0, b1;
  asm("mov.b64 {%0,%1}, %2;" : "=r"(a0), "=r"(a1) : "l"(a));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(b0), "=r"(b1) : "l"(b));
  uint64_t t, u, h;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(t) : "r"(a0), "r"(b1));
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(u) : "r"(a1), "r"(b0));
  asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(h) : "r"(a1), "r"(b1), "l"(t >> 32));
  return h + (u >> 32);
#endif
}

__device__ __forceinline__ uint64_t lo_madd64(uint64_t x, uint64_t w, uint64_t h, uint64_t nq) {
#if defined(CERIUM_EMU)
  return x * w + h * nq;
#else
  uint32_t x0, x1, w0, w1, h0, h1, n0, n1, lo, hi;
  asm("mov.b64 {%0,%1}, %2;" : "=r"(x0), "=r"(x1) : "l"(x));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(w0), "=r"(w1) : "l"(w));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(h0), "=r"(h1) : "l"(h));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(n0), "=r"(n1) : "l"(nq));
  uint64_t acc;
  asm("mul.wide.u32 %0, %1, %2;" : "=l"(acc) : "r"(x0), "r"(w0));
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(acc) : "r"(h0), "r"(n0));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(lo), "=r"(hi) : "l"(acc));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(x0), "r"(w1));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(x1), "r"(w0));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(h0), "r"(n1));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(h1), "r"(n0));
  uint64_t r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
#endif
}

// x*w mod q in [0, 4q) for any 64-bit x; nq = 2^64 - q.
__device__ __forceinline__ uint64_t mul_shoup_approx(uint64_t x, uint64_t w, uint64_t ws, uint64_t nq) {
  return lo_madd64(x, w, mulhi_approx64(x, ws), nq);
}
// 32-bit words have no fast path: the exact product (in [0, 2q)) stands in.
__device__ __forceinline__ uint32_t mul_shoup_approx(uint32_t x, uint32_t w, uint32_t ws, uint32_t nq) {
  return x * w + __umulhi(x, ws) * nq;
}

// Lazy butterflies (primes below 2^52): no range correction inside a pass.
//   forward: inputs below B -> outputs below B + 4q           (B <= 61q keeps 16 layers exact)
//   inverse: layer k of a pass takes inputs below 4q * 2^k, c = 4q * 2^k keeps a - b positive;
//            sums double per layer, products come back below 4q
template <typename W>
__device__ __forceinline__ void butterfly_fwd_lazy(W& a, W& b, W w, W ws, W nq, W q4) {
  const W v = mul_shoup_approx(b, w, ws, nq);
  const W u = a;
  a = u + v;
  b = u + q4 - v;
}
template <typename W>
__device__ __forceinline__ void butterfly_inv_lazy(W& a, W& b, W w, W ws, W nq, W c) {
  const W d = a + c - b;
  a = a + b;
  b = mul_shoup_approx(d, w, ws, nq);
}
// any value -> [0, 4q): x - floor~(x / q) * q, the multiplication by 1 left out
__device__ __forceinline__ uint64_t reduce_lazy(uint64_t x, uint64_t one_shoup, uint64_t nq) {
  const uint64_t h = mulhi_approx64(x, one_shoup);
#if defined(CERIUM_EMU)
  return x + h * nq;
#else
  uint32_t h0, h1, n0, n1, lo, hi;
  asm("mov.b64 {%0,%1}, %2;" : "=r"(h0), "=r"(h1) : "l"(h));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(n0), "=r"(n1) : "l"(nq));
  uint64_t acc = x;
  asm("mad.wide.u32 %0, %1, %2, %0;" : "+l"(acc) : "r"(h0), "r"(n0));
  asm("mov.b64 {%0,%1}, %2;" : "=r"(lo), "=r"(hi) : "l"(acc));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(h0), "r"(n1));
  asm("mad.lo.u32 %0, %1, %2, %0;" : "+r"(hi) : "r"(h1), "r"(n0));
  uint64_t r;
  asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
#endif
}
__device__ __forceinline__ uint32_t reduce_lazy(uint32_t x, uint32_t one_shoup, uint32_t nq) {
  return x + __umulhi(x, one_shoup) * nq;
}

// ---------------------------------------------------------------------------------------
// Double-precision modular arithmetic (primes below 2^50).
//
// B200 issues FP64 multiply-adds at the rate of 32-bit integer multiply-adds, on a pipe of their
// own, and a 64-bit modular product costs 6 of them against 9 integer multiply-adds plus the
// carries; the butterflies of the transforms therefore run on doubles holding exact integers.
// Values are signed residues |x| <= B*q with B < 8 (so every sum is an exact integer below 2^53);
// twiddles are centred, |w| < q/2, and come with wq = RN(w / q).
//
//   fp_mulmod(y, w, wq):  h = RN(y*w), l = y*w - h (exact, one FMA), c = RN(y*wq) by the
//   2^52-magic addition (needs |y*wq| <= 2^51, i.e. |y| <= 4q), r = (h - c*q) + l.  h - c*q is an
//   integer below 2^53 in magnitude, hence exact, and so is the last sum: r = y*w - c*q exactly,
//   with |c - y*w/q| <= 1/2 + |y| * 2^-55, i.e.  |r| <= q * (1/2 + B/32)  for |y| <= B*q.
//   fp_reduce(x) is the same with w = 1: |r| <= q * (1/2 + 2^-50).
// A host-side plan (ntt_kernels.cuh) tracks B through the layers and places the reductions.
// ---------------------------------------------------------------------------------------
constexpr double kFpMagic = 6755399441055744.0;  // 1.5 * 2^52
constexpr double kFpTwo52 = 4503599627370496.0;  // 2^52

__device__ __forceinline__ double fp_mulmod(double y, double w, double wq, double nq) {
  const double h = __dmul_rn(y, w);
  const double l = __fma_rn(y, w, -h);
  const double c = __dadd_rn(__fma_rn(y, wq, kFpMagic), -kFpMagic);
  return __dadd_rn(__fma_rn(c, nq, h), l);
}
__device__ __forceinline__ double fp_reduce(double x, double qinv, double nq) {
  const double c = __dadd_rn(__fma_rn(x, qinv, kFpMagic), -kFpMagic);
  return __fma_rn(c, nq, x);
}
// integer in [0, 2^52) <-> double, through the mantissa of 2^52 + x
__device__ __forceinline__ double fp_from_u64(uint64_t x) {
  return __dadd_rn(__longlong_as_double((long long)(x | 0x4330000000000000ull)), -kFpTwo52);
}
__device__ __forceinline__ uint64_t fp_to_u64(double x) {
  return (uint64_t)__double_as_longlong(__dadd_rn(x, kFpTwo52)) & 0x000fffffffffffffull;
}

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

// NTT-domain Galois automorphism out[i] = in[pi(i)] with
//   pi(i) = brev16( ((elt * (2*brev16(i) + 1)) >> 1) & (N-1) )
// (cerium/runtime/math/galois.cpp:30-62 builds this as a table; the reference kernels scatter
// through its inverse, cerium/compiler/backend/cuda_kernel.cc:228-300).  The map sends every
// aligned block of 2^k indices onto an aligned block of 2^k indices, so a warp's 32 gathered
// words always come from one aligned 32-word segment: the gather is sector-exact without a
// table and without staging.
__device__ __forceinline__ uint32_t galois_source_index(uint32_t i, uint32_t elt) {
  const uint32_t r = (__brev(i) >> (32 - kLogN)) * 2u + 1u;
  const uint32_t raw = ((elt * r) >> 1) & (uint32_t)(kN - 1);
  return __brev(raw) >> (32 - kLogN);
}


}  // namespace cerium
