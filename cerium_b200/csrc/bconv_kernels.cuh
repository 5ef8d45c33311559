// Fast base conversion between RNS bases (ModUp / ModDown building block).
//
// Replaces convert<I,O> and its launcher (cerium/compiler/backend/kernels/fhe_bconv.cuh:98-151,
// cerium/compiler/backend/kernels/function.cuh:61-122) and the factor tables of
// DeviceBaseConverter::set_output_bases (cerium/runtime/execution/evaluator.cpp:1516-1608).
//
//   out_j[c] = ( sum_i y_i[c] * F[j][i] ) mod p_j,         c = 0..N-1
//
// "lazy" mode (the reference's): y_i = x_i and F[j][i] = [Qhat_i^-1]_{q_i} * Qhat_i mod p_j.
// "exact" mode: y_i = x_i * [Qhat_i^-1]_{q_i} mod q_i and F[j][i] = Qhat_i mod p_j.
// The mode only changes how the tables are filled and whether `inv` is non-null.
//
// One thread owns one coefficient: it reads the I input residues once (coalesced across the
// warp), keeps them in registers (I <= 8) or in its own shared-memory column (larger I), and
// streams over the O output primes with the factor matrix and the per-output constants
// broadcast from shared memory.  Sums are reduced once per output (primes below 2^60 leave
// room for 256 terms), instead of the reference's trims at i = 15, 30.
#pragma once
#include "modarith.cuh"

namespace cerium {

// 160 threads: with the kernel's ~70 registers five CTAs fit an SM (740 slots on 148 SMs), and the
// 7 x 410 CTAs of a ModUp over seven digits are 3.9 waves; 256-thread CTAs gave 4.04 waves of 444,
// i.e. a fifth wave of 16 CTAs
constexpr int kBconvThreads = 160;
constexpr int kBconvBlocks = (kN + kBconvThreads - 1) / kBconvThreads;  // the last block is partial
constexpr int kBconvRegInputs = 8;
// grid.z splits the output primes of a conversion when the batch alone gives too few CTAs

template <typename W>
struct BconvOut;

template <typename W>
struct BconvDesc {
  const W* in;             // I limbs, coefficient form
  W* out;                  // O limbs
  size_t in_stride;        // words between input limbs
  size_t out_stride;       // words between output limbs
  const W* factors;        // [O][I]
  const W* inv;            // [I] or null (lazy mode)
  const W* inv_shoup;      // [I]
  const W* in_add;         // [I] added to the inputs mod q_i (rounding), or null
  const W* out_sub;        // [O] subtracted from the outputs mod p_j (rounding), or null
  const uint32_t* in_prime;   // [I] prime index of each input limb
  const uint32_t* out_prime;  // [O]
  const uint32_t* out_pos;    // [O] limb slot of output j inside `out`, or null (slot j)
  const uint32_t* in_pos;     // [I] limb slot of input i inside `in`, or null (slot i)
  // tables built when the converter is created (device memory, never change): per-output constants,
  // and for the 64-bit split path the factors as 30-bit pieces and as double-precision pairs
  const BconvOut<W>* outc;    // [O]
  const uint2* split_fac;     // [O][I] or null
  const double2* fp_fac;      // [O][I] {bit pattern of the centred factor as int64, RN(centred factor / q)} or null
  int lazy_out;               // 64-bit split path only: leave outputs in [0, 8q) / [0, 4q) for the forward NTT
  int fp_in;                  // 64-bit split path only: fp_fac is present and some outputs take their quotient
                              // from the FP64 pipe (see bconv_body_split64)
  int I;
  int O;
};

// Per-output constants staged in shared memory next to the factor matrix, so the output loop
// has no dependent global loads.
template <typename W>
struct BconvOut {
  W q, q2, mu_hi, mu_lo, sub;  // sub = rounding term (0 when unused)
  W fp_qinv;                   // bit pattern of RN(1 / q) when fp is set
  uint32_t pos;                // limb slot of this output
  uint16_t has_sub;            // rounding term present
  uint8_t strict;              // the prime's transform needs inputs below 4q (all but the lazy integer butterflies)
  uint8_t fp;                  // 1 / 2: quotient estimated in double precision, without / with a second step
                               // (see bconv_body_split64); 0: integer Barrett path
};

// Barrett reduction with the 3-multiply high products: qhat may be up to 7 short, so the
// remainder lies in [0, 8q) (q < 2^60) and takes three conditional subtractions.
__device__ __forceinline__ uint64_t barrett2_fast(uint64_t hi, uint64_t lo, uint64_t q, uint64_t q2, uint64_t mu_hi,
                                                  uint64_t mu_lo) {
  const uint64_t qhat = hi * mu_hi + mulhi_approx64(lo, mu_hi) + mulhi_approx64(hi, mu_lo);
  uint64_t r = lo - qhat * q;
  r = csub<uint64_t>(r, q2 + q2);
  r = csub<uint64_t>(r, q2);
  return csub<uint64_t>(r, q);
}

// rounding term and [Qhat_i^-1] applied to a residue of input i as it is read
template <typename W>
__device__ __forceinline__ W bconv_prepare(const BconvDesc<W>& d, const PrimeConst<W>* __restrict__ pcs, int i, W v) {
  if (d.in_add != nullptr || d.inv != nullptr) {
    const W qi = pcs[d.in_prime[i]].q;
    if (d.in_add != nullptr) v = add_mod<W>(v, d.in_add[i], qi);
    if (d.inv != nullptr) v = csub<W>(mul_shoup_lazy<W>(v, d.inv[i], d.inv_shoup[i], qi), qi);
  }
  return v;
}

template <typename W>
__device__ __forceinline__ W bconv_input(const BconvDesc<W>& d, const PrimeConst<W>* __restrict__ pcs, int i,
                                         int coeff) {
  return bconv_prepare<W>(d, pcs, i,
                          d.in[(size_t)(d.in_pos != nullptr ? d.in_pos[i] : (uint32_t)i) * d.in_stride + coeff]);
}

// 64-bit words, at most 8 inputs.
//
// Outputs flagged `fp` take the quotient from the FP64 pipe and the remainder from wrapping 64-bit
// integer arithmetic: with S = sum_i y_i * f_i (f_i the factor centred in (-q/2, q/2]) the kernel
// estimates c ~ S / q as the double-precision sum of y_i * RN(f_i / q), one FMA per term, rounds it to
// an integer and forms r = S - c q modulo 2^64 (three IMAD per 64-bit product, no high words, no
// carries).  r is the exact value of S - c q whenever |S - c q| < 2^63, i.e. whenever the estimate's
// error e satisfies (e + 1) q < 2^63; the host bounds e per output when the converter is created
// ((I + 2) 2^-53 sum_i q_i |f_i| / q) and sets fp = 1 when |r| < 3q is guaranteed (50-bit inputs:
// e < 2.5), fp = 2 when a second quotient step is needed (60-bit inputs into 50-bit outputs:
// |r| < 2^62; c2 = rint(r / q) in double precision, r -= c2 q), fp = 0 when neither holds (60-bit
// inputs into 60-bit outputs).  5 FMA + 18 IMAD + two conversions per 5-term output instead of 41
// FP64 operations (exact products on the FP64 pipe) or ~120 integer instructions (Barrett on a
// 128-bit sum).  sfp holds {bit pattern of the centred factor as int64, RN(factor / q)} per (output, input).
//
// Outputs with fp = 0: residues and factors are split at bit 30 so that every partial product is a
// 32x32->64 multiply-add into one of three column sums (y0*f0, y0*f1 + y1*f0, y1*f1).  With pieces
// below 2^30 and at most 8 terms no column overflows, so a multiply-accumulate is four IMAD.WIDE and
// no carry handling; one Barrett reduction of the 128-bit sum follows.
template <int kI, bool kLazyOut>  // kI = exact number of inputs, 1..8
__device__ __forceinline__ void bconv_body_split64(const BconvDesc<uint64_t>& d,
                                                   const PrimeConst<uint64_t>* __restrict__ pcs,
                                                   const uint2* sfac, const BconvOut<uint64_t>* sout,
                                                   const double2* sfp, int coeff) {
  const int O = d.O;
  uint64_t y[kI];
  double yd[kI];
#pragma unroll
  for (int i = 0; i < kI; i++) {
    y[i] = bconv_input<uint64_t>(d, pcs, i, coeff);
    yd[i] = d.fp_in ? __ull2double_rn(y[i]) : 0.0;
  }
#pragma unroll 2
  for (int j = 0; j < O; j++) {
    if (sout[j].fp) {
      const BconvOut<uint64_t> o = sout[j];
      const double2* f = sfp + j * kI;
      double cf = __dmul_rn(yd[0], f[0].y);
      uint64_t s = y[0] * (uint64_t)__double_as_longlong(f[0].x);
#pragma unroll
      for (int i = 1; i < kI; i++) {
        cf = __fma_rn(yd[i], f[i].y, cf);
        s += y[i] * (uint64_t)__double_as_longlong(f[i].x);
      }
      long long r = (long long)(s - (uint64_t)__double2ll_rn(cf) * o.q);
      if (kLazyOut && o.fp == 1) {
        // |r| < 3q: [0, 3q) is as good as [0, q) for the forward transform that follows
        if (r < 0) r += (long long)(o.q2 + o.q);
      } else {
        const long long c2 = __double2ll_rn(__dmul_rn(__ll2double_rn(r), __longlong_as_double((long long)o.fp_qinv)));
        r -= c2 * (long long)o.q;  // within q/2 of zero (and a rounding sliver)
        if (r < 0) r += (long long)o.q;
        if (o.has_sub) r = (long long)sub_mod<uint64_t>((uint64_t)r, o.sub, o.q);
      }
      d.out[(size_t)o.pos * d.out_stride + coeff] = (uint64_t)r;
      continue;
    }
    const uint2* f = sfac + j * kI;
    uint64_t c0 = 0, c1 = 0, c2 = 0;
#pragma unroll
    for (int i = 0; i < kI; i++) {
      const uint2 fi = f[i];
      const uint32_t y0 = (uint32_t)y[i] & 0x3fffffffu, y1 = (uint32_t)(y[i] >> 30);
      c0 += (uint64_t)y0 * fi.x;
      c1 += (uint64_t)y0 * fi.y;
      c1 += (uint64_t)y1 * fi.x;
      c2 += (uint64_t)y1 * fi.y;
    }
    // value = c0 + c1 * 2^30 + c2 * 2^60 as hi:lo (128-bit adds: carry chains, no compares)
#if defined(CERIUM_EMU)
    const unsigned __int128 v128 = (unsigned __int128)c0 + ((unsigned __int128)c1 << 30) + ((unsigned __int128)c2 << 60);
    const uint64_t lo = (uint64_t)v128, hi = (uint64_t)(v128 >> 64);
#else
    uint64_t lo, hi;
    {
      const uint64_t t1l = c1 << 30, t1h = c1 >> 34, t2l = c2 << 60, t2h = c2 >> 4;
      asm("add.cc.u64 %0, %2, %3;\n\taddc.u64 %1, %4, 0;" : "=l"(lo), "=l"(hi) : "l"(c0), "l"(t1l), "l"(t1h));
      asm("add.cc.u64 %0, %0, %2;\n\taddc.u64 %1, %1, %3;" : "+l"(lo), "+l"(hi) : "l"(t2l), "l"(t2h));
    }
#endif
    const BconvOut<uint64_t> o = sout[j];
    uint64_t r;
    if (kLazyOut) {
      // consumer is the forward transform: [0, 8q) is fine for lazy integer butterflies, the others take [0, 4q)
      const uint64_t qhat = hi * o.mu_hi + mulhi_approx64(lo, o.mu_hi) + mulhi_approx64(hi, o.mu_lo);
      r = lo - qhat * o.q;
      if (o.strict) r = csub<uint64_t>(r, o.q2 + o.q2);
    } else {
      r = barrett2_fast(hi, lo, o.q, o.q2, o.mu_hi, o.mu_lo);
      if (o.has_sub) r = sub_mod<uint64_t>(r, o.sub, o.q);
    }
    d.out[(size_t)o.pos * d.out_stride + coeff] = r;
  }
}

// Generic path (32-bit words, or more than 8 inputs): two-word accumulator, one Barrett
// reduction per output; inputs in registers (kRegI > 0) or in the thread's shared-memory column.
template <typename W, int kRegI>
__device__ __forceinline__ void bconv_body(const BconvDesc<W>& d, const PrimeConst<W>* __restrict__ pcs,
                                           const W* sfac, const BconvOut<W>* sout, W* scol, int coeff) {
  const int tid = threadIdx.x;
  const int I = kRegI > 0 ? kRegI : d.I, O = d.O;  // kRegI > 0: exact number of inputs
  W y[kRegI > 0 ? kRegI : 1];
  if (kRegI > 0) {
#pragma unroll
    for (int i = 0; i < kRegI; i++) y[i] = bconv_input<W>(d, pcs, i, coeff);
  } else {
    for (int i = 0; i < I; i++) scol[i * kBconvThreads + tid] = bconv_input<W>(d, pcs, i, coeff);
  }
#pragma unroll 2
  for (int j = 0; j < O; j++) {
    const W* f = sfac + j * I;
    W acc_hi, acc_lo;
    if (sizeof(W) == 4 && kRegI > 0) {
      // 32-bit words, at most 8 terms below 2^60 each: the sum fits one 64-bit register, so a
      // multiply-accumulate is a single wide multiply-add
      uint64_t a64 = 0;
#pragma unroll
      for (int i = 0; i < kRegI; i++) a64 += (uint64_t)y[i] * (uint64_t)f[i];
      acc_hi = (W)(a64 >> 32);
      acc_lo = (W)a64;
    } else {
      Acc2<W> acc;
      acc.clear();
      if (kRegI > 0) {
#pragma unroll
        for (int i = 0; i < kRegI; i++) acc.mad(y[i], f[i]);
      } else {
        for (int i = 0; i < I; i++) acc.mad(scol[i * kBconvThreads + tid], f[i]);
      }
      acc_hi = acc.hi();
      acc_lo = acc.lo();
    }
    const BconvOut<W> o = sout[j];
    PrimeConst<W> pc;
    pc.q = o.q;
    pc.q2 = o.q2;
    pc.mu_hi = o.mu_hi;
    pc.mu_lo = o.mu_lo;
    W r = barrett2<W>(acc_hi, acc_lo, pc);
    if (o.has_sub) r = sub_mod<W>(r, o.sub, o.q);
    d.out[(size_t)o.pos * d.out_stride + coeff] = r;
  }
}

// 32-bit words, at most 8 inputs, every limb 8-byte aligned: a thread converts the two coefficients
// coeff, coeff + 1 (coeff even) with 8-byte loads and stores, so the factor row and the output's
// constants are fetched from shared memory once per pair; the sum of at most 8 products below 2^60
// fits one 64-bit register (a multiply-accumulate is one wide multiply-add).
template <int kRegI>
__device__ __forceinline__ void bconv_body_pair32(const BconvDesc<uint32_t>& d,
                                                  const PrimeConst<uint32_t>* __restrict__ pcs, const uint32_t* sfac,
                                                  const BconvOut<uint32_t>* sout, int coeff) {
  uint32_t ya[kRegI], yb[kRegI];
#pragma unroll
  for (int i = 0; i < kRegI; i++) {
    const uint2 v = *reinterpret_cast<const uint2*>(
        d.in + (size_t)(d.in_pos != nullptr ? d.in_pos[i] : (uint32_t)i) * d.in_stride + coeff);
    ya[i] = bconv_prepare<uint32_t>(d, pcs, i, v.x);
    yb[i] = bconv_prepare<uint32_t>(d, pcs, i, v.y);
  }
  const int O = d.O;
#pragma unroll 2
  for (int j = 0; j < O; j++) {
    const uint32_t* f = sfac + j * kRegI;
    uint64_t a = 0, b = 0;
#pragma unroll
    for (int i = 0; i < kRegI; i++) {
      const uint64_t fi = f[i];
      a += (uint64_t)ya[i] * fi;
      b += (uint64_t)yb[i] * fi;
    }
    const BconvOut<uint32_t> o = sout[j];
    PrimeConst<uint32_t> pc;
    pc.q = o.q;
    pc.q2 = o.q2;
    pc.mu_hi = o.mu_hi;
    pc.mu_lo = o.mu_lo;
    uint32_t ra = barrett2<uint32_t>((uint32_t)(a >> 32), (uint32_t)a, pc);
    uint32_t rb = barrett2<uint32_t>((uint32_t)(b >> 32), (uint32_t)b, pc);
    if (o.has_sub) {
      ra = sub_mod<uint32_t>(ra, o.sub, o.q);
      rb = sub_mod<uint32_t>(rb, o.sub, o.q);
    }
    *reinterpret_cast<uint2*>(d.out + (size_t)o.pos * d.out_stride + coeff) = make_uint2(ra, rb);
  }
}

// 32-bit words, 9 to 32 inputs (the digits of the reference's 28-bit parameter sets hold 10 to 28 limbs): one
// coefficient per thread, every input in a register, the factor rows padded with zeros to kP = a multiple of
// four words and read as 16-byte vectors (one shared-memory load per four terms, the same address in every
// lane).  Residues and factors are below 2^30 (the widest primes a 32-bit context takes), a product is below
// 2^60, so sixteen of them fit one 64-bit sum: a multiply-accumulate is one wide multiply-add, and an output
// takes one Barrett reduction (two and an addition beyond sixteen inputs) - against a two-word accumulator
// with carries and a shared-memory column of inputs in the generic path.  Like the path for at most eight
// inputs, this one takes canonical residues.
template <int kP>
__device__ __forceinline__ void bconv_body_wide32(const BconvDesc<uint32_t>& d, const PrimeConst<uint32_t>* __restrict__ pcs,
                                                  const uint32_t* sfac, const BconvOut<uint32_t>* sout, int coeff) {
  static_assert(kP % 4 == 0 && kP > 8 && kP <= 32, "padded input count");
  uint32_t y[kP];
#pragma unroll
  for (int i = 0; i < kP; i++) y[i] = i < d.I ? bconv_input<uint32_t>(d, pcs, i, coeff) : 0u;
  const int O = d.O;
#pragma unroll 2
  for (int j = 0; j < O; j++) {
    const uint4* f = reinterpret_cast<const uint4*>(sfac + (size_t)j * kP);
    uint64_t a = 0, b = 0;  // inputs 0..15 and 16..31
#pragma unroll
    for (int g = 0; g < kP / 4; g++) {
      const uint4 v = f[g];
      uint64_t t = (uint64_t)y[4 * g] * v.x;
      t += (uint64_t)y[4 * g + 1] * v.y;
      t += (uint64_t)y[4 * g + 2] * v.z;
      t += (uint64_t)y[4 * g + 3] * v.w;
      if (g < 4) a += t; else b += t;
    }
    const BconvOut<uint32_t> o = sout[j];
    PrimeConst<uint32_t> pc;
    pc.q = o.q;
    pc.q2 = o.q2;
    pc.mu_hi = o.mu_hi;
    pc.mu_lo = o.mu_lo;
    uint32_t r = barrett2<uint32_t>((uint32_t)(a >> 32), (uint32_t)a, pc);
    if (kP > 16) r = add_mod<uint32_t>(r, barrett2<uint32_t>((uint32_t)(b >> 32), (uint32_t)b, pc), o.q);
    if (o.has_sub) r = sub_mod<uint32_t>(r, o.sub, o.q);
    d.out[(size_t)o.pos * d.out_stride + coeff] = r;
  }
}

// The wide path's dispatch on the padded input count.
__device__ __forceinline__ void bconv_wide32(const BconvDesc<uint32_t>& d, const PrimeConst<uint32_t>* __restrict__ pcs,
                                             const uint32_t* sfac, const BconvOut<uint32_t>* sout, int coeff) {
  switch ((d.I + 3) / 4) {
    case 3: bconv_body_wide32<12>(d, pcs, sfac, sout, coeff); break;
    case 4: bconv_body_wide32<16>(d, pcs, sfac, sout, coeff); break;
    case 5: bconv_body_wide32<20>(d, pcs, sfac, sout, coeff); break;
    case 6: bconv_body_wide32<24>(d, pcs, sfac, sout, coeff); break;
    case 7: bconv_body_wide32<28>(d, pcs, sfac, sout, coeff); break;
    default: bconv_body_wide32<32>(d, pcs, sfac, sout, coeff); break;
  }
}
constexpr int kBconvWideMaxInputs = 32;
template <typename W>
__host__ __device__ inline bool bconv_is_wide32(int I) {
  return sizeof(W) == 4 && I > kBconvRegInputs && I <= kBconvWideMaxInputs;
}

constexpr int kBconvMaxBatch = 24;  // conversions per launch (descriptors travel as parameters)

template <typename W>
struct BconvBatch {
  BconvDesc<W> d[kBconvMaxBatch];
};

// Shared-memory need of one conversion (bytes): factor matrix, per-output constants and, for
// more than kBconvRegInputs inputs, one column of inputs per thread.
template <typename W>
__host__ __device__ inline size_t bconv_smem_bytes(int I, int O) {
  size_t n = (size_t)O * I * sizeof(W);
  n = (n + 15) / 16 * 16 + ((size_t)O * sizeof(BconvOut<W>) + 15) / 16 * 16;
  if (I > kBconvRegInputs) n += (size_t)I * kBconvThreads * sizeof(W);
  else if (sizeof(W) == 8) n += (size_t)O * I * 16;  // double-precision factor pairs
  if (bconv_is_wide32<W>(I)) {  // padded factor rows in place of the plain matrix (and no input column)
    const size_t wide = ((size_t)O * ((I + 3) / 4 * 4) * sizeof(W) + 15) / 16 * 16 + ((size_t)O * sizeof(BconvOut<W>) + 15) / 16 * 16;
    if (wide > n) n = wide;
  }
  return n;
}

// grid = (ceil(N / kBconvThreads), conversions, ceil(max O / out_chunk)), block = kBconvThreads,
// dynamic smem = max bconv_smem_bytes over the batch.  CTA z handles outputs
// [z * out_chunk, min(O, (z + 1) * out_chunk)) of its conversion.
// kPair (32-bit words only, every conversion of the batch with at most 8 inputs and 8-byte aligned
// limbs): two coefficients per thread, grid.x = ceil(N / (2 kBconvThreads)).
template <typename W, bool kPair>
__global__ void __launch_bounds__(kBconvThreads, 5)
    bconv_kernel(const BconvBatch<W> batch, const int out_chunk, const PrimeConst<W>* __restrict__ pcs) {
  CERIUM_DYN_SMEM(smem_raw);
  grid_dependency_launch();
  BconvDesc<W> d = batch.d[blockIdx.y];
  const int j_first = blockIdx.z * out_chunk;
  if (j_first >= d.O) return;
  // restrict the descriptor to this CTA's slice of the outputs
  const int I = d.I, O = (d.O - j_first) < out_chunk ? (d.O - j_first) : out_chunk;
  d.factors += (size_t)j_first * I;
  d.O = O;
  W* sfac = reinterpret_cast<W*>(smem_raw);
  const bool wide = !kPair && bconv_is_wide32<W>(I);
  const int P = wide ? (I + 3) / 4 * 4 : I;  // words per staged factor row
  const size_t fac_bytes = ((size_t)O * P * sizeof(W) + 15) / 16 * 16;
  BconvOut<W>* sout = reinterpret_cast<BconvOut<W>*>(smem_raw + fac_bytes);
  const size_t out_bytes = ((size_t)O * sizeof(BconvOut<W>) + 15) / 16 * 16;
  W* scol = reinterpret_cast<W*>(smem_raw + fac_bytes + out_bytes);
  double2* sfp = reinterpret_cast<double2*>(smem_raw + fac_bytes + out_bytes);  // split path only (no scol then)
  const bool split = sizeof(W) == 8 && I <= kBconvRegInputs;
  // stage this CTA's slice of the converter's tables
  if (wide) {
    for (int k = threadIdx.x; k < O * P; k += kBconvThreads) {
      const int j = k / P, i = k - j * P;
      sfac[k] = i < I ? d.factors[(size_t)j * I + i] : (W)0;
    }
  }
  for (int k = threadIdx.x; k < (wide ? 0 : O * I); k += kBconvThreads) {
    if (split) {
      reinterpret_cast<uint2*>(sfac)[k] = d.split_fac[(size_t)j_first * I + k];
      if (d.fp_in != 0) sfp[k] = d.fp_fac[(size_t)j_first * I + k];
    } else {
      sfac[k] = d.factors[k];
    }
  }
  for (int j = threadIdx.x; j < O; j += kBconvThreads) sout[j] = d.outc[j_first + j];
  grid_dependency_wait();  // the tables above never change; the input limbs below come from the previous kernel
  __syncthreads();
  if (kPair && sizeof(W) == 4) {
    const int coeff = (blockIdx.x * kBconvThreads + threadIdx.x) * 2;
    if (coeff >= kN) return;  // partial last block (after the only barrier)
    const BconvDesc<uint32_t>& d32 = reinterpret_cast<const BconvDesc<uint32_t>&>(d);
    const PrimeConst<uint32_t>* p32 = reinterpret_cast<const PrimeConst<uint32_t>*>(pcs);
    const uint32_t* f32 = reinterpret_cast<const uint32_t*>(sfac);
    const BconvOut<uint32_t>* so = reinterpret_cast<const BconvOut<uint32_t>*>(sout);
    switch (I) {
      case 1: bconv_body_pair32<1>(d32, p32, f32, so, coeff); break;
      case 2: bconv_body_pair32<2>(d32, p32, f32, so, coeff); break;
      case 3: bconv_body_pair32<3>(d32, p32, f32, so, coeff); break;
      case 4: bconv_body_pair32<4>(d32, p32, f32, so, coeff); break;
      case 5: bconv_body_pair32<5>(d32, p32, f32, so, coeff); break;
      case 6: bconv_body_pair32<6>(d32, p32, f32, so, coeff); break;
      case 7: bconv_body_pair32<7>(d32, p32, f32, so, coeff); break;
      default: bconv_body_pair32<8>(d32, p32, f32, so, coeff); break;
    }
    return;
  }
  const int coeff = blockIdx.x * kBconvThreads + threadIdx.x;
  if (coeff >= kN) return;  // partial last block (after the only barrier)
  if (wide) {
    bconv_wide32(reinterpret_cast<const BconvDesc<uint32_t>&>(d), reinterpret_cast<const PrimeConst<uint32_t>*>(pcs),
                 reinterpret_cast<const uint32_t*>(sfac), reinterpret_cast<const BconvOut<uint32_t>*>(sout), coeff);
    return;
  }
  if (sizeof(W) == 8 && I <= kBconvRegInputs) {
    const BconvDesc<uint64_t>& d64 = reinterpret_cast<const BconvDesc<uint64_t>&>(d);
    const PrimeConst<uint64_t>* p64 = reinterpret_cast<const PrimeConst<uint64_t>*>(pcs);
    const uint2* f2 = reinterpret_cast<const uint2*>(sfac);
    const BconvOut<uint64_t>* so = reinterpret_cast<const BconvOut<uint64_t>*>(sout);
    switch (I) {
      case 1: if (d.lazy_out) bconv_body_split64<1, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<1, false>(d64, p64, f2, so, sfp, coeff); break;
      case 2: if (d.lazy_out) bconv_body_split64<2, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<2, false>(d64, p64, f2, so, sfp, coeff); break;
      case 3: if (d.lazy_out) bconv_body_split64<3, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<3, false>(d64, p64, f2, so, sfp, coeff); break;
      case 4: if (d.lazy_out) bconv_body_split64<4, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<4, false>(d64, p64, f2, so, sfp, coeff); break;
      case 5: if (d.lazy_out) bconv_body_split64<5, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<5, false>(d64, p64, f2, so, sfp, coeff); break;
      case 6: if (d.lazy_out) bconv_body_split64<6, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<6, false>(d64, p64, f2, so, sfp, coeff); break;
      case 7: if (d.lazy_out) bconv_body_split64<7, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<7, false>(d64, p64, f2, so, sfp, coeff); break;
      default: if (d.lazy_out) bconv_body_split64<8, true>(d64, p64, f2, so, sfp, coeff); else bconv_body_split64<8, false>(d64, p64, f2, so, sfp, coeff); break;
    }
  } else {
    switch (I) {
      case 1: bconv_body<W, 1>(d, pcs, sfac, sout, scol, coeff); break;
      case 2: bconv_body<W, 2>(d, pcs, sfac, sout, scol, coeff); break;
      case 3: bconv_body<W, 3>(d, pcs, sfac, sout, scol, coeff); break;
      case 4: bconv_body<W, 4>(d, pcs, sfac, sout, scol, coeff); break;
      case 5: bconv_body<W, 5>(d, pcs, sfac, sout, scol, coeff); break;
      case 6: bconv_body<W, 6>(d, pcs, sfac, sout, scol, coeff); break;
      case 7: bconv_body<W, 7>(d, pcs, sfac, sout, scol, coeff); break;
      case 8: bconv_body<W, 8>(d, pcs, sfac, sout, scol, coeff); break;
      default: bconv_body<W, 0>(d, pcs, sfac, sout, scol, coeff); break;
    }
  }
}

// The same conversion driven entirely by device-resident tables, the argument layout of the
// reference's launcher (_kernel_bco, cerium/compiler/backend/kernels/function.cuh:61-78, filled by
// Evaluator::fn_bco, cerium/runtime/execution/evaluator.cpp:861-940): conversion j reads
// ins[j] = [n_in[j]][N], writes outs[j] = [n_out[j]][N], with factors[j] = [O][I] residues and
// out_moduli[j] = [O] primes.  The host knows neither shapes nor primes, so the Barrett constants
// are derived here from the moduli (one division per output and CTA).  Lazy conversion only
// (the reference's), canonical outputs.
// The shared memory was sized on the host from the caller's shape bounds; a table entry above them
// (or above the smem_limit bytes the launch has) must not be staged: such a CTA touches no memory,
// records kStatusBconvShape in *status and returns.
// grid = (ceil(N / kBconvThreads), conversions), block = kBconvThreads, dynamic smem >= bconv_smem_bytes(I, O).
constexpr uint32_t kStatusBconvShape = 1u;  // bit of the context's status word
template <typename W>
__global__ void __launch_bounds__(kBconvThreads, 5)
    bconv_ptrs_kernel(W* const* __restrict__ outs, const size_t* __restrict__ n_out, const W* const* __restrict__ ins,
                      const size_t* __restrict__ n_in, const W* const* __restrict__ factors,
                      const W* const* __restrict__ out_moduli, const size_t max_in, const size_t max_out,
                      const size_t smem_limit, uint32_t* __restrict__ status) {
  CERIUM_DYN_SMEM(smem_raw);
  grid_dependency_launch();
  grid_dependency_wait();  // the tables may have been written by the stream's previous work
  const int j = blockIdx.y;
  const size_t In = n_in[j], On = n_out[j];
  if (In < 1 || On < 1 || In > max_in || On > max_out || bconv_smem_bytes<W>((int)In, (int)On) > smem_limit) {
    if (threadIdx.x == 0 && status != nullptr) atomicOr(status, kStatusBconvShape);
    return;
  }
  const int I = (int)In, O = (int)On;
  BconvDesc<W> d{};
  d.in = ins[j];
  d.out = outs[j];
  d.in_stride = kN;
  d.out_stride = kN;
  d.I = I;
  d.O = O;
  W* sfac = reinterpret_cast<W*>(smem_raw);
  const bool wide = bconv_is_wide32<W>(I);
  const int P = wide ? (I + 3) / 4 * 4 : I;  // words per staged factor row
  const size_t fac_bytes = ((size_t)O * P * sizeof(W) + 15) / 16 * 16;
  BconvOut<W>* sout = reinterpret_cast<BconvOut<W>*>(smem_raw + fac_bytes);
  const size_t out_bytes = ((size_t)O * sizeof(BconvOut<W>) + 15) / 16 * 16;
  W* scol = reinterpret_cast<W*>(smem_raw + fac_bytes + out_bytes);
  const W* fac = factors[j];
  const W* omod = out_moduli[j];
  for (int k = threadIdx.x; k < O * P; k += kBconvThreads) {
    const int jj = k / P, i = k - jj * P;
    sfac[k] = i < I ? fac[(size_t)jj * I + i] : (W)0;
  }
  for (int o = threadIdx.x; o < O; o += kBconvThreads) {
    const W q = omod[o];
    BconvOut<W> c{};
    c.q = q;
    c.q2 = q + q;
    if (sizeof(W) == 4) {
      // floor(2^64 / q) = floor((2^64 - 1) / q) for a q that is not a power of two
      const uint64_t mu = ~(uint64_t)0 / (uint64_t)q;
      c.mu_hi = (W)(mu >> 32);
      c.mu_lo = (W)(mu & 0xffffffffu);
    } else {
      // floor(2^128 / q) by two divisions: 2^64 = a q + r, then 2^128 / q = a 2^64 + floor(r 2^64 / q)
      const uint64_t a = ~(uint64_t)0 / (uint64_t)q;
      uint64_t r = ~(uint64_t)0 - a * (uint64_t)q + 1;  // 2^64 mod q (or q itself, fixed below)
      uint64_t hi = a;
      if (r >= (uint64_t)q) { r -= (uint64_t)q; hi += 1; }
      // long division of r * 2^64 by q, one bit at a time (r < q < 2^60, so 2r never overflows)
      uint64_t lo = 0;
      for (int bit = 0; bit < 64; bit++) {
        r <<= 1;
        lo <<= 1;
        if (r >= (uint64_t)q) { r -= (uint64_t)q; lo |= 1; }
      }
      c.mu_hi = (W)hi;
      c.mu_lo = (W)lo;
    }
    c.pos = (uint32_t)o;
    sout[o] = c;
  }
  __syncthreads();
  const int coeff = blockIdx.x * kBconvThreads + threadIdx.x;
  if (coeff >= kN) return;
  if (wide) {
    bconv_wide32(reinterpret_cast<const BconvDesc<uint32_t>&>(d), nullptr, reinterpret_cast<const uint32_t*>(sfac),
                 reinterpret_cast<const BconvOut<uint32_t>*>(sout), coeff);
    return;
  }
  switch (I) {
    case 1: bconv_body<W, 1>(d, nullptr, sfac, sout, scol, coeff); break;
    case 2: bconv_body<W, 2>(d, nullptr, sfac, sout, scol, coeff); break;
    case 3: bconv_body<W, 3>(d, nullptr, sfac, sout, scol, coeff); break;
    case 4: bconv_body<W, 4>(d, nullptr, sfac, sout, scol, coeff); break;
    case 5: bconv_body<W, 5>(d, nullptr, sfac, sout, scol, coeff); break;
    case 6: bconv_body<W, 6>(d, nullptr, sfac, sout, scol, coeff); break;
    case 7: bconv_body<W, 7>(d, nullptr, sfac, sout, scol, coeff); break;
    case 8: bconv_body<W, 8>(d, nullptr, sfac, sout, scol, coeff); break;
    default: bconv_body<W, 0>(d, nullptr, sfac, sout, scol, coeff); break;
  }
}

}  // namespace cerium
