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
// streams over the O output primes with the factor matrix broadcast from shared memory.  Sums
// are kept in a two-word accumulator and reduced once per output (primes below 2^60 leave room
// for 256 terms), instead of the reference's trims at i = 15, 30.
#pragma once
#include "modarith.cuh"

namespace cerium {

constexpr int kBconvThreads = 256;
constexpr int kBconvRegInputs = 8;

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
  int I;
  int O;
};

template <typename W, int kRegI>
__device__ __forceinline__ void bconv_body(const BconvDesc<W>& d, const PrimeConst<W>* __restrict__ pcs,
                                           W* sfac, W* scol, int coeff) {
  const int tid = threadIdx.x;
  const int I = d.I, O = d.O;
  W y[kRegI > 0 ? kRegI : 1];
  // gather (and pre-scale) the inputs
  if (kRegI > 0) {
#pragma unroll
    for (int i = 0; i < kRegI; i++) {
      if (i < I) {
        W v = d.in[(size_t)i * d.in_stride + coeff];
        if (d.in_add != nullptr || d.inv != nullptr) {
          const W qi = pcs[d.in_prime[i]].q;
          if (d.in_add != nullptr) v = add_mod<W>(v, d.in_add[i], qi);
          if (d.inv != nullptr) v = csub<W>(mul_shoup_lazy<W>(v, d.inv[i], d.inv_shoup[i], qi), qi);
        }
        y[i] = v;
      } else {
        y[i] = 0;
      }
    }
  } else {
    for (int i = 0; i < I; i++) {
      W v = d.in[(size_t)i * d.in_stride + coeff];
      if (d.in_add != nullptr || d.inv != nullptr) {
        const W qi = pcs[d.in_prime[i]].q;
        if (d.in_add != nullptr) v = add_mod<W>(v, d.in_add[i], qi);
        if (d.inv != nullptr) v = csub<W>(mul_shoup_lazy<W>(v, d.inv[i], d.inv_shoup[i], qi), qi);
      }
      scol[i * kBconvThreads + tid] = v;
    }
  }
  for (int j = 0; j < O; j++) {
    const PrimeConst<W> pc = pcs[d.out_prime[j]];
    const W* f = sfac + j * I;
    Acc2<W> acc;
    acc.clear();
    if (kRegI > 0) {
#pragma unroll
      for (int i = 0; i < kRegI; i++)
        if (i < I) acc.mad(y[i], f[i]);
    } else {
      for (int i = 0; i < I; i++) acc.mad(scol[i * kBconvThreads + tid], f[i]);
    }
    W r = barrett2<W>(acc.hi, acc.lo, pc);
    if (d.out_sub != nullptr) r = sub_mod<W>(r, d.out_sub[j], pc.q);
    d.out[(size_t)(d.out_pos != nullptr ? d.out_pos[j] : (uint32_t)j) * d.out_stride + coeff] = r;
  }
}

// grid = (N / 256, conversions), block = 256,
// dynamic smem = O*I*sizeof(W) (+ I*256*sizeof(W) when I > kBconvRegInputs), maxima over the batch.
constexpr int kBconvMaxBatch = 24;  // conversions per launch (descriptors travel as parameters)

template <typename W>
struct BconvBatch {
  BconvDesc<W> d[kBconvMaxBatch];
};

template <typename W>
__global__ void __launch_bounds__(kBconvThreads)
    bconv_kernel(const BconvBatch<W> batch, const PrimeConst<W>* __restrict__ pcs) {
  CERIUM_DYN_SMEM(smem_raw);
  const BconvDesc<W>& d = batch.d[blockIdx.y];
  W* sfac = reinterpret_cast<W*>(smem_raw);
  W* scol = sfac + d.O * d.I;
  for (int k = threadIdx.x; k < d.O * d.I; k += kBconvThreads) sfac[k] = d.factors[k];
  __syncthreads();
  const int coeff = blockIdx.x * kBconvThreads + threadIdx.x;
  if (d.I <= 4)
    bconv_body<W, 4>(d, pcs, sfac, scol, coeff);
  else if (d.I <= kBconvRegInputs)
    bconv_body<W, kBconvRegInputs>(d, pcs, sfac, scol, coeff);
  else
    bconv_body<W, 0>(d, pcs, sfac, scol, coeff);
}

}  // namespace cerium
