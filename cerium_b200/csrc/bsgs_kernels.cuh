// Kernels of the baby-step / giant-step multiply-accumulate (the linear-transform building block of
// bootstrapping): the plaintext multiply-accumulate of a group of giant steps in one pass, and the
// sum of several polynomials read through (different) Galois automorphisms.
//
// The reference lowers BsgsMultiplyAccumulate to one MuP and one Add instruction per diagonal and
// polynomial inside a generated kernel group (cerium/compiler/backend/compiler.cc:2495-2522) and one
// rotation + Add per giant step (:2562-2590).  Here a thread keeps the sums of up to kBsgsGroup giant
// steps in two-word accumulators while it walks the baby steps, so the rotated copies of the input
// are read once per group and every diagonal exactly once; one reduction per output.
#pragma once
#include "ewise_kernels.cuh"

namespace cerium {

constexpr int kBsgsMaxBaby = 16;   // baby steps (rotated copies of the input)
constexpr int kBsgsGroup = 4;      // giant steps whose inner sums one launch produces
constexpr int kBsgsMaxGiant = 32;  // giant steps of one multiply-accumulate

template <typename W>
struct PtMacArgs {
  const W* src0[kBsgsMaxBaby];            // baby step j, polynomial 0: [limbs][N]
  const W* src1[kBsgsMaxBaby];            // baby step j, polynomial 1
  const W* pt[kBsgsGroup][kBsgsMaxBaby];  // diagonal of (giant step of the group, baby step); null = absent
  W* out0[kBsgsGroup];                    // inner sum of the group's giant step, polynomial 0
  W* out1[kBsgsGroup];
  int g;                                  // baby steps
  uint8_t prime[kEwMaxLimbs];
};

// One thread owns kPtMacWords consecutive words of a limb: one 8-byte access per operand for both word
// sizes (a warp still moves whole 256-byte runs).  Wider accesses would double the accumulator
// registers: with four giant steps, two polynomials and two-word sums that costs the occupancy a
// streaming kernel lives on (136 registers and one CTA per SM when measured with 16-byte accesses).
template <typename W>
struct PtMacLanes {
  static constexpr int kWords = 8 / sizeof(W);
};
template <typename W>
__device__ __forceinline__ void ptmac_load(const W* p, W (&v)[PtMacLanes<W>::kWords]) {
  if constexpr (sizeof(W) == 8) {
    v[0] = __ldg(p);
  } else {
    const uint2 t = __ldg(reinterpret_cast<const uint2*>(p));
    v[0] = t.x;
    v[1] = t.y;
  }
}
template <typename W>
__device__ __forceinline__ void ptmac_store(W* p, const W (&v)[PtMacLanes<W>::kWords]) {
  if constexpr (sizeof(W) == 8) {
    *p = v[0];
  } else {
    *reinterpret_cast<uint2*>(p) = make_uint2(v[0], v[1]);
  }
}

// out[i][p] = sum_j pt[i][j] * src_p[j] for the GI giant steps of a group.
// grid = (N / (256 * kWords), limbs).
template <typename W, int GI>
__global__ void __launch_bounds__(kEwThreads, 3) pt_mac_kernel(const PtMacArgs<W> a, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  constexpr int kWords = PtMacLanes<W>::kWords;
  const int b = blockIdx.y;
  const PrimeConst<W> pc = pcs[a.prime[b]];
  const size_t off = (size_t)b * kN + (size_t)(blockIdx.x * kEwThreads + threadIdx.x) * kWords;
  Acc2<W> acc[GI][2][kWords];
#pragma unroll
  for (int i = 0; i < GI; i++)
#pragma unroll
    for (int l = 0; l < kWords; l++) {
      acc[i][0][l].clear();
      acc[i][1][l].clear();
    }
#pragma unroll 2
  for (int j = 0; j < a.g; j++) {
    W s0[kWords], s1[kWords];
    ptmac_load<W>(a.src0[j] + off, s0);
    ptmac_load<W>(a.src1[j] + off, s1);
#pragma unroll
    for (int i = 0; i < GI; i++) {
      const W* pp = a.pt[i][j];
      if (pp == nullptr) continue;
      W p[kWords];
      ptmac_load<W>(pp + off, p);
#pragma unroll
      for (int l = 0; l < kWords; l++) {
        acc[i][0][l].mad(s0[l], p[l]);
        acc[i][1][l].mad(s1[l], p[l]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < GI; i++) {
    W o0[kWords], o1[kWords];
#pragma unroll
    for (int l = 0; l < kWords; l++) {
      o0[l] = barrett2<W>(acc[i][0][l].hi(), acc[i][0][l].lo(), pc);
      o1[l] = barrett2<W>(acc[i][1][l].hi(), acc[i][1][l].lo(), pc);
    }
    ptmac_store<W>(a.out0[i] + off, o0);
    ptmac_store<W>(a.out1[i] + off, o1);
  }
}

template <typename W>
struct AutoSumArgs {
  const W* in[kBsgsMaxGiant];   // [limbs][N] each
  uint32_t elt[kBsgsMaxGiant];  // Galois element the polynomial is read through (1 = as it is)
  int count;
  W* out;                       // [limbs][N]; must not overlap an input
  uint8_t prime[kEwMaxLimbs];
};

// out[b][i] = sum_k in_k[b][pi_k(i)] mod q.  grid = (N / 256, limbs).
template <typename W>
__global__ void __launch_bounds__(kEwThreads) automorph_sum_kernel(const AutoSumArgs<W> a, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int b = blockIdx.y;
  const W q = pcs[a.prime[b]].q;
  const uint32_t i = blockIdx.x * kEwThreads + threadIdx.x;
  W s = 0;
  for (int k = 0; k < a.count; k++) {
    const uint32_t src = a.elt[k] == 1u ? i : galois_source_index(i, a.elt[k]);
    s = add_mod<W>(s, a.in[k][(size_t)b * kN + src], q);
  }
  a.out[(size_t)b * kN + i] = s;
}

}  // namespace cerium
