// Element-wise limb kernels: modular add / sub / neg / mul / multiply-add, P-multiply,
// ciphertext tensor product, Galois automorphism and the key-switching inner product.
//
// Replaces the kernels Cerium's compiler generates per program
// (cerium/compiler/backend/cuda_kernel.cc:64-399 handlers, :1142-1280 generic kernel,
// :2669-2765 PMU) with a fixed hand-written set.  Differences from the generated code:
// 16-byte vector accesses (2 u64 / 4 u32 per thread) instead of one word per thread, the
// automorphism index computed from bit reversals instead of a permutation table in global
// memory, and the evaluation-key inner product accumulated over all digits in registers
// (two-word sums, one Barrett reduction at the end) instead of one Mul/Mad launch per digit
// with a reduction mod q^2 after every term.
#pragma once
#include "modarith.cuh"

namespace cerium {

constexpr int kEwThreads = 256;
constexpr int kEwMaxLimbs = 128;  // limbs per launch (per-limb scalars travel as parameters)

template <typename W>
struct Vec16;
template <>
struct Vec16<uint64_t> {
  static constexpr int kLanes = 2;
  uint64_t v[2];
  static __device__ __forceinline__ Vec16 load(const uint64_t* p) {
    const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(p);
    Vec16 r;
    r.v[0] = t.x;
    r.v[1] = t.y;
    return r;
  }
  __device__ __forceinline__ void store(uint64_t* p) const {
    *reinterpret_cast<ulonglong2*>(p) = make_ulonglong2(v[0], v[1]);
  }
};
template <>
struct Vec16<uint32_t> {
  static constexpr int kLanes = 4;
  uint32_t v[4];
  static __device__ __forceinline__ Vec16 load(const uint32_t* p) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    Vec16 r;
    r.v[0] = t.x;
    r.v[1] = t.y;
    r.v[2] = t.z;
    r.v[3] = t.w;
    return r;
  }
  __device__ __forceinline__ void store(uint32_t* p) const {
    *reinterpret_cast<uint4*>(p) = make_uint4(v[0], v[1], v[2], v[3]);
  }
};

// A stack of limbs: limb b at p + b * stride (words).
template <typename W>
struct Limbs {
  W* p;
  size_t stride;
  __device__ __forceinline__ W* at(int b, int idx) const { return p + (size_t)b * stride + idx; }
};

enum EwOp : int {
  kEwAdd = 0,   // out = a + b
  kEwSub = 1,   // out = a - b
  kEwNeg = 2,   // out = -a
  kEwMul = 3,   // out = a * b
  kEwMad = 4,   // out = a * b + c
  kEwPmu = 5,   // out = a + b * s[limb]
  kEwMulScalar = 6,  // out = a * s[limb]
  kEwReduce = 7,     // out = a mod q for ANY word a (sums of residues after a reduce-scatter / all-reduce)
  kEwMulPeriodic = 8,  // out = a * b[i >> shift]      (b: a plaintext that repeats, stored once per period)
  kEwMadPeriodic = 9,  // out = a * b[i >> shift] + c
};

template <typename W>
struct EwArgs {
  Limbs<W> out, a, b, c;
  W scalar[kEwMaxLimbs];        // per limb (kEwPmu, kEwMulScalar)
  W scalar_shoup[kEwMaxLimbs];  // per limb
  uint8_t prime[kEwMaxLimbs];
  int shift;                    // kEwMulPeriodic / kEwMadPeriodic: log2 of the repeat count
};

// grid = (N / (256 * lanes), limbs), block = 256.
template <typename W, int kOp>
__global__ void __launch_bounds__(kEwThreads)
    ewise_kernel(const EwArgs<W> g, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  using V = Vec16<W>;
  const int b = blockIdx.y;
  const uint32_t pi = g.prime[b];
  const PrimeConst<W> pc = pcs[pi];
  const int idx = (blockIdx.x * kEwThreads + threadIdx.x) * V::kLanes;
  V a = V::load(g.a.at(b, idx)), o;
  V bb, cc;
  if (kOp == kEwAdd || kOp == kEwSub || kOp == kEwMul || kOp == kEwMad || kOp == kEwPmu)
    bb = V::load(g.b.at(b, idx));
  if (kOp == kEwMad || kOp == kEwMadPeriodic) cc = V::load(g.c.at(b, idx));
  if (kOp == kEwMulPeriodic || kOp == kEwMadPeriodic) {
#pragma unroll
    for (int l = 0; l < V::kLanes; l++) bb.v[l] = *g.b.at(b, (idx + l) >> g.shift);
  }
  W s = 0, ss = 0;
  if (kOp == kEwPmu || kOp == kEwMulScalar) {
    s = g.scalar[b];
    ss = g.scalar_shoup[b];
  }
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) {
    if (kOp == kEwAdd) o.v[l] = add_mod<W>(a.v[l], bb.v[l], pc.q);
    if (kOp == kEwSub) o.v[l] = sub_mod<W>(a.v[l], bb.v[l], pc.q);
    if (kOp == kEwNeg) o.v[l] = a.v[l] ? pc.q - a.v[l] : (W)0;
    if (kOp == kEwMul || kOp == kEwMulPeriodic) o.v[l] = mul_mod<W>(a.v[l], bb.v[l], pc);
    if (kOp == kEwMad || kOp == kEwMadPeriodic) o.v[l] = add_mod<W>(mul_mod<W>(a.v[l], bb.v[l], pc), cc.v[l], pc.q);
    if (kOp == kEwPmu)
      o.v[l] = add_mod<W>(a.v[l], csub<W>(mul_shoup_lazy<W>(bb.v[l], s, ss, pc.q), pc.q), pc.q);
    if (kOp == kEwMulScalar) o.v[l] = csub<W>(mul_shoup_lazy<W>(a.v[l], s, ss, pc.q), pc.q);
    if (kOp == kEwReduce) o.v[l] = reduce_word<W>(a.v[l], pc);
  }
  o.store(g.out.at(b, idx));
}

// Ciphertext tensor product (cerium/compiler/backend/compiler.cc:443-467):
// d0 = a0*b0, d1 = a0*b1 + a1*b0, d2 = a1*b1.  Reads 4 limbs, writes 3, one pass.
template <typename W>
struct TensorArgs {
  Limbs<W> a0, a1, b0, b1, d0, d1, d2;
  uint8_t prime[kEwMaxLimbs];
};

template <typename W>
__global__ void __launch_bounds__(kEwThreads)
    tensor_kernel(const TensorArgs<W> g, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  using V = Vec16<W>;
  const int b = blockIdx.y;
  const PrimeConst<W> pc = pcs[g.prime[b]];
  const int idx = (blockIdx.x * kEwThreads + threadIdx.x) * V::kLanes;
  const V a0 = V::load(g.a0.at(b, idx)), a1 = V::load(g.a1.at(b, idx));
  const V b0 = V::load(g.b0.at(b, idx)), b1 = V::load(g.b1.at(b, idx));
  V d0, d1, d2;
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) {
    d0.v[l] = mul_mod<W>(a0.v[l], b0.v[l], pc);
    d2.v[l] = mul_mod<W>(a1.v[l], b1.v[l], pc);
    Acc2<W> acc;
    acc.clear();
    acc.mad(a0.v[l], b1.v[l]);
    acc.mad(a1.v[l], b0.v[l]);
    d1.v[l] = barrett2<W>(acc.hi(), acc.lo(), pc);
  }
  d0.store(g.d0.at(b, idx));
  d1.store(g.d1.at(b, idx));
  d2.store(g.d2.at(b, idx));
}

template <typename W>
struct AutomorphArgs {
  Limbs<W> out, in;
  Limbs<W> out2, in2;  // entries b >= split: limb b - split of a second polynomial (same launch)
  int split;
  uint32_t elt;
};

// grid = (N / 256, limbs), block = 256; in and out must not overlap.
template <typename W>
__global__ void __launch_bounds__(kEwThreads) automorph_kernel(const AutomorphArgs<W> g) {
  grid_dependency_launch();
  grid_dependency_wait();
  const int b = blockIdx.y;
  const uint32_t i = blockIdx.x * kEwThreads + threadIdx.x;
  const uint32_t src = galois_source_index(i, g.elt);
  if (b < g.split) *g.out.at(b, (int)i) = *g.in.at(b, (int)src);
  else *g.out2.at(b - g.split, (int)i) = *g.in2.at(b - g.split, (int)src);
}

// Exact CRT composition of two limbs into a two-word integer ("resolve") and its reduction
// modulo other primes ("mod"): the pair bootstrapping's ModRaise and the double rescale are
// built from (cerium/compiler/backend/compiler_rescale.cc:69-121, 367-521).
// Replaces rsv_write_2 / mod_read_2 (cerium/compiler/backend/kernels/fhe_bconv.cuh:31-96) and
// the generated RSV / MOD kernels (cerium/compiler/backend/cuda_kernel.cc:2767-2952) with their
// factor tables (cerium/runtime/execution/function_execution.cpp:53-99).  The reference sums
// x_i * (Mhat_i * [Mhat_i^-1]) modulo M = m0*m1 with a 128-bit Barrett step; the same integer -
// the unique v in [0, M) with v = x0 mod m0 and v = x1 mod m1 - is obtained here by Garner's
// formula v = x0 + m0 * ((x1 - x0) * m0^-1 mod m1): one modular product and one word multiply.
template <typename W>
struct Rsv2Args {
  Limbs<W> x0, x1, lo, hi;  // `count` polynomials each
  W m0;                     // first modulus
  W inv;                    // m0^-1 mod m1
  W inv_shoup;
  uint32_t prime1;          // index of m1
};

// grid = (N / (256 * lanes), count), block = 256
template <typename W>
__global__ void __launch_bounds__(kEwThreads) rsv2_kernel(const Rsv2Args<W> g, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  using V = Vec16<W>;
  const int b = blockIdx.y;
  const PrimeConst<W> pc1 = pcs[g.prime1];
  const int idx = (blockIdx.x * kEwThreads + threadIdx.x) * V::kLanes;
  const V x0 = V::load(g.x0.at(b, idx)), x1 = V::load(g.x1.at(b, idx));
  V lo, hi;
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) {
    const W x0r = reduce_word<W>(x0.v[l], pc1);                    // x0 mod m1
    const W d = sub_mod<W>(x1.v[l], x0r, pc1.q);
    const W t = csub<W>(mul_shoup_lazy<W>(d, g.inv, g.inv_shoup, pc1.q), pc1.q);
    Acc2<W> acc;
    acc.clear();
    acc.mad(g.m0, t);
    // + x0 with carry
    const W l0 = acc.lo() + x0.v[l];
    lo.v[l] = l0;
    hi.v[l] = acc.hi() + (l0 < x0.v[l] ? (W)1 : (W)0);
  }
  lo.store(g.lo.at(b, idx));
  hi.store(g.hi.at(b, idx));
}

template <typename W>
struct Mod2Args {
  const W* lo;  // one two-word polynomial
  const W* hi;
  Limbs<W> out; // `count` limbs
  uint8_t prime[kEwMaxLimbs];
};

// grid = (N / (256 * lanes), count), block = 256: out[b] = (hi:lo) mod q_{prime[b]}
template <typename W>
__global__ void __launch_bounds__(kEwThreads) mod2_kernel(const Mod2Args<W> g, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  using V = Vec16<W>;
  const int b = blockIdx.y;
  const PrimeConst<W> pc = pcs[g.prime[b]];
  const int idx = (blockIdx.x * kEwThreads + threadIdx.x) * V::kLanes;
  const V lo = V::load(g.lo + idx), hi = V::load(g.hi + idx);
  V o;
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) o.v[l] = barrett2<W>(hi.v[l], lo.v[l], pc);
  o.store(g.out.at(b, idx));
}

// Key-switching inner product over the extended basis (L + K limbs):
//   out0[b] = sum_d a_d[b] * evk[d][0][b],   out1[b] = sum_d a_d[b] * evk[d][1][b]
// where a_d[b] is the raised digit d at limb b.  For the limbs that belong to digit d itself
// (own_digit[b] == d) the raised value is the NTT-form input limb, which is read in
// place from `own` instead of from `raised` (cerium/compiler/backend/kernel_instruction.h:
// 823-838 moves it; here it is never copied).
// Restates the EVKMUL / EVKMUL_EXT groups of cerium/compiler/backend/compiler_keyswitch.cc:
// 336-358 and :695-772 as one launch.
template <typename W>
struct InnerProductArgs {
  const W* raised;        // [dnum][LK][N]
  size_t raised_digit_stride;
  size_t raised_limb_stride;
  const W* own;           // [L][N] NTT-form input
  size_t own_stride;
  const W* evk;           // [dnum][2][LK][N]
  size_t evk_digit_stride;
  size_t evk_poly_stride;
  size_t evk_limb_stride;
  Limbs<W> out0, out1;    // [LK][N]
  int first_limb;         // grid.y covers extended limbs first_limb, first_limb + 1, ...
  int dnum;
  uint32_t own_elt;       // not 0: `own` is read through the Galois automorphism of this element
                          // (word i of a limb is own[pi(i)]), i.e. the rotation of the input is folded in
  int accumulate;         // not 0: the products are added to the (canonical) values out0 / out1 already hold
  uint8_t prime[kEwMaxLimbs];     // prime index of extended limb b
  int8_t own_digit[kEwMaxLimbs];  // digit that limb b belongs to (-1 for extension limbs)
};

template <typename W>
__global__ void __launch_bounds__(kEwThreads)
    inner_product_kernel(const InnerProductArgs<W> g, const PrimeConst<W>* __restrict__ pcs) {
  grid_dependency_launch();
  grid_dependency_wait();
  using V = Vec16<W>;
  const int b = g.first_limb + blockIdx.y;
  const PrimeConst<W> pc = pcs[g.prime[b]];
  const int idx = (blockIdx.x * kEwThreads + threadIdx.x) * V::kLanes;
  Acc2<W> acc0[V::kLanes], acc1[V::kLanes];
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) {
    acc0[l].clear();
    acc1[l].clear();
  }
  const int own_digit = g.own_digit[b];
#pragma unroll 2
  for (int d = 0; d < g.dnum; d++) {
    const bool is_own = d == own_digit;
    const W* ap = is_own ? g.own + (size_t)b * g.own_stride + idx
                         : g.raised + (size_t)d * g.raised_digit_stride +
                               (size_t)b * g.raised_limb_stride + idx;
    const W* kp = g.evk + (size_t)d * g.evk_digit_stride + (size_t)b * g.evk_limb_stride + idx;
    V a;
    if (is_own && g.own_elt != 0) {
      const W* limb = g.own + (size_t)b * g.own_stride;
#pragma unroll
      for (int l = 0; l < V::kLanes; l++) a.v[l] = limb[galois_source_index((uint32_t)(idx + l), g.own_elt)];
    } else {
      a = V::load(ap);
    }
    const V k0 = V::load(kp);
    const V k1 = V::load(kp + g.evk_poly_stride);
#pragma unroll
    for (int l = 0; l < V::kLanes; l++) {
      acc0[l].mad(a.v[l], k0.v[l]);
      acc1[l].mad(a.v[l], k1.v[l]);
    }
  }
  V o0, o1;
#pragma unroll
  for (int l = 0; l < V::kLanes; l++) {
    o0.v[l] = barrett2<W>(acc0[l].hi(), acc0[l].lo(), pc);
    o1.v[l] = barrett2<W>(acc1[l].hi(), acc1[l].lo(), pc);
  }
  if (g.accumulate != 0) {
    const V p0 = V::load(g.out0.at(b, idx)), p1 = V::load(g.out1.at(b, idx));
#pragma unroll
    for (int l = 0; l < V::kLanes; l++) {
      o0.v[l] = add_mod<W>(o0.v[l], p0.v[l], pc.q);
      o1.v[l] = add_mod<W>(o1.v[l], p1.v[l], pc.q);
    }
  }
  o0.store(g.out0.at(b, idx));
  o1.store(g.out1.at(b, idx));
}

}  // namespace cerium
