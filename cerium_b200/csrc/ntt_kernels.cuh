// Negacyclic NTT kernels for N = 2^16 over batches of RNS limbs.
//
// Replaces the reference's four NTT kernels and their launchers:
//   forward  ntt0/ntt1   cerium/compiler/backend/kernels/fhe_ntt.cuh:114-273,
//                        cerium/compiler/backend/kernels/function.cu:22-99
//   inverse  intt0/intt1 cerium/compiler/backend/kernels/fhe_ntt.cuh:470-601,
//                        cerium/compiler/backend/kernels/function.cu:199-280
//   SuD tail ntt1_sud    cerium/compiler/backend/kernels/fhe_ntt.cuh:278-359
// Same contract (standard order in -> bit-reversed order out for the forward transform,
// the inverse undoes it and scales by 1/N), different design:
//
//  * The 16 radix-2 layers are four radix-16 levels.  A level keeps 16 coefficients of one
//    thread in registers; two levels make a pass, with one shared-memory exchange between
//    them, so one limb crosses HBM twice per transform (once per pass) and the exchange
//    never leaves the SM.
//  * Twiddles are addressed through the "root prefix" S of a radix-16 group: layer t of the
//    group uses table entries (S << t) + (j >> (4 - t)), j the register index.  Level 0 has
//    S = 1, level 1 S = 16 + a, level 2 S = 256 + h, level 3 S = 4096 + 16 h + u.
//    The 255 twiddles of the column pass are the same for every column and sit in shared
//    memory; the row pass reads its twiddles in contiguous runs of 1, 2, 4, 8 entries.
//  * The column pass moves 128-byte row segments (16 u64 / 32 u32 columns per CTA); the row
//    pass gives each thread 16 consecutive coefficients and stores them as 16-byte vectors.
//  * Values stay lazy inside a transform ([0,4q) forward, [0,2q) inverse) and are reduced to
//    [0,q) by the last pass, so every buffer a caller sees is canonical.
#pragma once
#include "modarith.cuh"

namespace cerium {

template <typename W>
struct NttCfg;
template <>
struct NttCfg<uint64_t> {
  static constexpr int kCols = 16;  // 16 * 8 B = 128 B segments in the column pass
};
template <>
struct NttCfg<uint32_t> {
  static constexpr int kCols = 32;  // 32 * 4 B = 128 B
};

constexpr int kRowsPerCta = 16;    // row pass: 16 rows of 256 coefficients, 256 threads
// Lane-interleaved level-3 twiddles: [row h (256)][e = 2^t - 1 + g (15)][thread u (16)] pairs per
// prime; entry = bit-reversed table[((4096 + 16 h + u) << t) + g].
constexpr int kRowTwPerPrime = 256 * 15 * 16;
constexpr int kMaxBatch = 512;     // limbs per launch

// Addressing of a batch of limbs: batch entry b lives at base + pos[b] * stride; its modulus
// is prime[b] (index into the context's prime list).  Passed by value as a kernel parameter.
// in_stride = 0 makes every entry read the same source limb (rescale broadcasts the last limb).
template <typename W>
struct StridedBatch {
  const W* in;
  W* out;
  size_t in_stride;   // in words
  size_t out_stride;  // in words
  W* out2;            // entries b >= split write to out2 instead of out (two result stacks, one launch)
  int split;          // kMaxBatch when unused
  uint32_t in_elt;    // inverse transform only, not 0: word i of an input limb is read at pi(i), the Galois
                      // automorphism of this element (modarith.cuh), so a rotation costs no pass of its own
  uint16_t pos[kMaxBatch];
  uint8_t prime[kMaxBatch];
  __device__ __forceinline__ const W* in_limb(int b) const { return in + (size_t)pos[b] * in_stride; }
  __device__ __forceinline__ W* out_limb(int b) const {
    return (b >= split ? out2 : out) + (size_t)pos[b] * out_stride;
  }
  __device__ __forceinline__ uint32_t prime_of(int b) const { return prime[b]; }
  __device__ __forceinline__ uint32_t gather_elt() const { return in_elt; }
};

// StridedBatch whose entries read from a slot of their own: entry b reads limb in_pos[b] of `in`
// and writes limb pos[b] of `out` (one coefficient-form limb transformed under many primes).
template <typename W>
struct GatherBatch : StridedBatch<W> {
  uint16_t in_pos[kMaxBatch];
  __device__ __forceinline__ const W* in_limb(int b) const {
    return this->in + (size_t)in_pos[b] * this->in_stride;
  }
};

// Addressing through device-resident pointer tables, the layout the reference's launchers
// take (args_outputs / args_inputs / bases, cerium/compiler/backend/kernels/function.cu:22-39).
template <typename W>
struct PointerBatch {
  W* const* outs;
  const W* const* ins;
  const uint32_t* bases;
  int in_step;  // entry b reads ins[b * in_step + in_off] (the SuD launcher passes two inputs per entry)
  int in_off;
  __device__ __forceinline__ const W* in_limb(int b) const { return ins[b * in_step + in_off]; }
  __device__ __forceinline__ W* out_limb(int b) const { return outs[b]; }
  __device__ __forceinline__ uint32_t prime_of(int b) const { return bases[b]; }
  __device__ __forceinline__ uint32_t gather_elt() const { return 0u; }
};

// ---------------------------------------------------------------------------------------
// arithmetic policies
// ---------------------------------------------------------------------------------------

// Strict (Harvey) butterflies keep every value below 4q (forward) / 2q (inverse) with one
// correction per butterfly; they serve 32-bit words and 64-bit primes of 52 bits or more.
// Lazy butterflies (64-bit words, primes below 2^52) use the headroom above the prime instead
// of corrections and the 32-bit-piece products of modarith.cuh.
// Fp butterflies (64-bit words, primes below 2^50) run on the FP64 pipe: the registers hold the
// bit patterns of doubles, signed residues whose bound a compile-time plan tracks.
enum : int { kArithStrict = 0, kArithLazy = 1, kArithFp = 2 };

template <typename W, int kMode>
struct Arith {
  static constexpr bool kLazy = kMode == kArithLazy;
  W q, q2, q4, nq;
  __device__ __forceinline__ explicit Arith(const PrimeConst<W>& pc)
      : q(pc.q), q2(pc.q + pc.q), q4(pc.q * 4), nq((W)0 - pc.q) {}
  // canonical residue -> the form the butterflies work on
  __device__ __forceinline__ W enter(W x) const { return x; }
  __device__ __forceinline__ W reduce(W x) const { return x; }
  __device__ __forceinline__ void fwd(W& a, W& b, W w, W ws) const {
    if (kLazy) butterfly_fwd_lazy<W>(a, b, w, ws, nq, q4);
    else butterfly_fwd<W>(a, b, w, ws, q, q2);
  }
  // k = layer number inside the pass (0..7)
  __device__ __forceinline__ void inv(W& a, W& b, W w, W ws, int k) const {
    if (kLazy) butterfly_inv_lazy<W>(a, b, w, ws, nq, q4 << k);
    else butterfly_inv<W>(a, b, w, ws, q, q2);
  }
  // value at the end of a forward transform -> [0, q), or only below 4q when the consumer
  // takes lazy residues (kCanonical = false)
  template <bool kCanonical>
  __device__ __forceinline__ W finish_fwd(W x, W one_shoup) const {
    if (kLazy) x = reduce_lazy(x, one_shoup, nq);
    if (!kCanonical) return x;
    return csub<W>(csub<W>(x, q2), q);
  }
  // last inverse layer: (a + b) * N^-1 and (a - b) * w1 * N^-1, reduced to [0, q)
  __device__ __forceinline__ void inv_last(W& a, W& b, const PrimeConst<W>& pc) const {
    const W s = a + b;
    const W d = a + (kLazy ? (q4 << 7) : q2) - b;
    if (kLazy) {
      a = csub<W>(csub<W>(mul_shoup_approx(s, pc.ninv, pc.ninv_shoup, nq), q2), q);
      b = csub<W>(csub<W>(mul_shoup_approx(d, pc.w1ninv, pc.w1ninv_shoup, nq), q2), q);
    } else {
      a = csub<W>(mul_shoup_lazy<W>(s, pc.ninv, pc.ninv_shoup, q), q);
      b = csub<W>(mul_shoup_lazy<W>(d, pc.w1ninv, pc.w1ninv_shoup, q), q);
    }
  }
};

template <>
struct Arith<uint64_t, kArithFp> {
  using W = uint64_t;
  double q, nq, qinv;
  __device__ __forceinline__ explicit Arith(const PrimeConst<W>& pc) {
    q = fp_from_u64(pc.q);
    nq = -q;
    qinv = d(pc.fp_qinv);
  }
  static __device__ __forceinline__ double d(W x) { return __longlong_as_double((long long)x); }
  static __device__ __forceinline__ W u(double x) { return (W)__double_as_longlong(x); }
  __device__ __forceinline__ W enter(W x) const { return u(fp_from_u64(x)); }
  __device__ __forceinline__ W reduce(W x) const { return u(fp_reduce(d(x), qinv, nq)); }
  // quotient of a twiddle by q when the table holds the twiddle alone
  __device__ __forceinline__ W quotient(W w) const { return u(__dmul_rn(d(w), qinv)); }
  __device__ __forceinline__ void fwd(W& a, W& b, W w, W wq) const {
    const double r = fp_mulmod(d(b), d(w), d(wq), nq);
    const double x = d(a);
    a = u(__dadd_rn(x, r));
    b = u(__dadd_rn(x, -r));
  }
  __device__ __forceinline__ void inv(W& a, W& b, W w, W wq, int /*k*/) const {
    const double x = d(a), y = d(b);
    a = u(__dadd_rn(x, y));
    b = u(fp_mulmod(__dadd_rn(x, -y), d(w), d(wq), nq));
  }
  // |x| <= 0.63 q -> [0, q) as an integer word
  __device__ __forceinline__ W canonical(double x) const {
    return fp_to_u64(x < 0.0 ? __dadd_rn(x, q) : x);
  }
  template <bool kCanonical>
  __device__ __forceinline__ W finish_fwd(W x, W /*one_shoup*/) const {
    const double r = fp_reduce(d(x), qinv, nq);
    if (kCanonical) return canonical(r);
    return fp_to_u64(__dadd_rn(r, q));  // (0.49 q, 1.51 q): a lazy residue
  }
  __device__ __forceinline__ void inv_last(W& a, W& b, const PrimeConst<W>& pc) const {
    const double x = d(a), y = d(b);
    a = canonical(fp_mulmod(__dadd_rn(x, y), d(pc.fp_ninv), d(pc.fp_ninv_q), nq));
    b = canonical(fp_mulmod(__dadd_rn(x, -y), d(pc.fp_w1ninv), d(pc.fp_w1ninv_q), nq));
  }
};

// ---------------------------------------------------------------------------------------
// Compile-time plan of the Fp butterflies: bounds in units of q / 1024, rounded up.
// A product's operand may reach 4q and comes back within q * (1/2 + operand / 32q); sums stay
// below 8q.  The plan walks the layers of a radix-16 group and reduces, just in time, the
// values whose bound would break the operand limit.
// ---------------------------------------------------------------------------------------
constexpr int kFpCanon = 1024;       // canonical input, [0, q)
constexpr int kFpReduced = 513;      // after fp_reduce
constexpr int kFpOperandMax = 4096;  // operand of a product
// k32 = 1: the twiddle comes with its tabulated quotient RN(w / q); k32 = 3: the quotient is
// computed as RN(w * RN(1 / q)) (last level of the row pass, whose table then holds w only), three
// times the error: |r| <= q * (1/2 + 3 * operand / 32q)
__host__ __device__ constexpr int fp_product_bound(int operand, int k32 = 1) {
  return 512 + (k32 * operand + 31) / 32;
}

// forward (Cooley-Tukey): a' = a + w*b, b' = a - w*b; all 16 values share one bound
struct FpFwdPlan {
  bool before[4];  // reduce every value before layer t
  int out;
};
__host__ __device__ constexpr FpFwdPlan fp_plan_fwd(int bin, int k32 = 1) {
  FpFwdPlan p{};
  int b = bin;
  for (int t = 0; t < 4; t++) {
    p.before[t] = b > kFpOperandMax;
    if (p.before[t]) b = kFpReduced;
    b += fp_product_bound(b, k32);
  }
  p.out = b;
  return p;
}

// inverse (Gentleman-Sande): a' = a + b, b' = w * (a - b); the operand a - b needs
// bound(a) + bound(b) <= 4q.  before[t] is the mask of registers to reduce before layer t.
struct FpInvPlan {
  unsigned before[4];
  int bound[16];
  int max_out;
};
__host__ __device__ constexpr FpInvPlan fp_plan_inv(int bin, int k32 = 1) {
  FpInvPlan p{};
  for (int j = 0; j < 16; j++) p.bound[j] = bin;
  for (int t = 3; t >= 0; t--) {
    const int half = 8 >> t;
    unsigned mask = 0;
    for (int g = 0; g < (1 << t); g++)
      for (int k = 0; k < half; k++) {
        const int j = g * 2 * half + k, i = j + half;
        if (p.bound[j] + p.bound[i] > kFpOperandMax) {
          const int big = p.bound[j] >= p.bound[i] ? j : i;
          p.bound[big] = kFpReduced;
          mask |= 1u << big;
          if (p.bound[j] + p.bound[i] > kFpOperandMax) {
            const int other = big == j ? i : j;
            p.bound[other] = kFpReduced;
            mask |= 1u << other;
          }
        }
        const int sum = p.bound[j] + p.bound[i];
        p.bound[j] = sum;
        p.bound[i] = fp_product_bound(sum, k32);
      }
    p.before[t] = mask;
  }
  p.max_out = 0;
  for (int j = 0; j < 16; j++) p.max_out = p.bound[j] > p.max_out ? p.bound[j] : p.max_out;
  return p;
}
// Registers above `threshold` are reduced before they are exchanged (the next group mixes the
// registers of 16 threads, so it starts from the largest bound).
struct FpExchange {
  unsigned mask;
  int out;
};
__host__ __device__ constexpr FpExchange fp_plan_exchange(const FpInvPlan& p, int threshold) {
  FpExchange e{};
  for (int j = 0; j < 16; j++) {
    int b = p.bound[j];
    if (b > threshold) {
      e.mask |= 1u << j;
      b = kFpReduced;
    }
    e.out = b > e.out ? b : e.out;
  }
  return e;
}
constexpr int kFpInvExchangeMax = 2048;

// bounds along the forward transform: the column pass starts from its loader's bound (canonical
// words, or lazy ones below 4q) and stores at most kFpFwdMid, from which the row pass starts
constexpr int kFpLazyIn = 4096;
constexpr int kFpFwdMid = fp_plan_fwd(fp_plan_fwd(kFpLazyIn).out).out;
static_assert(fp_plan_fwd(fp_plan_fwd(kFpCanon).out).out <= kFpFwdMid, "the lazy loader is the worst case");
constexpr int kFpFwdL3 = fp_plan_fwd(kFpFwdMid).out;
constexpr int kFpLaneK32 = 3;  // level 3 (lane table) computes its quotients
static_assert(fp_plan_fwd(kFpFwdL3, kFpLaneK32).out < 8192, "the transform's last values must stay exact integers");
// bounds along the inverse transform: row pass (levels 3, 2) stores kFpInvMid
constexpr int kFpInvL3 = fp_plan_exchange(fp_plan_inv(kFpCanon, kFpLaneK32), kFpInvExchangeMax).out;
constexpr int kFpInvMid = fp_plan_inv(kFpInvL3).max_out;
constexpr int kFpInvL1 = fp_plan_exchange(fp_plan_inv(kFpInvMid), kFpInvExchangeMax).out;
constexpr unsigned kFpInvRowsExMask = fp_plan_exchange(fp_plan_inv(kFpCanon, kFpLaneK32), kFpInvExchangeMax).mask;
constexpr unsigned kFpInvColsExMask = fp_plan_exchange(fp_plan_inv(kFpInvMid), kFpInvExchangeMax).mask;
static_assert(kFpFwdMid < 8192 && kFpInvMid < 8192, "stored intermediates must stay exact integers");

template <typename W, int kMode>
__device__ __forceinline__ void fp_reduce_masked(W (&x)[16], unsigned mask, const Arith<W, kMode>& ar) {
#pragma unroll
  for (int j = 0; j < 16; j++)
    if (mask >> j & 1u) x[j] = ar.reduce(x[j]);
}

// ---------------------------------------------------------------------------------------
// radix-16 register kernels
// ---------------------------------------------------------------------------------------

template <typename W, bool kGlobalTw>
__device__ __forceinline__ typename WordTraits<W>::Pair load_tw(const typename WordTraits<W>::Pair* t,
                                                                 uint32_t idx) {
  if (kGlobalTw) return __ldg(t + idx);
  return t[idx];
}

// Twiddle addressing of a radix-16 group.  Plain: entry (S << t) + g of the bit-reversed table.
// Lane-interleaved (kLaneTable): the group's 15 twiddles sit at entries e * 16, e = 2^t - 1 + g,
// of a table pre-permuted so that the 16 threads of a row read 16 consecutive entries.
template <bool kLaneTable>
__device__ __forceinline__ uint32_t tw_index(uint32_t S, int t, int g) {
  return kLaneTable ? (uint32_t)(((1 << t) - 1 + g) * 16) : (S << t) + (uint32_t)g;
}

// Lane-interleaved table of a prime with double-precision butterflies: twiddles only, two per
// 16-byte entry; twiddle e = 2^t - 1 + g sits in double number e + 1 of the group's 16 (number 0
// is padding, so that every layer starts on an entry boundary), entry v of thread u at (v * 16).
template <typename W>
__device__ __forceinline__ W lane_tw_fp(const typename WordTraits<W>::Pair* tw, int t, int g) {
  const int slot = (1 << t) + g;
  const auto pv = __ldg(tw + (slot >> 1) * 16);
  return (slot & 1) ? pv.y : pv.x;
}

// Four forward layers on x[0..15]; layer t pairs (j, j + (8 >> t)).  kBin: bound of the inputs
// (Fp arithmetic only).
template <typename W, bool kGlobalTw, int kMode, bool kLaneTable = false, int kBin = 0>
__device__ __forceinline__ void radix16_fwd(W (&x)[16], const typename WordTraits<W>::Pair* tw,
                                            uint32_t S, const Arith<W, kMode>& ar) {
  constexpr bool kPacked = kLaneTable && kMode == kArithFp;
  constexpr FpFwdPlan plan = fp_plan_fwd(kBin, kPacked ? kFpLaneK32 : 1);
#pragma unroll
  for (int t = 0; t < 4; t++) {
    const int half = 8 >> t;
    if (kMode == kArithFp && plan.before[t]) fp_reduce_masked<W, kMode>(x, 0xffffu, ar);
#pragma unroll
    for (int g = 0; g < (1 << t); g++) {
      W w0, w1;
      if constexpr (kPacked) {
        w0 = lane_tw_fp<W>(tw, t, g);
        w1 = ar.quotient(w0);
      } else {
        const auto w = load_tw<W, kGlobalTw>(tw, tw_index<kLaneTable>(S, t, g));
        w0 = w.x;
        w1 = w.y;
      }
#pragma unroll
      for (int k = 0; k < half; k++) {
        const int j = g * 2 * half + k;
        ar.fwd(x[j], x[j + half], w0, w1);
      }
    }
  }
}

// The four inverse layers of the same group, in reverse order; kLayer0 is the pass-local
// number of the first layer executed (0 for the first level of a pass, 4 for the second).
template <typename W, bool kGlobalTw, int kMode, int kLayer0, bool kLaneTable = false, int kBin = 0>
__device__ __forceinline__ void radix16_inv(W (&x)[16], const typename WordTraits<W>::Pair* twi,
                                            uint32_t S, const Arith<W, kMode>& ar) {
  constexpr bool kPacked = kLaneTable && kMode == kArithFp;
  constexpr FpInvPlan plan = fp_plan_inv(kBin, kPacked ? kFpLaneK32 : 1);
#pragma unroll
  for (int t = 3; t >= 0; t--) {
    const int half = 8 >> t;
    if (kMode == kArithFp) fp_reduce_masked<W, kMode>(x, plan.before[t], ar);
#pragma unroll
    for (int g = 0; g < (1 << t); g++) {
      W w0, w1;
      if constexpr (kPacked) {
        w0 = lane_tw_fp<W>(twi, t, g);
        w1 = ar.quotient(w0);
      } else {
        const auto w = load_tw<W, kGlobalTw>(twi, tw_index<kLaneTable>(S, t, g));
        w0 = w.x;
        w1 = w.y;
      }
#pragma unroll
      for (int k = 0; k < half; k++) {
        const int j = g * 2 * half + k;
        ar.inv(x[j], x[j + half], w0, w1, kLayer0 + 3 - t);
      }
    }
  }
}

// Level 0 of the inverse transform (S = 1, layers 4..7 of the column pass): the last layer
// also multiplies by N^-1 and reduces to [0, q).
template <typename W, int kMode, int kBin = 0>
__device__ __forceinline__ void radix16_inv_final(W (&x)[16], const typename WordTraits<W>::Pair* twi,
                                                  const PrimeConst<W>& pc, const Arith<W, kMode>& ar) {
  constexpr FpInvPlan plan = fp_plan_inv(kBin);
#pragma unroll
  for (int t = 3; t >= 1; t--) {
    const int half = 8 >> t;
    if (kMode == kArithFp) fp_reduce_masked<W, kMode>(x, plan.before[t], ar);
#pragma unroll
    for (int g = 0; g < (1 << t); g++) {
      const auto w = twi[(1u << t) + g];
#pragma unroll
      for (int k = 0; k < half; k++) {
        const int j = g * 2 * half + k;
        ar.inv(x[j], x[j + half], w.x, w.y, 4 + 3 - t);
      }
    }
  }
  if (kMode == kArithFp) fp_reduce_masked<W, kMode>(x, plan.before[0], ar);
#pragma unroll
  for (int j = 0; j < 8; j++) ar.inv_last(x[j], x[j + 8], pc);
}

// Row-pass exchange buffer: one pad word after every 16 keeps both the strided and the
// consecutive access pattern free of bank conflicts.
__device__ __forceinline__ int row_pos(int i) { return i + (i >> 4); }
constexpr int kRowPitch = 256 + 16;

// Staging buffer that turns "each thread owns 16 consecutive words of its row" into
// "consecutive threads own consecutive 16-byte vectors" (and back) without bank conflicts.
// A row is 256 words = kVecPerRow vectors of 16 bytes; thread u owns vectors u * kVecPerThread
// + jj.  Vector v is stored at slot v ^ ((v >> 3) & (kVecPerThread - 1)) of its row: both the
// owner's accesses (8 threads, same jj) and the coalesced accesses (8 consecutive v) then fall
// into 8 different 16-byte bank groups.
template <typename W>
struct RowVec;
template <>
struct RowVec<uint64_t> {
  using Vec = ulonglong2;
  static constexpr int kWords = 2, kPerThread = 8, kPerRow = 128;
};
template <>
struct RowVec<uint32_t> {
  using Vec = uint4;
  static constexpr int kWords = 4, kPerThread = 4, kPerRow = 64;
};
template <typename W>
__device__ __forceinline__ int row_vec_slot(int v) {
  return v ^ ((v >> 3) & (RowVec<W>::kPerThread - 1));
}
__device__ __forceinline__ void vec_unpack(const ulonglong2& v, uint64_t* w) { w[0] = v.x; w[1] = v.y; }
__device__ __forceinline__ void vec_unpack(const uint4& v, uint32_t* w) { w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
__device__ __forceinline__ ulonglong2 vec_pack(const uint64_t* w) { return make_ulonglong2(w[0], w[1]); }
__device__ __forceinline__ uint4 vec_pack(const uint32_t* w) { return make_uint4(w[0], w[1], w[2], w[3]); }

// Runs one of the instantiations of a kernel body: the arithmetic policy of this CTA's prime
// (BODY is a template name taking <W, mode, ...>; ARGS its call arguments in parentheses).
#define CERIUM_TARGS(...) __VA_ARGS__
#define CERIUM_DISPATCH_ARITH(W, pc, BODY, TARGS, ARGS)                   \
  do {                                                                   \
    if constexpr (sizeof(W) == 8) {                                      \
      if ((pc).fp_ok != 0) { BODY<W, kArithFp, TARGS> ARGS; break; }     \
      if ((pc).lazy_ok != 0) { BODY<W, kArithLazy, TARGS> ARGS; break; } \
    }                                                                    \
    BODY<W, kArithStrict, TARGS> ARGS;                                   \
  } while (0)

// ---------------------------------------------------------------------------------------
// forward transform
// ---------------------------------------------------------------------------------------

// What the column pass does with a word it has just read.
template <typename W>
struct PlainLoader {
  static constexpr bool kHasSmall = false;
  static constexpr int kFpBound = kFpCanon;
  __device__ __forceinline__ W apply(W x, int /*b*/, const PrimeConst<W>& /*pc*/) const { return x; }
};

// Source residues belong to another modulus: any word -> [0, q) of the entry's prime.  This is
// the whole base conversion of a one-limb digit (Qhat = 1), fused into the transform's first read.
template <typename W>
struct ModLoader {
  static constexpr int kFpBound = kFpCanon;
  static constexpr bool kHasSmall = true;
  // small[b] != 0: the words of entry b are below 2^50 (their source prime is), so a prime with
  // double-precision butterflies converts and reduces them on the FP64 pipe (5 operations)
  // instead of the integer Shoup reduction
  uint8_t small[kMaxBatch];
  __device__ __forceinline__ W apply(W x, int /*b*/, const PrimeConst<W>& pc) const {
    return reduce_word<W>(x, pc);
  }
};

// Words below 4q, as the ModUp base conversion leaves them for the transform.
template <typename W>
struct LazyLoader {
  static constexpr bool kHasSmall = false;
  static constexpr int kFpBound = kFpLazyIn;
  __device__ __forceinline__ W apply(W x, int /*b*/, const PrimeConst<W>& /*pc*/) const { return x; }
};

constexpr int kSudMaxBatch = 96;  // limbs per launch when per-limb scalars travel as parameters

// Source residues belong to another (possibly larger) modulus src_q: optionally add pre_add
// mod src_q (rounding), reduce into [0, q) of the target prime, optionally subtract
// post_sub[b] mod q.  Used when one coefficient-form limb is re-read under many primes
// (rescale, cerium/compiler/backend/compiler_rescale.cc:262-284).
template <typename W>
struct ReduceLoader {
  static constexpr bool kHasSmall = false;
  static constexpr int kFpBound = kFpCanon;
  W src_q;
  W pre_add;
  W post_sub[kSudMaxBatch];
  __device__ __forceinline__ W apply(W x, int b, const PrimeConst<W>& pc) const {
    W v = csub<W>(x + pre_add, src_q);
    v = reduce_word<W>(v, pc);
    return sub_mod<W>(v, post_sub[b], pc.q);
  }
};

template <typename W, int kMode, typename Batch, typename Loader>
__device__ __forceinline__ void ntt_fwd_cols_body(const Batch& batch, const Loader& loader, int b,
                                                  const PrimeConst<W>& pc, W* tile,
                                                  const typename WordTraits<W>::Pair* stw) {
  constexpr int kCols = NttCfg<W>::kCols;
  const Arith<W, kMode> ar(pc);
  const int tid = threadIdx.x, c = tid % kCols, u = tid / kCols;
  const int col = blockIdx.x * kCols + c;
  // one base pointer per access pattern; the unrolled accesses are then constant offsets from it
  const W* in = batch.in_limb(b) + (unsigned)(u * 256 + col);
  W* out = batch.out_limb(b) + (unsigned)(u * 16 * 256 + col);
  W* t_strided = tile + (unsigned)(u * kCols + c);
  W* t_own = tile + (unsigned)(u * 16 * kCols + c);
  W x[16];
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = in[j * 16 * 256];
  bool entered = false;
  if constexpr (Loader::kHasSmall && kMode == kArithFp) {
    if (loader.small[b] != 0) {
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = ar.reduce(ar.enter(x[j]));
      entered = true;
    }
  }
  if (!entered) {
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] = ar.enter(loader.apply(x[j], b, pc));
  }
  __syncthreads();
  radix16_fwd<W, false, kMode, false, Loader::kFpBound>(x, stw, 1u, ar);
#pragma unroll
  for (int j = 0; j < 16; j++) t_strided[j * 16 * kCols] = x[j];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = t_own[j * kCols];
  radix16_fwd<W, false, kMode, false, fp_plan_fwd(Loader::kFpBound).out>(x, stw, 16u + (uint32_t)u, ar);
#pragma unroll
  for (int j = 0; j < 16; j++) out[j * 256] = x[j];
}

// Column pass (levels 0 and 1).  grid = (256 / kCols, limbs), block = 16 * kCols.
// Element (h, l) of a limb is word h * 256 + l; the CTA owns kCols adjacent columns.
template <typename W, typename Batch, typename Loader>
__global__ void __launch_bounds__(NttCfg<W>::kCols * 16, sizeof(W) == 8 ? 3 : 2)
    ntt_fwd_cols_kernel(const Batch batch, const Loader loader,
                        const typename WordTraits<W>::Pair* __restrict__ tw_all,
                        const PrimeConst<W>* __restrict__ pcs) {
  using Pair = typename WordTraits<W>::Pair;
  constexpr int kCols = NttCfg<W>::kCols;
  __shared__ W tile[256 * kCols];
  __shared__ Pair stw[256];
  grid_dependency_launch();
  const int b = blockIdx.y;
  const uint32_t pi = batch.prime_of(b);
  const PrimeConst<W> pc = pcs[pi];
  if (threadIdx.x < 256) stw[threadIdx.x] = __ldg(tw_all + (size_t)pi * kN + threadIdx.x);
  grid_dependency_wait();
  CERIUM_DISPATCH_ARITH(W, pc, ntt_fwd_cols_body, CERIUM_TARGS(Batch, Loader), (batch, loader, b, pc, tile, stw));
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
#if !defined(CERIUM_EMU)
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
#else
  (void)p;
#endif
}

// What the row pass does with the finished NTT value.  kCanonicalInput says whether the
// epilogue wants the value reduced to [0, q) first or takes it below 4q.
template <typename W>
struct StoreEpilogue {
  static constexpr bool kCanonicalInput = true;
  __device__ __forceinline__ uint32_t scatter_elt() const { return 0u; }
  template <int kWords>
  __device__ __forceinline__ void apply_vec(W (&)[kWords], int, int, uint32_t, const PrimeConst<W>&) const {}
  __device__ __forceinline__ void prefetch(int /*b*/, int /*idx*/) const {}
};

// Stores the transform below 4q.  Only for buffers whose one reader multiplies the values into a
// wide accumulator (the raised digits of a key switch, read by the inner product).
template <typename W>
struct LazyStoreEpilogue {
  static constexpr bool kCanonicalInput = false;
  __device__ __forceinline__ uint32_t scatter_elt() const { return 0u; }
  template <int kWords>
  __device__ __forceinline__ void apply_vec(W (&)[kWords], int, int, uint32_t, const PrimeConst<W>&) const {}
  __device__ __forceinline__ void prefetch(int /*b*/, int /*idx*/) const {}
};

// SuD tail: out = (minuend - NTT(in)) * factor[b] [+ addend]   (all mod q).
// minuend / addend are stacks of limbs: entry b at base + b * stride; entries b >= split belong
// to a second polynomial and use minuend2 / addend2 at (b - split) * stride.
template <typename W>
struct SudEpilogue {
  static constexpr bool kCanonicalInput = false;  // takes the transform below 4q
  const W* minuend;
  const W* minuend2;
  size_t minuend_stride;
  const W* addend;   // may be null
  const W* addend2;  // may be null
  size_t addend_stride;
  int split;         // kSudMaxBatch when there is one polynomial
  uint32_t addend_elt;  // not 0: the addends are read through the Galois automorphism of this element
  uint32_t store_elt;   // not 0: word i of the result is stored at pi(i), the index map of this element, so
                        // the output is the automorphism of the INVERSE element applied to the result
  __device__ __forceinline__ uint32_t scatter_elt() const { return store_elt; }
  W factor[kSudMaxBatch];
  W factor_shoup[kSudMaxBatch];
  // starts the 16 bytes at word idx of the operands towards L2 (called before the transform, whose
  // arithmetic then hides their latency)
  __device__ __forceinline__ void prefetch(int b, int idx) const {
    const bool second = b >= split;
    const int e = second ? b - split : b;
    prefetch_l2((second ? minuend2 : minuend) + (size_t)e * minuend_stride + idx);
    const W* ap = second ? addend2 : addend;
    if (ap != nullptr && addend_elt == 0) prefetch_l2(ap + (size_t)e * addend_stride + idx);
  }
  // The kWords results of one 16-byte vector (idx0 a multiple of kWords): minuend and addend come in
  // as one 16-byte load each.  With an automorphism the aligned group idx0 .. idx0 + kWords - 1 is the
  // image of ONE aligned group of the addend (the index map sends aligned 2^k blocks onto aligned 2^k
  // blocks), so that is one load as well and the words are picked from it.
  template <int kWords>
  __device__ __forceinline__ void apply_vec(W (&w)[kWords], int b, int idx0, uint32_t /*pi*/,
                                            const PrimeConst<W>& pc) const {
    using Vec = typename RowVec<W>::Vec;
    const bool second = b >= split;
    const int e_ = second ? b - split : b;
    const W* mp = (second ? minuend2 : minuend) + (size_t)e_ * minuend_stride;
    const W* ap = second ? addend2 : addend;
    W m[kWords], a[kWords] = {};
    vec_unpack(*reinterpret_cast<const Vec*>(mp + idx0), m);
    if (ap != nullptr) {
      ap += (size_t)e_ * addend_stride;
      if (addend_elt != 0) {
        uint32_t src[kWords];
#pragma unroll
        for (int e = 0; e < kWords; e++) src[e] = galois_source_index((uint32_t)(idx0 + e), addend_elt);
        W t[kWords];
        vec_unpack(*reinterpret_cast<const Vec*>(ap + (src[0] & ~(uint32_t)(kWords - 1))), t);
#pragma unroll
        for (int e = 0; e < kWords; e++) {
          a[e] = t[0];
#pragma unroll
          for (int k = 1; k < kWords; k++)
            if ((src[e] & (uint32_t)(kWords - 1)) == (uint32_t)k) a[e] = t[k];
        }
      } else {
        vec_unpack(*reinterpret_cast<const Vec*>(ap + idx0), a);
      }
    }
#pragma unroll
    for (int e = 0; e < kWords; e++) {
      W d;
      if (sizeof(W) == 4) {
        // 32-bit words hold primes up to 2^30: m + 4q would pass 2^32, so the transform comes below 2q first
        d = m[e] + pc.q2 - csub<W>(w[e], pc.q2);
      } else {
        d = m[e] + (pc.q2 + pc.q2) - w[e];  // w < 4q: positive, and the Shoup product takes any word
      }
      d = csub<W>(mul_shoup_lazy<W>(d, factor[b], factor_shoup[b], pc.q), pc.q);
      if (ap != nullptr) d = add_mod<W>(d, a[e], pc.q);
      w[e] = d;
    }
  }
};

// SuD tail with the argument tables of the reference's launcher (_kernel_sud_1,
// cerium/compiler/backend/kernels/function.cu:123-149): entry b has two inputs, ins[2b] the minuend
// and ins[2b + 1] the coefficient-form limb whose transform is subtracted; factors holds one
// residue per prime of the context, indexed by the entry's prime.
template <typename W>
struct PtrSudEpilogue {
  static constexpr bool kCanonicalInput = false;
  const W* const* ins;
  const W* factors;
  __device__ __forceinline__ uint32_t scatter_elt() const { return 0u; }
  __device__ __forceinline__ void prefetch(int b, int idx) const { prefetch_l2(ins[2 * b] + idx); }
  template <int kWords>
  __device__ __forceinline__ void apply_vec(W (&w)[kWords], int b, int idx0, uint32_t pi,
                                            const PrimeConst<W>& pc) const {
#pragma unroll
    for (int e = 0; e < kWords; e++) w[e] = apply(w[e], b, idx0 + e, pi, pc);  // caller's limbs may be unaligned
  }
  __device__ __forceinline__ W apply(W x, int b, int idx, uint32_t pi, const PrimeConst<W>& pc) const {
    const W m = ins[2 * b][idx];
    // x < 4q and m < q: bring the difference to [0, q) before the Barrett product
    W d = m + pc.q2 - csub<W>(x, pc.q2);  // (m, m + 2q]
    d = csub<W>(csub<W>(d, pc.q2), pc.q);
    return mul_mod<W>(d, csub<W>(factors[pi], pc.q), pc);
  }
};

template <typename W>
__device__ __forceinline__ void store16(W* dst, const W (&x)[16]);
template <>
__device__ __forceinline__ void store16<uint64_t>(uint64_t* dst, const uint64_t (&x)[16]) {
  ulonglong2* d = reinterpret_cast<ulonglong2*>(dst);
#pragma unroll
  for (int j = 0; j < 8; j++) d[j] = make_ulonglong2(x[2 * j], x[2 * j + 1]);
}
template <>
__device__ __forceinline__ void store16<uint32_t>(uint32_t* dst, const uint32_t (&x)[16]) {
  uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int j = 0; j < 4; j++) d[j] = make_uint4(x[4 * j], x[4 * j + 1], x[4 * j + 2], x[4 * j + 3]);
}
template <typename W>
__device__ __forceinline__ void load16(const W* src, W (&x)[16]);
template <>
__device__ __forceinline__ void load16<uint64_t>(const uint64_t* src, uint64_t (&x)[16]) {
  const ulonglong2* s = reinterpret_cast<const ulonglong2*>(src);
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const ulonglong2 v = s[j];
    x[2 * j] = v.x;
    x[2 * j + 1] = v.y;
  }
}
template <>
__device__ __forceinline__ void load16<uint32_t>(const uint32_t* src, uint32_t (&x)[16]) {
  const uint4* s = reinterpret_cast<const uint4*>(src);
#pragma unroll
  for (int j = 0; j < 4; j++) {
    const uint4 v = s[j];
    x[4 * j] = v.x;
    x[4 * j + 1] = v.y;
    x[4 * j + 2] = v.z;
    x[4 * j + 3] = v.w;
  }
}

template <typename W, int kMode, typename Batch, typename Epilogue>
__device__ __forceinline__ void ntt_fwd_rows_body(const Batch& batch, const Epilogue& epi, int b, uint32_t pi,
                                                  const PrimeConst<W>& pc, W* tile,
                                                  const typename WordTraits<W>::Pair* tw,
                                                  const typename WordTraits<W>::Pair* twr) {
  using RV = RowVec<W>;
  using Vec = typename RV::Vec;
  const Arith<W, kMode> ar(pc);
  const int tid = threadIdx.x, r = tid >> 4, u = tid & 15;
  const int h = blockIdx.x * kRowsPerCta + r;
  const W* row = batch.in_limb(b) + (unsigned)(h * 256 + u);
  W* limb_out = batch.out_limb(b);
  W* drow = limb_out + (unsigned)(h * 256);
  const uint32_t selt = epi.scatter_elt();
  W* trow = tile + (unsigned)(r * kRowPitch);
  W* t_strided = trow + u;             // row_pos(j * 16 + u) = j * 17 + u
  W* t_own = trow + (unsigned)(u * 17);  // row_pos(u * 16 + j) = u * 17 + j
  W x[16];
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = row[j * 16];
#pragma unroll
  for (int k = 0; k < RV::kPerThread; k++) epi.prefetch(b, h * 256 + (u + 16 * k) * RV::kWords);
  radix16_fwd<W, true, kMode, false, kFpFwdMid>(x, tw, 256u + (uint32_t)h, ar);
#pragma unroll
  for (int j = 0; j < 16; j++) t_strided[j * 17] = x[j];
  __syncwarp();  // a row's 16 threads share a warp; no other warp touches its staging rows
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = t_own[j];
  // level 3: this thread's 15 twiddles from the lane-interleaved table of row h
  radix16_fwd<W, true, kMode, true, kFpFwdL3>(x, twr + ((size_t)h * (kMode == kArithFp ? 8 : 15) * 16 + u), 0u, ar);
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = ar.template finish_fwd<Epilogue::kCanonicalInput>(x[j], pc.one_shoup);
  // own 16 words -> swizzled vectors -> coalesced vectors, then epilogue and store
  __syncwarp();  // a row's 16 threads share a warp; no other warp touches its staging rows
  Vec* vrow = reinterpret_cast<Vec*>(tile + r * kRowPitch);  // same private region as the exchange rows
#pragma unroll
  for (int jj = 0; jj < RV::kPerThread; jj++)
    vrow[row_vec_slot<W>(u * RV::kPerThread + jj)] = vec_pack(&x[jj * RV::kWords]);
  __syncwarp();  // a row's 16 threads share a warp; no other warp touches its staging rows
#pragma unroll
  for (int k = 0; k < RV::kPerThread; k++) {
    const int v = u + 16 * k;
    W w[RV::kWords];
    vec_unpack(vrow[row_vec_slot<W>(v)], w);
#pragma unroll
    epi.apply_vec(w, b, h * 256 + v * RV::kWords, pi, pc);
    if (selt != 0) {
      // the row's aligned 256-word block lands on one aligned block of the output limb
#pragma unroll
      for (int e = 0; e < RV::kWords; e++)
        limb_out[galois_source_index((uint32_t)(h * 256 + v * RV::kWords + e), selt)] = w[e];
    } else {
      reinterpret_cast<Vec*>(drow)[v] = vec_pack(w);
    }
  }
}

// Row pass (levels 2 and 3): reads the column pass's result from the batch's `in` stack and
// writes the finished transform to its `out` stack (the two may be the same buffer).
// grid = (256 / kRowsPerCta, limbs), block = 16 * kRowsPerCta; 16 threads own one row.
template <typename W, typename Batch, typename Epilogue>
__global__ void __launch_bounds__(kRowsPerCta * 16, 3)
    ntt_fwd_rows_kernel(const Batch batch, const Epilogue epi,
                        const typename WordTraits<W>::Pair* __restrict__ tw_all,
                        const typename WordTraits<W>::Pair* __restrict__ twr_all,
                        const PrimeConst<W>* __restrict__ pcs) {
  using Pair = typename WordTraits<W>::Pair;
  __shared__ __align__(16) W tile[kRowsPerCta * kRowPitch];
  grid_dependency_launch();
  const int b = blockIdx.y;
  const uint32_t pi = batch.prime_of(b);
  const PrimeConst<W> pc = pcs[pi];
  const Pair* tw = tw_all + (size_t)pi * kN;
  const Pair* twr = twr_all + (size_t)pi * kRowTwPerPrime;
  grid_dependency_wait();
  CERIUM_DISPATCH_ARITH(W, pc, ntt_fwd_rows_body, CERIUM_TARGS(Batch, Epilogue), (batch, epi, b, pi, pc, tile, tw, twr));
}

// ---------------------------------------------------------------------------------------
// inverse transform
// ---------------------------------------------------------------------------------------

template <typename W, int kMode, typename Batch>
__device__ __forceinline__ void ntt_inv_rows_body(const Batch& batch, int b, const PrimeConst<W>& pc, W* tile,
                                                  const typename WordTraits<W>::Pair* twi,
                                                  const typename WordTraits<W>::Pair* twri) {
  using RV = RowVec<W>;
  using Vec = typename RV::Vec;
  const Arith<W, kMode> ar(pc);
  const int tid = threadIdx.x, r = tid >> 4, u = tid & 15;
  const int h = blockIdx.x * kRowsPerCta + r;
  const W* limb_in = batch.in_limb(b);
  const W* src = limb_in + h * 256;
  const uint32_t elt = batch.gather_elt();
  W* dst = batch.out_limb(b) + h * 256;
  W* trow = tile + r * kRowPitch;
  // coalesced vectors -> swizzled staging -> own 16 consecutive words
  Vec* vrow = reinterpret_cast<Vec*>(tile + r * kRowPitch);  // same private region as the exchange rows
#pragma unroll
  for (int k = 0; k < RV::kPerThread; k++) {
    const int v = u + 16 * k;
    if (elt != 0) {
      // the automorphism maps the aligned 256-word block of this row onto one aligned block:
      // the gathered words use whole sectors
      W w[RV::kWords];
#pragma unroll
      for (int e = 0; e < RV::kWords; e++)
        w[e] = limb_in[galois_source_index((uint32_t)(h * 256 + v * RV::kWords + e), elt)];
      vrow[row_vec_slot<W>(v)] = vec_pack(w);
    } else {
      vrow[row_vec_slot<W>(v)] = reinterpret_cast<const Vec*>(src)[v];
    }
  }
  __syncwarp();
  W x[16];
#pragma unroll
  for (int jj = 0; jj < RV::kPerThread; jj++)
    vec_unpack(vrow[row_vec_slot<W>(u * RV::kPerThread + jj)], &x[jj * RV::kWords]);
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = ar.enter(x[j]);
  radix16_inv<W, true, kMode, 0, true, kFpCanon>(x, twri + ((size_t)h * (kMode == kArithFp ? 8 : 15) * 16 + u), 0u, ar);
  if (kMode == kArithFp) fp_reduce_masked<W, kMode>(x, kFpInvRowsExMask, ar);
  __syncwarp();
  W* t_own = trow + (unsigned)(u * 17);  // row_pos(u * 16 + j) = u * 17 + j
  W* t_strided = trow + u;             // row_pos(j * 16 + u) = j * 17 + u
#pragma unroll
  for (int j = 0; j < 16; j++) t_own[j] = x[j];
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = t_strided[j * 17];
  radix16_inv<W, true, kMode, 4, false, kFpInvL3>(x, twi, 256u + (uint32_t)h, ar);
  W* dcol = dst + u;
#pragma unroll
  for (int j = 0; j < 16; j++) dcol[j * 16] = x[j];
}

// Row pass (levels 3 and 2): in -> out; values leave in [0, 2q) (strict) or below 2^10 q (lazy).
template <typename W, typename Batch>
__global__ void __launch_bounds__(kRowsPerCta * 16, 3)
    ntt_inv_rows_kernel(const Batch batch, const typename WordTraits<W>::Pair* __restrict__ twi_all,
                        const typename WordTraits<W>::Pair* __restrict__ twri_all,
                        const PrimeConst<W>* __restrict__ pcs) {
  using Pair = typename WordTraits<W>::Pair;
  __shared__ __align__(16) W tile[kRowsPerCta * kRowPitch];
  grid_dependency_launch();
  const int b = blockIdx.y;
  const uint32_t pi = batch.prime_of(b);
  const PrimeConst<W> pc = pcs[pi];
  const Pair* twi = twi_all + (size_t)pi * kN;
  const Pair* twri = twri_all + (size_t)pi * kRowTwPerPrime;
  grid_dependency_wait();
  CERIUM_DISPATCH_ARITH(W, pc, ntt_inv_rows_body, Batch, (batch, b, pc, tile, twi, twri));
}

// Optional per-limb scalar applied to the finished inverse transform (exact base
// conversion wants x * [Qhat^-1] mod q; null = none).
template <typename W>
struct InvScale {
  const W* scale;        // per batch entry, may be null
  const W* scale_shoup;  // per batch entry
};

template <typename W, int kMode, typename Batch>
__device__ __forceinline__ void ntt_inv_cols_body(const Batch& batch, const InvScale<W>& sc, int b,
                                                  const PrimeConst<W>& pc, W* tile,
                                                  const typename WordTraits<W>::Pair* stw) {
  constexpr int kCols = NttCfg<W>::kCols;
  const Arith<W, kMode> ar(pc);
  const W q = pc.q;
  const int tid = threadIdx.x, c = tid % kCols, u = tid / kCols;
  const int col = blockIdx.x * kCols + c;
  W* buf_own = batch.out_limb(b) + (unsigned)(u * 16 * 256 + col);
  W* buf_strided = batch.out_limb(b) + (unsigned)(u * 256 + col);
  W* t_strided = tile + (unsigned)(u * kCols + c);
  W* t_own = tile + (unsigned)(u * 16 * kCols + c);
  W x[16];
#pragma unroll
  for (int j = 0; j < 16; j++) {
    x[j] = buf_own[j * 256];
    if (kMode == kArithLazy) x[j] = reduce_lazy(x[j], pc.one_shoup, (W)0 - pc.q);  // back below 4q for the second pass
  }
  __syncthreads();
  radix16_inv<W, false, kMode, 0, false, kFpInvMid>(x, stw, 16u + (uint32_t)u, ar);
  if (kMode == kArithFp) fp_reduce_masked<W, kMode>(x, kFpInvColsExMask, ar);
#pragma unroll
  for (int j = 0; j < 16; j++) t_own[j * kCols] = x[j];
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 16; j++) x[j] = t_strided[j * 16 * kCols];
  radix16_inv_final<W, kMode, kFpInvL1>(x, stw, pc, ar);
  if (sc.scale != nullptr) {
    const W s = __ldg(sc.scale + b), ss = __ldg(sc.scale_shoup + b);
#pragma unroll
    for (int j = 0; j < 16; j++) x[j] = csub<W>(mul_shoup_lazy<W>(x[j], s, ss, q), q);
  }
#pragma unroll
  for (int j = 0; j < 16; j++) buf_strided[j * 16 * 256] = x[j];
}

// Column pass (levels 1 and 0), in place on the output limb of the row pass; scales by
// N^-1 and reduces to [0, q).
template <typename W, typename Batch>
__global__ void __launch_bounds__(NttCfg<W>::kCols * 16, sizeof(W) == 8 ? 3 : 2)
    ntt_inv_cols_kernel(const Batch batch, const InvScale<W> sc,
                        const typename WordTraits<W>::Pair* __restrict__ twi_all,
                        const PrimeConst<W>* __restrict__ pcs) {
  using Pair = typename WordTraits<W>::Pair;
  constexpr int kCols = NttCfg<W>::kCols;
  __shared__ W tile[256 * kCols];
  __shared__ Pair stw[256];
  grid_dependency_launch();
  const int b = blockIdx.y;
  const uint32_t pi = batch.prime_of(b);
  const PrimeConst<W> pc = pcs[pi];
  if (threadIdx.x < 256) stw[threadIdx.x] = __ldg(twi_all + (size_t)pi * kN + threadIdx.x);
  grid_dependency_wait();
  CERIUM_DISPATCH_ARITH(W, pc, ntt_inv_cols_body, Batch, (batch, sc, b, pc, tile, stw));
}

}  // namespace cerium
