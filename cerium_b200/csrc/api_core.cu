// Context, NTT, SuD, element-wise, automorphism and base-conversion entry points of the C ABI.
// Host code here only validates arguments, fills by-value parameter blocks and launches; the
// arithmetic lives in the *_kernels.cuh headers.  Mirrors the role of
// cerium/runtime/execution/evaluator.cpp (Evaluator::fn_*) and device_utils.cu (execute_*).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "internal.h"

namespace cerium {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename W>
static int fill_batch(cerium_context* ctx, StridedBatch<W>& sb, const uint32_t* pos, const uint32_t* prime,
                      int first, int count) {
  for (int b = 0; b < count; b++) {
    const uint32_t p = prime[first + b];
    if (p >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "prime index out of range");
    const uint32_t s = pos ? pos[first + b] : (uint32_t)(first + b);
    if (s > 0xffffu) return fail(CERIUM_ERR_INVALID, "limb slot exceeds 65535");
    sb.prime[b] = (uint8_t)p;
    sb.pos[b] = (uint16_t)s;
  }
  return CERIUM_OK;
}

static int check_stack(const void* p, size_t stride_words, size_t word_bytes, const char* what,
                       bool allow_zero_stride = false) {
  if (p == nullptr) return fail(CERIUM_ERR_INVALID, std::string(what) + " is null");
  if (!aligned16(p)) return fail(CERIUM_ERR_INVALID, std::string(what) + " is not 16-byte aligned");
  if ((stride_words * word_bytes) % 16) return fail(CERIUM_ERR_INVALID, std::string(what) + " stride is not a multiple of 16 bytes");
  if (!allow_zero_stride && stride_words < (size_t)kN) return fail(CERIUM_ERR_INVALID, std::string(what) + " stride is smaller than N");
  return CERIUM_OK;
}

// ---------------------------------------------------------------------------------------
// NTT launchers
// ---------------------------------------------------------------------------------------

int launch_ntt_forward(cerium_context* ctx, const NttCall& c, cudaStream_t stream, bool lazy_out) {
  if (c.count == 0) return CERIUM_OK;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    constexpr int kCols = NttCfg<W>::kCols;
    for (int first = 0; first < c.count; first += kMaxBatch) {
      const int cnt = std::min(kMaxBatch, c.count - first);
      StridedBatch<W> cols{};
      cols.in = static_cast<const W*>(c.in);
      cols.out = static_cast<W*>(c.out);
      cols.in_stride = c.in_stride;
      cols.out_stride = c.out_stride;
      cols.split = kMaxBatch;
      if (int rc = fill_batch<W>(ctx, cols, c.pos, c.prime, first, cnt)) return rc;
      StridedBatch<W> rows = cols;
      rows.in = static_cast<const W*>(c.out);
      rows.in_stride = c.out_stride;
      if (c.src_pos != nullptr) {
        GatherBatch<W> gb{};
        static_cast<StridedBatch<W>&>(gb) = cols;
        for (int b = 0; b < cnt; b++) {
          if (c.src_pos[first + b] > 0xffffu) return fail(CERIUM_ERR_INVALID, "limb slot exceeds 65535");
          gb.in_pos[b] = (uint16_t)c.src_pos[first + b];
        }
        ModLoader<W> ml{};
        for (int b = 0; b < cnt; b++)
          ml.small[b] = (c.src_prime != nullptr && ctx->moduli[c.src_prime[first + b]] < ((uint64_t)1 << 50)) ? 1 : 0;
        auto kfn = ntt_fwd_cols_kernel<W, GatherBatch<W>, ModLoader<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, gb, ml, static_cast<const Pair*>(ctx->d_tw_fwd), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      } else if (c.lazy_in) {
        auto kfn = ntt_fwd_cols_kernel<W, StridedBatch<W>, LazyLoader<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, cols, LazyLoader<W>{}, static_cast<const Pair*>(ctx->d_tw_fwd), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      } else {
        auto kfn = ntt_fwd_cols_kernel<W, StridedBatch<W>, PlainLoader<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, cols, PlainLoader<W>{}, static_cast<const Pair*>(ctx->d_tw_fwd), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      }
      if (lazy_out) {
        auto kfn = ntt_fwd_rows_kernel<W, StridedBatch<W>, LazyStoreEpilogue<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, stream, rows, LazyStoreEpilogue<W>{}, static_cast<const Pair*>(ctx->d_tw_fwd), static_cast<const Pair*>(ctx->d_twr_fwd), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      } else {
        auto kfn = ntt_fwd_rows_kernel<W, StridedBatch<W>, StoreEpilogue<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, stream, rows, StoreEpilogue<W>{}, static_cast<const Pair*>(ctx->d_tw_fwd), static_cast<const Pair*>(ctx->d_twr_fwd), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      }
    }
    CERIUM_LAUNCH_CHECK("ntt_forward");
    return CERIUM_OK;
  });
}

int launch_ntt_inverse(cerium_context* ctx, const NttCall& c, const void* scale, const void* scale_shoup,
                       cudaStream_t stream) {
  if (c.count == 0) return CERIUM_OK;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    constexpr int kCols = NttCfg<W>::kCols;
    for (int first = 0; first < c.count; first += kMaxBatch) {
      const int cnt = std::min(kMaxBatch, c.count - first);
      StridedBatch<W> sb{};
      sb.in = static_cast<const W*>(c.in);
      sb.out = static_cast<W*>(c.out);
      sb.in_stride = c.in_stride;
      sb.out_stride = c.out_stride;
      sb.split = kMaxBatch;
      sb.in_elt = c.in_galois;
      if (int rc = fill_batch<W>(ctx, sb, c.pos, c.prime, first, cnt)) return rc;
      InvScale<W> sc{};
      if (scale != nullptr) {
        sc.scale = static_cast<const W*>(scale) + first;
        sc.scale_shoup = static_cast<const W*>(scale_shoup) + first;
      }
      if (c.src_pos != nullptr) {
        // entry b reads limb src_pos[b] of `in` and writes limb pos[b] of `out`
        GatherBatch<W> gb{};
        static_cast<StridedBatch<W>&>(gb) = sb;
        for (int b = 0; b < cnt; b++) {
          if (c.src_pos[first + b] > 0xffffu) return fail(CERIUM_ERR_INVALID, "limb slot exceeds 65535");
          gb.in_pos[b] = (uint16_t)c.src_pos[first + b];
        }
        auto kfn = ntt_inv_rows_kernel<W, GatherBatch<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, stream, gb, static_cast<const Pair*>(ctx->d_tw_inv), static_cast<const Pair*>(ctx->d_twr_inv), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      } else {
        auto kfn = ntt_inv_rows_kernel<W, StridedBatch<W>>;
        CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, stream, sb, static_cast<const Pair*>(ctx->d_tw_inv), static_cast<const Pair*>(ctx->d_twr_inv), static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      }
      { auto kfn = ntt_inv_cols_kernel<W, StridedBatch<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, sb, sc, static_cast<const Pair*>(ctx->d_tw_inv), static_cast<const PrimeConst<W>*>(ctx->d_pcs)); }
    }
    CERIUM_LAUNCH_CHECK("ntt_inverse");
    return CERIUM_OK;
  });
}

int launch_sud(cerium_context* ctx, const SudCall& c, cudaStream_t stream) {
  if (c.count == 0) return CERIUM_OK;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    constexpr int kCols = NttCfg<W>::kCols;
    const int bits = ctx->word_bits;
    if (c.split > 0 && c.count > kSudMaxBatch) return fail(CERIUM_ERR_INVALID, "sud: a two-polynomial launch holds at most 96 limbs");
    {
      // the tail reads minuend and addend as 16-byte vectors
      const size_t wb = sizeof(W);
      const uintptr_t ptrs = (uintptr_t)c.minuend | (uintptr_t)c.minuend2 | (uintptr_t)c.addend | (uintptr_t)c.addend2;
      if (ptrs % 16 != 0 || (c.minuend_stride * wb) % 16 != 0 || (c.addend != nullptr && (c.addend_stride * wb) % 16 != 0))
        return fail(CERIUM_ERR_INVALID, "sud: minuend and addend limbs must be 16-byte aligned");
    }
    for (int first = 0; first < c.count; first += kSudMaxBatch) {
      const int cnt = std::min(kSudMaxBatch, c.count - first);
      StridedBatch<W> cols{};
      cols.in = static_cast<const W*>(c.src) + (c.src_stride ? (size_t)first * c.src_stride : 0);
      cols.out = static_cast<W*>(c.work) + (size_t)first * c.work_stride;
      cols.in_stride = c.src_stride;
      cols.out_stride = c.work_stride;
      cols.split = kMaxBatch;
      if (int rc = fill_batch<W>(ctx, cols, nullptr, c.prime + first, 0, cnt)) return rc;
      StridedBatch<W> rows = cols;
      rows.in = cols.out;
      rows.in_stride = c.work_stride;
      rows.out = static_cast<W*>(c.dst) + (size_t)first * c.dst_stride;
      rows.out_stride = c.dst_stride;
      SudEpilogue<W> epi{};
      epi.minuend = static_cast<const W*>(c.minuend) + (size_t)first * c.minuend_stride;
      epi.minuend_stride = c.minuend_stride;
      epi.addend = c.addend ? static_cast<const W*>(c.addend) + (size_t)first * c.addend_stride : nullptr;
      epi.addend_stride = c.addend_stride;
      epi.addend_elt = c.addend_galois;
      epi.store_elt = c.store_galois;
      epi.split = kSudMaxBatch;
      if (c.split > 0) {
        // second polynomial: entry b lands at slot b - split of dst2 (the slot number itself stays b,
        // it also addresses the work stack), so the base is moved back by split limbs
        rows.split = c.split;
        rows.out2 = static_cast<W*>(c.dst2) - (ptrdiff_t)c.split * (ptrdiff_t)c.dst_stride;
        epi.split = c.split;
        epi.minuend2 = static_cast<const W*>(c.minuend2);
        epi.addend2 = static_cast<const W*>(c.addend2);
      }
      for (int b = 0; b < cnt; b++) {
        const uint64_t q = ctx->moduli[c.prime[first + b]];
        const uint64_t f = c.factor[first + b] % q;
        epi.factor[b] = (W)f;
        epi.factor_shoup[b] = (W)host::shoup(f, q, bits);
      }
      const Pair* tw = static_cast<const Pair*>(ctx->d_tw_fwd);
      const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
      if (c.reduce_src) {
        ReduceLoader<W> ld{};
        ld.src_q = (W)c.src_q;
        ld.pre_add = (W)c.pre_add;
        for (int b = 0; b < cnt; b++) ld.post_sub[b] = c.post_sub ? (W)c.post_sub[first + b] : (W)0;
        if (c.src_pos != nullptr) {
          GatherBatch<W> gb{};
          static_cast<StridedBatch<W>&>(gb) = cols;
          gb.in = static_cast<const W*>(c.src);
          for (int b = 0; b < cnt; b++) gb.in_pos[b] = (uint16_t)c.src_pos[first + b];
          auto kfn = ntt_fwd_cols_kernel<W, GatherBatch<W>, ReduceLoader<W>>;
          CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, gb, ld, tw, pcs);
        } else {
          auto kfn = ntt_fwd_cols_kernel<W, StridedBatch<W>, ReduceLoader<W>>;
          CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, cols, ld, tw, pcs);
        }
      } else {
        { auto kfn = ntt_fwd_cols_kernel<W, StridedBatch<W>, PlainLoader<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, stream, cols, PlainLoader<W>{}, tw, pcs); }
      }
      { auto kfn = ntt_fwd_rows_kernel<W, StridedBatch<W>, SudEpilogue<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, stream, rows, epi, tw, static_cast<const Pair*>(ctx->d_twr_fwd), pcs); }
    }
    CERIUM_LAUNCH_CHECK("sud");
    return CERIUM_OK;
  });
}

// ---------------------------------------------------------------------------------------
// base conversion
// ---------------------------------------------------------------------------------------

// Packs several small tables into one device allocation: append() returns the byte offset
// of a 16-byte aligned copy of the data.
struct Blob {
  std::vector<char> bytes;
  size_t append(const void* p, size_t n) {
    const size_t off = bytes.size();
    bytes.resize(off + (n + 15) / 16 * 16, 0);
    if (n) std::memcpy(bytes.data() + off, p, n);
    return off;
  }
  template <typename W>
  size_t append_words(const std::vector<uint64_t>& v) {
    std::vector<W> t(v.size());
    for (size_t i = 0; i < v.size(); i++) t[i] = (W)v[i];
    return append(t.data(), t.size() * sizeof(W));
  }
};

int create_bconv(cerium_context* ctx, cerium_bconv** out, int mode, const uint32_t* in_primes, int n_in,
                 const uint32_t* out_primes, int n_out, const BconvOptions& opt) {
  if (!ctx || !out || !in_primes || !out_primes) return fail(CERIUM_ERR_INVALID, "bconv_create: null argument");
  if (mode != CERIUM_BCONV_LAZY && mode != CERIUM_BCONV_EXACT) return fail(CERIUM_ERR_INVALID, "bconv_create: unknown mode");
  if (n_in < 1 || n_in > 64 || n_out < 1 || n_out > 255) return fail(CERIUM_ERR_INVALID, "bconv_create: need 1..64 inputs and 1..255 outputs");
  if (!opt.out_pos.empty() && (int)opt.out_pos.size() != n_out) return fail(CERIUM_ERR_INVALID, "bconv_create: out_pos size");
  if (!opt.in_pos.empty() && (int)opt.in_pos.size() != n_in) return fail(CERIUM_ERR_INVALID, "bconv_create: in_pos size");
  for (int i = 0; i < n_in; i++)
    if (in_primes[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "bconv_create: input prime index out of range");
  for (int j = 0; j < n_out; j++)
    if (out_primes[j] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "bconv_create: output prime index out of range");
  // the unreduced sum of products must fit the two-word accumulator
  for (int j = 0; j < n_out; j++) {
    long double sum = 0;
    for (int i = 0; i < n_in; i++) sum += (long double)ctx->moduli[in_primes[i]] * (long double)ctx->moduli[out_primes[j]];
    if (sum >= (ctx->word_bits == 32 ? 1.8e19L : 3.4e38L))
      return fail(CERIUM_ERR_UNSUPPORTED, "bconv_create: too many inputs for primes this wide (sum of products overflows)");
  }
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "bconv_create: cannot select device");
  auto* bc = new cerium_bconv();
  bc->ctx = ctx;
  bc->mode = mode;
  bc->lazy_out = opt.lazy_out;
  bc->I = n_in;
  bc->O = n_out;
  bc->in_primes.assign(in_primes, in_primes + n_in);
  bc->out_primes.assign(out_primes, out_primes + n_out);
  const auto& m = ctx->moduli;
  const int bits = ctx->word_bits;
  // [Qhat_i^-1]_{q_i}
  std::vector<uint64_t> inv(n_in), inv_shoup(n_in);
  for (int i = 0; i < n_in; i++) {
    const uint64_t qi = m[in_primes[i]];
    uint64_t p = 1 % qi;
    for (int k = 0; k < n_in; k++)
      if (k != i) p = host::mulmod(p, m[in_primes[k]] % qi, qi);
    inv[i] = host::invmod(p, qi);
    if (qi > 1 && inv[i] == 0 && n_in > 1) {
      delete bc;
      return fail(CERIUM_ERR_INVALID, "bconv_create: input primes are not pairwise distinct");
    }
    if (n_in == 1) inv[i] = 1;
    inv_shoup[i] = host::shoup(inv[i], qi, bits);
  }
  bc->inv_host = inv;
  std::vector<uint64_t> factors((size_t)n_out * n_in);
  for (int j = 0; j < n_out; j++) {
    const uint64_t pj = m[out_primes[j]];
    for (int i = 0; i < n_in; i++) {
      uint64_t qhat = 1 % pj;
      for (int k = 0; k < n_in; k++)
        if (k != i) qhat = host::mulmod(qhat, m[in_primes[k]] % pj, pj);
      factors[(size_t)j * n_in + i] =
          mode == CERIUM_BCONV_LAZY ? host::mulmod(inv[i] % pj, qhat, pj) : qhat;
    }
  }
  std::vector<uint64_t> in_add, out_sub;
  if (opt.round_half) {
    // floor(P/2) = (P-1)/2 for odd P = prod of input primes
    in_add.resize(n_in);
    out_sub.resize(n_out);
    std::vector<uint32_t> idx(in_primes, in_primes + n_in);
    auto half_mod = [&](uint64_t q) {
      const uint64_t p = host::product_mod(m, idx, q);
      const uint64_t pm1 = (p + q - 1 % q) % q;
      return host::mulmod(pm1, host::invmod(2, q), q);
    };
    for (int i = 0; i < n_in; i++) {
      in_add[i] = half_mod(m[in_primes[i]]);
      // inputs that arrive pre-scaled by [Qhat_i^-1] need the rounding term scaled alike:
      // (x + h) * inv = x * inv + h * inv  (mod q_i)
      if (mode == CERIUM_BCONV_EXACT && opt.prescaled) in_add[i] = host::mulmod(in_add[i], inv[i], m[in_primes[i]]);
    }
    for (int j = 0; j < n_out; j++) out_sub[j] = half_mod(m[out_primes[j]]);
  }
  // 64-bit words, at most 8 inputs: outputs may take their quotient from the FP64 pipe.  The estimate
  // c ~ sum_i y_i f_i / p_j (f_i centred) is off by at most e = (I + 2) 2^-53 sum_i q_i |f_i| / p_j + 1/2
  // (rounding of RN(f_i / p_j), of y_i as a double, of every partial sum; then rounding to an integer),
  // so |sum - c p_j| <= e p_j: class 1 when that is below 3 p_j, class 2 when it is below 2^62.
  bc->fp_in = bits == 64 && n_in <= kBconvRegInputs && ctx->allow_fp;
  std::vector<uint8_t> fp_class(n_out, 0);
  if (bc->fp_in) {
    bool any = false;
    for (int j = 0; j < n_out; j++) {
      const uint64_t pj = m[out_primes[j]];
      long double b = 0.0L;
      for (int i = 0; i < n_in; i++) {
        const uint64_t f = factors[(size_t)j * n_in + i];
        const uint64_t mag = f > pj / 2 ? pj - f : f;
        b += (long double)m[in_primes[i]] * (long double)mag / (long double)pj;
      }
      const long double e = (long double)(n_in + 2) * b * 0x1p-53L + 0.5L;
      if (e < 2.9L) fp_class[j] = 1;
      else if ((e + 1.0L) * (long double)pj < 0x1p62L) fp_class[j] = 2;
      any = any || fp_class[j] != 0;
    }
    bc->fp_in = any;
  }
  const bool use_inv = mode == CERIUM_BCONV_EXACT && !opt.prescaled && n_in > 1;
  Blob blob;
  size_t o_fac = 0, o_inv = 0, o_invs = 0, o_add = 0, o_sub = 0;
  dispatch_word(bits, [&](auto tag) -> int {
    using W = decltype(tag);
    o_fac = blob.append_words<W>(factors);
    o_inv = blob.append_words<W>(inv);
    o_invs = blob.append_words<W>(inv_shoup);
    o_add = blob.append_words<W>(in_add);
    o_sub = blob.append_words<W>(out_sub);
    return 0;
  });
  size_t o_outc = 0, o_split = 0, o_fpfac = 0;
  const bool split = bits == 64 && n_in <= kBconvRegInputs;
  dispatch_word(bits, [&](auto tag) -> int {
    using W = decltype(tag);
    std::vector<BconvOut<W>> outc(n_out);
    for (int j = 0; j < n_out; j++) {
      const uint32_t pj = out_primes[j];
      BconvOut<W>& o = outc[j];
      std::memset(&o, 0, sizeof(o));
      o.q = (W)m[pj];
      o.q2 = (W)(2 * m[pj]);
      o.mu_hi = (W)ctx->mu_hi[pj];
      o.mu_lo = (W)ctx->mu_lo[pj];
      o.sub = out_sub.empty() ? (W)0 : (W)out_sub[j];
      o.pos = opt.out_pos.empty() ? (uint32_t)j : opt.out_pos[j];
      o.has_sub = out_sub.empty() ? 0 : 1;
      o.strict = (ctx->lazy_ok[pj] && !ctx->fp_ok[pj]) ? 0 : 1;
      o.fp = (split && bc->fp_in) ? fp_class[j] : 0;
      const double qinv = 1.0 / (double)m[pj];
      uint64_t qinv_bits;
      std::memcpy(&qinv_bits, &qinv, 8);
      o.fp_qinv = (W)qinv_bits;
    }
    o_outc = blob.append(outc.data(), outc.size() * sizeof(BconvOut<W>));
    return 0;
  });
  if (split) {
    std::vector<uint2> sf(factors.size());
    std::vector<double2> ff(factors.size());
    for (size_t k = 0; k < factors.size(); k++) {
      const uint64_t f = factors[k], q = m[out_primes[k / n_in]];
      sf[k] = make_uint2((uint32_t)f & 0x3fffffffu, (uint32_t)(f >> 30));
      // centred factor (as the bit pattern of an int64) and its quotient by q rounded to a double
      const long long fc = f > q / 2 ? -(long long)(q - f) : (long long)f;
      double fbits;
      std::memcpy(&fbits, &fc, 8);
      ff[k] = make_double2(fbits, (double)((long double)fc / (long double)q));
    }
    o_split = blob.append(sf.data(), sf.size() * sizeof(uint2));
    o_fpfac = blob.append(ff.data(), ff.size() * sizeof(double2));
  }
  const size_t o_ip = blob.append(bc->in_primes.data(), bc->in_primes.size() * 4);
  const size_t o_op = blob.append(bc->out_primes.data(), bc->out_primes.size() * 4);
  const size_t o_pos = blob.append(opt.out_pos.data(), opt.out_pos.size() * 4);
  const size_t o_ipos = blob.append(opt.in_pos.data(), opt.in_pos.size() * 4);
  if (cudaMalloc(&bc->d_block, blob.bytes.size() + 16) != cudaSuccess) {
    delete bc;
    return fail(CERIUM_ERR_CUDA, "bconv_create: cudaMalloc failed");
  }
  if (cudaMemcpy(bc->d_block, blob.bytes.data(), blob.bytes.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaFree(bc->d_block);
    delete bc;
    return fail(CERIUM_ERR_CUDA, "bconv_create: upload failed");
  }
  char* base = static_cast<char*>(bc->d_block);
  bc->d_factors = base + o_fac;
  bc->d_outc = base + o_outc;
  bc->d_split_fac = split ? base + o_split : nullptr;
  bc->d_fp_fac = (split && bc->fp_in) ? base + o_fpfac : nullptr;
  bc->d_inv = use_inv ? base + o_inv : nullptr;
  bc->d_inv_shoup = use_inv ? base + o_invs : nullptr;
  bc->d_in_add = in_add.empty() ? nullptr : base + o_add;
  bc->d_out_sub = out_sub.empty() ? nullptr : base + o_sub;
  bc->d_in_prime = reinterpret_cast<uint32_t*>(base + o_ip);
  bc->d_out_prime = reinterpret_cast<uint32_t*>(base + o_op);
  bc->d_out_pos = opt.out_pos.empty() ? nullptr : reinterpret_cast<uint32_t*>(base + o_pos);
  bc->d_in_pos = opt.in_pos.empty() ? nullptr : reinterpret_cast<uint32_t*>(base + o_ipos);
  *out = bc;
  return CERIUM_OK;
}

int launch_bconv(cerium_context* ctx, const BconvCall* calls, int count, cudaStream_t stream) {
  if (count == 0) return CERIUM_OK;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    static bool smem_opt_in[kMaxDevices][2] = {};  // the attribute is per device
    for (int first = 0; first < count; first += kBconvMaxBatch) {
      const int cnt = std::min(kBconvMaxBatch, count - first);
      BconvBatch<W> batch{};
      size_t smem = 0;
      int max_o = 1;
      bool pair = sizeof(W) == 4;  // two coefficients per thread (see bconv_body_pair32)
      for (int k = 0; k < cnt; k++) {
        const BconvCall& c = calls[first + k];
        const cerium_bconv* bc = c.bc;
        BconvDesc<W>& d = batch.d[k];
        d.in = static_cast<const W*>(c.in);
        d.out = static_cast<W*>(c.out);
        d.in_stride = c.in_stride;
        d.out_stride = c.out_stride;
        d.factors = static_cast<const W*>(bc->d_factors);
        d.inv = static_cast<const W*>(bc->d_inv);
        d.inv_shoup = static_cast<const W*>(bc->d_inv_shoup);
        d.in_add = static_cast<const W*>(bc->d_in_add);
        d.out_sub = static_cast<const W*>(bc->d_out_sub);
        d.in_prime = bc->d_in_prime;
        d.out_prime = bc->d_out_prime;
        d.out_pos = bc->d_out_pos;
        d.in_pos = bc->d_in_pos;
        d.outc = static_cast<const BconvOut<W>*>(bc->d_outc);
        d.split_fac = static_cast<const uint2*>(bc->d_split_fac);
        d.fp_fac = static_cast<const double2*>(bc->d_fp_fac);
        d.lazy_out = bc->lazy_out ? 1 : 0;
        d.fp_in = bc->fp_in ? 1 : 0;
        d.I = bc->I;
        d.O = bc->O;
        smem = std::max(smem, bconv_smem_bytes<W>(bc->I, bc->O));
        max_o = std::max(max_o, bc->O);
        pair = pair && bc->I <= kBconvRegInputs && ((uintptr_t)c.in | (uintptr_t)c.out) % 8 == 0 &&
               (c.in_stride * sizeof(W)) % 8 == 0 && (c.out_stride * sizeof(W)) % 8 == 0;
      }
      if (smem > 48 * 1024) {
        if (smem > 200 * 1024) return fail(CERIUM_ERR_UNSUPPORTED, "bconv: conversion needs more than 200 KiB of shared memory");
        const int slot = sizeof(W) == 4 ? 0 : 1;
        const int dev = ctx->device;
        if (dev < 0 || dev >= kMaxDevices || !smem_opt_in[dev][slot]) {
          CERIUM_CUDA(cudaFuncSetAttribute(bconv_kernel<W, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
          CERIUM_CUDA(cudaFuncSetAttribute(bconv_kernel<W, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
          if (dev >= 0 && dev < kMaxDevices) smem_opt_in[dev][slot] = true;
        }
      }
      {
        // grid.z splits the outputs of a conversion over nz CTAs (each reloads the inputs and restages its
        // tables): take the nz in 1..4 with the best waves x per-CTA-work estimate on this GPU
        auto kfn = pair ? bconv_kernel<W, true> : bconv_kernel<W, false>;
        const int blocks = pair ? (kBconvBlocks + 1) / 2 : kBconvBlocks;
        const int slots = 5 * ctx->sm_count;
        int nz = 1;
        double best = 1e30;
        for (int cand = 1; cand <= std::min(4, (max_o + 3) / 4); cand++) {
          const int ctas = blocks * cnt * cand;
          const double cost = (double)((ctas + slots - 1) / slots) * (1.0 / cand + 0.15);
          if (cost < best - 1e-9) {
            best = cost;
            nz = cand;
          }
        }
        const int out_chunk = (max_o + nz - 1) / nz;
        CERIUM_LAUNCH(kfn, dim3(blocks, cnt, (max_o + out_chunk - 1) / out_chunk), kBconvThreads, smem, stream,
                      batch, out_chunk, static_cast<const PrimeConst<W>*>(ctx->d_pcs));
      }
    }
    CERIUM_LAUNCH_CHECK("bconv");
    return CERIUM_OK;
  });
}

}  // namespace cerium

using namespace cerium;

// ---------------------------------------------------------------------------------------
// extern "C"
// ---------------------------------------------------------------------------------------

extern "C" {

int cerium_version(void) { return 100; }

const char* cerium_last_error(void) { return g_last_error.c_str(); }

int cerium_context_create(cerium_context** out, int device, int log_n, int word_bits, const uint64_t* moduli,
                          int n_moduli) {
  if (!out || !moduli) return fail(CERIUM_ERR_INVALID, "context_create: null argument");
  if (log_n != kLogN) return fail(CERIUM_ERR_UNSUPPORTED, "context_create: only log_n = 16 is built");
  if (word_bits != 32 && word_bits != 64) return fail(CERIUM_ERR_INVALID, "context_create: word_bits must be 32 or 64");
  if (n_moduli < 1 || n_moduli > 255) return fail(CERIUM_ERR_INVALID, "context_create: need 1..255 moduli");
  const uint64_t limit = word_bits == 32 ? ((uint64_t)1 << 30) : ((uint64_t)1 << 60);
  for (int k = 0; k < n_moduli; k++) {
    if (moduli[k] >= limit) return fail(CERIUM_ERR_INVALID, "context_create: modulus too large for the word size");
    if (!host::is_prime(moduli[k]) || (moduli[k] - 1) % ((uint64_t)2 << log_n))
      return fail(CERIUM_ERR_INVALID, "context_create: modulus is not a prime congruent to 1 mod 2N");
    for (int j = 0; j < k; j++)
      if (moduli[j] == moduli[k]) return fail(CERIUM_ERR_INVALID, "context_create: duplicate modulus");
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
    return fail(CERIUM_ERR_CUDA, "context_create: no CUDA device (this library has no CPU path)");
  if (device < 0 || device >= ndev) return fail(CERIUM_ERR_INVALID, "context_create: device out of range");
  DeviceGuard guard(device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "context_create: cannot select device");
  auto* ctx = new cerium_context();
  ctx->device = device;
  ctx->logn = log_n;
  ctx->word_bits = word_bits;
  ctx->n_primes = n_moduli;
  ctx->moduli.assign(moduli, moduli + n_moduli);
  ctx->psi.resize(n_moduli);
  if (cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || ctx->sm_count < 1) {
    delete ctx;
    return fail(CERIUM_ERR_CUDA, "context_create: cannot read the number of SMs");
  }
  if (const char* arith = std::getenv("CERIUM_B200_NTT_ARITH")) ctx->allow_fp = std::strcmp(arith, "int") != 0;
  const size_t n = kN;
  int rc = dispatch_word(word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    std::vector<Pair> fwd(n * n_moduli), inv(n * n_moduli);
    std::vector<Pair> rfwd((size_t)kRowTwPerPrime * n_moduli), rinv((size_t)kRowTwPerPrime * n_moduli);
    std::vector<PrimeConst<W>> pcs(n_moduli);
    for (int k = 0; k < n_moduli; k++) {
      const uint64_t q = moduli[k];
      host::PrimeTables t = host::build_prime_tables(q, log_n, word_bits);
      ctx->psi[k] = t.psi;
      // primes below 2^50 run their butterflies on doubles: the tables then hold the centred
      // twiddle and its correctly rounded quotient by q instead of the twiddle and its Shoup word
      const bool fp = word_bits == 64 && q < ((uint64_t)1 << 50) && ctx->allow_fp;
      auto fp_pair = [&](uint64_t w) {
        const double wd = w > q / 2 ? -(double)(q - w) : (double)w;
        const double wq = wd / (double)q;
        uint64_t a, b;
        std::memcpy(&a, &wd, 8);
        std::memcpy(&b, &wq, 8);
        return WordTraits<W>::make((W)a, (W)b);
      };
      for (size_t i = 0; i < n; i++) {
        if (fp) {
          fwd[k * n + i] = fp_pair(t.w[i]);
          inv[k * n + i] = fp_pair(t.wi[i]);
        } else {
          fwd[k * n + i] = WordTraits<W>::make((W)t.w[i], (W)host::shoup(t.w[i], q, word_bits));
          inv[k * n + i] = WordTraits<W>::make((W)t.wi[i], (W)host::shoup(t.wi[i], q, word_bits));
        }
      }
      for (int h = 0; h < 256; h++)
        for (int t = 0; t < 4; t++)
          for (int g = 0; g < (1 << t); g++)
            for (int u = 0; u < 16; u++) {
              const size_t src = k * n + (((size_t)(4096 + 16 * h + u)) << t) + g;
              if (fp) {
                // twiddles only (the kernel computes their quotients), two per entry: double number
                // 2^t + g of the group's 16 (see lane_tw_fp)
                const int slot = (1 << t) + g;
                const size_t dst = (size_t)k * kRowTwPerPrime + ((size_t)h * 8 + (slot >> 1)) * 16 + u;
                if (slot & 1) {
                  rfwd[dst].y = fwd[src].x;
                  rinv[dst].y = inv[src].x;
                } else {
                  rfwd[dst].x = fwd[src].x;
                  rinv[dst].x = inv[src].x;
                }
              } else {
                const size_t dst = (size_t)k * kRowTwPerPrime + ((size_t)h * 15 + ((1 << t) - 1 + g)) * 16 + u;
                rfwd[dst] = fwd[src];
                rinv[dst] = inv[src];
              }
            }
      PrimeConst<W>& pc = pcs[k];
      std::memset(&pc, 0, sizeof(pc));
      pc.q = (W)q;
      pc.q2 = (W)(2 * q);
      pc.mu_hi = (W)t.mu_hi;
      pc.mu_lo = (W)t.mu_lo;
      pc.one_shoup = (W)host::shoup(1, q, word_bits);
      pc.ninv = (W)t.ninv;
      pc.ninv_shoup = (W)host::shoup(t.ninv, q, word_bits);
      const uint64_t w1 = host::mulmod(t.wi[1], t.ninv, q);
      pc.w1ninv = (W)w1;
      pc.w1ninv_shoup = (W)host::shoup(w1, q, word_bits);
      pc.lazy_ok = (W)((word_bits == 64 && q < ((uint64_t)1 << 52)) ? 1 : 0);
      ctx->mu_hi.push_back(t.mu_hi);
      ctx->mu_lo.push_back(t.mu_lo);
      ctx->lazy_ok.push_back(pc.lazy_ok != 0 ? 1 : 0);
      ctx->fp_ok.push_back(fp ? 1 : 0);
      if (fp) {
        const double qinv = 1.0 / (double)q;
        uint64_t bits;
        std::memcpy(&bits, &qinv, 8);
        pc.fp_ok = 1;
        pc.fp_qinv = (W)bits;
        const auto ni = fp_pair(t.ninv), w1 = fp_pair(host::mulmod(t.wi[1], t.ninv, q));
        pc.fp_ninv = ni.x;
        pc.fp_ninv_q = ni.y;
        pc.fp_w1ninv = w1.x;
        pc.fp_w1ninv_q = w1.y;
      }
    }
    CERIUM_CUDA(cudaMalloc(&ctx->d_tw_fwd, fwd.size() * sizeof(Pair)));
    CERIUM_CUDA(cudaMalloc(&ctx->d_tw_inv, inv.size() * sizeof(Pair)));
    CERIUM_CUDA(cudaMalloc(&ctx->d_pcs, pcs.size() * sizeof(PrimeConst<W>)));
    CERIUM_CUDA(cudaMalloc(&ctx->d_twr_fwd, rfwd.size() * sizeof(Pair)));
    CERIUM_CUDA(cudaMalloc(&ctx->d_twr_inv, rinv.size() * sizeof(Pair)));
    CERIUM_CUDA(cudaMalloc(reinterpret_cast<void**>(&ctx->d_status), 16));
    CERIUM_CUDA(cudaMemset(ctx->d_status, 0, 16));
    CERIUM_CUDA(cudaMemcpy(ctx->d_twr_fwd, rfwd.data(), rfwd.size() * sizeof(Pair), cudaMemcpyHostToDevice));
    CERIUM_CUDA(cudaMemcpy(ctx->d_twr_inv, rinv.data(), rinv.size() * sizeof(Pair), cudaMemcpyHostToDevice));
    CERIUM_CUDA(cudaMemcpy(ctx->d_tw_fwd, fwd.data(), fwd.size() * sizeof(Pair), cudaMemcpyHostToDevice));
    CERIUM_CUDA(cudaMemcpy(ctx->d_tw_inv, inv.data(), inv.size() * sizeof(Pair), cudaMemcpyHostToDevice));
    CERIUM_CUDA(cudaMemcpy(ctx->d_pcs, pcs.data(), pcs.size() * sizeof(PrimeConst<W>), cudaMemcpyHostToDevice));
    return CERIUM_OK;
  });
  if (rc != CERIUM_OK) {
    cerium_context_destroy(ctx);
    return rc;
  }
  *out = ctx;
  return CERIUM_OK;
}

int cerium_context_destroy(cerium_context* ctx) {
  if (!ctx) return CERIUM_OK;
  DeviceGuard guard(ctx->device);
  cudaFree(ctx->d_tw_fwd);
  cudaFree(ctx->d_tw_inv);
  cudaFree(ctx->d_pcs);
  cudaFree(ctx->d_twr_fwd);
  cudaFree(ctx->d_twr_inv);
  cudaFree(ctx->d_status);
  delete ctx;
  return CERIUM_OK;
}

int cerium_context_check(cerium_context* ctx) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "context_check: null context");
  DeviceGuard guard(ctx->device);
  uint32_t st = 0;
  CERIUM_CUDA(cudaMemcpy(&st, ctx->d_status, sizeof(st), cudaMemcpyDeviceToHost));  // waits for the device's work
  if (st == 0) return CERIUM_OK;
  CERIUM_CUDA(cudaMemset(ctx->d_status, 0, sizeof(st)));
  std::string msg = "context_check:";
  if (st & kStatusBconvShape) msg += " a base-conversion table entry exceeded the shape bounds of its launch (that conversion was skipped);";
  if (st & ~kStatusBconvShape) msg += " unknown status bits;";
  return fail(CERIUM_ERR_INVALID, msg);
}

int cerium_context_word_bits(const cerium_context* ctx) { return ctx ? ctx->word_bits : 0; }
int cerium_context_num_moduli(const cerium_context* ctx) { return ctx ? ctx->n_primes : 0; }
uint64_t cerium_context_modulus(const cerium_context* ctx, int k) {
  return (ctx && k >= 0 && k < ctx->n_primes) ? ctx->moduli[k] : 0;
}
uint64_t cerium_context_root(const cerium_context* ctx, int k) {
  return (ctx && k >= 0 && k < ctx->n_primes) ? ctx->psi[k] : 0;
}

static int ntt_common(cerium_context* ctx, bool forward, void* out, size_t out_stride, const void* in,
                      size_t in_stride, const uint32_t* prime_idx, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "ntt: null context");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "ntt: negative count");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx) return fail(CERIUM_ERR_INVALID, "ntt: null prime_idx");
  if (count > 65536) return fail(CERIUM_ERR_INVALID, "ntt: more than 65536 limbs in one call");
  if (int rc = check_stack(out, out_stride, ctx->word_bytes(), "ntt: out")) return rc;
  if (int rc = check_stack(in, in_stride, ctx->word_bytes(), "ntt: in")) return rc;
  DeviceGuard guard(ctx->device);
  NttCall c{in, out, in_stride, out_stride, nullptr, prime_idx, count};
  return forward ? launch_ntt_forward(ctx, c, (cudaStream_t)stream)
                 : launch_ntt_inverse(ctx, c, nullptr, nullptr, (cudaStream_t)stream);
}

int cerium_ntt_forward(cerium_context* ctx, void* out, size_t out_stride, const void* in, size_t in_stride,
                       const uint32_t* prime_idx, int count, void* stream) {
  return ntt_common(ctx, true, out, out_stride, in, in_stride, prime_idx, count, stream);
}

int cerium_ntt_inverse(cerium_context* ctx, void* out, size_t out_stride, const void* in, size_t in_stride,
                       const uint32_t* prime_idx, int count, void* stream) {
  return ntt_common(ctx, false, out, out_stride, in, in_stride, prime_idx, count, stream);
}

static int ntt_ptrs_common(cerium_context* ctx, bool forward, void* const* outs, const void* const* ins,
                           const uint32_t* bases, size_t num_bases, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "ntt_ptrs: null context");
  if (num_bases == 0) return CERIUM_OK;
  if (!outs || !ins || !bases) return fail(CERIUM_ERR_INVALID, "ntt_ptrs: null table");
  if (num_bases > 65535) return fail(CERIUM_ERR_INVALID, "ntt_ptrs: more than 65535 limbs in one call");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    constexpr int kCols = NttCfg<W>::kCols;
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    PointerBatch<W> pb{reinterpret_cast<W* const*>(outs), reinterpret_cast<const W* const*>(ins), bases, 1, 0};
    PointerBatch<W> inplace{reinterpret_cast<W* const*>(outs), reinterpret_cast<const W* const*>(outs), bases, 1, 0};
    const int cnt = (int)num_bases;
    if (forward) {
      const Pair* tw = static_cast<const Pair*>(ctx->d_tw_fwd);
      { auto kfn = ntt_fwd_cols_kernel<W, PointerBatch<W>, PlainLoader<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, s, pb, PlainLoader<W>{}, tw, pcs); }
      { auto kfn = ntt_fwd_rows_kernel<W, PointerBatch<W>, StoreEpilogue<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, s, inplace, StoreEpilogue<W>{}, tw, static_cast<const Pair*>(ctx->d_twr_fwd), pcs); }
    } else {
      const Pair* tw = static_cast<const Pair*>(ctx->d_tw_inv);
      { auto kfn = ntt_inv_rows_kernel<W, PointerBatch<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, s, pb, tw, static_cast<const Pair*>(ctx->d_twr_inv), pcs); }
      { auto kfn = ntt_inv_cols_kernel<W, PointerBatch<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, s, pb, InvScale<W>{}, tw, pcs); }
    }
    CERIUM_LAUNCH_CHECK("ntt_ptrs");
    return CERIUM_OK;
  });
}

int cerium_ntt_forward_ptrs(cerium_context* ctx, void* const* outs, const void* const* ins, const uint32_t* bases,
                            size_t num_bases, void* stream) {
  return ntt_ptrs_common(ctx, true, outs, ins, bases, num_bases, stream);
}

int cerium_ntt_inverse_ptrs(cerium_context* ctx, void* const* outs, const void* const* ins, const uint32_t* bases,
                            size_t num_bases, void* stream) {
  return ntt_ptrs_common(ctx, false, outs, ins, bases, num_bases, stream);
}

int cerium_sud_ptrs(cerium_context* ctx, void* const* outs, const void* const* ins, const uint32_t* bases,
                    size_t num_bases, const void* factors, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "sud_ptrs: null context");
  if (num_bases == 0) return CERIUM_OK;
  if (!outs || !ins || !bases || !factors) return fail(CERIUM_ERR_INVALID, "sud_ptrs: null table");
  if (num_bases > 65535) return fail(CERIUM_ERR_INVALID, "sud_ptrs: more than 65535 limbs in one call");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using Pair = typename WordTraits<W>::Pair;
    constexpr int kCols = NttCfg<W>::kCols;
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    const Pair* tw = static_cast<const Pair*>(ctx->d_tw_fwd);
    const int cnt = (int)num_bases;
    // column pass: second input of every entry -> output limb; row pass in place on the output
    PointerBatch<W> cols{reinterpret_cast<W* const*>(outs), reinterpret_cast<const W* const*>(ins), bases, 2, 1};
    PointerBatch<W> rows{reinterpret_cast<W* const*>(outs), reinterpret_cast<const W* const*>(outs), bases, 1, 0};
    PtrSudEpilogue<W> epi{reinterpret_cast<const W* const*>(ins), static_cast<const W*>(factors)};
    { auto kfn = ntt_fwd_cols_kernel<W, PointerBatch<W>, PlainLoader<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kCols, cnt), kCols * 16, 0, s, cols, PlainLoader<W>{}, tw, pcs); }
    { auto kfn = ntt_fwd_rows_kernel<W, PointerBatch<W>, PtrSudEpilogue<W>>; CERIUM_LAUNCH(kfn, dim3(256 / kRowsPerCta, cnt), kRowsPerCta * 16, 0, s, rows, epi, tw, static_cast<const Pair*>(ctx->d_twr_fwd), pcs); }
    CERIUM_LAUNCH_CHECK("sud_ptrs");
    return CERIUM_OK;
  });
}

int cerium_bconv_ptrs(cerium_context* ctx, void* const* outs, const size_t* n_out, const void* const* ins,
                      const size_t* n_in, const void* const* factors, const void* const* out_moduli,
                      size_t max_in, size_t max_out, size_t num_conversions, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "bconv_ptrs: null context");
  if (num_conversions == 0) return CERIUM_OK;
  if (!outs || !n_out || !ins || !n_in || !factors || !out_moduli) return fail(CERIUM_ERR_INVALID, "bconv_ptrs: null table");
  if (max_in < 1 || max_out < 1 || max_in > 64 || max_out > 128) return fail(CERIUM_ERR_INVALID, "bconv_ptrs: bad shape bound");
  if (num_conversions > 65535) return fail(CERIUM_ERR_INVALID, "bconv_ptrs: more than 65535 conversions in one call");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    static bool smem_opt_in[kMaxDevices][2] = {};  // the attribute is per device
    // the shapes live on the device: size the shared memory for the caller's bounds (inputs staged per
    // thread when there are more than kBconvRegInputs of them); smaller shapes inside the bounds may need
    // more than the bound shape itself (the double-precision factor pairs of up to 8 inputs)
    size_t smem = bconv_smem_bytes<W>((int)max_in, (int)max_out);
    smem = std::max(smem, bconv_smem_bytes<W>((int)std::min<size_t>(max_in, kBconvRegInputs), (int)max_out));
    if (smem > 200 * 1024) return fail(CERIUM_ERR_UNSUPPORTED, "bconv_ptrs: conversion needs more than 200 KiB of shared memory");
    if (smem > 48 * 1024) {
      const int slot = sizeof(W) == 4 ? 0 : 1;
      const int dev = ctx->device;
      if (dev < 0 || dev >= kMaxDevices || !smem_opt_in[dev][slot]) {
        CERIUM_CUDA(cudaFuncSetAttribute(bconv_ptrs_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        if (dev >= 0 && dev < kMaxDevices) smem_opt_in[dev][slot] = true;
      }
    }
    auto kfn = bconv_ptrs_kernel<W>;
    CERIUM_LAUNCH(kfn, dim3(kBconvBlocks, (unsigned)num_conversions), kBconvThreads, smem, s,
                  reinterpret_cast<W* const*>(outs), n_out, reinterpret_cast<const W* const*>(ins), n_in,
                  reinterpret_cast<const W* const*>(factors), reinterpret_cast<const W* const*>(out_moduli),
                  max_in, max_out, smem, ctx->d_status);
    CERIUM_LAUNCH_CHECK("bconv_ptrs");
    return CERIUM_OK;
  });
}

int cerium_sud(cerium_context* ctx, void* out, size_t out_stride, const void* minuend, size_t minuend_stride,
               void* in_coeff, size_t in_stride, const void* addend, size_t addend_stride,
               const uint32_t* prime_idx, int count, const uint32_t* divide_primes, int n_divide, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "sud: null context");
  if (count < 0 || n_divide < 1) return fail(CERIUM_ERR_INVALID, "sud: bad count");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx || !divide_primes) return fail(CERIUM_ERR_INVALID, "sud: null index array");
  const size_t wb = ctx->word_bytes();
  if (int rc = check_stack(out, out_stride, wb, "sud: out")) return rc;
  if (int rc = check_stack(minuend, minuend_stride, wb, "sud: minuend")) return rc;
  if (int rc = check_stack(in_coeff, in_stride, wb, "sud: in_coeff")) return rc;
  if (addend)
    if (int rc = check_stack(addend, addend_stride, wb, "sud: addend")) return rc;
  std::vector<uint32_t> div(divide_primes, divide_primes + n_divide);
  for (uint32_t d : div)
    if (d >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "sud: divide prime index out of range");
  std::vector<uint64_t> factor(count);
  for (int i = 0; i < count; i++) {
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "sud: prime index out of range");
    const uint64_t q = ctx->moduli[prime_idx[i]];
    // a prime that divides the product has no inverse: factor 0, as compute_sud_factors leaves it
    factor[i] = host::invmod(host::product_mod(ctx->moduli, div, q), q);
  }
  DeviceGuard guard(ctx->device);
  SudCall c{};
  c.src = in_coeff;
  c.src_stride = in_stride;
  c.work = in_coeff;
  c.work_stride = in_stride;
  c.dst = out;
  c.dst_stride = out_stride;
  c.minuend = minuend;
  c.minuend_stride = minuend_stride;
  c.addend = addend;
  c.addend_stride = addend_stride;
  c.prime = prime_idx;
  c.factor = factor.data();
  c.count = count;
  return launch_sud(ctx, c, (cudaStream_t)stream);
}

int cerium_ewise(cerium_context* ctx, int op, void* out, size_t out_stride, const void* a, size_t a_stride,
                 const void* b, size_t b_stride, const void* c, size_t c_stride, const uint64_t* scalars,
                 const uint32_t* prime_idx, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "ewise: null context");
  if (op < CERIUM_EW_ADD || op > CERIUM_EW_REDUCE) return fail(CERIUM_ERR_INVALID, "ewise: unknown op");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "ewise: negative count");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx) return fail(CERIUM_ERR_INVALID, "ewise: null prime_idx");
  const size_t wb = ctx->word_bytes();
  const bool need_b = op == CERIUM_EW_ADD || op == CERIUM_EW_SUB || op == CERIUM_EW_MUL || op == CERIUM_EW_MAD ||
                      op == CERIUM_EW_PMU;
  const bool need_c = op == CERIUM_EW_MAD;
  const bool need_s = op == CERIUM_EW_PMU || op == CERIUM_EW_MUL_SCALAR;
  if (int rc = check_stack(out, out_stride, wb, "ewise: out")) return rc;
  if (int rc = check_stack(a, a_stride, wb, "ewise: a")) return rc;
  if (need_b)
    if (int rc = check_stack(b, b_stride, wb, "ewise: b")) return rc;
  if (need_c)
    if (int rc = check_stack(c, c_stride, wb, "ewise: c")) return rc;
  if (need_s && !scalars) return fail(CERIUM_ERR_INVALID, "ewise: null scalars");
  for (int i = 0; i < count; i++)
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "ewise: prime index out of range");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    for (int first = 0; first < count; first += kEwMaxLimbs) {
      const int cnt = std::min(kEwMaxLimbs, count - first);
      EwArgs<W> g{};
      g.out = {static_cast<W*>(out) + (size_t)first * out_stride, out_stride};
      g.a = {const_cast<W*>(static_cast<const W*>(a)) + (size_t)first * a_stride, a_stride};
      if (need_b) g.b = {const_cast<W*>(static_cast<const W*>(b)) + (size_t)first * b_stride, b_stride};
      if (need_c) g.c = {const_cast<W*>(static_cast<const W*>(c)) + (size_t)first * c_stride, c_stride};
      for (int k = 0; k < cnt; k++) {
        g.prime[k] = (uint8_t)prime_idx[first + k];
        if (need_s) {
          const uint64_t q = ctx->moduli[prime_idx[first + k]];
          const uint64_t sv = scalars[first + k] % q;
          g.scalar[k] = (W)sv;
          g.scalar_shoup[k] = (W)host::shoup(sv, q, ctx->word_bits);
        }
      }
      const dim3 grid(kN / (kEwThreads * V::kLanes), cnt);
      switch (op) {
        case CERIUM_EW_ADD: { auto kfn = ewise_kernel<W, kEwAdd>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_SUB: { auto kfn = ewise_kernel<W, kEwSub>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_NEG: { auto kfn = ewise_kernel<W, kEwNeg>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_MUL: { auto kfn = ewise_kernel<W, kEwMul>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_MAD: { auto kfn = ewise_kernel<W, kEwMad>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_PMU: { auto kfn = ewise_kernel<W, kEwPmu>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        case CERIUM_EW_REDUCE: { auto kfn = ewise_kernel<W, kEwReduce>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
        default: { auto kfn = ewise_kernel<W, kEwMulScalar>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); } break;
      }
    }
    CERIUM_LAUNCH_CHECK("ewise");
    return CERIUM_OK;
  });
}

int cerium_mul_plain_periodic(cerium_context* ctx, void* out, size_t out_stride, const void* a, size_t a_stride,
                              const void* pt, size_t pt_stride, int log2_repeat, const void* addend, size_t addend_stride,
                              const uint32_t* prime_idx, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: null context");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: negative count");
  if (log2_repeat < 0 || log2_repeat > ctx->logn) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: repeat count out of range");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: null prime_idx");
  const size_t wb = ctx->word_bytes();
  if (int rc = check_stack(out, out_stride, wb, "mul_plain_periodic: out")) return rc;
  if (int rc = check_stack(a, a_stride, wb, "mul_plain_periodic: a")) return rc;
  if (!pt) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: null plaintext");
  if (pt_stride < ((size_t)kN >> log2_repeat)) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: plaintext stride is smaller than one period");
  if (addend)
    if (int rc = check_stack(addend, addend_stride, wb, "mul_plain_periodic: addend")) return rc;
  for (int i = 0; i < count; i++)
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "mul_plain_periodic: prime index out of range");
  DeviceGuard guard(ctx->device);
  cudaStream_t s = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    for (int first = 0; first < count; first += kEwMaxLimbs) {
      const int cnt = std::min(kEwMaxLimbs, count - first);
      EwArgs<W> g{};
      g.out = {static_cast<W*>(out) + (size_t)first * out_stride, out_stride};
      g.a = {const_cast<W*>(static_cast<const W*>(a)) + (size_t)first * a_stride, a_stride};
      g.b = {const_cast<W*>(static_cast<const W*>(pt)) + (size_t)first * pt_stride, pt_stride};
      if (addend) g.c = {const_cast<W*>(static_cast<const W*>(addend)) + (size_t)first * addend_stride, addend_stride};
      g.shift = log2_repeat;
      for (int k = 0; k < cnt; k++) g.prime[k] = (uint8_t)prime_idx[first + k];
      const dim3 grid(kN / (kEwThreads * V::kLanes), cnt);
      if (addend) { auto kfn = ewise_kernel<W, kEwMadPeriodic>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); }
      else { auto kfn = ewise_kernel<W, kEwMulPeriodic>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, s, g, pcs); }
    }
    CERIUM_LAUNCH_CHECK("mul_plain_periodic");
    return CERIUM_OK;
  });
}

int cerium_tensor(cerium_context* ctx, void* d0, void* d1, void* d2, const void* a0, const void* a1,
                  const void* b0, const void* b1, size_t stride, const uint32_t* prime_idx, int count,
                  void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "tensor: null context");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "tensor: negative count");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx) return fail(CERIUM_ERR_INVALID, "tensor: null prime_idx");
  const size_t wb = ctx->word_bytes();
  const void* ptrs[7] = {d0, d1, d2, a0, a1, b0, b1};
  for (const void* p : ptrs)
    if (int rc = check_stack(p, stride, wb, "tensor: operand")) return rc;
  for (int i = 0; i < count; i++)
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "tensor: prime index out of range");
  DeviceGuard guard(ctx->device);
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    for (int first = 0; first < count; first += kEwMaxLimbs) {
      const int cnt = std::min(kEwMaxLimbs, count - first);
      const size_t off = (size_t)first * stride;
      auto mk = [&](const void* p) { return Limbs<W>{const_cast<W*>(static_cast<const W*>(p)) + off, stride}; };
      TensorArgs<W> g{};
      g.a0 = mk(a0); g.a1 = mk(a1); g.b0 = mk(b0); g.b1 = mk(b1);
      g.d0 = mk(d0); g.d1 = mk(d1); g.d2 = mk(d2);
      for (int k = 0; k < cnt; k++) g.prime[k] = (uint8_t)prime_idx[first + k];
      { auto kfn = tensor_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / (kEwThreads * V::kLanes), cnt), kEwThreads, 0, (cudaStream_t)stream, g, static_cast<const PrimeConst<W>*>(ctx->d_pcs)); }
    }
    CERIUM_LAUNCH_CHECK("tensor");
    return CERIUM_OK;
  });
}

uint32_t cerium_galois_elt_from_step(int step, int log_n) {
  if (log_n < 1 || log_n > 30) return 0;
  const uint64_t n = (uint64_t)1 << log_n, m = 2 * n;
  if (step == 0) return (uint32_t)(m - 1);
  const uint64_t a = step < 0 ? (uint64_t)(-(int64_t)step) : (uint64_t)step;
  if (a >= (n >> 1)) return 0;  // "step count too large" in the reference
  uint64_t s = step < 0 ? (n >> 1) - a : a;
  uint64_t e = 1, g = 5;
  for (; s; s >>= 1) {
    if (s & 1) e = (e * g) & (m - 1);
    g = (g * g) & (m - 1);
  }
  return (uint32_t)e;
}

int cerium_automorph(cerium_context* ctx, void* out, size_t out_stride, const void* in, size_t in_stride,
                     uint32_t galois_elt, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "automorph: null context");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "automorph: negative count");
  if (!(galois_elt & 1) || galois_elt >= 2u * kN) return fail(CERIUM_ERR_INVALID, "automorph: Galois element is not valid");
  if (count == 0) return CERIUM_OK;
  if (count > 65535) return fail(CERIUM_ERR_INVALID, "automorph: more than 65535 limbs in one call");
  const size_t wb = ctx->word_bytes();
  if (int rc = check_stack(out, out_stride, wb, "automorph: out")) return rc;
  if (int rc = check_stack(in, in_stride, wb, "automorph: in")) return rc;
  if (out == in) return fail(CERIUM_ERR_INVALID, "automorph: result cannot alias the operand");
  DeviceGuard guard(ctx->device);
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    AutomorphArgs<W> g{};
    g.out = {static_cast<W*>(out), out_stride};
    g.in = {const_cast<W*>(static_cast<const W*>(in)), in_stride};
    g.split = count;
    g.elt = galois_elt;
    { auto kfn = automorph_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / kEwThreads, count), kEwThreads, 0, (cudaStream_t)stream, g); }
    CERIUM_LAUNCH_CHECK("automorph");
    return CERIUM_OK;
  });
}

}  // extern "C"

namespace cerium {
// Automorphism of two polynomials of `count` limbs each (stride N) in one launch.
int launch_automorph_pair(cerium_context* ctx, void* out_a, const void* in_a, void* out_b, const void* in_b,
                          uint32_t galois_elt, int count, cudaStream_t stream) {
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    AutomorphArgs<W> g{};
    g.out = {static_cast<W*>(out_a), (size_t)kN};
    g.in = {const_cast<W*>(static_cast<const W*>(in_a)), (size_t)kN};
    g.out2 = {static_cast<W*>(out_b), (size_t)kN};
    g.in2 = {const_cast<W*>(static_cast<const W*>(in_b)), (size_t)kN};
    g.split = count;
    g.elt = galois_elt;
    { auto kfn = automorph_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / kEwThreads, 2 * count), kEwThreads, 0, stream, g); }
    CERIUM_LAUNCH_CHECK("automorph");
    return CERIUM_OK;
  });
}
}  // namespace cerium

extern "C" {

int cerium_resolve2(cerium_context* ctx, void* lo, void* hi, const void* x0, const void* x1, size_t stride,
                    uint32_t prime0, uint32_t prime1, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "resolve2: null context");
  if (count < 0 || count > 65535) return fail(CERIUM_ERR_INVALID, "resolve2: bad count");
  if (count == 0) return CERIUM_OK;
  if (prime0 >= (uint32_t)ctx->n_primes || prime1 >= (uint32_t)ctx->n_primes || prime0 == prime1)
    return fail(CERIUM_ERR_INVALID, "resolve2: need two different prime indices of the context");
  const size_t wb = ctx->word_bytes();
  const void* ptrs[4] = {lo, hi, x0, x1};
  for (const void* p : ptrs)
    if (int rc = check_stack(p, stride, wb, "resolve2: operand")) return rc;
  const uint64_t m0 = ctx->moduli[prime0], m1 = ctx->moduli[prime1];
  const uint64_t inv = host::invmod(m0 % m1, m1);
  DeviceGuard guard(ctx->device);
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    auto mk = [&](const void* p) { return Limbs<W>{const_cast<W*>(static_cast<const W*>(p)), stride}; };
    Rsv2Args<W> g{};
    g.x0 = mk(x0); g.x1 = mk(x1); g.lo = mk(lo); g.hi = mk(hi);
    g.m0 = (W)m0;
    g.inv = (W)inv;
    g.inv_shoup = (W)host::shoup(inv, m1, ctx->word_bits);
    g.prime1 = prime1;
    { auto kfn = rsv2_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / (kEwThreads * V::kLanes), count), kEwThreads, 0, (cudaStream_t)stream, g, static_cast<const PrimeConst<W>*>(ctx->d_pcs)); }
    CERIUM_LAUNCH_CHECK("resolve2");
    return CERIUM_OK;
  });
}

int cerium_mod2(cerium_context* ctx, void* out, size_t out_stride, const void* lo, const void* hi,
                const uint32_t* prime_idx, int count, void* stream) {
  if (!ctx) return fail(CERIUM_ERR_INVALID, "mod2: null context");
  if (count < 0) return fail(CERIUM_ERR_INVALID, "mod2: negative count");
  if (count == 0) return CERIUM_OK;
  if (!prime_idx) return fail(CERIUM_ERR_INVALID, "mod2: null prime_idx");
  const size_t wb = ctx->word_bytes();
  if (int rc = check_stack(out, out_stride, wb, "mod2: out")) return rc;
  if (int rc = check_stack(lo, kN, wb, "mod2: lo")) return rc;
  if (int rc = check_stack(hi, kN, wb, "mod2: hi")) return rc;
  for (int i = 0; i < count; i++)
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "mod2: prime index out of range");
  DeviceGuard guard(ctx->device);
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    for (int first = 0; first < count; first += kEwMaxLimbs) {
      const int cnt = std::min(kEwMaxLimbs, count - first);
      Mod2Args<W> g{};
      g.lo = static_cast<const W*>(lo);
      g.hi = static_cast<const W*>(hi);
      g.out = {static_cast<W*>(out) + (size_t)first * out_stride, out_stride};
      for (int k = 0; k < cnt; k++) g.prime[k] = (uint8_t)prime_idx[first + k];
      { auto kfn = mod2_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / (kEwThreads * V::kLanes), cnt), kEwThreads, 0, (cudaStream_t)stream, g, static_cast<const PrimeConst<W>*>(ctx->d_pcs)); }
    }
    CERIUM_LAUNCH_CHECK("mod2");
    return CERIUM_OK;
  });
}

int cerium_bconv_create(cerium_context* ctx, cerium_bconv** out, int mode, const uint32_t* in_primes, int n_in,
                        const uint32_t* out_primes, int n_out) {
  return create_bconv(ctx, out, mode, in_primes, n_in, out_primes, n_out, BconvOptions{});
}

int cerium_bconv_destroy(cerium_bconv* bc) {
  if (!bc) return CERIUM_OK;
  DeviceGuard guard(bc->ctx->device);
  cudaFree(bc->d_block);
  delete bc;
  return CERIUM_OK;
}

int cerium_bconv_apply(cerium_bconv* bc, void* out, size_t out_stride, const void* in, size_t in_stride,
                       void* stream) {
  if (!bc) return fail(CERIUM_ERR_INVALID, "bconv_apply: null converter");
  const size_t wb = bc->ctx->word_bytes();
  if (int rc = check_stack(out, out_stride, wb, "bconv_apply: out")) return rc;
  if (int rc = check_stack(in, in_stride, wb, "bconv_apply: in")) return rc;
  DeviceGuard guard(bc->ctx->device);
  BconvCall c{bc, out, out_stride, in, in_stride};
  return launch_bconv(bc->ctx, &c, 1, (cudaStream_t)stream);
}

int cerium_bconv_apply_batch(cerium_bconv* const* bcs, void* const* outs, const void* const* ins, int count,
                             size_t out_stride, size_t in_stride, void* stream) {
  if (count < 0) return fail(CERIUM_ERR_INVALID, "bconv_apply_batch: negative count");
  if (count == 0) return CERIUM_OK;
  if (!bcs || !outs || !ins) return fail(CERIUM_ERR_INVALID, "bconv_apply_batch: null array");
  std::vector<BconvCall> calls(count);
  for (int k = 0; k < count; k++) {
    if (!bcs[k]) return fail(CERIUM_ERR_INVALID, "bconv_apply_batch: null converter");
    if (bcs[k]->ctx != bcs[0]->ctx) return fail(CERIUM_ERR_INVALID, "bconv_apply_batch: converters of different contexts");
    const size_t wb = bcs[k]->ctx->word_bytes();
    if (int rc = check_stack(outs[k], out_stride, wb, "bconv_apply_batch: out")) return rc;
    if (int rc = check_stack(ins[k], in_stride, wb, "bconv_apply_batch: in")) return rc;
    calls[k] = BconvCall{bcs[k], outs[k], out_stride, ins[k], in_stride};
  }
  DeviceGuard guard(bcs[0]->ctx->device);
  return launch_bconv(bcs[0]->ctx, calls.data(), count, (cudaStream_t)stream);
}

}  // extern "C"
