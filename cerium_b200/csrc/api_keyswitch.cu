// Hybrid key switching and the CKKS operators built on it (HRot, HMult + relinearise,
// rescale).  The sequence of kernels is the one Cerium's compiler emits for these operators
// (cerium/compiler/backend/compiler_keyswitch.cc:253-432: INTT, BCONV, NTT, EVKMUL, PMU, INTT,
// BCONV, SUD; cerium/compiler/backend/compiler.cc:443-467, 701-726;
// cerium/compiler/backend/compiler_rescale.cc:209-284), issued here by a fixed host routine
// instead of being compiled per program:
//   1 launch pair  iNTT of the switched polynomial            (L limbs)
//   1 launch       base conversion of every digit             (dnum conversions in one grid)
//   1 launch pair  NTT of all converted limbs of all digits   (dnum*(L+K) - L limbs)
//   1 launch       inner product with the key over all digits (L+K limbs, 2 outputs)
//   1 launch pair  iNTT of the 2*K extension limbs
//   1 launch       base conversion P -> Q for both outputs
//   2 launch pairs SuD (NTT fused with subtract, multiply by P^-1 and the final addition)
#include <algorithm>
#include <cstring>

#include "internal.h"

using namespace cerium;

struct cerium_keyswitch {
  cerium_context* ctx = nullptr;
  int bconv_mode = 0, round_mode = 0;
  int L = 0, K = 0, dnum = 0, LK = 0;
  std::vector<uint32_t> q_idx, p_idx, all_idx;
  std::vector<cerium_bconv*> up;   // one converter per non-empty digit
  std::vector<int> up_digit;       // digit number of up[k]
  cerium_bconv* down = nullptr;    // P -> Q
  std::vector<uint64_t> pinv;      // [L] P^-1 mod q_i
  // transform batches
  std::vector<uint32_t> ntt_pos, ntt_prime;  // converted limbs of all digits inside `raised`
  std::vector<uint32_t> ext_pos, ext_prime;  // extension limbs of both accumulators
  // exact mode: per-limb scalars folded into the inverse transforms (device, one word per entry)
  void* d_scale = nullptr;  // [L] then [2K]: scale, and at +count their Shoup companions
  void* d_scale_q = nullptr;
  void* d_scale_q_shoup = nullptr;
  void* d_scale_p = nullptr;
  void* d_scale_p_shoup = nullptr;
  // workspace
  void* ws = nullptr;
  size_t ws_bytes = 0;
  size_t o_coef = 0, o_raised = 0, o_acc = 0, o_conv = 0, o_tmp = 0, o_ksout = 0, o_scratch = 0;  // words
};

namespace {

template <typename W>
W* ws_at(const cerium_keyswitch* ks, size_t off_words) {
  return static_cast<W*>(ks->ws) + off_words;
}

int rescale_impl(cerium_context* ctx, int round_mode, void* out, const void* in, const uint32_t* q_idx, int L,
                 int n_polys, void* scratch, cudaStream_t stream) {
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  const uint32_t last = q_idx[L - 1];
  const uint64_t ql = ctx->moduli[last];
  // 1. inverse transform of the last limb of every polynomial -> scratch[poly][N]
  std::vector<uint32_t> pos(n_polys), prime(n_polys, last);
  for (int p = 0; p < n_polys; p++) pos[p] = (uint32_t)p;
  {
    // input limb of poly p sits at in + (p*L + L-1)*N: base shifted to the first such limb, stride L*N
    NttCall c{};
    c.in = static_cast<const char*>(in) + (size_t)(L - 1) * n * wb;
    c.in_stride = (size_t)L * n;
    c.out = scratch;
    c.out_stride = n;
    c.pos = pos.data();
    c.prime = prime.data();
    c.count = n_polys;
    if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, stream)) return rc;
  }
  // 2. SuD of the remaining limbs against the re-reduced last limb
  std::vector<uint64_t> factor(L - 1), post_sub(L - 1);
  const uint64_t half = ql >> 1;
  for (int i = 0; i < L - 1; i++) {
    const uint64_t q = ctx->moduli[q_idx[i]];
    factor[i] = host::invmod(ql % q, q);
    post_sub[i] = round_mode == CERIUM_ROUND_HALF ? half % q : 0;
  }
  for (int p = 0; p < n_polys; p++) {
    SudCall s{};
    s.src = static_cast<const char*>(scratch) + (size_t)p * n * wb;
    s.src_stride = 0;
    s.work = static_cast<char*>(out) + (size_t)p * (L - 1) * n * wb;
    s.work_stride = n;
    s.dst = s.work;
    s.dst_stride = n;
    s.minuend = static_cast<const char*>(in) + (size_t)p * L * n * wb;
    s.minuend_stride = n;
    s.addend = nullptr;
    s.addend_stride = 0;
    s.prime = q_idx;
    s.factor = factor.data();
    s.count = L - 1;
    s.reduce_src = true;
    s.src_q = ql;
    s.pre_add = round_mode == CERIUM_ROUND_HALF ? half : 0;
    s.post_sub = post_sub.data();
    if (int rc = launch_sud(ctx, s, stream)) return rc;
  }
  return CERIUM_OK;
}

int keyswitch_impl(cerium_keyswitch* ks, void* out0, void* out1, const void* cpoly, const void* evk,
                   const void* add0, const void* add1, cudaStream_t stream) {
  cerium_context* ctx = ks->ctx;
  const size_t n = kN;
  const int L = ks->L, K = ks->K, LK = ks->LK, dnum = ks->dnum;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    W* coef = ws_at<W>(ks, ks->o_coef);
    W* raised = ws_at<W>(ks, ks->o_raised);
    W* acc = ws_at<W>(ks, ks->o_acc);
    W* conv = ws_at<W>(ks, ks->o_conv);
    // 1. iNTT of the switched polynomial (exact mode: times [Qhat_i^-1] of its digit)
    {
      NttCall c{cpoly, coef, n, n, nullptr, ks->q_idx.data(), L};
      if (int rc = launch_ntt_inverse(ctx, c, ks->d_scale_q, ks->d_scale_q_shoup, stream)) return rc;
    }
    // 2. ModUp base conversion, every digit in one launch.  Digit d reads limbs d, d+dnum, ...
    {
      std::vector<BconvCall> calls;
      for (size_t k = 0; k < ks->up.size(); k++) {
        const int d = ks->up_digit[k];
        calls.push_back(BconvCall{ks->up[k], raised + (size_t)d * LK * n, n, coef + (size_t)d * n, (size_t)dnum * n});
      }
      if (int rc = launch_bconv(ctx, calls.data(), (int)calls.size(), stream)) return rc;
    }
    // 3. NTT of every converted limb
    {
      NttCall c{raised, raised, n, n, ks->ntt_pos.data(), ks->ntt_prime.data(), (int)ks->ntt_pos.size()};
      if (int rc = launch_ntt_forward(ctx, c, stream)) return rc;
    }
    // 4. inner product with the key
    {
      InnerProductArgs<W> g{};
      g.raised = raised;
      g.raised_digit_stride = (size_t)LK * n;
      g.raised_limb_stride = n;
      g.own = static_cast<const W*>(cpoly);
      g.own_stride = n;
      g.evk = static_cast<const W*>(evk);
      g.evk_digit_stride = (size_t)2 * LK * n;
      g.evk_poly_stride = (size_t)LK * n;
      g.evk_limb_stride = n;
      g.out0 = {acc, n};
      g.out1 = {acc + (size_t)LK * n, n};
      g.L = L;
      g.dnum = dnum;
      for (int b = 0; b < LK; b++) g.prime[b] = (uint8_t)ks->all_idx[b];
      { auto kfn = inner_product_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / (kEwThreads * V::kLanes), LK), kEwThreads, 0, stream, g, static_cast<const PrimeConst<W>*>(ctx->d_pcs)); }
      CERIUM_LAUNCH_CHECK("inner_product");
    }
    // 5. iNTT of the extension limbs of both accumulators, in place
    {
      NttCall c{acc, acc, n, n, ks->ext_pos.data(), ks->ext_prime.data(), 2 * K};
      if (int rc = launch_ntt_inverse(ctx, c, ks->d_scale_p, ks->d_scale_p_shoup, stream)) return rc;
    }
    // 6. ModDown base conversion P -> Q
    {
      BconvCall calls[2] = {
          {ks->down, conv, n, acc + (size_t)L * n, n},
          {ks->down, conv + (size_t)L * n, n, acc + (size_t)(LK + L) * n, n},
      };
      if (int rc = launch_bconv(ctx, calls, 2, stream)) return rc;
    }
    // 7. SuD: out = (acc_Q - NTT(conv)) * P^-1 (+ add)
    for (int p = 0; p < 2; p++) {
      SudCall s{};
      s.src = conv + (size_t)p * L * n;
      s.src_stride = n;
      s.work = conv + (size_t)p * L * n;
      s.work_stride = n;
      s.dst = p == 0 ? out0 : out1;
      s.dst_stride = n;
      s.minuend = acc + (size_t)p * LK * n;
      s.minuend_stride = n;
      s.addend = p == 0 ? add0 : add1;
      s.addend_stride = n;
      s.prime = ks->q_idx.data();
      s.factor = ks->pinv.data();
      s.count = L;
      if (int rc = launch_sud(ctx, s, stream)) return rc;
    }
    return CERIUM_OK;
  });
}

}  // namespace

extern "C" {

int cerium_keyswitch_create(cerium_context* ctx, cerium_keyswitch** out, int bconv_mode, int round_mode,
                            const uint32_t* q_idx, int L, const uint32_t* p_idx, int K, int dnum) {
  if (!ctx || !out || !q_idx || !p_idx) return fail(CERIUM_ERR_INVALID, "keyswitch_create: null argument");
  if (bconv_mode != CERIUM_BCONV_LAZY && bconv_mode != CERIUM_BCONV_EXACT) return fail(CERIUM_ERR_INVALID, "keyswitch_create: unknown bconv mode");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "keyswitch_create: unknown round mode");
  if (L < 1 || K < 1 || dnum < 1 || dnum > L) return fail(CERIUM_ERR_INVALID, "keyswitch_create: need L >= 1, K >= 1, 1 <= dnum <= L");
  if (L + K > kEwMaxLimbs || L > kSudMaxBatch) return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch_create: too many limbs (L <= 64, L + K <= 128)");
  const int alpha = (L + dnum - 1) / dnum;
  if (alpha > K) return fail(CERIUM_ERR_INVALID, "keyswitch_create: digit size exceeds the number of extension primes");
  if ((size_t)dnum * (L + K) > 0xffff) return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch_create: dnum * (L + K) too large");
  std::vector<bool> seen(ctx->n_primes, false);
  for (int i = 0; i < L + K; i++) {
    const uint32_t p = i < L ? q_idx[i] : p_idx[i - L];
    if (p >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "keyswitch_create: prime index out of range");
    if (seen[p]) return fail(CERIUM_ERR_INVALID, "keyswitch_create: a prime appears twice");
    seen[p] = true;
  }
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "keyswitch_create: cannot select device");
  auto* ks = new cerium_keyswitch();
  ks->ctx = ctx;
  ks->bconv_mode = bconv_mode;
  ks->round_mode = round_mode;
  ks->L = L;
  ks->K = K;
  ks->dnum = dnum;
  ks->LK = L + K;
  ks->q_idx.assign(q_idx, q_idx + L);
  ks->p_idx.assign(p_idx, p_idx + K);
  ks->all_idx = ks->q_idx;
  ks->all_idx.insert(ks->all_idx.end(), ks->p_idx.begin(), ks->p_idx.end());
  const int LK = ks->LK;
  const int bits = ctx->word_bits;
  const bool exact = bconv_mode == CERIUM_BCONV_EXACT;
  std::vector<uint64_t> scale_q(L, 1), scale_p(2 * K, 1);
  int rc = CERIUM_OK;
  // per-digit converters: inputs {d, d+dnum, ...}, outputs every other extended limb
  for (int d = 0; d < dnum && rc == CERIUM_OK; d++) {
    std::vector<uint32_t> in_primes, out_primes, out_pos;
    std::vector<int> in_limb;
    for (int i = 0; i < LK; i++) {
      if (i < L && i % dnum == d) {
        in_primes.push_back(ks->all_idx[i]);
        in_limb.push_back(i);
      } else {
        out_primes.push_back(ks->all_idx[i]);
        out_pos.push_back((uint32_t)i);
        ks->ntt_pos.push_back((uint32_t)(d * LK + i));
        ks->ntt_prime.push_back(ks->all_idx[i]);
      }
    }
    if (in_primes.empty()) continue;
    BconvOptions opt;
    opt.prescaled = exact;
    opt.out_pos = out_pos;
    cerium_bconv* bc = nullptr;
    rc = create_bconv(ctx, &bc, bconv_mode, in_primes.data(), (int)in_primes.size(), out_primes.data(),
                      (int)out_primes.size(), opt);
    if (rc != CERIUM_OK) break;
    ks->up.push_back(bc);
    ks->up_digit.push_back(d);
    if (exact)
      for (size_t k = 0; k < in_limb.size(); k++) scale_q[in_limb[k]] = bc->inv_host[k];
  }
  if (rc == CERIUM_OK) {
    BconvOptions opt;
    opt.prescaled = exact;
    opt.round_half = round_mode == CERIUM_ROUND_HALF;
    rc = create_bconv(ctx, &ks->down, bconv_mode, ks->p_idx.data(), K, ks->q_idx.data(), L, opt);
    if (rc == CERIUM_OK && exact)
      for (int k = 0; k < K; k++) scale_p[k] = scale_p[K + k] = ks->down->inv_host[k];
  }
  if (rc != CERIUM_OK) {
    cerium_keyswitch_destroy(ks);
    return rc;
  }
  ks->pinv.resize(L);
  for (int i = 0; i < L; i++) {
    const uint64_t q = ctx->moduli[ks->q_idx[i]];
    ks->pinv[i] = host::invmod(host::product_mod(ctx->moduli, ks->p_idx, q), q);
  }
  for (int p = 0; p < 2; p++)
    for (int k = 0; k < K; k++) {
      ks->ext_pos.push_back((uint32_t)(p * LK + L + k));
      ks->ext_prime.push_back(ks->p_idx[k]);
    }
  const size_t wb = ctx->word_bytes();
  const size_t n = kN;
  if (exact) {
    // [scale_q | scale_q_shoup | scale_p | scale_p_shoup]
    std::vector<uint64_t> all;
    for (int i = 0; i < L; i++) all.push_back(scale_q[i]);
    for (int i = 0; i < L; i++) all.push_back(host::shoup(scale_q[i], ctx->moduli[ks->q_idx[i]], bits));
    for (int i = 0; i < 2 * K; i++) all.push_back(scale_p[i]);
    for (int i = 0; i < 2 * K; i++) all.push_back(host::shoup(scale_p[i], ctx->moduli[ks->p_idx[i % K]], bits));
    std::vector<char> bytes(all.size() * wb);
    for (size_t i = 0; i < all.size(); i++) {
      if (bits == 32) reinterpret_cast<uint32_t*>(bytes.data())[i] = (uint32_t)all[i];
      else reinterpret_cast<uint64_t*>(bytes.data())[i] = all[i];
    }
    if (cudaMalloc(&ks->d_scale, bytes.size()) != cudaSuccess ||
        cudaMemcpy(ks->d_scale, bytes.data(), bytes.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
      cerium_keyswitch_destroy(ks);
      return fail(CERIUM_ERR_CUDA, "keyswitch_create: scale upload failed");
    }
    char* b = static_cast<char*>(ks->d_scale);
    ks->d_scale_q = b;
    ks->d_scale_q_shoup = b + (size_t)L * wb;
    ks->d_scale_p = b + (size_t)2 * L * wb;
    ks->d_scale_p_shoup = b + (size_t)(2 * L + 2 * K) * wb;
  }
  // workspace layout (in words)
  size_t off = 0;
  auto take = [&](size_t limbs) {
    const size_t o = off;
    off += limbs * n;
    return o;
  };
  ks->o_coef = take(L);
  ks->o_raised = take((size_t)dnum * LK);
  ks->o_acc = take(2 * (size_t)LK);
  ks->o_conv = take(2 * (size_t)L);
  ks->o_tmp = take(3 * (size_t)L);
  ks->o_ksout = take(2 * (size_t)L);
  ks->o_scratch = take(2);
  ks->ws_bytes = off * wb;
  if (cudaMalloc(&ks->ws, ks->ws_bytes) != cudaSuccess) {
    cerium_keyswitch_destroy(ks);
    return fail(CERIUM_ERR_CUDA, "keyswitch_create: cannot allocate the workspace");
  }
  *out = ks;
  return CERIUM_OK;
}

int cerium_keyswitch_destroy(cerium_keyswitch* ks) {
  if (!ks) return CERIUM_OK;
  DeviceGuard guard(ks->ctx->device);
  for (cerium_bconv* b : ks->up) cerium_bconv_destroy(b);
  cerium_bconv_destroy(ks->down);
  cudaFree(ks->d_scale);
  cudaFree(ks->ws);
  delete ks;
  return CERIUM_OK;
}

size_t cerium_keyswitch_workspace_bytes(const cerium_keyswitch* ks) { return ks ? ks->ws_bytes : 0; }

int cerium_keyswitch_apply(cerium_keyswitch* ks, void* out0, void* out1, const void* cpoly, const void* evk,
                           const void* add0, const void* add1, void* stream) {
  if (!ks || !out0 || !out1 || !cpoly || !evk) return fail(CERIUM_ERR_INVALID, "keyswitch_apply: null argument");
  DeviceGuard guard(ks->ctx->device);
  return keyswitch_impl(ks, out0, out1, cpoly, evk, add0, add1, (cudaStream_t)stream);
}

int cerium_hrot(cerium_keyswitch* ks, void* out0, void* out1, const void* c0, const void* c1, const void* evk,
                uint32_t galois_elt, void* stream) {
  if (!ks || !out0 || !out1 || !c0 || !c1 || !evk) return fail(CERIUM_ERR_INVALID, "hrot: null argument");
  if (!(galois_elt & 1) || galois_elt >= 2u * kN) return fail(CERIUM_ERR_INVALID, "hrot: Galois element is not valid");
  cerium_context* ctx = ks->ctx;
  DeviceGuard guard(ctx->device);
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  char* tmp = static_cast<char*>(ks->ws) + ks->o_tmp * wb;
  void* rot0 = tmp;
  void* rot1 = tmp + (size_t)ks->L * n * wb;
  if (int rc = cerium_automorph(ctx, rot0, n, c0, n, galois_elt, ks->L, stream)) return rc;
  if (int rc = cerium_automorph(ctx, rot1, n, c1, n, galois_elt, ks->L, stream)) return rc;
  return keyswitch_impl(ks, out0, out1, rot1, evk, rot0, nullptr, (cudaStream_t)stream);
}

int cerium_hmult(cerium_keyswitch* ks, void* out0, void* out1, const void* a0, const void* a1, const void* b0,
                 const void* b1, const void* evk, int do_rescale, void* stream) {
  if (!ks || !out0 || !out1 || !a0 || !a1 || !b0 || !b1 || !evk) return fail(CERIUM_ERR_INVALID, "hmult: null argument");
  cerium_context* ctx = ks->ctx;
  if (do_rescale && ks->L < 2) return fail(CERIUM_ERR_INVALID, "hmult: cannot rescale a one-limb ciphertext");
  DeviceGuard guard(ctx->device);
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  const size_t limb = n * wb;
  char* tmp = static_cast<char*>(ks->ws) + ks->o_tmp * wb;
  void* d0 = tmp;
  void* d1 = tmp + (size_t)ks->L * limb;
  void* d2 = tmp + (size_t)2 * ks->L * limb;
  if (int rc = cerium_tensor(ctx, d0, d1, d2, a0, a1, b0, b1, n, ks->q_idx.data(), ks->L, stream)) return rc;
  if (!do_rescale) return keyswitch_impl(ks, out0, out1, d2, evk, d0, d1, (cudaStream_t)stream);
  char* kso = static_cast<char*>(ks->ws) + ks->o_ksout * wb;  // [2][L][N], contiguous: two polynomials
  if (int rc = keyswitch_impl(ks, kso, kso + (size_t)ks->L * limb, d2, evk, d0, d1, (cudaStream_t)stream)) return rc;
  void* scratch = static_cast<char*>(ks->ws) + ks->o_scratch * wb;
  // out0 / out1 are separate buffers: rescale each polynomial on its own
  if (int rc = rescale_impl(ctx, ks->round_mode, out0, kso, ks->q_idx.data(), ks->L, 1, scratch, (cudaStream_t)stream)) return rc;
  return rescale_impl(ctx, ks->round_mode, out1, kso + (size_t)ks->L * limb, ks->q_idx.data(), ks->L, 1,
                      static_cast<char*>(scratch) + limb, (cudaStream_t)stream);
}

int cerium_rescale(cerium_context* ctx, int round_mode, void* out, const void* in, const uint32_t* q_idx, int L,
                   int n_polys, void* scratch, void* stream) {
  if (!ctx || !out || !in || !q_idx || !scratch) return fail(CERIUM_ERR_INVALID, "rescale: null argument");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "rescale: unknown round mode");
  if (L < 2 || L - 1 > kSudMaxBatch) return fail(CERIUM_ERR_INVALID, "rescale: need 2 <= L <= 65");
  if (n_polys < 1 || n_polys > 4096) return fail(CERIUM_ERR_INVALID, "rescale: need 1 <= n_polys <= 4096");
  for (int i = 0; i < L; i++)
    if (q_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "rescale: prime index out of range");
  if (((uintptr_t)out | (uintptr_t)in | (uintptr_t)scratch) & 15u) return fail(CERIUM_ERR_INVALID, "rescale: pointers must be 16-byte aligned");
  DeviceGuard guard(ctx->device);
  return rescale_impl(ctx, round_mode, out, in, q_idx, L, n_polys, scratch, (cudaStream_t)stream);
}

}  // extern "C"
