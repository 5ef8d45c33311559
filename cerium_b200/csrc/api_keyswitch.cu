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

// A plan covers the limbs one GPU owns.  With `world` GPUs, Q-limb i lives on rank i % world
// (cerium/compiler/backend/terms.h:672-685) and the K extension limbs are replicated on every
// rank (Term::Ext): "local extended limb" e < nloc is global limb loc[e], e >= nloc is extension
// limb e - nloc.  L and LK below are the LOCAL counts (nloc and nloc + K); world = 1 makes them
// the global ones.
struct cerium_keyswitch {
  cerium_context* ctx = nullptr;
  int bconv_mode = 0, round_mode = 0;
  int L = 0, K = 0, dnum = 0, LK = 0;
  int L_global = 0, rank = 0, world = 1, gather_limbs = 0;  // gather_limbs = ceil(L_global / world)
  // extension limbs: replicated on every rank (K == K_global), or split over the ranks like the Q limbs
  // (extension limb k lives on rank (L_global + k) % world; K is then the LOCAL count and the coefficient-
  // form extension limbs of the accumulators are all-gathered before the ModDown conversion)
  bool ext_split = false;
  int K_global = 0, pgather_limbs = 0;  // pgather_limbs = ceil(K_global / world), per polynomial and rank
  std::vector<int> ploc;           // global index of local extension limb
  std::vector<uint32_t> ext_dst;   // ext_split: slot of each entry of ext_pos inside this rank's block of `pgather`
  std::vector<int> loc;            // global index of local Q-limb e
  std::vector<int> own_digit;      // [LK] digit of local extended limb e, -1 for extension limbs
  std::vector<uint32_t> q_idx, p_idx, all_idx;  // prime indices of the LOCAL limbs
  std::vector<cerium_bconv*> up;   // one converter per non-empty digit
  std::vector<int> up_digit;       // digit number of up[k]
  cerium_bconv* down = nullptr;    // P -> Q
  std::vector<uint64_t> pinv;      // [L] P^-1 mod q_i
  std::vector<uint64_t> pmod;      // [L] P mod q_i (the PMU factor, cerium/runtime/execution/function.cpp:733-755)
  // ModDown with r = 1, 2 rescale levels in the same division (one-GPU plans): converter
  // (dropped Q limbs, P) -> remaining Q limbs, (P * dropped primes)^-1, the limbs to inverse-transform
  struct FusedDown {
    cerium_bconv* down = nullptr;
    std::vector<uint64_t> pinv;              // [L - r]
    std::vector<uint32_t> ext_pos, ext_prime;  // both accumulators: slots [L - r, LK) of each
    void* d_scale = nullptr;                 // exact mode: per entry of ext_pos, then the Shoup companions
    void* d_scale_shoup = nullptr;
  };
  std::vector<FusedDown> fused;
  // transform batches
  std::vector<uint32_t> ntt_pos, ntt_prime;  // converted limbs of all digits inside `raised`
  // one-limb digits: the conversion is a plain reduction, done by the transform as it reads the
  // digit's limb (slot ntt_src[b] of the gathered buffer); no converters exist then
  bool direct_raise = false;
  std::vector<uint32_t> ntt_src, ntt_src_prime;
  // lifted plan (ModRaise): one digit whose value arrives as an exact integer and is reduced modulo
  // every prime of the plan by the caller of keyswitch_inner_moddown; no converters, no own limbs
  bool lifted = false;
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
  // sharded plans: [world][gather_limbs] coefficient-form limbs of the switched polynomial, and with
  // ext_split [world][2][pgather_limbs] coefficient-form extension limbs of the two accumulators; a rank
  // writes its own block in place and the all-gather fills the others
  size_t o_gathered = 0, o_pgather = 0;
};

namespace {

template <typename W>
W* ws_at(const cerium_keyswitch* ks, size_t off_words) {
  return static_cast<W*>(ks->ws) + off_words;
}

// Drops the last limb of n_polys polynomials stored back to back in `in` ([n_polys][L][N]);
// polynomial p goes to outs[p] ([L-1][N]).  Two polynomials share a launch pair when their
// results are adjacent in memory or `pair_work` (a [2(L-1)][N] stack) is given.
// addend0 (optional, [L-1][N]) is added to polynomial 0.
// have_last: `scratch` already holds the coefficient-form last limbs (another rank produced them)
// and `in` is [n_polys][L-1][N], the remaining limbs only.
int rescale_impl(cerium_context* ctx, int round_mode, void* const* outs, void* pair_work, const void* in,
                 const uint32_t* q_idx, int L, int n_polys, void* scratch, cudaStream_t stream,
                 const void* addend0 = nullptr, bool have_last = false) {
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  const size_t limb = n * wb;
  const uint32_t last = q_idx[L - 1];
  const uint64_t ql = ctx->moduli[last];
  const int R = L - 1;
  const int in_limbs = have_last ? R : L;  // limbs per polynomial in `in`
  // 1. inverse transform of the last limb of every polynomial -> scratch[poly][N]
  std::vector<uint32_t> pos(n_polys), prime(n_polys, last);
  for (int p = 0; p < n_polys; p++) pos[p] = (uint32_t)p;
  if (!have_last) {
    // input limb of poly p sits at in + (p*L + L-1)*N: base shifted to the first such limb, stride L*N
    NttCall c{};
    c.in = static_cast<const char*>(in) + (size_t)R * limb;
    c.in_stride = (size_t)L * n;
    c.out = scratch;
    c.out_stride = n;
    c.pos = pos.data();
    c.prime = prime.data();
    c.count = n_polys;
    if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, stream)) return rc;
  }
  // 2. SuD of the remaining limbs against the re-reduced last limb
  std::vector<uint64_t> factor(2 * R), post_sub(2 * R);
  std::vector<uint32_t> prime2(2 * R), src_pos(2 * R);
  const uint64_t half = ql >> 1;
  for (int i = 0; i < 2 * R; i++) {
    const uint64_t q = ctx->moduli[q_idx[i % R]];
    prime2[i] = q_idx[i % R];
    factor[i] = host::invmod(ql % q, q);
    post_sub[i] = round_mode == CERIUM_ROUND_HALF ? half % q : 0;
    src_pos[i] = i < R ? 0 : 1;
  }
  for (int p = 0; p < n_polys;) {
    SudCall s{};
    s.src = static_cast<const char*>(scratch) + (size_t)p * limb;
    s.work_stride = n;
    s.dst = outs[p];
    s.dst_stride = n;
    s.minuend = static_cast<const char*>(in) + (size_t)p * in_limbs * limb;
    s.minuend_stride = n;
    if (p == 0 && addend0 != nullptr) {
      s.addend = addend0;
      s.addend_stride = n;
    }
    s.prime = prime2.data();
    s.factor = factor.data();
    s.reduce_src = true;
    s.src_q = ql;
    s.pre_add = round_mode == CERIUM_ROUND_HALF ? half : 0;
    s.post_sub = post_sub.data();
    const bool adjacent = p + 1 < n_polys && outs[p + 1] == static_cast<char*>(outs[p]) + (size_t)R * limb;
    if (p + 1 < n_polys && 2 * R <= kSudMaxBatch && (adjacent || pair_work != nullptr)) {
      s.src_stride = n;
      s.src_pos = src_pos.data();
      s.work = adjacent ? outs[p] : pair_work;
      s.count = 2 * R;
      s.split = R;
      s.dst2 = outs[p + 1];
      s.minuend2 = static_cast<const char*>(in) + (size_t)(p + 1) * in_limbs * limb;
      p += 2;
    } else {
      s.src_stride = 0;
      s.work = outs[p];
      s.count = R;
      p += 1;
    }
    if (int rc = launch_sud(ctx, s, stream)) return rc;
  }
  return CERIUM_OK;
}

// Step 1: inverse transform of the local limbs of the switched polynomial into `dst`
// ([gather_limbs][N]; exact mode: times [Qhat_i^-1] of the limb's digit).
// pre_elt (here and below), not 0: the key switch runs on the Galois automorphism of this element
// applied to cpoly and to add0 / add1, which are read through the index map wherever they are used
// (a rotation then needs no pass and no copy of its own).
int keyswitch_begin(cerium_keyswitch* ks, void* dst, const void* cpoly, cudaStream_t stream, uint32_t pre_elt = 0) {
  const size_t n = kN;
  NttCall c{cpoly, dst, n, n, nullptr, ks->q_idx.data(), ks->L};
  c.in_galois = pre_elt;
  return launch_ntt_inverse(ks->ctx, c, ks->d_scale_q, ks->d_scale_q_shoup, stream);
}

// Steps 2-7 from the coefficient-form limbs of ALL ranks (`gathered`: global limb i at slot
// (i % world) * gather_limbs + i / world).
// Steps 2-3: base conversion of every digit and forward transform of the converted limbs into
// the plan's `raised` buffer.
int keyswitch_raise(cerium_keyswitch* ks, const void* gathered, cudaStream_t stream) {
  cerium_context* ctx = ks->ctx;
  const size_t n = kN;
  const int LK = ks->LK;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    W* raised = ws_at<W>(ks, ks->o_raised);
    if (ks->direct_raise) {
      NttCall c{gathered, raised, n, n, ks->ntt_pos.data(), ks->ntt_prime.data(), (int)ks->ntt_pos.size()};
      c.src_pos = ks->ntt_src.data();
      c.src_prime = ks->ntt_src_prime.data();
      return launch_ntt_forward(ctx, c, stream, /*lazy_out=*/true);
    }
    // 2. ModUp base conversion, every digit in one launch
    {
      std::vector<BconvCall> calls;
      for (size_t k = 0; k < ks->up.size(); k++) {
        const int d = ks->up_digit[k];
        calls.push_back(BconvCall{ks->up[k], raised + (size_t)d * LK * n, n, gathered, n});
      }
      if (int rc = launch_bconv(ctx, calls.data(), (int)calls.size(), stream)) return rc;
    }
    // 3. NTT of every converted limb
    {
      NttCall c{raised, raised, n, n, ks->ntt_pos.data(), ks->ntt_prime.data(), (int)ks->ntt_pos.size()};
      c.lazy_in = true;  // the converters of step 2 are created with lazy_out
      if (int rc = launch_ntt_forward(ctx, c, stream, /*lazy_out=*/true)) return rc;
    }
    return CERIUM_OK;
  });
}

// Step 4 on the digits that keyswitch_raise left in the plan: inner product with `evk` into the
// plan's accumulators (both polynomials, every local extended limb).  accumulate: add to what the
// accumulators hold (the giant steps of a BSGS multiply-accumulate sum up in the extended basis).
int keyswitch_inner(cerium_keyswitch* ks, const void* cpoly, const void* evk, cudaStream_t stream, uint32_t pre_elt = 0,
                    bool accumulate = false) {
  cerium_context* ctx = ks->ctx;
  const size_t n = kN;
  const int LK = ks->LK, dnum = ks->dnum;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    W* acc = ws_at<W>(ks, ks->o_acc);
    InnerProductArgs<W> g{};
    g.raised = ws_at<W>(ks, ks->o_raised);
    g.raised_digit_stride = (size_t)LK * n;
    g.raised_limb_stride = n;
    g.own = static_cast<const W*>(cpoly);
    g.own_stride = n;
    g.own_elt = pre_elt;
    g.accumulate = accumulate ? 1 : 0;
    g.evk = static_cast<const W*>(evk);
    g.evk_digit_stride = (size_t)2 * LK * n;
    g.evk_poly_stride = (size_t)LK * n;
    g.evk_limb_stride = n;
    g.out0 = {acc, n};
    g.out1 = {acc + (size_t)LK * n, n};
    g.dnum = dnum;
    for (int b = 0; b < LK; b++) {
      g.prime[b] = (uint8_t)ks->all_idx[b];
      g.own_digit[b] = (int8_t)ks->own_digit[b];
    }
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    // every local extended limb (Q and extension) in one launch
    g.first_limb = 0;
    { auto kfn = inner_product_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / (kEwThreads * V::kLanes), LK), dim3(kEwThreads), 0, stream, g, pcs); }
    CERIUM_LAUNCH_CHECK("inner_product");
    return CERIUM_OK;
  });
}

// Steps 5-7: ModDown of the plan's accumulators, optional additions.
// comm: needed by plans with split extension limbs, whose accumulators' extension limbs are
// all-gathered (coefficient form) between steps 5 and 6.
// r > 0: the last r Q limbs are divided away in the same step (they join the extension limbs:
// cerium/compiler/backend/compiler_keyswitch.cc:26-39, 402-412); add0 / add1 then enter as the
// reference's PMU group does, acc += [P] * add on the Q limbs, and the outputs hold L - r limbs.
int keyswitch_moddown(cerium_keyswitch* ks, void* out0, void* out1, const void* add0, const void* add1,
                      cudaStream_t stream, uint32_t pre_elt = 0, uint32_t store_elt = 0, cerium_comm* comm = nullptr,
                      int r = 0) {
  if (ks->ext_split && comm == nullptr)
    return fail(CERIUM_ERR_INVALID, "keyswitch: a plan with split extension limbs needs a communicator");
  cerium_context* ctx = ks->ctx;
  const size_t n = kN;
  const int L = ks->L, K = ks->K, LK = ks->LK;
  if (r > 0) {
    if (r > 2 || (size_t)r > ks->fused.size() || ks->fused[r - 1].down == nullptr)
      return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch: this plan has no ModDown with that many rescale levels (1 or 2, one GPU, L - r >= 1)");
    if (pre_elt != 0 || store_elt != 0) return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch: a rotation cannot be folded into a ModDown with rescale levels");
  }
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    W* acc = ws_at<W>(ks, ks->o_acc);
    W* conv = ws_at<W>(ks, ks->o_conv);
    if (r > 0) {
      const cerium_keyswitch::FusedDown& fd = ks->fused[r - 1];
      const int Lr = L - r;
      // PMU: acc_p += [P] * add_p on all Q limbs (the dropped ones as well: they are divided away below)
      for (int p = 0; p < 2; p++) {
        const void* add = p == 0 ? add0 : add1;
        if (add == nullptr) continue;
        W* ap = acc + (size_t)p * LK * n;
        if (int rc = cerium_ewise(ctx, CERIUM_EW_PMU, ap, n, ap, n, add, n, nullptr, 0, ks->pmod.data(), ks->q_idx.data(), L, stream)) return rc;
      }
      // 5. iNTT of the extension limbs and the dropped Q limbs of both accumulators, in place
      {
        NttCall c{acc, acc, n, n, fd.ext_pos.data(), fd.ext_prime.data(), (int)fd.ext_pos.size()};
        if (int rc = launch_ntt_inverse(ctx, c, fd.d_scale, fd.d_scale_shoup, stream)) return rc;
      }
      // 6. base conversion (dropped Q limbs, P) -> remaining Q limbs
      {
        BconvCall calls[2] = {
            {fd.down, conv, n, acc + (size_t)Lr * n, n},
            {fd.down, conv + (size_t)Lr * n, n, acc + (size_t)(LK + Lr) * n, n},
        };
        if (int rc = launch_bconv(ctx, calls, 2, stream)) return rc;
      }
      // 7. SuD: out = (acc - NTT(conv)) * (P * dropped primes)^-1
      std::vector<uint32_t> prime2(ks->q_idx.begin(), ks->q_idx.begin() + Lr);
      prime2.insert(prime2.end(), ks->q_idx.begin(), ks->q_idx.begin() + Lr);
      std::vector<uint64_t> factor2(fd.pinv);
      factor2.insert(factor2.end(), fd.pinv.begin(), fd.pinv.end());
      for (int p = 0; p < 2; p++) {
        const bool both = 2 * Lr <= kSudMaxBatch;
        if (p == 1 && both) break;
        SudCall s{};
        s.src = conv + (size_t)p * Lr * n;
        s.src_stride = n;
        s.work = conv + (size_t)p * Lr * n;
        s.work_stride = n;
        s.dst = p == 0 ? out0 : out1;
        s.dst_stride = n;
        s.minuend = acc + (size_t)p * LK * n;
        s.minuend_stride = n;
        s.prime = prime2.data();
        s.factor = factor2.data();
        s.count = both ? 2 * Lr : Lr;
        if (both) {
          s.split = Lr;
          s.dst2 = out1;
          s.minuend2 = acc + (size_t)LK * n;
        }
        if (int rc = launch_sud(ctx, s, stream)) return rc;
      }
      return CERIUM_OK;
    }
    {
      const W* p0 = acc + (size_t)L * n;          // coefficient-form extension limbs of accumulator 0 ...
      const W* p1 = acc + (size_t)(LK + L) * n;   // ... and 1, as the ModDown conversion reads them
      if (!ks->ext_split) {
        // 5. iNTT of the extension limbs of both accumulators, in place
        NttCall c{acc, acc, n, n, ks->ext_pos.data(), ks->ext_prime.data(), 2 * K};
        if (int rc = launch_ntt_inverse(ctx, c, ks->d_scale_p, ks->d_scale_p_shoup, stream)) return rc;
      } else {
        // 5. iNTT of the LOCAL extension limbs into this rank's block of the gather buffer
        //    ([world][2][pgather_limbs]), then the all-gather: every rank needs all K limbs to convert
        W* pg = ws_at<W>(ks, ks->o_pgather);
        const size_t block = (size_t)2 * ks->pgather_limbs * n;
        W* mine = pg + (size_t)ks->rank * block;
        NttCall c{acc, mine, n, n, ks->ext_dst.data(), ks->ext_prime.data(), 2 * K};
        c.src_pos = ks->ext_pos.data();
        if (int rc = launch_ntt_inverse(ctx, c, ks->d_scale_p, ks->d_scale_p_shoup, stream)) return rc;
        if (int rc = comm_allgather(comm, pg, mine, block * sizeof(W), stream)) return rc;
        p0 = pg;
        p1 = pg + (size_t)ks->pgather_limbs * n;
      }
      if (L == 0) return CERIUM_OK;  // a rank without Q limbs only feeds the gathers
      // 6. ModDown base conversion P -> local Q limbs
      {
        BconvCall calls[2] = {
            {ks->down, conv, n, p0, n},
            {ks->down, conv + (size_t)L * n, n, p1, n},
        };
        if (int rc = launch_bconv(ctx, calls, 2, stream)) return rc;
      }
    }
    // 7. SuD: out = (acc_Q - NTT(conv)) * P^-1 (+ add); both polynomials in one launch pair
    if (2 * L <= kSudMaxBatch) {
      std::vector<uint32_t> prime2(ks->q_idx);
      prime2.insert(prime2.end(), ks->q_idx.begin(), ks->q_idx.end());
      std::vector<uint64_t> factor2(ks->pinv);
      factor2.insert(factor2.end(), ks->pinv.begin(), ks->pinv.end());
      SudCall s{};
      s.src = conv;
      s.src_stride = n;
      s.work = conv;
      s.work_stride = n;
      s.dst = out0;
      s.dst_stride = n;
      s.minuend = acc;
      s.minuend_stride = n;
      s.addend = add0;
      s.addend_stride = n;
      s.prime = prime2.data();
      s.factor = factor2.data();
      s.count = 2 * L;
      s.split = L;
      s.dst2 = out1;
      s.minuend2 = acc + (size_t)LK * n;
      s.addend2 = add1;
      s.addend_galois = pre_elt;
      s.store_galois = store_elt;
      if (int rc = launch_sud(ctx, s, stream)) return rc;
    } else {
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
        s.addend_galois = pre_elt;
        s.store_galois = store_elt;
        if (int rc = launch_sud(ctx, s, stream)) return rc;
      }
    }
    return CERIUM_OK;
  });
}

// Steps 4-7.  Can be repeated with different keys on the same raised digits (hoisting).
int keyswitch_inner_moddown(cerium_keyswitch* ks, void* out0, void* out1, const void* cpoly, const void* evk,
                            const void* add0, const void* add1, cudaStream_t stream, uint32_t pre_elt = 0,
                            uint32_t store_elt = 0, cerium_comm* comm = nullptr, int r = 0) {
  if (ks->ext_split && comm == nullptr)
    return fail(CERIUM_ERR_INVALID, "keyswitch: a plan with split extension limbs needs a communicator");
  if (int rc = keyswitch_inner(ks, cpoly, evk, stream, pre_elt)) return rc;
  return keyswitch_moddown(ks, out0, out1, add0, add1, stream, pre_elt, store_elt, comm, r);
}

int keyswitch_finish(cerium_keyswitch* ks, void* out0, void* out1, const void* gathered, const void* cpoly,
                     const void* evk, const void* add0, const void* add1, cudaStream_t stream, uint32_t pre_elt = 0,
                     cerium_comm* comm = nullptr) {
  if (int rc = keyswitch_raise(ks, gathered, stream)) return rc;
  return keyswitch_inner_moddown(ks, out0, out1, cpoly, evk, add0, add1, stream, pre_elt, 0, comm);
}

// The whole key switch of a limb-sharded plan: inverse transform of the local limbs straight into
// this rank's block of the gather buffer, all-gather (in place), steps 2-7 on the local limbs.
int keyswitch_sharded_impl(cerium_keyswitch* ks, cerium_comm* comm, void* out0, void* out1, const void* cpoly,
                           const void* evk, const void* add0, const void* add1, cudaStream_t stream,
                           uint32_t pre_elt = 0) {
  if (ks->world == 1) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded: the plan is not sharded");
  if (!comm || comm->world != ks->world || comm->rank != ks->rank)
    return fail(CERIUM_ERR_INVALID, "keyswitch_sharded: the communicator does not match the plan's rank and world");
  const size_t wb = ks->ctx->word_bytes();
  char* gathered = static_cast<char*>(ks->ws) + ks->o_gathered * wb;
  const size_t block = (size_t)ks->gather_limbs * kN * wb;
  char* mine = gathered + (size_t)ks->rank * block;
  if (int rc = keyswitch_begin(ks, mine, cpoly, stream, pre_elt)) return rc;
  if (int rc = comm_allgather(comm, gathered, mine, block, stream)) return rc;
  return keyswitch_finish(ks, out0, out1, gathered, cpoly, evk, add0, add1, stream, pre_elt, comm);
}

int keyswitch_impl(cerium_keyswitch* ks, void* out0, void* out1, const void* cpoly, const void* evk,
                   const void* add0, const void* add1, cudaStream_t stream, uint32_t pre_elt = 0, int r = 0) {
  if (ks->world != 1) return fail(CERIUM_ERR_INVALID, "keyswitch: a sharded plan needs the begin / finish calls around the all-gather");
  if (ks->lifted) return fail(CERIUM_ERR_INVALID, "keyswitch: a lifted plan only serves cerium_mod_raise");
  void* coef = static_cast<char*>(ks->ws) + ks->o_coef * ks->ctx->word_bytes();
  if (int rc = keyswitch_begin(ks, coef, cpoly, stream, pre_elt)) return rc;
  if (int rc = keyswitch_raise(ks, coef, stream)) return rc;
  return keyswitch_inner_moddown(ks, out0, out1, cpoly, evk, add0, add1, stream, pre_elt, 0, nullptr, r);
}

}  // namespace

extern "C" {

static int keyswitch_create_impl(cerium_context* ctx, cerium_keyswitch** out, int bconv_mode, int round_mode,
                                 const uint32_t* q_idx, int Lg, const uint32_t* p_idx, int Kg, int dnum, int rank,
                                 int world, bool lifted = false, bool ext_split = false) {
  const int K = Kg;  // the checks below are on the global shape
  if (!ctx || !out || !q_idx || !p_idx) return fail(CERIUM_ERR_INVALID, "keyswitch_create: null argument");
  if (bconv_mode != CERIUM_BCONV_LAZY && bconv_mode != CERIUM_BCONV_EXACT) return fail(CERIUM_ERR_INVALID, "keyswitch_create: unknown bconv mode");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "keyswitch_create: unknown round mode");
  if (Lg < 1 || K < 1 || dnum < 1 || dnum > Lg) return fail(CERIUM_ERR_INVALID, "keyswitch_create: need L >= 1, K >= 1, 1 <= dnum <= L");
  if (world < 1 || rank < 0 || rank >= world) return fail(CERIUM_ERR_INVALID, "keyswitch_create: need 0 <= rank < world");
  if (Lg + K > kEwMaxLimbs || Lg > 64) return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch_create: too many limbs (L <= 64, L + K <= 128)");
  const int alpha = (Lg + dnum - 1) / dnum;
  if (alpha > K && !lifted) return fail(CERIUM_ERR_INVALID, "keyswitch_create: digit size exceeds the number of extension primes");
  if ((size_t)dnum * (Lg + K) > 0xffff) return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch_create: dnum * (L + K) too large");
  std::vector<bool> seen(ctx->n_primes, false);
  for (int i = 0; i < Lg + K; i++) {
    const uint32_t p = i < Lg ? q_idx[i] : p_idx[i - Lg];
    if (p >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "keyswitch_create: prime index out of range");
    if (seen[p]) return fail(CERIUM_ERR_INVALID, "keyswitch_create: a prime appears twice");
    seen[p] = true;
  }
  for (int i = 0; i < Lg + K; i++) {
    const long double q = (long double)ctx->moduli[i < Lg ? q_idx[i] : p_idx[i - Lg]];
    // raised digits reach the inner product below 4q, the key below q
    if (4 * q * q * dnum >= (ctx->word_bits == 32 ? 1.8e19L : 3.4e38L))
      return fail(CERIUM_ERR_UNSUPPORTED, "keyswitch_create: dnum products of primes this wide overflow the accumulator");
  }
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "keyswitch_create: cannot select device");
  auto* ks = new cerium_keyswitch();
  ks->ctx = ctx;
  ks->bconv_mode = bconv_mode;
  ks->round_mode = round_mode;
  ks->dnum = dnum;
  ks->L_global = Lg;
  ks->K_global = Kg;
  ks->rank = rank;
  ks->world = world;
  ks->gather_limbs = (Lg + world - 1) / world;
  ks->ext_split = ext_split && world > 1;
  ks->pgather_limbs = (Kg + world - 1) / world;
  for (int i = rank; i < Lg; i += world) {
    ks->loc.push_back(i);
    ks->q_idx.push_back(q_idx[i]);
  }
  const int L = (int)ks->loc.size();
  ks->L = L;
  // the extension limbs this rank computes: all of them, or (split) those that continue the round robin
  for (int k = 0; k < Kg; k++)
    if (!ks->ext_split || (Lg + k) % world == rank) {
      ks->ploc.push_back(k);
      ks->p_idx.push_back(p_idx[k]);
    }
  ks->K = (int)ks->ploc.size();
  ks->LK = L + ks->K;
  ks->all_idx = ks->q_idx;
  ks->all_idx.insert(ks->all_idx.end(), ks->p_idx.begin(), ks->p_idx.end());
  const int LK = ks->LK;
  const int Kl = ks->K;  // local extension limbs
  ks->lifted = lifted;
  for (int e = 0; e < LK; e++) ks->own_digit.push_back((e < L && !lifted) ? ks->loc[e] % dnum : -1);
  const int bits = ctx->word_bits;
  const bool exact = bconv_mode == CERIUM_BCONV_EXACT;
  std::vector<uint64_t> scale_q(std::max(L, 1), 1), scale_p(2 * std::max(Kl, 1), 1);
  ks->direct_raise = alpha == 1;
  auto slot_of = [&](int i) { return (uint32_t)((i % world) * ks->gather_limbs + i / world); };
  int rc = CERIUM_OK;
  // per-digit converters: inputs = global limbs {d, d+dnum, ...} (read from the gathered buffer),
  // outputs = every local extended limb outside the digit
  for (int d = 0; d < dnum && rc == CERIUM_OK && !lifted; d++) {
    std::vector<uint32_t> in_primes, in_pos, out_primes, out_pos;
    std::vector<int> in_limb;
    for (int i = d; i < Lg; i += dnum) {
      in_primes.push_back(q_idx[i]);
      in_pos.push_back(slot_of(i));
      in_limb.push_back(i);
    }
    for (int e = 0; e < LK; e++) {
      if (ks->own_digit[e] == d) continue;
      out_primes.push_back(ks->all_idx[e]);
      out_pos.push_back((uint32_t)e);
      ks->ntt_pos.push_back((uint32_t)(d * LK + e));
      ks->ntt_prime.push_back(ks->all_idx[e]);
      ks->ntt_src.push_back(slot_of(d));
      ks->ntt_src_prime.push_back(q_idx[d]);
    }
    if (in_primes.empty() || out_primes.empty() || ks->direct_raise) continue;
    BconvOptions opt;
    opt.prescaled = exact;
    opt.out_pos = out_pos;
    opt.in_pos = in_pos;
    opt.lazy_out = true;  // ModUp outputs go straight into the forward transform
    cerium_bconv* bc = nullptr;
    rc = create_bconv(ctx, &bc, bconv_mode, in_primes.data(), (int)in_primes.size(), out_primes.data(),
                      (int)out_primes.size(), opt);
    if (rc != CERIUM_OK) break;
    ks->up.push_back(bc);
    ks->up_digit.push_back(d);
  }
  if (exact && !lifted && !ks->direct_raise) {
    // exact conversion: the inverse transform of local limb i leaves x_i * [Qhat_i^-1]_{q_i}, Qhat_i the
    // product of the other limbs of its digit (every rank scales its own limbs, whoever converts them)
    for (int e = 0; e < L; e++) {
      const int i = ks->loc[e];
      const uint64_t qi = ctx->moduli[q_idx[i]];
      uint64_t prod = 1 % qi;
      for (int j = i % dnum; j < Lg; j += dnum)
        if (j != i) prod = host::mulmod(prod, ctx->moduli[q_idx[j]] % qi, qi);
      scale_q[e] = host::invmod(prod, qi);
    }
  }
  if (rc == CERIUM_OK && L > 0) {
    // P -> Q over ALL extension primes; with split extension limbs the inputs are read from the gathered
    // buffer: limb k of a polynomial sits at slot owner(k) * 2 * pgather_limbs + (its index on the owner)
    BconvOptions opt;
    opt.prescaled = exact;
    opt.round_half = round_mode == CERIUM_ROUND_HALF;
    if (ks->ext_split) {
      std::vector<int> seen(world, 0);
      for (int k = 0; k < Kg; k++) {
        const int owner = (Lg + k) % world;
        opt.in_pos.push_back((uint32_t)(owner * 2 * ks->pgather_limbs + seen[owner]++));
      }
    }
    rc = create_bconv(ctx, &ks->down, bconv_mode, p_idx, Kg, ks->q_idx.data(), L, opt);
  }
  if (rc == CERIUM_OK && exact) {
    // [Phat_k^-1]_{p_k} does not depend on the output set
    for (int j = 0; j < Kl; j++) {
      const int k = ks->ploc[j];
      const uint64_t pk = ctx->moduli[p_idx[k]];
      uint64_t prod = 1 % pk;
      for (int i = 0; i < Kg; i++)
        if (i != k) prod = host::mulmod(prod, ctx->moduli[p_idx[i]] % pk, pk);
      scale_p[j] = scale_p[Kl + j] = Kg > 1 ? host::invmod(prod, pk) : 1;
    }
  }
  if (rc != CERIUM_OK) {
    cerium_keyswitch_destroy(ks);
    return rc;
  }
  ks->pinv.resize(L);
  {
    const std::vector<uint32_t> p_all(p_idx, p_idx + Kg);
    for (int i = 0; i < L; i++) {
      const uint64_t q = ctx->moduli[ks->q_idx[i]];
      ks->pinv[i] = host::invmod(host::product_mod(ctx->moduli, p_all, q), q);
    }
  }
  for (int p = 0; p < 2; p++)
    for (int k = 0; k < Kl; k++) {
      ks->ext_pos.push_back((uint32_t)(p * LK + L + k));
      ks->ext_prime.push_back(ks->p_idx[k]);
      ks->ext_dst.push_back((uint32_t)(p * ks->pgather_limbs + k));
    }
  ks->pmod.resize(L);
  {
    const std::vector<uint32_t> p_all(p_idx, p_idx + Kg);
    for (int i = 0; i < L; i++) ks->pmod[i] = host::product_mod(ctx->moduli, p_all, ctx->moduli[ks->q_idx[i]]);
  }
  const size_t wb = ctx->word_bytes();
  const size_t n = kN;
  // ModDown with rescale levels folded in (one-GPU plans only)
  for (int r = 1; r <= 2 && world == 1 && !lifted && L - r >= 1; r++) {
    cerium_keyswitch::FusedDown fd;
    const int Lr = L - r, E = Kg + r;
    std::vector<uint32_t> e_idx;
    for (int k = 0; k < r; k++) e_idx.push_back(q_idx[Lr + k]);
    for (int k = 0; k < Kg; k++) e_idx.push_back(p_idx[k]);
    BconvOptions opt;
    opt.prescaled = exact;
    opt.round_half = round_mode == CERIUM_ROUND_HALF;
    if (create_bconv(ctx, &fd.down, bconv_mode, e_idx.data(), E, ks->q_idx.data(), Lr, opt) != CERIUM_OK) {
      // a shape the converter cannot take (sum of products too wide): the plan simply has no fused variant
      fd.down = nullptr;
      ks->fused.push_back(fd);
      continue;
    }
    fd.pinv.resize(Lr);
    for (int i = 0; i < Lr; i++) {
      const uint64_t q = ctx->moduli[ks->q_idx[i]];
      fd.pinv[i] = host::invmod(host::product_mod(ctx->moduli, e_idx, q), q);
    }
    std::vector<uint64_t> sc, scs;
    for (int p = 0; p < 2; p++)
      for (int k = 0; k < E; k++) {
        fd.ext_pos.push_back((uint32_t)(p * LK + Lr + k));
        fd.ext_prime.push_back(e_idx[k]);
        const uint64_t ek = ctx->moduli[e_idx[k]];
        sc.push_back(exact ? fd.down->inv_host[k] : 1);
        scs.push_back(host::shoup(sc.back(), ek, bits));
      }
    if (exact) {
      std::vector<char> bytes(2 * sc.size() * wb);
      for (size_t i = 0; i < 2 * sc.size(); i++) {
        const uint64_t v = i < sc.size() ? sc[i] : scs[i - sc.size()];
        if (bits == 32) reinterpret_cast<uint32_t*>(bytes.data())[i] = (uint32_t)v;
        else reinterpret_cast<uint64_t*>(bytes.data())[i] = v;
      }
      if (cudaMalloc(&fd.d_scale, bytes.size()) != cudaSuccess ||
          cudaMemcpy(fd.d_scale, bytes.data(), bytes.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
        cerium_bconv_destroy(fd.down);
        cerium_keyswitch_destroy(ks);
        return fail(CERIUM_ERR_CUDA, "keyswitch_create: scale upload failed");
      }
      fd.d_scale_shoup = static_cast<char*>(fd.d_scale) + sc.size() * wb;
    }
    ks->fused.push_back(fd);
  }
  if (exact) {
    // [scale_q | scale_q_shoup | scale_p | scale_p_shoup]
    std::vector<uint64_t> all;
    for (int i = 0; i < L; i++) all.push_back(scale_q[i]);
    for (int i = 0; i < L; i++) all.push_back(host::shoup(scale_q[i], ctx->moduli[ks->q_idx[i]], bits));
    for (int i = 0; i < 2 * Kl; i++) all.push_back(scale_p[i]);
    for (int i = 0; i < 2 * Kl; i++) all.push_back(host::shoup(scale_p[i], ctx->moduli[ks->p_idx[i % Kl]], bits));
    if (all.empty()) all.push_back(0);
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
    ks->d_scale_p_shoup = b + (size_t)(2 * L + 2 * Kl) * wb;
  }
  // workspace layout (in words)
  size_t off = 0;
  auto take = [&](size_t limbs) {
    const size_t o = off;
    off += limbs * n;
    return o;
  };
  ks->o_coef = take(world == 1 ? Lg : 0);
  ks->o_gathered = take(world == 1 ? 0 : (size_t)world * ks->gather_limbs);
  ks->o_pgather = take(ks->ext_split ? (size_t)world * 2 * ks->pgather_limbs : 0);
  ks->o_raised = take((size_t)dnum * LK);
  ks->o_acc = take(2 * (size_t)LK);
  ks->o_conv = take(2 * (size_t)std::max(L, 1));
  ks->o_tmp = take(3 * (size_t)std::max(L, 1));
  ks->o_ksout = take(2 * (size_t)std::max(L, 1));
  ks->o_scratch = take(2);
  ks->ws_bytes = off * wb;
  if (cudaMalloc(&ks->ws, ks->ws_bytes) != cudaSuccess) {
    cerium_keyswitch_destroy(ks);
    return fail(CERIUM_ERR_CUDA, "keyswitch_create: cannot allocate the workspace");
  }
  *out = ks;
  return CERIUM_OK;
}

int cerium_keyswitch_create(cerium_context* ctx, cerium_keyswitch** out, int bconv_mode, int round_mode,
                            const uint32_t* q_idx, int L, const uint32_t* p_idx, int K, int dnum) {
  return keyswitch_create_impl(ctx, out, bconv_mode, round_mode, q_idx, L, p_idx, K, dnum, 0, 1);
}

int cerium_keyswitch_create_sharded(cerium_context* ctx, cerium_keyswitch** out, int bconv_mode, int round_mode,
                                    const uint32_t* q_idx, int L, const uint32_t* p_idx, int K, int dnum, int rank,
                                    int world, int ext_split) {
  return keyswitch_create_impl(ctx, out, bconv_mode, round_mode, q_idx, L, p_idx, K, dnum, rank, world, false,
                               ext_split != 0);
}

int cerium_keyswitch_create_lifted(cerium_context* ctx, cerium_keyswitch** out, int bconv_mode, int round_mode,
                                   const uint32_t* q_idx, int L, const uint32_t* p_idx, int K) {
  if (L < 4) return fail(CERIUM_ERR_INVALID, "keyswitch_create_lifted: need L >= 4");
  return keyswitch_create_impl(ctx, out, bconv_mode, round_mode, q_idx, L, p_idx, K, 1, 0, 1, /*lifted=*/true);
}

int cerium_mod_raise(cerium_keyswitch* ks, void* out0, void* out1, const void* c0, const void* c1, uint32_t base0,
                     uint32_t base1, const void* evk, void* stream) {
  if (!ks || !out0 || !out1 || !c0 || !c1 || !evk) return fail(CERIUM_ERR_INVALID, "mod_raise: null argument");
  if (!ks->lifted) return fail(CERIUM_ERR_INVALID, "mod_raise: the plan was not made by cerium_keyswitch_create_lifted");
  cerium_context* ctx = ks->ctx;
  if (base0 >= (uint32_t)ctx->n_primes || base1 >= (uint32_t)ctx->n_primes || base0 == base1)
    return fail(CERIUM_ERR_INVALID, "mod_raise: need two different base primes of the context");
  DeviceGuard guard(ctx->device);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = kN, wb = ctx->word_bytes(), limb = n * wb;
  const int L = ks->L, LK = ks->LK, Lt = L - 1;
  char* ws = static_cast<char*>(ks->ws);
  char* tmp = ws + ks->o_conv * wb;     // 8 limbs, free until the ModDown: [c0b0 c0b1 c1b0 c1b1 | lo0 hi0 lo1 hi1]
  char* t6 = ws + ks->o_tmp * wb;       // [Lt] the lifted c0
  char* raised = ws + ks->o_raised * wb;
  char* kso = ws + ks->o_ksout * wb;
  // 1. the four input limbs to coefficient form
  for (int k = 0; k < 2; k++) {
    const uint32_t prime[2] = {base0, base1};
    NttCall c{k == 0 ? c0 : c1, tmp + (size_t)2 * k * limb, n, n, nullptr, prime, 2};
    if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, st)) return rc;
  }
  // 2. exact CRT of each polynomial's pair of limbs: integers in [0, q_base0 * q_base1)
  if (int rc = cerium_resolve2(ctx, tmp + 4 * limb, tmp + 5 * limb, tmp, tmp + limb, 2 * n, base0, base1, 2, stream)) return rc;
  // 3. c0 lifted to the target primes
  if (int rc = cerium_mod2(ctx, t6, n, tmp + 4 * limb, tmp + 5 * limb, ks->q_idx.data(), Lt, stream)) return rc;
  {
    NttCall c{t6, t6, n, n, nullptr, ks->q_idx.data(), Lt};
    if (int rc = launch_ntt_forward(ctx, c, st)) return rc;
  }
  // 4. c1 lifted to every prime of the plan: the one digit of the key switch
  if (int rc = cerium_mod2(ctx, raised, n, tmp + 6 * limb, tmp + 7 * limb, ks->all_idx.data(), LK, stream)) return rc;
  {
    NttCall c{raised, raised, n, n, nullptr, ks->all_idx.data(), LK};
    if (int rc = launch_ntt_forward(ctx, c, st, /*lazy_out=*/true)) return rc;
  }
  // 5-6. product with the key, ModDown
  if (int rc = keyswitch_inner_moddown(ks, kso, kso + (size_t)L * limb, nullptr, evk, nullptr, nullptr, st)) return rc;
  // 7-8. drop the plan's last Q limb; add the lifted c0
  void* outs[2] = {out0, out1};
  void* scratch = ws + ks->o_scratch * wb;
  return rescale_impl(ctx, ks->round_mode, outs, tmp, kso, ks->q_idx.data(), L, 2, scratch, st, t6);
}

int cerium_keyswitch_local_limbs(const cerium_keyswitch* ks) { return ks ? ks->L : 0; }
int cerium_keyswitch_gather_limbs(const cerium_keyswitch* ks) { return ks ? ks->gather_limbs : 0; }

int cerium_keyswitch_sharded_begin(cerium_keyswitch* ks, void* send, const void* cpoly_local, void* stream) {
  if (!ks || !send) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_begin: null argument");
  if (ks->L > 0 && !cpoly_local) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_begin: null polynomial");
  if (ks->ext_split) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_begin: plans with split extension limbs exchange twice; use cerium_keyswitch_sharded_apply");
  DeviceGuard guard(ks->ctx->device);
  return keyswitch_begin(ks, send, cpoly_local, (cudaStream_t)stream);
}

int cerium_keyswitch_sharded_finish(cerium_keyswitch* ks, void* out0, void* out1, const void* gathered,
                                    const void* cpoly_local, const void* evk_local, const void* add0,
                                    const void* add1, void* stream) {
  if (!ks || !gathered || !evk_local) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_finish: null argument");
  if (ks->L > 0 && (!out0 || !out1 || !cpoly_local)) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_finish: null argument");
  if (ks->ext_split) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_finish: plans with split extension limbs exchange twice; use cerium_keyswitch_sharded_apply");
  DeviceGuard guard(ks->ctx->device);
  return keyswitch_finish(ks, out0, out1, gathered, cpoly_local, evk_local, add0, add1, (cudaStream_t)stream);
}

int cerium_keyswitch_local_ext_limbs(const cerium_keyswitch* ks) { return ks ? ks->K : 0; }

int cerium_keyswitch_sharded_apply(cerium_keyswitch* ks, cerium_comm* comm, void* out0, void* out1,
                                   const void* cpoly_local, const void* evk_local, const void* add0, const void* add1,
                                   void* stream) {
  if (!ks || !comm || !evk_local) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_apply: null argument");
  if (ks->L > 0 && (!out0 || !out1 || !cpoly_local)) return fail(CERIUM_ERR_INVALID, "keyswitch_sharded_apply: null argument");
  DeviceGuard guard(ks->ctx->device);
  return keyswitch_sharded_impl(ks, comm, out0, out1, cpoly_local, evk_local, add0, add1, (cudaStream_t)stream);
}

int cerium_hrot_sharded(cerium_keyswitch* ks, cerium_comm* comm, void* out0, void* out1, const void* c0_local,
                        const void* c1_local, const void* evk_local, uint32_t galois_elt, void* stream) {
  if (!ks || !comm || !evk_local) return fail(CERIUM_ERR_INVALID, "hrot_sharded: null argument");
  if (ks->L > 0 && (!out0 || !out1 || !c0_local || !c1_local)) return fail(CERIUM_ERR_INVALID, "hrot_sharded: null argument");
  if (!(galois_elt & 1) || galois_elt >= 2u * kN) return fail(CERIUM_ERR_INVALID, "hrot_sharded: Galois element is not valid");
  cerium_context* ctx = ks->ctx;
  DeviceGuard guard(ctx->device);
  const size_t wb = ctx->word_bytes();
  if (((uintptr_t)c0_local | (uintptr_t)c1_local) & 15u) return fail(CERIUM_ERR_INVALID, "hrot_sharded: pointers must be 16-byte aligned");
  // as in cerium_hrot: the rotation is folded into the key switch's reads of the local limbs unless an
  // output overlaps an input
  const size_t poly_bytes = (size_t)ks->L * kN * wb;
  auto overlaps = [&](const void* a, const void* b) {
    const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
    return x < y + poly_bytes && y < x + poly_bytes;
  };
  if (ks->L == 0 || (!overlaps(out0, c0_local) && !overlaps(out1, c0_local) && !overlaps(out0, c1_local) && !overlaps(out1, c1_local)))
    return keyswitch_sharded_impl(ks, comm, out0, out1, c1_local, evk_local, c0_local, nullptr, (cudaStream_t)stream, galois_elt);
  char* tmp = static_cast<char*>(ks->ws) + ks->o_tmp * wb;
  void* rot0 = tmp;
  void* rot1 = tmp + poly_bytes;
  if (int rc = launch_automorph_pair(ctx, rot0, c0_local, rot1, c1_local, galois_elt, ks->L, (cudaStream_t)stream)) return rc;
  return keyswitch_sharded_impl(ks, comm, out0, out1, rot1, evk_local, rot0, nullptr, (cudaStream_t)stream);
}

int cerium_rescale_sharded(cerium_context* ctx, cerium_comm* comm, int round_mode, void* out, const void* in,
                           const uint32_t* q_idx, int L, int n_polys, void* last_coef, void* stream) {
  if (!ctx || !comm || !q_idx || !last_coef) return fail(CERIUM_ERR_INVALID, "rescale_sharded: null argument");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "rescale_sharded: unknown round mode");
  if (L < 2 || L - 1 > 64 * comm->world) return fail(CERIUM_ERR_INVALID, "rescale_sharded: bad L");
  if (n_polys < 1 || n_polys > 4096) return fail(CERIUM_ERR_INVALID, "rescale_sharded: need 1 <= n_polys <= 4096");
  for (int i = 0; i < L; i++)
    if (q_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "rescale_sharded: prime index out of range");
  const int rank = comm->rank, world = comm->world;
  const int owner = (L - 1) % world;
  std::vector<uint32_t> mine, keep;
  for (int i = rank; i < L; i += world) {
    mine.push_back(q_idx[i]);
    if (i != L - 1) keep.push_back(q_idx[i]);
  }
  const int n_local = (int)mine.size();
  if ((n_local > 0 && !in) || (!keep.empty() && !out)) return fail(CERIUM_ERR_INVALID, "rescale_sharded: null argument");
  DeviceGuard guard(ctx->device);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = kN, wb = ctx->word_bytes();
  if (rank == owner) {
    // the dropped limb is the owner's last local limb of every polynomial
    std::vector<uint32_t> pos(n_polys), prime(n_polys, q_idx[L - 1]);
    for (int p = 0; p < n_polys; p++) pos[p] = (uint32_t)p;
    NttCall c{};
    c.in = static_cast<const char*>(in) + (size_t)(n_local - 1) * n * wb;
    c.in_stride = (size_t)n_local * n;
    c.out = last_coef;
    c.out_stride = n;
    c.pos = pos.data();
    c.prime = prime.data();
    c.count = n_polys;
    if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, st)) return rc;
  }
  if (int rc = comm_broadcast(comm, last_coef, (size_t)n_polys * n * wb, owner, st)) return rc;
  if (keep.empty()) return CERIUM_OK;
  // divide the remaining local limbs; on the owner they are strided by n_local inside `in`
  keep.push_back(q_idx[L - 1]);
  const int R = (int)keep.size() - 1;
  if (rank != owner) {
    std::vector<void*> outs(n_polys);
    for (int p = 0; p < n_polys; p++) outs[p] = static_cast<char*>(out) + (size_t)p * R * n * wb;
    return rescale_impl(ctx, round_mode, outs.data(), nullptr, in, keep.data(), R + 1, n_polys, last_coef, st, nullptr, true);
  }
  // owner: polynomial p's remaining limbs start at in + p * n_local limbs: one polynomial per call
  for (int p = 0; p < n_polys; p++) {
    void* o = static_cast<char*>(out) + (size_t)p * R * n * wb;
    const void* i = static_cast<const char*>(in) + (size_t)p * n_local * n * wb;
    void* lc = static_cast<char*>(last_coef) + (size_t)p * n * wb;
    if (int rc = rescale_impl(ctx, round_mode, &o, nullptr, i, keep.data(), R + 1, 1, lc, st, nullptr, true)) return rc;
  }
  return CERIUM_OK;
}

int cerium_keyswitch_destroy(cerium_keyswitch* ks) {
  if (!ks) return CERIUM_OK;
  DeviceGuard guard(ks->ctx->device);
  for (cerium_bconv* b : ks->up) cerium_bconv_destroy(b);
  if (ks->down) cerium_bconv_destroy(ks->down);
  for (auto& fd : ks->fused) {
    if (fd.down) cerium_bconv_destroy(fd.down);
    cudaFree(fd.d_scale);
  }
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

int cerium_keyswitch_apply_rescale(cerium_keyswitch* ks, void* out0, void* out1, const void* cpoly, const void* evk,
                                   const void* add0, const void* add1, int rescale_levels, void* stream) {
  if (!ks || !out0 || !out1 || !cpoly || !evk) return fail(CERIUM_ERR_INVALID, "keyswitch_apply_rescale: null argument");
  if (rescale_levels < 0 || rescale_levels > 2) return fail(CERIUM_ERR_INVALID, "keyswitch_apply_rescale: 0, 1 or 2 rescale levels");
  DeviceGuard guard(ks->ctx->device);
  return keyswitch_impl(ks, out0, out1, cpoly, evk, add0, add1, (cudaStream_t)stream, 0, rescale_levels);
}

int cerium_hrot(cerium_keyswitch* ks, void* out0, void* out1, const void* c0, const void* c1, const void* evk,
                uint32_t galois_elt, void* stream) {
  if (!ks || !out0 || !out1 || !c0 || !c1 || !evk) return fail(CERIUM_ERR_INVALID, "hrot: null argument");
  if (ks->world != 1) return fail(CERIUM_ERR_INVALID, "hrot: sharded plans are driven through the begin / finish calls");
  if (!(galois_elt & 1) || galois_elt >= 2u * kN) return fail(CERIUM_ERR_INVALID, "hrot: Galois element is not valid");
  cerium_context* ctx = ks->ctx;
  DeviceGuard guard(ctx->device);
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  char* tmp = static_cast<char*>(ks->ws) + ks->o_tmp * wb;
  void* rot0 = tmp;
  void* rot1 = tmp + (size_t)ks->L * n * wb;
  if (((uintptr_t)c0 | (uintptr_t)c1) & 15u) return fail(CERIUM_ERR_INVALID, "hrot: pointers must be 16-byte aligned");
  // The rotation is folded into the key switch's own reads of c0 and c1 (inverse transform, the
  // digits' own limbs in the inner product, the final addition) unless an output overlaps an input:
  // the last kernel writes out0 / out1 while it still gathers from c0, and the inner product reads c1.
  const size_t poly_bytes = (size_t)ks->L * n * wb;
  auto overlaps = [&](const void* a, const void* b) {
    const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
    return x < y + poly_bytes && y < x + poly_bytes;
  };
  if (!overlaps(out0, c0) && !overlaps(out1, c0) && !overlaps(out0, c1) && !overlaps(out1, c1))
    return keyswitch_impl(ks, out0, out1, c1, evk, c0, nullptr, (cudaStream_t)stream, galois_elt);
  if (int rc = launch_automorph_pair(ctx, rot0, c0, rot1, c1, galois_elt, ks->L, (cudaStream_t)stream)) return rc;
  return keyswitch_impl(ks, out0, out1, rot1, evk, rot0, nullptr, (cudaStream_t)stream);
}

int cerium_hoisted_begin(cerium_keyswitch* ks, const void* c1, void* stream) {
  if (!ks || !c1) return fail(CERIUM_ERR_INVALID, "hoisted_begin: null argument");
  if (ks->world != 1) return fail(CERIUM_ERR_INVALID, "hoisted_begin: sharded plans are driven through the begin / finish calls");
  if (ks->lifted) return fail(CERIUM_ERR_INVALID, "hoisted_begin: a lifted plan only serves cerium_mod_raise");
  DeviceGuard guard(ks->ctx->device);
  void* coef = static_cast<char*>(ks->ws) + ks->o_coef * ks->ctx->word_bytes();
  if (int rc = keyswitch_begin(ks, coef, c1, (cudaStream_t)stream)) return rc;
  return keyswitch_raise(ks, coef, (cudaStream_t)stream);
}

int cerium_hoisted_rotate(cerium_keyswitch* ks, void* out0, void* out1, const void* c0, const void* c1,
                          const void* evk_pre, uint32_t galois_elt, void* stream) {
  if (!ks || !out0 || !out1 || !c0 || !c1 || !evk_pre) return fail(CERIUM_ERR_INVALID, "hoisted_rotate: null argument");
  if (!(galois_elt & 1) || galois_elt >= 2u * kN) return fail(CERIUM_ERR_INVALID, "hoisted_rotate: Galois element is not valid");
  if (ks->world != 1) return fail(CERIUM_ERR_INVALID, "hoisted_rotate: sharded plans are driven through the begin / finish calls");
  cerium_context* ctx = ks->ctx;
  DeviceGuard guard(ctx->device);
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  char* tmp = static_cast<char*>(ks->ws) + ks->o_tmp * wb;
  void* t0 = tmp;
  void* t1 = tmp + (size_t)ks->L * n * wb;
  // (t0, t1) = KeySwitch(c1) + (c0, 0) on the un-rotated digits, then the automorphism: as the store
  // pattern of the last kernel (out[i] = t[pi_g(i)] is t[i] -> out[pi_{1/g}(i)]), unless an output
  // overlaps an input that kernel still reads
  {
    const size_t poly_bytes = (size_t)ks->L * n * wb;
    auto overlaps = [&](const void* a, const void* b) {
      const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
      return x < y + poly_bytes && y < x + poly_bytes;
    };
    if (!overlaps(out0, c0) && !overlaps(out1, c0) && !overlaps(out0, c1) && !overlaps(out1, c1)) {
      // inverse of the element modulo 2N (odd, so it exists): Newton steps double the valid bits
      uint32_t inv = galois_elt;
      for (int k = 0; k < 5; k++) inv *= 2u - galois_elt * inv;
      inv &= 2u * (uint32_t)kN - 1u;
      return keyswitch_inner_moddown(ks, out0, out1, c1, evk_pre, c0, nullptr, (cudaStream_t)stream, 0, inv);
    }
  }
  if (int rc = keyswitch_inner_moddown(ks, t0, t1, c1, evk_pre, c0, nullptr, (cudaStream_t)stream)) return rc;
  if (((uintptr_t)out0 | (uintptr_t)out1) & 15u) return fail(CERIUM_ERR_INVALID, "hoisted_rotate: pointers must be 16-byte aligned");
  return launch_automorph_pair(ctx, out0, t0, out1, t1, galois_elt, ks->L, (cudaStream_t)stream);
}

int cerium_hmult(cerium_keyswitch* ks, void* out0, void* out1, const void* a0, const void* a1, const void* b0,
                 const void* b1, const void* evk, int do_rescale, void* stream) {
  if (!ks || !out0 || !out1 || !a0 || !a1 || !b0 || !b1 || !evk) return fail(CERIUM_ERR_INVALID, "hmult: null argument");
  if (ks->world != 1) return fail(CERIUM_ERR_INVALID, "hmult: sharded plans are driven through the begin / finish calls");
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
  if (do_rescale < 0 || do_rescale > 2) return fail(CERIUM_ERR_INVALID, "hmult: do_rescale is 0, 1 or 2");
  if (int rc = cerium_tensor(ctx, d0, d1, d2, a0, a1, b0, b1, n, ks->q_idx.data(), ks->L, stream)) return rc;
  if (!do_rescale) return keyswitch_impl(ks, out0, out1, d2, evk, d0, d1, (cudaStream_t)stream);
  // one division by P * q_last: the last limb joins the extension limbs of the ModDown
  if (do_rescale == 2) return keyswitch_impl(ks, out0, out1, d2, evk, d0, d1, (cudaStream_t)stream, 0, 1);
  char* kso = static_cast<char*>(ks->ws) + ks->o_ksout * wb;  // [2][L][N], contiguous: two polynomials
  if (int rc = keyswitch_impl(ks, kso, kso + (size_t)ks->L * limb, d2, evk, d0, d1, (cudaStream_t)stream)) return rc;
  void* scratch = static_cast<char*>(ks->ws) + ks->o_scratch * wb;
  // out0 / out1 are separate buffers: the shared column pass works in the (now free) ModDown buffer
  void* outs[2] = {out0, out1};
  void* pair_work = static_cast<char*>(ks->ws) + ks->o_conv * wb;
  return rescale_impl(ctx, ks->round_mode, outs, pair_work, kso, ks->q_idx.data(), ks->L, 2, scratch, (cudaStream_t)stream);
}

int cerium_plaintext_mac(cerium_context* ctx, int n_out, int n_src, void* const* out0, void* const* out1,
                         const void* const* src0, const void* const* src1, const void* const* plaintexts,
                         const uint32_t* prime_idx, int count, void* stream) {
  if (!ctx || !out0 || !out1 || !src0 || !src1 || !plaintexts || !prime_idx) return fail(CERIUM_ERR_INVALID, "plaintext_mac: null argument");
  if (n_out < 1 || n_src < 1 || n_src > kBsgsMaxBaby) return fail(CERIUM_ERR_UNSUPPORTED, "plaintext_mac: 1..16 sources, at least one output");
  if (count < 1 || count > kEwMaxLimbs) return fail(CERIUM_ERR_INVALID, "plaintext_mac: 1..128 limbs");
  for (int b = 0; b < count; b++) {
    if (prime_idx[b] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "plaintext_mac: prime index out of range");
    const long double q = (long double)ctx->moduli[prime_idx[b]];
    if (q * q * n_src >= (ctx->word_bits == 32 ? 1.8e19L : 3.4e38L))
      return fail(CERIUM_ERR_UNSUPPORTED, "plaintext_mac: that many sources overflow the accumulator for primes this wide");
  }
  for (int j = 0; j < n_src; j++)
    if (!src0[j] || !src1[j] || (((uintptr_t)src0[j] | (uintptr_t)src1[j]) & 15u)) return fail(CERIUM_ERR_INVALID, "plaintext_mac: bad source pointer");
  for (int i = 0; i < n_out; i++)
    if (!out0[i] || !out1[i] || (((uintptr_t)out0[i] | (uintptr_t)out1[i]) & 15u)) return fail(CERIUM_ERR_INVALID, "plaintext_mac: bad output pointer");
  DeviceGuard guard(ctx->device);
  cudaStream_t st = (cudaStream_t)stream;
  return dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    for (int first = 0; first < n_out; first += kBsgsGroup) {
      const int cnt = std::min(kBsgsGroup, n_out - first);
      PtMacArgs<W> a{};
      a.g = n_src;
      for (int j = 0; j < n_src; j++) {
        a.src0[j] = static_cast<const W*>(src0[j]);
        a.src1[j] = static_cast<const W*>(src1[j]);
      }
      for (int i = 0; i < cnt; i++) {
        a.out0[i] = static_cast<W*>(out0[first + i]);
        a.out1[i] = static_cast<W*>(out1[first + i]);
        for (int j = 0; j < n_src; j++) {
          const void* p = plaintexts[(size_t)(first + i) * n_src + j];
          if (p != nullptr && ((uintptr_t)p & 15u)) return fail(CERIUM_ERR_INVALID, "plaintext_mac: pointers must be 16-byte aligned");
          a.pt[i][j] = static_cast<const W*>(p);
        }
      }
      for (int b = 0; b < count; b++) a.prime[b] = (uint8_t)prime_idx[b];
      const dim3 grid(kN / (kEwThreads * PtMacLanes<W>::kWords), count);
      switch (cnt) {
        case 1: { auto kfn = pt_mac_kernel<W, 1>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        case 2: { auto kfn = pt_mac_kernel<W, 2>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        case 3: { auto kfn = pt_mac_kernel<W, 3>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        default: { auto kfn = pt_mac_kernel<W, 4>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
      }
    }
    CERIUM_LAUNCH_CHECK("plaintext_mac");
    return CERIUM_OK;
  });
}

size_t cerium_bsgs_work_limbs(const cerium_keyswitch* ks, int g, int n_giant) {
  if (!ks || g < 1 || n_giant < 1) return 0;
  // rotated copies of the input, the giant steps' inner sums, the two pre-addition sums
  return ((size_t)(g - 1) * 2 + (size_t)n_giant * 2 + 2) * (size_t)ks->L;
}

int cerium_bsgs_apply(cerium_keyswitch* ks, void* out0, void* out1, const void* c0, const void* c1, int g, int n_giant,
                      const void* const* plaintexts, const void* const* baby_keys_pre, const uint32_t* baby_elts,
                      const void* const* giant_keys, const uint32_t* giant_elts, int rescale_levels, void* work,
                      void* stream) {
  if (!ks || !out0 || !out1 || !c0 || !c1 || !plaintexts || !giant_elts || !work)
    return fail(CERIUM_ERR_INVALID, "bsgs_apply: null argument");
  if (ks->world != 1 || ks->lifted) return fail(CERIUM_ERR_INVALID, "bsgs_apply: needs a one-GPU key-switching plan");
  if (g < 1 || g > kBsgsMaxBaby || n_giant < 1 || n_giant > kBsgsMaxGiant)
    return fail(CERIUM_ERR_UNSUPPORTED, "bsgs_apply: at most 16 baby steps and 32 giant steps");
  if (g > 1 && (!baby_keys_pre || !baby_elts)) return fail(CERIUM_ERR_INVALID, "bsgs_apply: baby steps need keys and elements");
  if (rescale_levels < 0 || rescale_levels > 2) return fail(CERIUM_ERR_INVALID, "bsgs_apply: 0, 1 or 2 rescale levels");
  cerium_context* ctx = ks->ctx;
  const int L = ks->L;
  if (((uintptr_t)work | (uintptr_t)c0 | (uintptr_t)c1 | (uintptr_t)out0 | (uintptr_t)out1) & 15u)
    return fail(CERIUM_ERR_INVALID, "bsgs_apply: pointers must be 16-byte aligned");
  for (int i = 0; i < L; i++) {
    // g products of two residues per accumulator
    const long double q = (long double)ctx->moduli[ks->q_idx[i]];
    if (q * q * g >= (ctx->word_bits == 32 ? 1.8e19L : 3.4e38L))
      return fail(CERIUM_ERR_UNSUPPORTED, "bsgs_apply: that many baby steps overflow the accumulator for primes this wide");
  }
  int n_rot = 0;
  for (int i = 0; i < n_giant; i++) {
    if (!(giant_elts[i] & 1) || giant_elts[i] >= 2u * kN) return fail(CERIUM_ERR_INVALID, "bsgs_apply: Galois element is not valid");
    if (giant_elts[i] != 1) {
      if (!giant_keys || !giant_keys[i]) return fail(CERIUM_ERR_INVALID, "bsgs_apply: a rotated giant step has no key");
      n_rot++;
    }
  }
  if (n_rot == 0 && rescale_levels != 0) return fail(CERIUM_ERR_UNSUPPORTED, "bsgs_apply: rescale levels need at least one rotated giant step");
  DeviceGuard guard(ctx->device);
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = kN, wb = ctx->word_bytes(), poly = (size_t)L * n * wb;
  char* w = static_cast<char*>(work);
  char* baby = w;                                        // [g-1][2][L]
  char* inner = baby + (size_t)(g - 1) * 2 * poly;       // [n_giant][2][L]
  char* sum0 = inner + (size_t)n_giant * 2 * poly;       // [L]  sum of the rotated first polynomials
  char* sum1 = sum0 + poly;                              // [L]  sum of the un-rotated second polynomials
  // 1. baby steps: g - 1 hoisted rotations of the input (one ModUp)
  if (g > 1) {
    if (int rc = cerium_hoisted_begin(ks, c1, stream)) return rc;
    for (int j = 1; j < g; j++) {
      if (!baby_keys_pre[j]) return fail(CERIUM_ERR_INVALID, "bsgs_apply: a baby step has no key");
      char* bj = baby + (size_t)(j - 1) * 2 * poly;
      if (int rc = cerium_hoisted_rotate(ks, bj, bj + poly, c0, c1, baby_keys_pre[j], baby_elts[j], stream)) return rc;
    }
  }
  // 2. inner sums s_i = sum_j pt[i][j] * baby_j, kBsgsGroup giant steps per pass over the baby steps
  std::vector<char> have(n_giant, 0);
  int rc = dispatch_word(ctx->word_bits, [&](auto tag) -> int {
    using W = decltype(tag);
    using V = Vec16<W>;
    const PrimeConst<W>* pcs = static_cast<const PrimeConst<W>*>(ctx->d_pcs);
    for (int first = 0; first < n_giant; first += kBsgsGroup) {
      const int cnt = std::min(kBsgsGroup, n_giant - first);
      PtMacArgs<W> a{};
      a.g = g;
      for (int j = 0; j < g; j++) {
        const char* b = j == 0 ? nullptr : baby + (size_t)(j - 1) * 2 * poly;
        a.src0[j] = reinterpret_cast<const W*>(j == 0 ? static_cast<const char*>(c0) : b);
        a.src1[j] = reinterpret_cast<const W*>(j == 0 ? static_cast<const char*>(c1) : b + poly);
      }
      for (int i = 0; i < kBsgsGroup; i++) {
        const int gi = first + std::min(i, cnt - 1);   // unused slots of the last group repeat its last giant step
        a.out0[i] = reinterpret_cast<W*>(inner + (size_t)gi * 2 * poly);
        a.out1[i] = reinterpret_cast<W*>(inner + (size_t)gi * 2 * poly + poly);
        for (int j = 0; j < g; j++) {
          const void* p = i < cnt ? plaintexts[(size_t)(first + i) * g + j] : nullptr;
          if (p != nullptr && ((uintptr_t)p & 15u)) return fail(CERIUM_ERR_INVALID, "bsgs_apply: pointers must be 16-byte aligned");
          a.pt[i][j] = static_cast<const W*>(p);
          if (p != nullptr) have[first + i] = 1;
        }
      }
      for (int b = 0; b < L; b++) a.prime[b] = (uint8_t)ks->q_idx[b];
      const dim3 grid(kN / (kEwThreads * PtMacLanes<W>::kWords), L);
      switch (cnt) {
        case 1: { auto kfn = pt_mac_kernel<W, 1>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        case 2: { auto kfn = pt_mac_kernel<W, 2>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        case 3: { auto kfn = pt_mac_kernel<W, 3>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
        default: { auto kfn = pt_mac_kernel<W, 4>; CERIUM_LAUNCH(kfn, grid, kEwThreads, 0, st, a, pcs); } break;
      }
    }
    CERIUM_LAUNCH_CHECK("bsgs plaintext multiply-accumulate");
    // 3. sum0 = sum_i phi_i(s_i.c0) over every giant step, sum1 = sum of s_i.c1 over the un-rotated ones
    for (int which = 0; which < 2; which++) {
      AutoSumArgs<W> s{};
      for (int i = 0; i < n_giant; i++) {
        if (!have[i] || (which == 1 && giant_elts[i] != 1)) continue;
        s.in[s.count] = reinterpret_cast<const W*>(inner + (size_t)i * 2 * poly + (which ? poly : 0));
        s.elt[s.count] = giant_elts[i];
        s.count++;
      }
      s.out = reinterpret_cast<W*>(which ? sum1 : sum0);
      for (int b = 0; b < L; b++) s.prime[b] = (uint8_t)ks->q_idx[b];
      { auto kfn = automorph_sum_kernel<W>; CERIUM_LAUNCH(kfn, dim3(kN / kEwThreads, L), kEwThreads, 0, st, s, pcs); }
    }
    CERIUM_LAUNCH_CHECK("bsgs rotation sums");
    return CERIUM_OK;
  });
  if (rc != CERIUM_OK) return rc;
  if (!have[0] && n_rot == 0) return fail(CERIUM_ERR_INVALID, "bsgs_apply: no diagonal at all");
  // 4. every rotated giant step: ModUp of phi_i(s_i.c1) (the rotation is the read pattern of the inverse
  //    transform and of the digits' own limbs) and its product with the key, summed in the extended basis
  void* coef = static_cast<char*>(ks->ws) + ks->o_coef * wb;
  bool first = true;
  for (int i = 0; i < n_giant; i++) {
    if (!have[i] || giant_elts[i] == 1) continue;
    const char* s1 = inner + (size_t)i * 2 * poly + poly;
    if (int r2 = keyswitch_begin(ks, coef, s1, st, giant_elts[i])) return r2;
    if (int r2 = keyswitch_raise(ks, coef, st)) return r2;
    if (int r2 = keyswitch_inner(ks, s1, giant_keys[i], st, giant_elts[i], !first)) return r2;
    first = false;
  }
  if (first) {
    // no rotated giant step: the sums are the result
    CERIUM_CUDA(cudaMemcpyAsync(out0, sum0, poly, cudaMemcpyDeviceToDevice, st));
    CERIUM_CUDA(cudaMemcpyAsync(out1, sum1, poly, cudaMemcpyDeviceToDevice, st));
    return CERIUM_OK;
  }
  // 5. ONE ModDown (with the rescale levels in the same division); the sums enter as the PMU
  //    pre-addition: as addends of the last kernel when nothing else is divided away
  return keyswitch_moddown(ks, out0, out1, sum0, sum1, st, 0, 0, nullptr, rescale_levels);
}

int cerium_rescale(cerium_context* ctx, int round_mode, void* out, const void* in, const uint32_t* q_idx, int L,
                   int n_polys, void* scratch, void* stream) {
  if (!ctx || !out || !in || !q_idx || !scratch) return fail(CERIUM_ERR_INVALID, "rescale: null argument");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "rescale: unknown round mode");
  if (L < 2 || L - 1 > 64) return fail(CERIUM_ERR_INVALID, "rescale: need 2 <= L <= 65");
  if (n_polys < 1 || n_polys > 4096) return fail(CERIUM_ERR_INVALID, "rescale: need 1 <= n_polys <= 4096");
  for (int i = 0; i < L; i++)
    if (q_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "rescale: prime index out of range");
  if (((uintptr_t)out | (uintptr_t)in | (uintptr_t)scratch) & 15u) return fail(CERIUM_ERR_INVALID, "rescale: pointers must be 16-byte aligned");
  DeviceGuard guard(ctx->device);
  std::vector<void*> outs(n_polys);
  for (int p = 0; p < n_polys; p++) outs[p] = static_cast<char*>(out) + (size_t)p * (L - 1) * kN * ctx->word_bytes();
  return rescale_impl(ctx, round_mode, outs.data(), nullptr, in, q_idx, L, n_polys, scratch, (cudaStream_t)stream);
}

int cerium_rescale_local(cerium_context* ctx, int round_mode, void* out, const void* in, const uint32_t* local_idx,
                         int n_local, uint32_t last_prime, const void* last_coef, int n_polys, void* stream) {
  if (!ctx || !out || !in || !local_idx || !last_coef) return fail(CERIUM_ERR_INVALID, "rescale_local: null argument");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF) return fail(CERIUM_ERR_INVALID, "rescale_local: unknown round mode");
  if (n_local < 1 || n_local > 64) return fail(CERIUM_ERR_INVALID, "rescale_local: need 1 <= n_local <= 64");
  if (n_polys < 1 || n_polys > 4096) return fail(CERIUM_ERR_INVALID, "rescale_local: need 1 <= n_polys <= 4096");
  if (last_prime >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "rescale_local: prime index out of range");
  std::vector<uint32_t> idx(local_idx, local_idx + n_local);
  for (uint32_t i : idx)
    if (i >= (uint32_t)ctx->n_primes || i == last_prime) return fail(CERIUM_ERR_INVALID, "rescale_local: bad local prime index");
  if (((uintptr_t)out | (uintptr_t)in | (uintptr_t)last_coef) & 15u) return fail(CERIUM_ERR_INVALID, "rescale_local: pointers must be 16-byte aligned");
  idx.push_back(last_prime);
  DeviceGuard guard(ctx->device);
  std::vector<void*> outs(n_polys);
  for (int p = 0; p < n_polys; p++) outs[p] = static_cast<char*>(out) + (size_t)p * n_local * kN * ctx->word_bytes();
  return rescale_impl(ctx, round_mode, outs.data(), nullptr, in, idx.data(), n_local + 1, n_polys,
                      const_cast<void*>(last_coef), (cudaStream_t)stream, nullptr, /*have_last=*/true);
}

int cerium_double_rescale(cerium_context* ctx, void* out, const void* in, const uint32_t* q_idx, int L, int n_polys,
                          void* scratch, void* stream) {
  if (!ctx || !out || !in || !q_idx || !scratch) return fail(CERIUM_ERR_INVALID, "double_rescale: null argument");
  if (L < 3 || L - 2 > 64) return fail(CERIUM_ERR_INVALID, "double_rescale: need 3 <= L <= 66");
  if (n_polys < 1 || n_polys > 128) return fail(CERIUM_ERR_INVALID, "double_rescale: need 1 <= n_polys <= 128");
  for (int i = 0; i < L; i++)
    if (q_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "double_rescale: prime index out of range");
  if (q_idx[L - 1] == q_idx[L - 2]) return fail(CERIUM_ERR_INVALID, "double_rescale: the two dropped primes are the same");
  if (((uintptr_t)out | (uintptr_t)in | (uintptr_t)scratch) & 15u) return fail(CERIUM_ERR_INVALID, "double_rescale: pointers must be 16-byte aligned");
  DeviceGuard guard(ctx->device);
  const size_t n = kN, wb = ctx->word_bytes(), limb = n * wb;
  const int R = L - 2;
  const uint32_t pa = q_idx[L - 2], pb = q_idx[L - 1];
  cudaStream_t st = (cudaStream_t)stream;
  char* sc = static_cast<char*>(scratch);  // per polynomial: [x_a | x_b | lo | hi]
  // 1. inverse transform of the two dropped limbs of every polynomial
  {
    // entry (p, k) reads limb p*L + L-2+k of `in`: one call per k with the input base shifted
    for (int k = 0; k < 2; k++) {
      std::vector<uint32_t> po(n_polys), pr(n_polys, k == 0 ? pa : pb);
      for (int p = 0; p < n_polys; p++) po[p] = (uint32_t)p;
      NttCall c{};
      c.in = static_cast<const char*>(in) + (size_t)(L - 2 + k) * limb;
      c.in_stride = (size_t)L * n;
      c.out = sc + (size_t)k * limb;
      c.out_stride = 4 * n;
      c.pos = po.data();
      c.prime = pr.data();
      c.count = n_polys;
      if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, st)) return rc;
    }
  }
  // 2. exact CRT composition of the pair, every polynomial in one launch
  if (int rc = cerium_resolve2(ctx, sc + 2 * limb, sc + 3 * limb, sc, sc + limb, 4 * n, pa, pb, n_polys, stream)) return rc;
  // 3. its residues modulo the remaining primes, written where the results will be
  for (int p = 0; p < n_polys; p++) {
    char* o = static_cast<char*>(out) + (size_t)p * R * limb;
    if (int rc = cerium_mod2(ctx, o, n, sc + (size_t)(4 * p + 2) * limb, sc + (size_t)(4 * p + 3) * limb, q_idx, R, stream)) return rc;
  }
  // 4. SuD in place: out = (in - NTT(out)) * (q_a q_b)^-1, two polynomials per launch pair
  std::vector<uint64_t> factor(2 * R);
  std::vector<uint32_t> prime2(2 * R);
  for (int i = 0; i < 2 * R; i++) {
    const uint64_t q = ctx->moduli[q_idx[i % R]];
    prime2[i] = q_idx[i % R];
    factor[i] = host::invmod(host::mulmod(ctx->moduli[pa] % q, ctx->moduli[pb] % q, q), q);
  }
  for (int p = 0; p < n_polys;) {
    char* o = static_cast<char*>(out) + (size_t)p * R * limb;
    SudCall s{};
    s.src = o;
    s.src_stride = n;
    s.work = o;
    s.work_stride = n;
    s.dst = o;
    s.dst_stride = n;
    s.minuend = static_cast<const char*>(in) + (size_t)p * L * limb;
    s.minuend_stride = n;
    s.prime = prime2.data();
    s.factor = factor.data();
    if (p + 1 < n_polys && 2 * R <= kSudMaxBatch) {
      s.count = 2 * R;
      s.split = R;
      s.dst2 = o + (size_t)R * limb;
      s.minuend2 = static_cast<const char*>(in) + (size_t)(p + 1) * L * limb;
      p += 2;
    } else {
      s.count = R;
      p += 1;
    }
    if (int rc = launch_sud(ctx, s, st)) return rc;
  }
  return CERIUM_OK;
}

}  // extern "C"
