/*
 * cerium_b200 - C ABI of the B200-native RNS-CKKS evaluation core.
 *
 * This is the boundary a Cerium runtime binds instead of the per-program
 * function_map_<p>.so it loads today (cerium/runtime/execution/function.cpp:144-177) and the
 * execute_* shims behind it (cerium/runtime/execution/device_utils.h:29-150).  Every entry
 * point is extern "C", takes plain pointers and sizes, returns a status code (no exceptions
 * cross the boundary; the reference throws std::runtime_error from CHECK_CUDA_ERROR,
 * cerium/compiler/backend/kernels/fhe.cuh:34-42) and enqueues work on the given CUDA stream
 * without synchronising.  Nothing here allocates device memory except the *_create calls.
 *
 * Data model
 *   - Ring degree N = 2^16 (fixed, as in cerium/compiler/backend/kernels/fhe_ntt.cuh:27).
 *   - A "limb" is N residues of one RNS prime: uint32_t words (primes below 2^30; the
 *     reference's 28-bit chain) or uint64_t words (primes below 2^60).  The word size is a
 *     property of the context.
 *   - A stack of limbs is addressed as base + i * stride (stride in WORDS); `prime_idx[i]`
 *     names the modulus of limb i as an index into the context's prime list.  The *_ptrs
 *     variants take device-resident pointer tables instead, the layout of the reference's
 *     launchers (cerium/compiler/backend/kernels/function.cu:22-39).
 *   - All residues that enter or leave a call are canonical, in [0, q).  (The reference's
 *     32-bit Barrett may leave values in [q, 2q); compare modulo q.)
 *   - NTT form is bit-reversed order with psi = the minimal primitive 2N-th root, i.e. the
 *     order of cerium/runtime/math/ntt.cpp:118-125.
 *   - Pointers must be 16-byte aligned and strides multiples of 16 bytes.
 */
#ifndef CERIUM_B200_H_
#define CERIUM_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CERIUM_API __attribute__((visibility("default")))
#else
#define CERIUM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define CERIUM_OK 0
#define CERIUM_ERR_INVALID 1     /* bad argument (null, size, alignment, unknown prime index) */
#define CERIUM_ERR_CUDA 2        /* a CUDA runtime call failed; see cerium_last_error()        */
#define CERIUM_ERR_UNSUPPORTED 3 /* parameter outside what the kernels are built for          */

/* base-conversion semantics */
#define CERIUM_BCONV_LAZY 0  /* Cerium: factors fold the CRT inverse (evaluator.cpp:1539-1578) */
#define CERIUM_BCONV_EXACT 1 /* inputs are multiplied by [Qhat_i^-1] mod q_i first             */
/* division semantics of ModDown / rescale */
#define CERIUM_ROUND_FLOOR 0 /* Cerium: no rounding term (fhe_ntt.cuh:346-358)                 */
#define CERIUM_ROUND_HALF 1  /* add floor(P/2) before dividing                                 */

/* element-wise operations of cerium_ewise() */
#define CERIUM_EW_ADD 0        /* out = a + b            */
#define CERIUM_EW_SUB 1        /* out = a - b            */
#define CERIUM_EW_NEG 2        /* out = -a               */
#define CERIUM_EW_MUL 3        /* out = a * b            */
#define CERIUM_EW_MAD 4        /* out = a * b + c        */
#define CERIUM_EW_PMU 5        /* out = a + b * s[i]     */
#define CERIUM_EW_MUL_SCALAR 6 /* out = a * s[i]         */
#define CERIUM_EW_REDUCE 7     /* out = a mod q, a any word (sums of residues after a collective) */

typedef struct cerium_context cerium_context;
typedef struct cerium_bconv cerium_bconv;
typedef struct cerium_keyswitch cerium_keyswitch;
typedef struct cerium_comm cerium_comm;
typedef struct cerium_program cerium_program;

/* Library version (major * 10000 + minor * 100 + patch). */
CERIUM_API int cerium_version(void);

/* Message of the last failing call on this host thread ("" if none). */
CERIUM_API const char *cerium_last_error(void);

/*
 * Context: device tables for a list of primes (moduli, Barrett constants, forward and
 * inverse twiddles with Shoup companions).  Replaces EvaluatorContext
 * (cerium/runtime/execution/evaluator.h:94-136, evaluator.cpp:58-269).
 * word_bits is 32 or 64; log_n must be 16; every modulus must be a prime = 1 mod 2N,
 * below 2^30 (32-bit words) or 2^60 (64-bit words); at most 255 moduli.
 */
CERIUM_API int cerium_context_create(cerium_context **out, int device, int log_n, int word_bits,
                          const uint64_t *moduli, int n_moduli);
CERIUM_API int cerium_context_destroy(cerium_context *ctx);
/*
 * Kernels never trap on a malformed work item (the reference's do no bounds checking at all,
 * cerium/compiler/backend/kernels/function.cuh:61-78): the affected CTAs skip it and set a bit in
 * a status word of the context.  cerium_context_check waits for the device, reads and clears that
 * word; it returns CERIUM_ERR_INVALID (and a message) when a bit was set since the last check.
 */
CERIUM_API int cerium_context_check(cerium_context *ctx);
CERIUM_API int cerium_context_word_bits(const cerium_context *ctx);
CERIUM_API int cerium_context_num_moduli(const cerium_context *ctx);
CERIUM_API uint64_t cerium_context_modulus(const cerium_context *ctx, int k);
CERIUM_API uint64_t cerium_context_root(const cerium_context *ctx, int k); /* psi of prime k */

/*
 * Forward / inverse negacyclic NTT of `count` limbs.  in == out is allowed.
 * Replaces _function_ntt_ / _function_int_ (cerium/compiler/backend/kernels/function.cu:
 * 58-72, 237-256) and Evaluator::fn_ntt / fn_int
 * (cerium/runtime/execution/evaluator.cpp:444-463, 540-551).
 */
CERIUM_API int cerium_ntt_forward(cerium_context *ctx, void *out, size_t out_stride, const void *in,
                       size_t in_stride, const uint32_t *prime_idx, int count, void *stream);
CERIUM_API int cerium_ntt_inverse(cerium_context *ctx, void *out, size_t out_stride, const void *in,
                       size_t in_stride, const uint32_t *prime_idx, int count, void *stream);

/*
 * The same with the reference launchers' argument layout: outs/ins are DEVICE arrays of
 * `num_bases` limb pointers, bases a DEVICE array of prime indices
 * (cerium/runtime/execution/device_utils.h:42-53).
 */
CERIUM_API int cerium_ntt_forward_ptrs(cerium_context *ctx, void *const *outs, const void *const *ins,
                            const uint32_t *bases, size_t num_bases, void *stream);
CERIUM_API int cerium_ntt_inverse_ptrs(cerium_context *ctx, void *const *outs, const void *const *ins,
                            const uint32_t *bases, size_t num_bases, void *stream);

/*
 * SuD with the argument tables of the reference's launcher (_function_sud_,
 * cerium/compiler/backend/kernels/function.cu:101-174; cerium/runtime/execution/device_utils.h:54-62):
 * all arrays are DEVICE resident.  Entry b has two inputs: ins[2b] is the minuend (NTT form),
 * ins[2b+1] the coefficient-form limb; outs[b] = (ins[2b] - NTT(ins[2b+1])) * factors[bases[b]] mod q.
 * `factors` has one word per prime of the context (compute_sud_factors layout,
 * cerium/runtime/execution/function.cpp:685-732).  outs[b] may alias either input.  Results are
 * canonical.
 */
CERIUM_API int cerium_sud_ptrs(cerium_context *ctx, void *const *outs, const void *const *ins,
                               const uint32_t *bases, size_t num_bases, const void *factors, void *stream);

/*
 * Base conversion with the argument tables of the reference's launcher (_function_bco_<I, O>,
 * cerium/compiler/backend/kernels/function.cuh:80-98, marshalled by Evaluator::fn_bco,
 * cerium/runtime/execution/evaluator.cpp:861-940): all arrays are DEVICE resident.  Conversion j
 * reads ins[j] = [n_in[j]][N] and writes outs[j] = [n_out[j]][N] with the factor matrix
 * factors[j] = [n_out[j]][n_in[j]] (DeviceBaseConverter, evaluator.cpp:1539-1578) and the output
 * primes out_moduli[j] = [n_out[j]]; no converter object and no prime index is involved.  max_in /
 * max_out are HOST upper bounds of the shapes (they size the shared memory); a table entry above
 * them is skipped on the device and reported by cerium_context_check.  The reference's lazy
 * conversion; results are canonical.
 */
CERIUM_API int cerium_bconv_ptrs(cerium_context *ctx, void *const *outs, const size_t *n_out,
                                 const void *const *ins, const size_t *n_in, const void *const *factors,
                                 const void *const *out_moduli, size_t max_in, size_t max_out,
                                 size_t num_conversions, void *stream);

/*
 * SuD: out[i] = (minuend[i] - NTT(in_coeff[i])) * [(prod divide primes)^-1] mod q_i,
 * optionally + addend[i] (addend may be NULL).  in_coeff holds coefficient-form residues
 * already reduced mod q_i.  out may alias minuend; in_coeff is overwritten (it is the
 * transform's work buffer).  Replaces _function_sud_
 * (cerium/compiler/backend/kernels/function.cu:151-169) and compute_sud_factors
 * (cerium/runtime/execution/function.cpp:685-732).
 */
CERIUM_API int cerium_sud(cerium_context *ctx, void *out, size_t out_stride, const void *minuend,
               size_t minuend_stride, void *in_coeff, size_t in_stride, const void *addend,
               size_t addend_stride, const uint32_t *prime_idx, int count,
               const uint32_t *divide_primes, int n_divide, void *stream);

/*
 * Element-wise modular arithmetic over `count` limbs (op = CERIUM_EW_*).  Unused operands
 * may be NULL.  `scalars` (host array, one canonical residue per limb) feeds PMU and
 * MUL_SCALAR.  Replaces the generated generic and PMU kernels
 * (cerium/compiler/backend/cuda_kernel.cc:1142-1280, 2669-2765) and Evaluator::fn_ewi
 * (cerium/runtime/execution/evaluator.cpp:279-463).
 */
CERIUM_API int cerium_ewise(cerium_context *ctx, int op, void *out, size_t out_stride, const void *a,
                 size_t a_stride, const void *b, size_t b_stride, const void *c, size_t c_stride,
                 const uint64_t *scalars, const uint32_t *prime_idx, int count, void *stream);

/*
 * Ciphertext tensor product d0 = a0*b0, d1 = a0*b1 + a1*b0, d2 = a1*b1 over `count` limbs
 * (all seven stacks share `stride`).  Restates mul_ct_ct
 * (cerium/compiler/backend/compiler.cc:443-467) as one kernel.
 */
CERIUM_API int cerium_tensor(cerium_context *ctx, void *d0, void *d1, void *d2, const void *a0,
                  const void *a1, const void *b0, const void *b1, size_t stride,
                  const uint32_t *prime_idx, int count, void *stream);

/*
 * Multiplication by a PERIODIC plaintext: a plaintext whose slots repeat 2^log2_repeat times is stored
 * once per period, N >> log2_repeat words per limb in NTT form (the reference's encoder transforms only
 * the first log2(N) - log2_repeat levels, cerium/runtime/io/ckks-encoder.h:205-372), and the generated
 * kernels read it as pt[i >> log2_repeat] (cerium/compiler/backend/cuda_kernel.cc:919-934):
 *   out[l][i] = a[l][i] * pt[l][i >> log2_repeat] (+ addend[l][i] when addend is not NULL)   mod q_l
 * pt_stride is the distance between the plaintext's limbs in words (>= N >> log2_repeat).
 */
CERIUM_API int cerium_mul_plain_periodic(cerium_context *ctx, void *out, size_t out_stride, const void *a,
                                         size_t a_stride, const void *pt, size_t pt_stride, int log2_repeat,
                                         const void *addend, size_t addend_stride, const uint32_t *prime_idx,
                                         int count, void *stream);

/*
 * Galois automorphism in NTT form: out[i][k] = in[i][pi(k)] for `count` limbs, pi as built by
 * GaloisTool::generate_table_ntt (cerium/runtime/math/galois.cpp:30-62).  in and out must not
 * overlap.  cerium_galois_elt_from_step restates get_elt_from_step (galois.cpp:79-113):
 * step 0 is conjugation.  Replaces the ROT_WRITE path of the generated kernels
 * (cerium/compiler/backend/cuda_kernel.cc:228-300) and
 * EvaluatorContext::get_rotation_map_ptr (evaluator.cpp:233-260); no table is uploaded.
 */
CERIUM_API uint32_t cerium_galois_elt_from_step(int step, int log_n);
CERIUM_API int cerium_automorph(cerium_context *ctx, void *out, size_t out_stride, const void *in,
                     size_t in_stride, uint32_t galois_elt, int count, void *stream);

/*
 * Resolve: exact CRT composition of the two limbs x0 (mod prime0) and x1 (mod prime1) of `count`
 * polynomials into the two-word integer v in [0, q0*q1) with v = x0 mod q0, v = x1 mod q1; the low
 * words go to `lo`, the high words to `hi`.  Mod: out[i] = (hi:lo) mod q_{prime_idx[i]} for one
 * two-word polynomial.  Together they are the reference's exact ModRaise / double-rescale pair
 * (rsv_write_2 and mod_read_2, cerium/compiler/backend/kernels/fhe_bconv.cuh:31-96; generated
 * RSV / MOD kernels, cerium/compiler/backend/cuda_kernel.cc:2767-2952; factors
 * cerium/runtime/execution/function_execution.cpp:53-99).  All four stacks of cerium_resolve2
 * share `stride`.
 */
CERIUM_API int cerium_resolve2(cerium_context *ctx, void *lo, void *hi, const void *x0, const void *x1,
                    size_t stride, uint32_t prime0, uint32_t prime1, int count, void *stream);
CERIUM_API int cerium_mod2(cerium_context *ctx, void *out, size_t out_stride, const void *lo, const void *hi,
                const uint32_t *prime_idx, int count, void *stream);

/*
 * Base converter from the primes in_primes[0..n_in) to out_primes[0..n_out).
 * Replaces DeviceBaseConverter (cerium/runtime/execution/evaluator.h:30-92,
 * evaluator.cpp:1483-1608) and _function_bco_ (cerium/compiler/backend/kernels/function.cuh:
 * 80-99).  Input limbs are in coefficient form.
 */
CERIUM_API int cerium_bconv_create(cerium_context *ctx, cerium_bconv **out, int mode,
                        const uint32_t *in_primes, int n_in, const uint32_t *out_primes, int n_out);
CERIUM_API int cerium_bconv_destroy(cerium_bconv *bc);
CERIUM_API int cerium_bconv_apply(cerium_bconv *bc, void *out, size_t out_stride, const void *in,
                       size_t in_stride, void *stream);
/*
 * `count` conversions in one launch (blockIdx.y = conversion, as num_conversions of
 * _function_bco_, cerium/compiler/backend/kernels/function.cuh:80-99).  bcs / outs / ins are HOST
 * arrays of `count` converters (of one context) and device pointers; every conversion uses the
 * same strides.
 */
CERIUM_API int cerium_bconv_apply_batch(cerium_bconv *const *bcs, void *const *outs, const void *const *ins,
                             int count, size_t out_stride, size_t in_stride, void *stream);

/*
 * Hybrid key-switching plan for ciphertexts over q_idx[0..L) with extension primes
 * p_idx[0..K) and dnum digits (limb i belongs to digit i % dnum, the stride split of
 * cerium/compiler/backend/compiler_keyswitch.cc:68-99).  Holds the per-digit converters,
 * P^-1 mod q_i and a device workspace of cerium_keyswitch_workspace_bytes().
 * An evaluation key is dnum x 2 x (L+K) limbs, [digit][c0|c1][q_idx..., p_idx...][N]
 * (cerium/runtime/io/ckks-encryptor.cpp:534-599).
 */
CERIUM_API int cerium_keyswitch_create(cerium_context *ctx, cerium_keyswitch **out, int bconv_mode,
                            int round_mode, const uint32_t *q_idx, int L, const uint32_t *p_idx,
                            int K, int dnum);
CERIUM_API int cerium_keyswitch_destroy(cerium_keyswitch *ks);
CERIUM_API size_t cerium_keyswitch_workspace_bytes(const cerium_keyswitch *ks);

/*
 * Communicator of the limb collectives: the `world` ranks of one job, one process and one GPU each.
 * Replaces the NCCL layer of the reference runtime (CUDA::NCCL::*, cerium/runtime/cuda/nccl_ops.cu:
 * 241-440, one host thread per GPU there) for the three exchange records of a compiled program:
 *   DRM  all-gather of coefficient-form limbs      Evaluator::drm  evaluator.cpp:1154-1251
 *   AGS  reduce-scatter of partial sums + mod      Evaluator::ags  evaluator.cpp:1253-1367
 *   ARD  all-reduce of partial sums + mod          Evaluator::ard  evaluator.cpp:1369-1481
 * Limb stacks are contiguous, so there is no pack / unpack pass around a collective (the reference's
 * copy_to_nccl_buffer / copy_from_nccl_buffer[_with_mod], device_utils.cu:290-413): the producer
 * writes the send block, the consumer reads the receive buffer, and the sums are reduced in place.
 * Two transports:
 *   cerium_comm_unique_id + cerium_comm_init   NCCL (libnccl.so.2, opened at run time).  Rank 0 makes
 *       the 128-byte id, the caller hands it to every rank (a file, a store, MPI, torch.distributed).
 *   cerium_comm_init_callbacks                 the caller's own collectives (a runtime that owns its
 *       communicators; a host-memory transport in tests).  A callback enqueues on `stream`, or
 *       completes before it returns, and returns 0 on success.  Unused entries may be NULL.
 * Every collective is enqueued on the given stream and lands in this GPU's own memory.  The ranks
 * must issue their collectives on one communicator in the same order.
 */
#define CERIUM_COMM_ID_BYTES 128
typedef struct cerium_comm_callbacks {
  void *user;
  /* recv [world][bytes_per_rank]; send is this rank's block, possibly recv + rank * bytes_per_rank */
  int (*allgather)(void *user, void *recv, const void *send, size_t bytes_per_rank, void *stream);
  /* send [world][words_per_rank]; recv [words_per_rank] = sum over the ranks of their block `rank` (plain
   * word sums, word_bits = 32 or 64) */
  int (*reducescatter)(void *user, void *recv, const void *send, size_t words_per_rank, int word_bits, void *stream);
  int (*allreduce)(void *user, void *recv, const void *send, size_t words, int word_bits, void *stream);
  int (*broadcast)(void *user, void *buf, size_t bytes, int root, void *stream);
} cerium_comm_callbacks;
CERIUM_API int cerium_comm_unique_id(void *id, size_t id_bytes);
CERIUM_API int cerium_comm_init(cerium_comm **out, const void *id, size_t id_bytes, int rank, int world, int device);
CERIUM_API int cerium_comm_init_callbacks(cerium_comm **out, int rank, int world, int device,
                                          const cerium_comm_callbacks *cb);
/* The communicator of the `size` consecutive ranks that hold this rank (rank / size * size ...), the
 * reference's comms[n][comm_size][device] (cerium/runtime/cuda/nccl_ops.cu:185-215): programs compiled
 * for 4 or 8 GPUs also exchange limbs inside half-size groups.  Collective over `comm` (every rank calls it,
 * in the same order); the result is owned by `comm`.  NCCL transport only. */
CERIUM_API int cerium_comm_split(cerium_comm *comm, int size, cerium_comm **out);
CERIUM_API int cerium_comm_destroy(cerium_comm *comm);
CERIUM_API int cerium_comm_rank(const cerium_comm *comm);
CERIUM_API int cerium_comm_world(const cerium_comm *comm);
/*
 * cerium_allgather_limbs      gathered [world][limbs_per_rank][N] <- every rank's send [limbs_per_rank][N]
 *                             (send may be the rank's own block of gathered)
 * cerium_reducescatter_limbs  in [world][limbs_per_rank][N] partial sums of canonical residues;
 *                             out [limbs_per_rank][N] = (sum over the ranks of their block `rank`) mod
 *                             q_{prime_idx[i]}, canonical.  out may be the rank's block of in.
 * cerium_allreduce_limbs      out [limbs][N] = (sum over the ranks of in) mod q_{prime_idx[i]}; in place allowed
 * cerium_broadcast_limbs      buf [limbs][N] of rank `root` to every rank
 * The sums are word additions on the wire: world * q must fit a word (refused otherwise).
 */
CERIUM_API int cerium_allgather_limbs(cerium_comm *comm, cerium_context *ctx, void *gathered, const void *send,
                                      size_t limbs_per_rank, void *stream);
CERIUM_API int cerium_reducescatter_limbs(cerium_comm *comm, cerium_context *ctx, void *out, const void *in,
                                          const uint32_t *prime_idx, int limbs_per_rank, void *stream);
CERIUM_API int cerium_allreduce_limbs(cerium_comm *comm, cerium_context *ctx, void *out, const void *in,
                                      const uint32_t *prime_idx, int limbs, void *stream);
CERIUM_API int cerium_broadcast_limbs(cerium_comm *comm, cerium_context *ctx, void *buf, size_t limbs, int root,
                                      void *stream);

/*
 * Limb-sharded plan for rank `rank` of `world` GPUs.  Q-limb i lives on rank i % world
 * (cerium/compiler/backend/terms.h:672-685); evaluation keys are sharded like the ciphertext
 * (cerium/compiler/backend/compiler_partition.cc:446-470).  The K extension limbs are
 *   ext_split = 0  replicated on every rank (the reference's Term::Ext): no second exchange, but every
 *                  rank repeats the extension limbs' share of the conversions, transforms and products;
 *   ext_split = 1  split over the ranks like the Q limbs (the reference's Ext_Split / PaE_Split terms,
 *                  cerium/compiler/backend/terms.h:623-790): extension limb k lives on rank
 *                  (L + k) % world, and the coefficient-form extension limbs of the two accumulators are
 *                  all-gathered (2 K limbs) before the ModDown conversion.
 * Every stack a sharded call takes holds the rank's own limbs only, in increasing global index:
 *   polynomial  [n_local][N]                       n_local = cerium_keyswitch_local_limbs()
 *   key         [dnum][c0|c1][n_local + k_local][N]   k_local = cerium_keyswitch_local_ext_limbs()
 *                                                  (= K when the extension limbs are replicated)
 * The one exchange of a key switch is the all-gather of the coefficient-form limbs before base
 * conversion (the reference's DRM group, cerium/compiler/backend/compiler_keyswitch.cc:323-335,
 * cerium/runtime/execution/evaluator.cpp:1154-1251); the caller performs it between the two
 * calls below with whatever transport it owns (NCCL all-gather):
 *   cerium_keyswitch_sharded_begin   inverse transform of the local limbs into `send`
 *                                    ([g][N], g = cerium_keyswitch_gather_limbs() = ceil(L / world);
 *                                    slots past n_local are not written)
 *   all-gather of `send` over the ranks into `gathered` ([world][g][N], rank-major)
 *   cerium_keyswitch_sharded_finish  base conversion, NTT, inner product, ModDown on local limbs
 * world = 1 reproduces cerium_keyswitch_create / cerium_keyswitch_apply.  The begin / finish pair
 * serves plans with replicated extension limbs only.
 *
 * With a communicator the library runs the exchanges itself, into buffers of the plan's workspace
 * (the inverse transform writes this rank's block of the gather buffer in place):
 *   cerium_keyswitch_sharded_apply   the whole key switch on the local limbs (either ext_split mode)
 *   cerium_hrot_sharded              HRot of a sharded ciphertext; the rotation is folded into the
 *                                    key switch's reads of the local limbs, as in cerium_hrot
 *   cerium_rescale_sharded           rescale of a sharded ciphertext (cerium/compiler/backend/
 *                                    compiler_rescale.cc:209-284 with several partitions): the owner of
 *                                    limb L-1 inverse-transforms it into last_coef ([n_polys][N], a
 *                                    caller-owned buffer on every rank), broadcast, every rank divides
 *                                    its remaining limbs.  in: [n_polys][n_local][N] (limbs i = rank,
 *                                    rank + world, ... of q_idx[0..L)); out: [n_polys][n_local'][N],
 *                                    n_local' = n_local - 1 on the owner of the dropped limb.
 * Every rank makes the same call in the same order.  Results equal the one-GPU plan's bit for bit.
 */
CERIUM_API int cerium_keyswitch_create_sharded(cerium_context *ctx, cerium_keyswitch **out, int bconv_mode,
                                    int round_mode, const uint32_t *q_idx, int L,
                                    const uint32_t *p_idx, int K, int dnum, int rank, int world,
                                    int ext_split);
CERIUM_API int cerium_keyswitch_local_limbs(const cerium_keyswitch *ks);
CERIUM_API int cerium_keyswitch_local_ext_limbs(const cerium_keyswitch *ks);
CERIUM_API int cerium_keyswitch_sharded_apply(cerium_keyswitch *ks, cerium_comm *comm, void *out0, void *out1,
                                              const void *cpoly_local, const void *evk_local, const void *add0,
                                              const void *add1, void *stream);
CERIUM_API int cerium_hrot_sharded(cerium_keyswitch *ks, cerium_comm *comm, void *out0, void *out1,
                                   const void *c0_local, const void *c1_local, const void *evk_local,
                                   uint32_t galois_elt, void *stream);
CERIUM_API int cerium_rescale_sharded(cerium_context *ctx, cerium_comm *comm, int round_mode, void *out,
                                      const void *in, const uint32_t *q_idx, int L, int n_polys, void *last_coef,
                                      void *stream);
CERIUM_API int cerium_keyswitch_gather_limbs(const cerium_keyswitch *ks);
CERIUM_API int cerium_keyswitch_sharded_begin(cerium_keyswitch *ks, void *send, const void *cpoly_local,
                                   void *stream);
CERIUM_API int cerium_keyswitch_sharded_finish(cerium_keyswitch *ks, void *out0, void *out1,
                                    const void *gathered, const void *cpoly_local,
                                    const void *evk_local, const void *add0, const void *add1,
                                    void *stream);

/*
 * out0,out1 [L][N] = ModDown( sum_d ModUp(digit d of cpoly) * evk[d] ); if add0 / add1 are
 * non-NULL they are added to out0 / out1 (the P*c0 pre-addition of the reference's PMU
 * group, which commutes with ModDown).  Restates keyswitch_ciphertext_impl
 * (cerium/compiler/backend/compiler_keyswitch.cc:253-432): INTT, BCONV, NTT, EVKMUL,
 * INTT, BCONV, SUD.  All stacks are contiguous ([limb][N], stride N).
 */
CERIUM_API int cerium_keyswitch_apply(cerium_keyswitch *ks, void *out0, void *out1, const void *cpoly,
                           const void *evk, const void *add0, const void *add1, void *stream);

/*
 * The key switch with the reference's PMU pre-addition and `rescale_levels` (0, 1 or 2) of the last Q
 * limbs divided away in the SAME division as P: the dropped limbs join the extension limbs of the
 * ModDown - inverse transform, base conversion (dropped limbs, P) -> remaining limbs, one SuD with
 * (P * dropped primes)^-1 - as keyswitch_ciphertext_impl does with rescale_levels > 0
 * (cerium/compiler/backend/compiler_keyswitch.cc:26-39, 360-417).  out0 / out1 hold L - rescale_levels
 * limbs.  One rounding, where cerium_keyswitch_apply followed by cerium_rescale rounds twice: the two
 * results may differ in the last unit.  One-GPU plans; rescale_levels = 0 is cerium_keyswitch_apply.
 */
CERIUM_API int cerium_keyswitch_apply_rescale(cerium_keyswitch *ks, void *out0, void *out1, const void *cpoly,
                                              const void *evk, const void *add0, const void *add1,
                                              int rescale_levels, void *stream);

/*
 * HRot: (out0,out1) = KeySwitch(phi(c1)) + (phi(c0), 0), phi the automorphism galois_elt.
 * Restates rotate_internal (cerium/compiler/backend/compiler.cc:701-726).  The rotated
 * polynomials are never materialised: the kernels of the key switch read c0 and c1 through the
 * automorphism's index map.  When an output overlaps an input (in-place rotation) the library
 * rotates into its workspace first, one more launch; both give the same result.
 */
CERIUM_API int cerium_hrot(cerium_keyswitch *ks, void *out0, void *out1, const void *c0, const void *c1,
                const void *evk, uint32_t galois_elt, void *stream);

/*
 * Hoisted rotations: several rotations of one ciphertext share the expensive half of the key
 * switch (inverse transform, base conversion and forward transform of c1's digits).  Restates the
 * reference's HoistedRotate lowering (cerium/compiler/backend/compiler.cc:958-1153: one
 * INTT -> BCONV -> NTT of c1, then per rotation an inner product with the RotationInv key,
 * ModDown, c0' = ks0 + c0, and the automorphism applied AFTER key switching, :1084-1135).
 *   cerium_hoisted_begin   raises c1 once into the plan's workspace
 *   cerium_hoisted_rotate  (out0,out1) = phi( KeySwitch(c1; evk_pre) + (c0, 0) ), phi = galois_elt
 * evk_pre is the rotation key of phi with every limb pre-permuted by phi^-1 (the reference's
 * "RotationInv" key): phi(sum_d a_d * phi^-1(k_d)) = sum_d phi(a_d) * k_d.  c1 must be the
 * polynomial given to cerium_hoisted_begin; any number of rotate calls may follow one begin.
 * The automorphism is the store pattern of the last kernel unless an output overlaps an input.
 */
CERIUM_API int cerium_hoisted_begin(cerium_keyswitch *ks, const void *c1, void *stream);
CERIUM_API int cerium_hoisted_rotate(cerium_keyswitch *ks, void *out0, void *out1, const void *c0,
                          const void *c1, const void *evk_pre, uint32_t galois_elt, void *stream);

/*
 * HMult + relinearize (+ rescale by the last limb when do_rescale != 0): tensor product,
 * key switch of d2, addition of d0/d1 (cerium/compiler/backend/compiler.cc:443-467,
 * compiler_keyswitch.cc:360-380) and rescale (compiler_rescale.cc:209-284).  Outputs hold
 * L limbs, or L-1 with rescale.  do_rescale = 1: ModDown, then rescale (two divisions, two
 * roundings); do_rescale = 2: the rescale folded into the ModDown (one division by P * q_last,
 * cerium_keyswitch_apply_rescale with one level: fewer kernels, one rounding).
 */
CERIUM_API int cerium_hmult(cerium_keyswitch *ks, void *out0, void *out1, const void *a0, const void *a1,
                 const void *b0, const void *b1, const void *evk, int do_rescale, void *stream);

/*
 * Baby-step / giant-step multiply-accumulate, out = sum_i phi_{G_i}( sum_j pt[i][j] (.) phi_{B_j}(ct) ):
 * the linear-transform building block of bootstrapping (CoeffToSlot / SlotToCoeff) and of matrix-vector
 * products.  Restates the reference's BsgsMultiplyAccumulate lowering
 * (cerium/compiler/backend/compiler.cc:2457-2822, entry :3001-3069): the baby steps are hoisted
 * rotations of the input (one ModUp); per giant step the plaintext products are summed (MuP, Add),
 * the sum is rotated, raised (INTT, BCONV, NTT) and multiplied with the giant step's key, and these
 * products are ACCUMULATED IN THE EXTENDED BASIS over all giant steps; the un-rotated parts enter as the
 * PMU pre-addition; ONE ModDown ends the operation, with `rescale_levels` (0, 1, 2) extra Q limbs
 * divided away in the same step.
 *   c0, c1            the input ciphertext, [L][N] each
 *   g, n_giant        baby steps (1..16, baby step 0 is the input itself) and giant steps (1..32)
 *   plaintexts        HOST array [n_giant * g] of device pointers to NTT-form diagonals [L][N], entry
 *                     i * g + j; NULL = that diagonal is absent
 *   baby_keys_pre     HOST array [g]: pre-permuted ("RotationInv") key of baby step j (entry 0 unused), as
 *   baby_elts         cerium_hoisted_rotate takes them; HOST array [g] of Galois elements (entry 0 unused)
 *   giant_keys        HOST array [n_giant]: ordinary rotation key of giant step i, as cerium_hrot takes it
 *   giant_elts        HOST array [n_giant] of Galois elements; 1 = this giant step is not rotated (no key)
 *   work              caller-owned device scratch of cerium_bsgs_work_limbs() limbs
 *   out0, out1        [L - rescale_levels][N]; must not overlap the inputs
 * Every diagonal and every key is read exactly once; the rotated copies once per four giant steps.
 */
/*
 * Plaintext multiply-accumulate on its own: n_out ciphertexts out_i = sum_j pt[i][j] (.) src_j over
 * n_src (1..16) source ciphertexts, both polynomials, `count` limbs - the MuP + Add kernel group of the
 * reference's lowerings (cerium/compiler/backend/compiler.cc:2495-2522) as one pass per four outputs.
 * All pointer arrays are HOST arrays of device pointers to [count][N] stacks; plaintexts has n_out *
 * n_src entries, entry i * n_src + j, NULL = no such term.  Outputs must not overlap sources.
 */
CERIUM_API int cerium_plaintext_mac(cerium_context *ctx, int n_out, int n_src, void *const *out0, void *const *out1,
                                    const void *const *src0, const void *const *src1,
                                    const void *const *plaintexts, const uint32_t *prime_idx, int count,
                                    void *stream);
CERIUM_API size_t cerium_bsgs_work_limbs(const cerium_keyswitch *ks, int g, int n_giant);
CERIUM_API int cerium_bsgs_apply(cerium_keyswitch *ks, void *out0, void *out1, const void *c0, const void *c1,
                                 int g, int n_giant, const void *const *plaintexts,
                                 const void *const *baby_keys_pre, const uint32_t *baby_elts,
                                 const void *const *giant_keys, const uint32_t *giant_elts, int rescale_levels,
                                 void *work, void *stream);

/*
 * Rescale `n_polys` polynomials of L limbs each ([poly][limb][N] contiguous) by their last
 * limb: out [poly][L-1][N].  `scratch` is a caller-owned device buffer of n_polys * N words.
 * Restates rescale (cerium/compiler/backend/compiler_rescale.cc:209-284): INTT of the last
 * limb, SuD on the others.
 */
CERIUM_API int cerium_rescale(cerium_context *ctx, int round_mode, void *out, const void *in,
                   const uint32_t *q_idx, int L, int n_polys, void *scratch, void *stream);

/*
 * Rescale of the limbs ONE rank owns when a ciphertext is sharded by limb: the rank that owns the
 * dropped limb inverse-transforms it (cerium_ntt_inverse) and broadcasts the coefficient-form
 * residues ([n_polys][N], last_coef here); every rank then calls this on its remaining limbs
 * (in, out: [n_polys][n_local][N], primes local_idx[0..n_local), none equal to last_prime).
 * Same arithmetic as cerium_rescale; the exchange is the reference's DRM of the last limb
 * (cerium/compiler/backend/compiler_rescale.cc:262-273).
 */
CERIUM_API int cerium_rescale_local(cerium_context *ctx, int round_mode, void *out, const void *in,
                         const uint32_t *local_idx, int n_local, uint32_t last_prime,
                         const void *last_coef, int n_polys, void *stream);

/*
 * Bootstrap ModRaise (cerium/compiler/backend/compiler_rescale.cc:32-207): a ciphertext with the
 * two limbs base0, base1 is lifted to the primes of a larger basis.  Each polynomial's pair of
 * limbs is composed to the exact integer in [0, q_base0 * q_base1) (INTT, Resolve); c0's integer
 * is reduced modulo the target primes (Mod, NTT); c1's integer is reduced modulo EVERY prime of
 * the plan (Q and P), multiplied with the bootstrap key (one digit), taken through ModDown by P
 * and rescaled by the plan's last Q prime; out0 = that + lifted c0, out1 = the other half.
 *   plan: cerium_keyswitch_create_lifted over q_idx[0..L) (the L-1 target primes followed by the
 *         prime the final rescale drops) and the K extension primes; no other call accepts it;
 *   c0, c1: [2][N] (limb base0, limb base1), NTT form;  evk: [1][2][L+K][N];
 *   out0, out1: [L-1][N].
 */
CERIUM_API int cerium_keyswitch_create_lifted(cerium_context *ctx, cerium_keyswitch **out, int bconv_mode,
                                   int round_mode, const uint32_t *q_idx, int L,
                                   const uint32_t *p_idx, int K);
CERIUM_API int cerium_mod_raise(cerium_keyswitch *ks, void *out0, void *out1, const void *c0, const void *c1,
                     uint32_t base0, uint32_t base1, const void *evk, void *stream);

/*
 * Double rescale: drops the last TWO limbs of n_polys polynomials at once (floor division by
 * q_{L-2} * q_{L-1}); in is [n_polys][L][N] in NTT form, out is [n_polys][L-2][N], scratch holds
 * 4 * n_polys limbs.  Restates double_rescale (cerium/compiler/backend/compiler_rescale.cc:
 * 367-521): INTT of the two limbs, Resolve (exact CRT of the pair), Mod (its residues modulo the
 * remaining primes), SuD with both primes as divide bases.  out must not overlap in.
 */
CERIUM_API int cerium_double_rescale(cerium_context *ctx, void *out, const void *in, const uint32_t *q_idx,
                          int L, int n_polys, void *scratch, void *stream);

/*
 * cerium_rescale for callers that cannot allocate (no counterpart in the reference, whose runtime
 * always owns its buffers).  Same result as cerium_rescale, but the n_polys * N words of scratch
 * live in a fixed 1 MiB device array inside the library instead of being passed in: meant for
 * hosts that have no device memory left to hand out, or that must not call cudaMalloc where they
 * evaluate (an arena-only runtime, a plug-in without an allocation budget, a latency-critical
 * section, since cudaMalloc synchronises the device).  Limits and rules:
 *   - n_polys <= 2 (one ciphertext); more is refused with CERIUM_ERR_UNSUPPORTED;
 *   - the first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress); make that first call before any stream capture begins;
 *   - neither this call nor anything under it calls cudaMalloc / cudaFree;
 *   - all calls on one device share the array.  It needs no clearing between calls (each call
 *     overwrites what it later reads), but two calls whose kernels overlap on the GPU - on
 *     different streams - race on it: keep them on one stream or order them with events;
 *   - the array costs 1 MiB on every GPU that loads the library, used or not.
 */
CERIUM_API int cerium_rescale_static(cerium_context *ctx, int round_mode, void *out, const void *in,
                                     const uint32_t *q_idx, int L, int n_polys, void *stream);

/*
 * The reference runtime's plugin contract.  The Cerium runtime resolves two C++ getters in every
 * function_map_<p>.so it loads, __GET_FUNCTION_MAP__ and __GET_FUNCTION_MAP_CUGRAPH__
 * (cerium/runtime/execution/function.cpp:144-177).  Here they live in a small shim
 * (cerium_b200/function_map_shim.so, source csrc/plugin_shim/function_map_shim.cpp) of which one
 * copy per partition is installed under that name; the shim asks this library for the maps of its
 * partition's records file `functions<p>`: the ids of the ntt / int / sud / bco records mapped to
 * launchers with the signatures of cerium/runtime/execution/device_utils.cu:33-113, stream and
 * graph variants, backed by cerium_ntt_*_ptrs, cerium_sud_ptrs and cerium_bconv_ptrs.  Launchers of
 * other record types are taken from the generated plugin when its path is given.
 *
 * cerium_function_map_bind     names the context whose tables the launchers use on `device`
 *                              (NULL unbinds).  Bind before the first launch.
 * cerium_function_map_get      the stream (cugraph = 0) or graph map of one records file, as a
 *                              `const std::unordered_map<uint32_t, void*> *`; built on first request
 *                              and kept for the life of the process, one pair per records file (so
 *                              per function and partition).  generated_plugin_path may be NULL.
 *                              Returns NULL on failure; cerium_function_map_error() says why.
 * cerium_function_map_size / _lookup / _launcher   inspect the maps (tests, diagnostics): number of
 *                              entries (-1 on failure), launcher of a kernel id, launcher of a
 *                              record type ("ntt", "int", "sud", "bco").
 */
CERIUM_API int cerium_function_map_bind(cerium_context *ctx, int device);
CERIUM_API const void *cerium_function_map_get(const char *functions_path, const char *generated_plugin_path,
                                               int cugraph);
CERIUM_API const char *cerium_function_map_error(void);
CERIUM_API int cerium_function_map_size(const char *functions_path, int cugraph);
CERIUM_API void *cerium_function_map_lookup(const char *functions_path, int cugraph, uint32_t kernel_id);
CERIUM_API void *cerium_function_map_launcher(const char *type, int cugraph);

/*
 * Executor of one partition of a compiled Cerium function: what CeriumFunction::make_program /
 * run_program do in the reference runtime for one GPU, in stream mode
 * (cerium/runtime/execution/function_execution.cpp:124-360 builds the argument tables, :437-611 replays
 * them).  cerium_program_load parses the compiler's kernel stream `functions<p>` (the ll.functions
 * records, cerium/compiler/backend/cuda_kernel.cc:1707-1916; fields as FunctionMetaData reads them,
 * cerium/runtime/execution/function.h:269-347), loads the kernel plugin function_map_<p>.so of the
 * function and resolves every term: `r<n>` in a register file, `b<k>(<prime>)` in the base-conversion
 * units (stateful like DeviceBaseConverter, evaluator.cpp:1483-1608), anything else as named program
 * memory, one limb per term (function.cpp:464-503).  The tables every record's launcher takes are built
 * once: pointer tables, `bases`, SuD and PMU factors (function.cpp:685-755), conversion matrices, and -
 * for the element-wise launchers the compiler generated - the modulus / Barrett / rotation tables of the
 * reference's EvaluatorContext.  cerium_program_run replays the records on a stream through the
 * plugin's launchers, by kernel id.  With this library's plugin shim installed, ntt / int / sud / bco
 * records run on this library's kernels and generic / pmu records on the program's generated ones.
 *   scalar_terms / scalar_values   values of the `.scalars` terms of generic records (may be empty)
 *   cerium_program_memory          device address of a named memory term, e.g. "i1(0)": the caller
 *                                  writes inputs and keys there before a run and reads outputs after it
 *                                  (names and meanings are listed in the function's `inputs<p>` file)
 *   cerium_program_write / _read   copy `n_limbs` limbs between host memory ([n_limbs][N] 32-bit words) and
 *                                  the memory terms "<name>(<limb_ids[i]>)", as the reference's
 *                                  copy_ciphertext_inputs_to_gpu / get_program_outputs do
 *                                  (cerium/runtime/execution/function_io.cpp:958-1100, :1360-1420);
 *                                  both wait for `stream` before they return
 *   cerium_program_capture         records one run into a CUDA graph (stream capture, the exchange records
 *                                  included); every later cerium_program_run launches that graph on the
 *                                  caller's stream - the reference's use_cudagraph mode
 *                                  (function_execution.cpp:670-1096 builds its graph node by node)
 *   cerium_program_inspect         parses only (no device): one line per record,
 *                                  "id type #outputs #inputs #bases #rots #units #sud #pmu #rsv #scalars
 *                                  comm_size comm_num_limbs #comm_srcs #comm_dests #call_args callee"
 *   comm                           the partitions of a function compiled for several GPUs run as the
 *                                  ranks of this communicator, one process each (partition p = rank p);
 *                                  its drm records (the all-gather of limbs between partitions,
 *                                  Evaluator::drm, evaluator.cpp:1154-1251) and its ags / ard records
 *                                  (reduce-scatter / all-reduce of partial sums, then reduction modulo
 *                                  each limb's prime, evaluator.cpp:1253-1481) run on it.  NULL for a
 *                                  function compiled for one GPU.
 *   call records                   the called function is loaded from the same program directory
 *                                  (<programs>/<function_name>/functions<p>, inputs<p>, function_map_<p>.so,
 *                                  so functions_path must be <programs>/<function>/functions<p>); its
 *                                  argument and result limbs are bound to the caller's limbs
 * 32-bit contexts (the generated kernels are 32-bit).  Not served: remapable inputs; a function that has one is refused at load.
 */
CERIUM_API int cerium_program_load(cerium_context *ctx, cerium_program **out, const char *functions_path,
                                   const char *plugin_path, const char *const *scalar_terms,
                                   const uint64_t *scalar_values, int n_scalars, cerium_comm *comm);
CERIUM_API int cerium_program_destroy(cerium_program *prog);
CERIUM_API int cerium_program_num_steps(const cerium_program *prog);
CERIUM_API int cerium_program_memory(cerium_program *prog, const char *term, void **device_ptr);
CERIUM_API int cerium_program_write(cerium_program *prog, const char *name, const uint32_t *limb_ids, int n_limbs,
                                    const void *host, void *stream);
CERIUM_API int cerium_program_read(cerium_program *prog, const char *name, const uint32_t *limb_ids, int n_limbs,
                                   void *host, void *stream);
CERIUM_API int cerium_program_run(cerium_program *prog, void *stream);
CERIUM_API int cerium_program_capture(cerium_program *prog);
CERIUM_API int cerium_program_inspect(const char *functions_path, char *buf, size_t buf_bytes, int *n_records);

#ifdef __cplusplus
}
#endif
#endif /* CERIUM_B200_H_ */
