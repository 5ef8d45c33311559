// Internal host-side structures behind the opaque handles of include/cerium_b200.h.
#pragma once
#if defined(CERIUM_EMU)
#include "emu_cuda.h"  // test-only host stand-ins; the shipped library is never built this way
#else
#include <cuda_runtime.h>
#endif

#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "../../include/cerium_b200.h"
#include "bconv_kernels.cuh"
#include "bsgs_kernels.cuh"
#include "ewise_kernels.cuh"
#include "host_math.h"
#include "ntt_kernels.cuh"

namespace cerium {

constexpr int kMaxDevices = 64;  // per-device host-side caches are indexed by the CUDA device ordinal

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define CERIUM_CUDA(call)                                                              \
  do {                                                                                 \
    cudaError_t e__ = (call);                                                          \
    if (e__ != cudaSuccess)                                                            \
      return ::cerium::fail(CERIUM_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
  } while (0)

#define CERIUM_LAUNCH_CHECK(what)                                                      \
  do {                                                                                 \
    cudaError_t e__ = cudaGetLastError();                                              \
    if (e__ != cudaSuccess)                                                            \
      return ::cerium::fail(CERIUM_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// Kernel launch through a function pointer (template-ids with commas stay out of the macro).
#if defined(CERIUM_EMU)
#define CERIUM_LAUNCH(kfn, grid, block, smem, stream, ...) \
  ::cerium_emu::launch((grid), (block), (smem), [=]() { kfn(__VA_ARGS__); })
#else
// Every kernel is launched with programmatic stream serialisation (see grid_dependency_wait in
// modarith.cuh): its CTAs may be placed while the previous kernel of the stream drains.
template <typename... KArgs, typename... Args>
inline void launch_dependent(void (*kfn)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kfn, std::forward<Args>(args)...);  // errors surface in CERIUM_LAUNCH_CHECK
}
#define CERIUM_LAUNCH(kfn, grid, block, smem, stream, ...) \
  ::cerium::launch_dependent(kfn, dim3(grid), dim3(block), (size_t)(smem), (stream), __VA_ARGS__)
#endif

// Runs fn(W{}) with W = uint32_t or uint64_t according to the context's word size.
template <typename F>
inline int dispatch_word(int word_bits, F&& fn) {
  if (word_bits == 32) return fn(uint32_t{});
  return fn(uint64_t{});
}

// RAII switch to the context's device for the duration of a call.
struct DeviceGuard {
  int prev = -1;
  bool ok = true;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) != cudaSuccess) ok = false;
    if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    if (prev == dev) prev = -1;
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

}  // namespace cerium

struct cerium_context {
  int device = 0;
  int logn = 0;
  int word_bits = 0;
  int n_primes = 0;
  std::vector<uint64_t> moduli;
  std::vector<uint64_t> psi;
  void* d_tw_fwd = nullptr;  // Pair[n_primes][N], bit-reversed powers of psi
  void* d_tw_inv = nullptr;  // Pair[n_primes][N], bit-reversed powers of psi^-1
  void* d_twr_fwd = nullptr; // Pair[n_primes][256][15][16], lane-interleaved level-3 twiddles (row pass)
  void* d_twr_inv = nullptr; // same for the inverse transform
  void* d_pcs = nullptr;     // PrimeConst<W>[n_primes]
  uint32_t* d_status = nullptr;  // device status word: kernels that skip a malformed work item set a bit here
  // 64-bit primes below 2^50 transform on the FP64 pipe unless the environment variable
  // CERIUM_B200_NTT_ARITH is "int" when the context is created (for comparisons)
  bool allow_fp = true;
  int sm_count = 1;  // SMs of the device (launch shapes are sized in multiples of it)
  std::vector<uint64_t> mu_hi, mu_lo;  // Barrett constants per prime (host copy)
  std::vector<uint8_t> fp_ok, lazy_ok; // arithmetic of each prime's transforms (host copy)
  size_t word_bytes() const { return (size_t)word_bits / 8; }
};

struct cerium_bconv {
  cerium_context* ctx = nullptr;
  int mode = 0;
  int I = 0, O = 0;
  std::vector<uint32_t> in_primes, out_primes;
  // one device allocation holding every table below
  void* d_block = nullptr;
  void* d_factors = nullptr;    // W[O][I]
  void* d_outc = nullptr;       // BconvOut<W>[O]
  void* d_split_fac = nullptr;  // uint2[O][I] (64-bit words, at most 8 inputs)
  void* d_fp_fac = nullptr;     // double2[O][I] (when fp_in)
  void* d_inv = nullptr;        // W[I] (exact mode, unless the caller pre-scales)
  void* d_inv_shoup = nullptr;  // W[I]
  void* d_in_add = nullptr;     // W[I]  rounding term, or null
  void* d_out_sub = nullptr;    // W[O]  rounding term, or null
  uint32_t* d_in_prime = nullptr;
  uint32_t* d_out_prime = nullptr;
  uint32_t* d_out_pos = nullptr;  // or null
  uint32_t* d_in_pos = nullptr;   // or null
  bool lazy_out = false;
  std::vector<uint64_t> inv_host;  // [Qhat_i^-1]_{q_i}
  bool fp_in = false;              // some outputs take their quotient from the FP64 pipe (d_fp_fac is present)
};

// Communicator of the limb collectives: the ranks of one job, one GPU each.  The transport is NCCL
// (loaded at run time) or a set of caller-provided functions.
struct cerium_comm {
  int rank = 0, world = 1, device = 0;
  void* nccl = nullptr;  // ncclComm_t when the transport is NCCL
  cerium_comm_callbacks cb = {};
  bool has_cb = false;
  std::map<int, cerium_comm*> subgroups;  // communicators of `size` consecutive ranks holding this rank (owned)
};

namespace cerium {

// Collectives on raw device buffers, enqueued on `stream`.  `send` of the all-gather may be the
// rank's own block of `recv` (in place).  Sums are plain word additions (no modular reduction).
int comm_allgather(cerium_comm* comm, void* recv, const void* send, size_t bytes_per_rank, cudaStream_t stream);
int comm_reducescatter_sum(cerium_comm* comm, void* recv, const void* send, size_t words_per_rank, int word_bits,
                           cudaStream_t stream);
int comm_allreduce_sum(cerium_comm* comm, void* recv, const void* send, size_t words, int word_bits, cudaStream_t stream);
int comm_broadcast(cerium_comm* comm, void* buf, size_t bytes, int root, cudaStream_t stream);
// The communicator of the `size` consecutive ranks [rank / size * size, ...) that hold this rank (`comm` itself
// when size is its world); created on first use - a collective call: every rank of `comm` makes it, in the
// same order - and owned by `comm`.
int comm_subgroup(cerium_comm* comm, int size, cerium_comm** out);

// Options of create_bconv beyond the public entry point.
struct BconvOptions {
  bool prescaled = false;            // exact mode, inputs already multiplied by [Qhat_i^-1]
  bool round_half = false;           // add floor(prod_in/2) to inputs, subtract it from outputs
  std::vector<uint32_t> out_pos;     // output limb slots (empty = 0..O-1)
  std::vector<uint32_t> in_pos;      // input limb slots (empty = 0..I-1)
  bool lazy_out = false;             // outputs feed the forward NTT directly: skip the final corrections
};

int create_bconv(cerium_context* ctx, cerium_bconv** out, int mode, const uint32_t* in_primes, int n_in,
                 const uint32_t* out_primes, int n_out, const BconvOptions& opt);

// One entry of a batched conversion launch.
struct BconvCall {
  cerium_bconv* bc;
  void* out;
  size_t out_stride;
  const void* in;
  size_t in_stride;
};
int launch_bconv(cerium_context* ctx, const BconvCall* calls, int count, cudaStream_t stream);

// Batched transforms with explicit limb slots (pos[b]) and prime indices.
struct NttCall {
  const void* in;
  void* out;
  size_t in_stride, out_stride;
  const uint32_t* pos;    // count entries, or null for 0..count-1
  const uint32_t* prime;  // count entries
  int count;
  // forward transform: entry b reads limb src_pos[b] of `in`, residues of another modulus, and
  // reduces them to its own prime on the way in (null: reads limb pos[b], already reduced).
  // inverse transform: entry b reads limb src_pos[b] of `in` (same modulus) instead of limb pos[b]
  const uint32_t* src_pos = nullptr;
  // with src_pos: prime index of the modulus the words of entry b are residues of (null: unknown)
  const uint32_t* src_prime = nullptr;
  // forward transform only: the input words are below 4q instead of canonical
  bool lazy_in = false;
  // inverse transform only, not 0: the input limbs are read through the Galois automorphism of this element
  uint32_t in_galois = 0;
};
// lazy_out: leave the results below 4q instead of canonical (internal buffers read by the inner product only)
int launch_ntt_forward(cerium_context* ctx, const NttCall& c, cudaStream_t stream, bool lazy_out = false);
// scale / scale_shoup: device arrays with one word per batch entry, or null.
int launch_ntt_inverse(cerium_context* ctx, const NttCall& c, const void* scale, const void* scale_shoup,
                       cudaStream_t stream);

// SuD over `count` limbs (count <= kSudMaxBatch per launch; chunked internally).
struct SudCall {
  const void* src;       // coefficient-form source; src_stride == 0 broadcasts one limb
  size_t src_stride;
  void* work;            // column-pass output / row-pass input (may equal src when src_stride != 0)
  size_t work_stride;
  void* dst;
  size_t dst_stride;
  const void* minuend;
  size_t minuend_stride;
  const void* addend;    // or null
  size_t addend_stride;
  const uint32_t* prime;  // count prime indices
  const uint64_t* factor; // count canonical residues (host)
  int count;
  // optional second polynomial in the same launch: entries [split, count) write dst2 and read
  // minuend2 / addend2 at index (b - split); src / work stay one stack of `count` limbs
  int split = 0;          // 0 = one polynomial
  void* dst2 = nullptr;
  const void* minuend2 = nullptr;
  const void* addend2 = nullptr;
  // source re-reduction (only when reduce_src): residues of modulus src_q, optional rounding
  bool reduce_src = false;
  uint64_t src_q = 0;
  uint64_t pre_add = 0;
  const uint64_t* post_sub = nullptr;  // count residues (host) or null
  // only with reduce_src: entry b reads limb src_pos[b] of src (null: limb b, or the one limb
  // when src_stride == 0)
  const uint32_t* src_pos = nullptr;
  // not 0: addend / addend2 are read through the Galois automorphism of this element
  uint32_t addend_galois = 0;
  // not 0: word i of every result limb is stored at pi(i) (index map of this element); dst / dst2 must
  // then not overlap minuend, addend or work
  uint32_t store_galois = 0;
};
int launch_sud(cerium_context* ctx, const SudCall& c, cudaStream_t stream);
int launch_automorph_pair(cerium_context* ctx, void* out_a, const void* in_a, void* out_b, const void* in_b,
                          uint32_t galois_elt, int count, cudaStream_t stream);

}  // namespace cerium
