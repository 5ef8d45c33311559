// Limb collectives of the multi-GPU path: the exchange steps of a limb-sharded ciphertext.
//
// Replaces Evaluator::drm / ags / ard (cerium/runtime/execution/evaluator.cpp:1154-1481), the NCCL
// wrappers behind them (cerium/runtime/cuda/nccl_ops.cu:241-440) and the pack / unpack kernels around
// them (cerium/runtime/execution/device_utils.cu:290-413):
//   DRM  all-gather of coefficient-form limbs before a base conversion      cerium_allgather_limbs
//   AGS  reduce-scatter of partial sums, then reduction modulo each prime   cerium_reducescatter_limbs
//   ARD  all-reduce of partial sums, then reduction modulo each prime       cerium_allreduce_limbs
// Differences: one process per GPU instead of one thread per GPU, limb stacks are contiguous so
// nothing is packed or unpacked (the producer kernel writes the send block, the consumer reads the
// receive buffer), the sums are reduced by a vectorised kernel with one Shoup step instead of nine
// conditional subtractions, and the transport is pluggable: NCCL, opened with dlopen at run time
// (libnccl.so.2; whichever copy the process already holds is used), or functions the caller
// provides (a runtime that owns its communicators, or a host-memory transport in tests).
// Every collective lands in this GPU's own memory; kernels never read a peer's memory.
#include <cstring>
#include <mutex>

#include "internal.h"

#if !defined(CERIUM_EMU)
#include <dlfcn.h>
#if __has_include(<nccl.h>)
#include <nccl.h>
#else
// the part of NCCL's public interface used here (stable across NCCL 2.x)
extern "C" {
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef enum { ncclSuccess = 0 } ncclResult_t;
typedef enum { ncclSum = 0 } ncclRedOp_t;
typedef enum { ncclUint8 = 1, ncclUint32 = 3, ncclUint64 = 5 } ncclDataType_t;
}
#endif
#endif

using namespace cerium;

namespace {

#if !defined(CERIUM_EMU)
struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommSplit)(ncclComm_t, int, int, ncclComm_t*, void*) = nullptr;  // NCCL 2.18 and later
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) {
      api.error = "libnccl.so.2 cannot be loaded";
      return;
    }
    auto sym = [&](const char* name) {
      void* p = dlsym(api.handle, name);
      if (!p && api.error.empty()) api.error = std::string("libnccl has no ") + name;
      return p;
    };
    api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
    api.AllGather = (decltype(api.AllGather))sym("ncclAllGather");
    api.ReduceScatter = (decltype(api.ReduceScatter))sym("ncclReduceScatter");
    api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
    api.Broadcast = (decltype(api.Broadcast))sym("ncclBroadcast");
    api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
    api.CommSplit = (decltype(api.CommSplit))dlsym(api.handle, "ncclCommSplit");  // optional
  });
  return &api;
}

int nccl_fail(const char* what, ncclResult_t r) {
  NcclApi* api = nccl_api();
  return fail(CERIUM_ERR_CUDA, std::string(what) + ": " + (api->GetErrorString ? api->GetErrorString(r) : "NCCL error"));
}
#define CERIUM_NCCL(call, what)                    \
  do {                                             \
    ncclResult_t r__ = (call);                     \
    if (r__ != ncclSuccess) return nccl_fail(what, r__); \
  } while (0)
#endif  // !CERIUM_EMU

int check_comm(const cerium_comm* comm, const char* what) {
  if (!comm) return fail(CERIUM_ERR_INVALID, std::string(what) + ": null communicator");
  if (!comm->nccl && !comm->has_cb) return fail(CERIUM_ERR_INVALID, std::string(what) + ": communicator has no transport");
  return CERIUM_OK;
}

}  // namespace

namespace cerium {

int comm_subgroup(cerium_comm* comm, int size, cerium_comm** out) {
  if (int rc = check_comm(comm, "comm_split")) return rc;
  if (size <= 0 || size > comm->world || comm->world % size) return fail(CERIUM_ERR_INVALID, "comm_split: the group size must divide the number of ranks");
  if (size == comm->world) {
    *out = comm;
    return CERIUM_OK;
  }
  auto it = comm->subgroups.find(size);
  if (it != comm->subgroups.end()) {
    *out = it->second;
    return CERIUM_OK;
  }
  if (comm->has_cb) return fail(CERIUM_ERR_UNSUPPORTED, "comm_split: the caller's transport has no sub-groups");
#if !defined(CERIUM_EMU)
  NcclApi* api = nccl_api();
  if (!api->CommSplit) return fail(CERIUM_ERR_UNSUPPORTED, "comm_split: this NCCL has no ncclCommSplit (2.18 or later is needed)");
  DeviceGuard guard(comm->device);
  ncclComm_t sub = nullptr;
  CERIUM_NCCL(api->CommSplit((ncclComm_t)comm->nccl, comm->rank / size, comm->rank % size, &sub, nullptr), "ncclCommSplit");
  auto* c = new cerium_comm();
  c->rank = comm->rank % size;
  c->world = size;
  c->device = comm->device;
  c->nccl = sub;
  comm->subgroups[size] = c;
  *out = c;
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "comm_split: no transport");
#endif
}

int comm_allgather(cerium_comm* comm, void* recv, const void* send, size_t bytes_per_rank, cudaStream_t stream) {
  if (int rc = check_comm(comm, "allgather")) return rc;
  if (bytes_per_rank == 0) return CERIUM_OK;
  if (comm->world == 1) {
    if (recv != send) CERIUM_CUDA(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, stream));
    return CERIUM_OK;
  }
  if (comm->has_cb) {
    if (!comm->cb.allgather) return fail(CERIUM_ERR_UNSUPPORTED, "allgather: the caller's transport has no all-gather");
    if (comm->cb.allgather(comm->cb.user, recv, send, bytes_per_rank, stream) != 0)
      return fail(CERIUM_ERR_CUDA, "allgather: the caller's transport failed");
    return CERIUM_OK;
  }
#if !defined(CERIUM_EMU)
  CERIUM_NCCL(nccl_api()->AllGather(send, recv, bytes_per_rank, ncclUint8, (ncclComm_t)comm->nccl, stream), "ncclAllGather");
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "allgather: no transport");
#endif
}

int comm_reducescatter_sum(cerium_comm* comm, void* recv, const void* send, size_t words_per_rank, int word_bits,
                           cudaStream_t stream) {
  if (int rc = check_comm(comm, "reducescatter")) return rc;
  if (words_per_rank == 0) return CERIUM_OK;
  const size_t wb = (size_t)word_bits / 8;
  if (comm->world == 1) {
    if (recv != send) CERIUM_CUDA(cudaMemcpyAsync(recv, send, words_per_rank * wb, cudaMemcpyDeviceToDevice, stream));
    return CERIUM_OK;
  }
  if (comm->has_cb) {
    if (!comm->cb.reducescatter) return fail(CERIUM_ERR_UNSUPPORTED, "reducescatter: the caller's transport has no reduce-scatter");
    if (comm->cb.reducescatter(comm->cb.user, recv, send, words_per_rank, word_bits, stream) != 0)
      return fail(CERIUM_ERR_CUDA, "reducescatter: the caller's transport failed");
    return CERIUM_OK;
  }
#if !defined(CERIUM_EMU)
  CERIUM_NCCL(nccl_api()->ReduceScatter(send, recv, words_per_rank, word_bits == 32 ? ncclUint32 : ncclUint64, ncclSum,
                                        (ncclComm_t)comm->nccl, stream),
              "ncclReduceScatter");
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "reducescatter: no transport");
#endif
}

int comm_allreduce_sum(cerium_comm* comm, void* recv, const void* send, size_t words, int word_bits, cudaStream_t stream) {
  if (int rc = check_comm(comm, "allreduce")) return rc;
  if (words == 0) return CERIUM_OK;
  const size_t wb = (size_t)word_bits / 8;
  if (comm->world == 1) {
    if (recv != send) CERIUM_CUDA(cudaMemcpyAsync(recv, send, words * wb, cudaMemcpyDeviceToDevice, stream));
    return CERIUM_OK;
  }
  if (comm->has_cb) {
    if (!comm->cb.allreduce) return fail(CERIUM_ERR_UNSUPPORTED, "allreduce: the caller's transport has no all-reduce");
    if (comm->cb.allreduce(comm->cb.user, recv, send, words, word_bits, stream) != 0)
      return fail(CERIUM_ERR_CUDA, "allreduce: the caller's transport failed");
    return CERIUM_OK;
  }
#if !defined(CERIUM_EMU)
  CERIUM_NCCL(nccl_api()->AllReduce(send, recv, words, word_bits == 32 ? ncclUint32 : ncclUint64, ncclSum,
                                    (ncclComm_t)comm->nccl, stream),
              "ncclAllReduce");
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "allreduce: no transport");
#endif
}

int comm_broadcast(cerium_comm* comm, void* buf, size_t bytes, int root, cudaStream_t stream) {
  if (int rc = check_comm(comm, "broadcast")) return rc;
  if (root < 0 || root >= comm->world) return fail(CERIUM_ERR_INVALID, "broadcast: root out of range");
  if (bytes == 0 || comm->world == 1) return CERIUM_OK;
  if (comm->has_cb) {
    if (!comm->cb.broadcast) return fail(CERIUM_ERR_UNSUPPORTED, "broadcast: the caller's transport has no broadcast");
    if (comm->cb.broadcast(comm->cb.user, buf, bytes, root, stream) != 0)
      return fail(CERIUM_ERR_CUDA, "broadcast: the caller's transport failed");
    return CERIUM_OK;
  }
#if !defined(CERIUM_EMU)
  CERIUM_NCCL(nccl_api()->Broadcast(buf, buf, bytes, ncclUint8, root, (ncclComm_t)comm->nccl, stream), "ncclBroadcast");
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "broadcast: no transport");
#endif
}

}  // namespace cerium

extern "C" {

int cerium_comm_unique_id(void* id, size_t id_bytes) {
  if (!id || id_bytes < CERIUM_COMM_ID_BYTES) return fail(CERIUM_ERR_INVALID, "comm_unique_id: need a buffer of 128 bytes");
#if !defined(CERIUM_EMU)
  NcclApi* api = nccl_api();
  if (!api->error.empty()) return fail(CERIUM_ERR_UNSUPPORTED, "comm_unique_id: " + api->error);
  static_assert(sizeof(ncclUniqueId) == CERIUM_COMM_ID_BYTES, "NCCL's id is 128 bytes");
  ncclUniqueId uid;
  CERIUM_NCCL(api->GetUniqueId(&uid), "ncclGetUniqueId");
  std::memcpy(id, &uid, sizeof(uid));
  return CERIUM_OK;
#else
  return fail(CERIUM_ERR_UNSUPPORTED, "comm_unique_id: NCCL is not part of the host-only test build");
#endif
}

int cerium_comm_init(cerium_comm** out, const void* id, size_t id_bytes, int rank, int world, int device) {
  if (!out || !id || id_bytes < CERIUM_COMM_ID_BYTES) return fail(CERIUM_ERR_INVALID, "comm_init: null argument or short id");
  if (world < 1 || rank < 0 || rank >= world) return fail(CERIUM_ERR_INVALID, "comm_init: need 0 <= rank < world");
#if !defined(CERIUM_EMU)
  NcclApi* api = nccl_api();
  if (!api->error.empty()) return fail(CERIUM_ERR_UNSUPPORTED, "comm_init: " + api->error);
  DeviceGuard guard(device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "comm_init: cannot select device");
  ncclUniqueId uid;
  std::memcpy(&uid, id, sizeof(uid));
  ncclComm_t c = nullptr;
  CERIUM_NCCL(api->CommInitRank(&c, world, uid, rank), "ncclCommInitRank");
  auto* comm = new cerium_comm();
  comm->rank = rank;
  comm->world = world;
  comm->device = device;
  comm->nccl = c;
  *out = comm;
  return CERIUM_OK;
#else
  (void)device;
  return fail(CERIUM_ERR_UNSUPPORTED, "comm_init: NCCL is not part of the host-only test build");
#endif
}

int cerium_comm_init_callbacks(cerium_comm** out, int rank, int world, int device, const cerium_comm_callbacks* cb) {
  if (!out || !cb) return fail(CERIUM_ERR_INVALID, "comm_init_callbacks: null argument");
  if (world < 1 || rank < 0 || rank >= world) return fail(CERIUM_ERR_INVALID, "comm_init_callbacks: need 0 <= rank < world");
  auto* comm = new cerium_comm();
  comm->rank = rank;
  comm->world = world;
  comm->device = device;
  comm->cb = *cb;
  comm->has_cb = true;
  *out = comm;
  return CERIUM_OK;
}

int cerium_comm_split(cerium_comm* comm, int size, cerium_comm** out) {
  if (!out) return fail(CERIUM_ERR_INVALID, "comm_split: null argument");
  return comm_subgroup(comm, size, out);
}

int cerium_comm_destroy(cerium_comm* comm) {
  if (!comm) return CERIUM_OK;
  for (auto& kv : comm->subgroups) cerium_comm_destroy(kv.second);
  comm->subgroups.clear();
#if !defined(CERIUM_EMU)
  if (comm->nccl) {
    DeviceGuard guard(comm->device);
    nccl_api()->CommDestroy((ncclComm_t)comm->nccl);
  }
#endif
  delete comm;
  return CERIUM_OK;
}

int cerium_comm_rank(const cerium_comm* comm) { return comm ? comm->rank : -1; }
int cerium_comm_world(const cerium_comm* comm) { return comm ? comm->world : 0; }

static int limb_args(const cerium_comm* comm, const cerium_context* ctx, const void* a, const void* b, const char* what) {
  if (!comm || !ctx || !a || !b) return fail(CERIUM_ERR_INVALID, std::string(what) + ": null argument");
  if (((uintptr_t)a | (uintptr_t)b) & 15u) return fail(CERIUM_ERR_INVALID, std::string(what) + ": pointers must be 16-byte aligned");
  return CERIUM_OK;
}

int cerium_allgather_limbs(cerium_comm* comm, cerium_context* ctx, void* gathered, const void* send,
                           size_t limbs_per_rank, void* stream) {
  if (int rc = limb_args(comm, ctx, gathered, send, "allgather_limbs")) return rc;
  DeviceGuard guard(ctx->device);
  return comm_allgather(comm, gathered, send, limbs_per_rank * kN * ctx->word_bytes(), (cudaStream_t)stream);
}

// Sums of `world` canonical residues are below world * q < 2^B for every prime the word size admits
// when world <= 4 (32-bit words, q < 2^30) or world <= 16 (64-bit words, q < 2^60).
static int check_sum_range(const cerium_comm* comm, const cerium_context* ctx, const uint32_t* prime_idx, int count,
                           const char* what) {
  if (!prime_idx && count > 0) return fail(CERIUM_ERR_INVALID, std::string(what) + ": null prime_idx");
  for (int i = 0; i < count; i++) {
    if (prime_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, std::string(what) + ": prime index out of range");
    const long double top = ctx->word_bits == 32 ? 4294967296.0L : 18446744073709551616.0L;
    if ((long double)ctx->moduli[prime_idx[i]] * comm->world >= top)
      return fail(CERIUM_ERR_UNSUPPORTED, std::string(what) + ": the sum over the ranks overflows a word for a prime this wide");
  }
  return CERIUM_OK;
}

int cerium_reducescatter_limbs(cerium_comm* comm, cerium_context* ctx, void* out, const void* in,
                               const uint32_t* prime_idx, int limbs_per_rank, void* stream) {
  if (int rc = limb_args(comm, ctx, out, in, "reducescatter_limbs")) return rc;
  if (limbs_per_rank < 0) return fail(CERIUM_ERR_INVALID, "reducescatter_limbs: negative count");
  if (limbs_per_rank == 0) return CERIUM_OK;
  if (int rc = check_sum_range(comm, ctx, prime_idx, limbs_per_rank, "reducescatter_limbs")) return rc;
  DeviceGuard guard(ctx->device);
  if (int rc = comm_reducescatter_sum(comm, out, in, (size_t)limbs_per_rank * kN, ctx->word_bits, (cudaStream_t)stream)) return rc;
  return cerium_ewise(ctx, CERIUM_EW_REDUCE, out, kN, out, kN, nullptr, 0, nullptr, 0, nullptr, prime_idx, limbs_per_rank, stream);
}

int cerium_allreduce_limbs(cerium_comm* comm, cerium_context* ctx, void* out, const void* in, const uint32_t* prime_idx,
                           int limbs, void* stream) {
  if (int rc = limb_args(comm, ctx, out, in, "allreduce_limbs")) return rc;
  if (limbs < 0) return fail(CERIUM_ERR_INVALID, "allreduce_limbs: negative count");
  if (limbs == 0) return CERIUM_OK;
  if (int rc = check_sum_range(comm, ctx, prime_idx, limbs, "allreduce_limbs")) return rc;
  DeviceGuard guard(ctx->device);
  if (int rc = comm_allreduce_sum(comm, out, in, (size_t)limbs * kN, ctx->word_bits, (cudaStream_t)stream)) return rc;
  return cerium_ewise(ctx, CERIUM_EW_REDUCE, out, kN, out, kN, nullptr, 0, nullptr, 0, nullptr, prime_idx, limbs, stream);
}

int cerium_broadcast_limbs(cerium_comm* comm, cerium_context* ctx, void* buf, size_t limbs, int root, void* stream) {
  if (int rc = limb_args(comm, ctx, buf, buf, "broadcast_limbs")) return rc;
  DeviceGuard guard(ctx->device);
  return comm_broadcast(comm, buf, limbs * kN * ctx->word_bytes(), root, (cudaStream_t)stream);
}

}  // extern "C"
