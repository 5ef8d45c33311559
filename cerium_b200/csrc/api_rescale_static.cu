// Rescale without any allocation.
//
// Some hosts of this library are not allowed to allocate device memory at the point where they
// evaluate: a runtime that sized its own arena at start-up and has handed every byte of it out,
// a plug-in loaded into a process whose memory budget belongs to someone else, or code on a
// latency-critical path where cudaMalloc would synchronise the device.  cerium_rescale() asks
// such a caller for a scratch buffer of n_polys * N words; the variant here carries that scratch
// inside the library image instead, as a fixed device array of 1 MiB that every GPU which loads
// the library holds from load until the process exits.
#include <atomic>

#include "internal.h"

using namespace cerium;

namespace {

constexpr int kStaticRescaleMaxPolys = 2;  // one ciphertext: c0 and c1
constexpr int kStaticMaxDevices = 64;

// Room for two polynomials of N 64-bit words.  Polynomial p sits at byte p * N * word size, so a
// 32-bit context packs its two polynomials into the first half of the array.
static __device__ __align__(256) unsigned char g_rescale_scratch[kStaticRescaleMaxPolys * kN * 8];

// In host code the name `g_rescale_scratch` only identifies the symbol; it is not an address a
// kernel may be given.  The device address is looked up once per device, with that device
// current, and cached here.
// Two host threads may make the first call on one device at the same time: both look the address
// up and store the same value; the flag is published with release order after the pointer.
void* g_scratch_ptr[kStaticMaxDevices] = {};
std::atomic<bool> g_scratch_ready[kStaticMaxDevices] = {};

int static_rescale_scratch(int device, void** out) {
  if (device < 0 || device >= kStaticMaxDevices)
    return fail(CERIUM_ERR_UNSUPPORTED, "rescale_static: device index above 63");
  if (!g_scratch_ready[device].load(std::memory_order_acquire)) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_rescale_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(CERIUM_ERR_CUDA, std::string("rescale_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    g_scratch_ptr[device] = p;
    g_scratch_ready[device].store(true, std::memory_order_release);
  }
  *out = g_scratch_ptr[device];
  return CERIUM_OK;
}

}  // namespace

extern "C" int cerium_rescale_static(cerium_context* ctx, int round_mode, void* out, const void* in,
                                     const uint32_t* q_idx, int L, int n_polys, void* stream) {
  if (!ctx || !out || !in || !q_idx) return fail(CERIUM_ERR_INVALID, "rescale_static: null argument");
  if (round_mode != CERIUM_ROUND_FLOOR && round_mode != CERIUM_ROUND_HALF)
    return fail(CERIUM_ERR_INVALID, "rescale_static: unknown round mode");
  if (L < 2 || L - 1 > 64) return fail(CERIUM_ERR_INVALID, "rescale_static: need 2 <= L <= 65");
  if (n_polys < 1) return fail(CERIUM_ERR_INVALID, "rescale_static: need at least one polynomial");
  if (n_polys > kStaticRescaleMaxPolys)
    return fail(CERIUM_ERR_UNSUPPORTED,
                "rescale_static: the built-in scratch holds 2 polynomials; call cerium_rescale with your own "
                "scratch buffer for more");
  for (int i = 0; i < L; i++)
    if (q_idx[i] >= (uint32_t)ctx->n_primes) return fail(CERIUM_ERR_INVALID, "rescale_static: prime index out of range");
  if (((uintptr_t)out | (uintptr_t)in) & 15u)
    return fail(CERIUM_ERR_INVALID, "rescale_static: pointers must be 16-byte aligned");
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "rescale_static: cannot select device");
  void* scratch = nullptr;
  if (int rc = static_rescale_scratch(ctx->device, &scratch)) return rc;

  // The two steps of cerium_rescale, with every host-side table on the stack.
  const size_t n = kN;
  const size_t wb = ctx->word_bytes();
  const uint32_t last = q_idx[L - 1];
  const uint64_t ql = ctx->moduli[last];
  cudaStream_t s = (cudaStream_t)stream;
  uint32_t pos[kStaticRescaleMaxPolys], prime[kStaticRescaleMaxPolys];
  for (int p = 0; p < n_polys; p++) {
    pos[p] = (uint32_t)p;
    prime[p] = last;
  }
  NttCall c{};
  c.in = static_cast<const char*>(in) + (size_t)(L - 1) * n * wb;
  c.in_stride = (size_t)L * n;
  // Nothing in the scratch has to start at zero: the inverse transform overwrites every word
  // that the second step reads, so what an earlier call left behind is never seen.
  c.out = scratch;
  c.out_stride = n;
  c.pos = pos;
  c.prime = prime;
  c.count = n_polys;
  if (int rc = launch_ntt_inverse(ctx, c, nullptr, nullptr, s)) return rc;
  uint64_t factor[kSudMaxBatch], post_sub[kSudMaxBatch];
  const uint64_t half = ql >> 1;
  for (int i = 0; i < L - 1; i++) {
    const uint64_t q = ctx->moduli[q_idx[i]];
    factor[i] = host::invmod(ql % q, q);
    post_sub[i] = round_mode == CERIUM_ROUND_HALF ? half % q : 0;
  }
  for (int p = 0; p < n_polys; p++) {
    SudCall sc{};
    sc.src = static_cast<const char*>(scratch) + (size_t)p * n * wb;
    sc.src_stride = 0;
    sc.work = static_cast<char*>(out) + (size_t)p * (L - 1) * n * wb;
    sc.work_stride = n;
    sc.dst = sc.work;
    sc.dst_stride = n;
    sc.minuend = static_cast<const char*>(in) + (size_t)p * L * n * wb;
    sc.minuend_stride = n;
    sc.prime = q_idx;
    sc.factor = factor;
    sc.count = L - 1;
    sc.reduce_src = true;
    sc.src_q = ql;
    sc.pre_add = round_mode == CERIUM_ROUND_HALF ? half : 0;
    sc.post_sub = post_sub;
    if (int rc = launch_sud(ctx, sc, s)) return rc;
  }
  return CERIUM_OK;
}
