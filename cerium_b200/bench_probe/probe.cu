// Integer-pipe probe: measures, on the GPU it runs on, the register-only rate of the
// instructions and butterflies the transforms are made of.  It is the "integer-multiply
// roofline" the 64-bit kernels are judged against (their HBM roofline is not the binding one):
// a transform cannot run its butterflies faster than these loops, which touch no memory.
// Benchmark infrastructure: built into its own shared object (libcerium_b200_probe.so), which only
// bench.py loads; the evaluation library does not contain it.  It allocates a small scratch buffer
// and synchronises the device.
#include <cstring>

#include "../csrc/internal.h"

using namespace cerium;

// the error plumbing of the evaluation library, restated for this stand-alone object
namespace cerium {
static thread_local std::string g_probe_error;
void set_error(const std::string& msg) { g_probe_error = msg; }
int fail(int code, const std::string& msg) {
  g_probe_error = msg;
  return code;
}
}  // namespace cerium

namespace {

constexpr int kProbeThreads = 256;

// OP: 0 mad.lo.u32, 1 mad.wide.u32, 2 mul.hi.u64, 3 mul.lo.u64, 4 add.u64, 5 fma.rn.f64 -- 8 chains per thread
template <int OP>
__global__ void __launch_bounds__(kProbeThreads) probe_raw_kernel(uint64_t* out, uint32_t a, uint32_t b, int iters) {
  grid_dependency_launch();
  grid_dependency_wait();
  uint32_t r[8];
  uint64_t R[8];
  double D[8];
  for (int j = 0; j < 8; j++) {
    r[j] = threadIdx.x + j;
    R[j] = threadIdx.x * 3 + j;
    D[j] = (double)(threadIdx.x + j);
  }
#if !defined(CERIUM_EMU)
  const uint64_t ab = (uint64_t)a << 32 | b;
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int rep = 0; rep < 4; rep++)
#pragma unroll
      for (int j = 0; j < 8; j++) {
        if (OP == 0) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(r[j]) : "r"(a), "r"(b));
        if (OP == 1) asm volatile("mad.wide.u32 %0, %1, %2, %0;" : "+l"(R[j]) : "r"(r[j]), "r"(a));
        if (OP == 2) asm volatile("mul.hi.u64 %0, %0, %1;" : "+l"(R[j]) : "l"(ab));
        if (OP == 3) asm volatile("mul.lo.u64 %0, %0, %1;" : "+l"(R[j]) : "l"(ab));
        if (OP == 4) asm volatile("add.u64 %0, %0, %1;" : "+l"(R[j]) : "l"(ab));
        if (OP == 5) asm volatile("fma.rn.f64 %0, %0, %1, %2;" : "+d"(D[j]) : "d"(0.999999 + a * 1e-9), "d"(0.5 + b));
      }
  }
#endif
  uint64_t s = 0;
  for (int j = 0; j < 8; j++) s ^= R[j] ^ r[j] ^ (uint64_t)__double_as_longlong(D[j]);
  out[blockIdx.x * blockDim.x + threadIdx.x] = s + iters;
}

// `iters` radix-16 groups (32 butterflies each) on 16 register-resident words per thread, with the
// library's own butterfly code; twiddles are loop-invariant registers.
template <typename W, int kMode>
__global__ void __launch_bounds__(kProbeThreads) probe_butterfly_kernel(W* out, PrimeConst<W> pc, W w0, W ws0, int iters) {
  grid_dependency_launch();
  grid_dependency_wait();
  constexpr bool kLazy = kMode == kArithLazy;
  const Arith<W, kMode> ar(pc);
  const W q = pc.q;
  W x[16], w[4], ws[4];
  for (int j = 0; j < 16; j++) x[j] = ar.enter((W)(threadIdx.x * 977u + j * 131u + blockIdx.x) % q);
  for (int t = 0; t < 4; t++) {
    w[t] = (w0 + (W)(t * 12345u + threadIdx.x)) % q;
    ws[t] = ws0 + (W)(t * 777u + threadIdx.x);
    if (kMode == kArithFp) {
      // centred twiddle and its quotient by q, as the bit patterns of doubles
      const double wd = (double)(long long)w[t] - (w[t] > q / 2 ? (double)(long long)q : 0.0);
      w[t] = (W)__double_as_longlong(wd);
      ws[t] = (W)__double_as_longlong(wd / (double)(long long)q);
    }
  }
  for (int it = 0; it < iters; it++) {
#pragma unroll
    for (int t = 0; t < 4; t++) {
      const int half = 8 >> t;
#pragma unroll
      for (int g = 0; g < (1 << t); g++)
#pragma unroll
        for (int k = 0; k < half; k++) {
          const int j = g * 2 * half + k;
          ar.fwd(x[j], x[j + half], w[t], ws[t]);
        }
    }
    if (kLazy) {
      // a transform reduces once per 16 layers; here a mask keeps the lazy values in range
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] &= (W)(~(W)0 >> 8);
    }
    if (kMode == kArithFp) {
      // the transforms reduce once per six layers at most; once per four here
#pragma unroll
      for (int j = 0; j < 16; j++) x[j] = ar.reduce(x[j]);
    }
  }
  W s = 0;
  for (int j = 0; j < 16; j++) s ^= x[j];
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

template <typename F>
float time_ms(F launch) {
  cudaEvent_t e0, e1;
  float ms = 0;
#if defined(CERIUM_EMU)
  launch();
  (void)e0; (void)e1;
  ms = 1.0f;
#else
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  launch();
  cudaDeviceSynchronize();
  cudaEventRecord(e0);
  launch();
  cudaEventRecord(e1);
  cudaDeviceSynchronize();
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
#endif
  return ms;
}

}  // namespace

// results (giga-operations per second, whole GPU):
//  [0] mad.lo.u32   [1] mad.wide.u32   [2] mul.hi.u64   [3] mul.lo.u64   [4] add.u64
//  [5] 64-bit strict (Harvey) butterfly   [6] 64-bit lazy butterfly   [7] 32-bit strict butterfly
//  and, when n_results >= 10:   [8] fma.rn.f64   [9] 64-bit double-precision butterfly
extern "C" __attribute__((visibility("default"))) const char* cerium_probe_last_error(void) {
  return cerium::g_probe_error.c_str();
}

extern "C" __attribute__((visibility("default"))) int cerium_probe_int_pipe(int device, double* gops, int n_results) {
  if (!gops || n_results < 8) return fail(CERIUM_ERR_INVALID, "probe_int_pipe: need room for 8 results");
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || device < 0 || device >= ndev)
    return fail(CERIUM_ERR_CUDA, "probe_int_pipe: no such CUDA device");
  DeviceGuard guard(device);
#if defined(CERIUM_EMU)
  const int sms = 1, iters = 1;
#else
  cudaDeviceProp prop;
  CERIUM_CUDA(cudaGetDeviceProperties(&prop, device));
  const int sms = prop.multiProcessorCount, iters = 2000;
#endif
  const int blocks = sms * 8;
  uint64_t* out = nullptr;
  CERIUM_CUDA(cudaMalloc(&out, (size_t)blocks * kProbeThreads * sizeof(uint64_t)));
  const double nthr = (double)blocks * kProbeThreads;
  const uint64_t q64 = 1125899903827969ull;  // 50-bit NTT prime
  const uint32_t q32 = 268042241u;           // 28-bit NTT prime
  auto rate = [&](float ms, double per_thread_iter) { return nthr * iters * per_thread_iter / (ms * 1e-3) / 1e9; };
  const dim3 g(blocks), b(kProbeThreads);
  gops[0] = rate(time_ms([&] { auto k = probe_raw_kernel<0>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
  gops[1] = rate(time_ms([&] { auto k = probe_raw_kernel<1>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
  gops[2] = rate(time_ms([&] { auto k = probe_raw_kernel<2>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
  gops[3] = rate(time_ms([&] { auto k = probe_raw_kernel<3>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
  gops[4] = rate(time_ms([&] { auto k = probe_raw_kernel<4>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
  PrimeConst<uint64_t> pc64{};
  pc64.q = q64;
  {
    const double qinv = 1.0 / (double)q64;
    std::memcpy(&pc64.fp_qinv, &qinv, sizeof(double));
  }
  PrimeConst<uint32_t> pc32{};
  pc32.q = q32;
  gops[5] = rate(time_ms([&] { auto k = probe_butterfly_kernel<uint64_t, kArithStrict>; CERIUM_LAUNCH(k, g, b, 0, 0, out, pc64, (uint64_t)12345, (uint64_t)67890, iters); }), 32);
  gops[6] = rate(time_ms([&] { auto k = probe_butterfly_kernel<uint64_t, kArithLazy>; CERIUM_LAUNCH(k, g, b, 0, 0, out, pc64, (uint64_t)12345, (uint64_t)67890, iters); }), 32);
  gops[7] = rate(time_ms([&] { auto k = probe_butterfly_kernel<uint32_t, kArithStrict>; CERIUM_LAUNCH(k, g, b, 0, 0, reinterpret_cast<uint32_t*>(out), pc32, 12345u, 67890u, iters); }), 32);
  if (n_results >= 10) {
    gops[8] = rate(time_ms([&] { auto k = probe_raw_kernel<5>; CERIUM_LAUNCH(k, g, b, 0, 0, out, 3u, 5u, iters); }), 32);
    gops[9] = rate(time_ms([&] { auto k = probe_butterfly_kernel<uint64_t, kArithFp>; CERIUM_LAUNCH(k, g, b, 0, 0, out, pc64, (uint64_t)12345, (uint64_t)67890, iters); }), 32);
  }
  cudaFree(out);
  CERIUM_LAUNCH_CHECK("probe_int_pipe");
  return CERIUM_OK;
}
