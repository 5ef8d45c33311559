// Reference-CUDA harness.  TEST / BASELINE INFRASTRUCTURE ONLY.
//
// Compiles the reference's own device headers (cerium/compiler/backend/kernels/{fhe,
// fhe_arith,fhe_mem,fhe_ntt,fhe_bconv,transpose}.cuh), unmodified and from where they lie in
// the reference tree (-I on the nvcc command line; no reference source is copied into this
// repository), behind thin __global__ wrappers.  The reference's own wrappers live in
// cerium/compiler/backend/kernels/function.cu, which does not compile with CUDA 12.9 (it calls
// the CUDA-13 five-argument cudaGraphAddDependencies at function.cu:97,195,278), so the wrappers
// below restate function.cu:22-56 (ntt), :101-149 (sud), :199-235 (int) and
// function.cuh:61-78 (bco): same launch shapes, same argument tables.
//
// Twiddle tables are laid out the way EvaluatorContext::init_ntt_params builds them
// (cerium/runtime/execution/evaluator.cpp:115-231): bit-reversed powers of the minimal
// primitive root with Shoup words floor(w * 2^32 / q) (cerium/runtime/math/util.h:140-143),
// inverse powers pre-divided by two, then permute_root_powers (evaluator.cpp:93-113) with
// (1,256,N,4), (256,N,N,4) for the forward table and (128,N,N,8) for the inverse table.
//
// The library produced here (oracle/_ref/libref_cuda.so) is (a) the 32-bit GPU oracle that
// pins the CPU oracle and the product's 32-bit kernels to the reference's real output and
// (b) the "reference kernel on the same B200" timing.  Outputs of the reference may lie in
// [q, 2q) (its Barrett does one conditional subtract); callers compare modulo q.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#define __FNAME__ refharness
#include "fhe.cuh"

namespace {

typedef unsigned __int128 u128;

uint64_t mulmod(uint64_t a, uint64_t b, uint64_t q) { return (uint64_t)((u128)a * b % q); }
uint64_t powmod(uint64_t a, uint64_t e, uint64_t q) {
  uint64_t r = 1;
  for (a %= q; e; e >>= 1, a = mulmod(a, a, q))
    if (e & 1) r = mulmod(r, a, q);
  return r;
}
uint32_t brev(uint32_t x, int bits) {
  uint32_t r = 0;
  for (int i = 0; i < bits; i++, x >>= 1) r = (r << 1) | (x & 1);
  return r;
}
uint64_t min_root(uint64_t q, int logn) {
  const uint64_t m = (uint64_t)2 << logn, e = (q - 1) / m;
  uint64_t r = 0;
  for (uint64_t g = 2; g < q; g++) {
    r = powmod(g, e, q);
    if (powmod(r, m / 2, q) == q - 1) break;
  }
  const uint64_t sq = mulmod(r, r, q);
  uint64_t best = r, cur = r;
  for (uint64_t i = 0; i < m / 2; i++, cur = mulmod(cur, sq, q))
    if (cur < best) best = cur;
  return best;
}
uint32_t shoup32(uint32_t w, uint32_t q) { return (uint32_t)(((uint64_t)w << 32) / q); }

// evaluator.cpp:93-113 for one prime's table
void permute(std::vector<uint32_t>& t, size_t m_start, size_t m_end, size_t per_thread) {
  std::vector<uint32_t> o(t);
  for (size_t mm = m_start; mm < m_end; mm *= per_thread)
    for (size_t tt = 1; tt < per_thread; tt *= 2)
      for (size_t k = 0; k < tt; k++)
        for (size_t i = 0; i < mm; i++) o[mm * (tt + k) + i] = t[(mm + i) * tt + k];
  t.swap(o);
}

struct Harness {
  int n_primes = 0;
  std::vector<uint32_t> primes;
  uint32_t *d_mod = nullptr, *d_ratio = nullptr, *d_k = nullptr;
  uint2 *d_fwd = nullptr, *d_inv = nullptr;
};

__global__ static void __launch_bounds__(NTT0_BLOCK_DIM_X, 32)
    k_ntt0(uint32_t** outs, const uint32_t** ins, const uint32_t* bases, const uint32_t* mod, const uint2* roots) {
  __shared__ uint32_t sh[nttShMemSize0];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  ntt0(outs[b], ins[b], roots + (size_t)t * NTT_TABLE_SIZE, mod[t], sh);
}
__global__ static void __launch_bounds__(NTT1_BLOCK_DIM_X, 32)
    k_ntt1(uint32_t** outs, const uint32_t* bases, const uint32_t* mod, const uint2* roots) {
  __shared__ uint32_t sh[nttShMemSize1];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  ntt1(outs[b], outs[b], roots + (size_t)t * NTT_TABLE_SIZE, mod[t], sh);
}
__global__ static void __launch_bounds__(NTT0_BLOCK_DIM_X, 32)
    k_sud0(uint32_t** outs, const uint32_t** ins2, const uint32_t* bases, const uint32_t* mod, const uint2* roots) {
  __shared__ uint32_t sh[nttShMemSize0];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  ntt0_sud(outs[b], ins2[b], roots + (size_t)t * NTT_TABLE_SIZE, mod[t], sh);
}
__global__ static void __launch_bounds__(NTT1_BLOCK_DIM_X, 32)
    k_sud1(uint32_t** outs, const uint32_t** ins1, const uint32_t* bases, const uint32_t* mod, const uint2* roots,
           const uint32_t* factors, const uint32_t* ratio, const uint32_t* bk) {
  __shared__ uint32_t sh[nttShMemSize1];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  ntt1_sud(outs[b], outs[b], ins1[b], roots + (size_t)t * NTT_TABLE_SIZE, factors[t], mod[t], ratio[t], bk[t], sh);
}
__global__ static void k_int0(uint32_t** outs, const uint32_t** ins, const uint32_t* bases, const uint32_t* mod,
                              const uint2* roots) {
  __shared__ uint32_t sh[intShMemSize0];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  intt0(outs[b], ins[b], roots + (size_t)t * NTT_TABLE_SIZE, mod[t], sh);
}
__global__ static void k_int1(uint32_t** outs, const uint32_t* bases, const uint32_t* mod, const uint2* roots) {
  __shared__ uint32_t sh[intShMemSize1];
  const auto b = blockIdx.y;
  const auto t = bases[b];
  intt1(outs[b], outs[b], roots + (size_t)t * NTT_TABLE_SIZE, mod[t], sh);
}
template <size_t I, size_t O>
__global__ static void __launch_bounds__(BLOCK_DIM_X)
    k_bco(uint32_t** outs, const uint32_t** ins, const uint32_t** factors, const uint32_t** omod,
          const uint32_t** ratio, const uint32_t** bk) {
  const size_t j = blockIdx.y;
  convert<I, O>(ins[j], outs[j], factors[j], omod[j], ratio[j], bk[j]);
}

template <typename T>
T* upload(const std::vector<T>& v) {
  T* d = nullptr;
  if (cudaMalloc(&d, v.size() * sizeof(T)) != cudaSuccess) return nullptr;
  cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}

// Device pointer tables for `count` contiguous limbs of N words starting at base.
uint32_t** limb_table(uint32_t* base, int count) {
  std::vector<uint32_t*> h(count);
  for (int i = 0; i < count; i++) h[i] = base + (size_t)i * LENGTH;
  return upload(h);
}

template <size_t I, size_t O>
int run_bco(Harness* h, uint32_t* out, const uint32_t* in, const uint32_t* in_idx, const uint32_t* out_idx,
            int n_conv, int iters, float* ms) {
  // factor matrix of DeviceBaseConverter::set_output_bases (evaluator.cpp:1539-1578)
  std::vector<uint32_t> fac(I * O), omod(O), ratio(O), bk(O, 58);
  std::vector<uint64_t> inv(I);
  for (size_t i = 0; i < I; i++) {
    const uint64_t qi = h->primes[in_idx[i]];
    uint64_t p = 1;
    for (size_t k = 0; k < I; k++)
      if (k != i) p = mulmod(p, h->primes[in_idx[k]] % qi, qi);
    inv[i] = powmod(p, qi - 2, qi);
  }
  for (size_t j = 0; j < O; j++) {
    const uint64_t pj = h->primes[out_idx[j]];
    omod[j] = (uint32_t)pj;
    ratio[j] = (uint32_t)(((uint64_t)1 << 58) / pj);
    for (size_t i = 0; i < I; i++) {
      uint64_t qhat = 1;
      for (size_t k = 0; k < I; k++)
        if (k != i) qhat = mulmod(qhat, h->primes[in_idx[k]] % pj, pj);
      fac[j * I + i] = (uint32_t)mulmod(inv[i] % pj, qhat, pj);
    }
  }
  uint32_t *d_fac = upload(fac), *d_omod = upload(omod), *d_ratio = upload(ratio), *d_bk = upload(bk);
  std::vector<uint32_t*> outs(n_conv), facs(n_conv, d_fac), omods(n_conv, d_omod), ratios(n_conv, d_ratio), bks(n_conv, d_bk);
  std::vector<const uint32_t*> ins(n_conv);
  for (int c = 0; c < n_conv; c++) {
    outs[c] = out + (size_t)c * O * LENGTH;
    ins[c] = in + (size_t)c * I * LENGTH;
  }
  uint32_t** d_outs = upload(outs);
  const uint32_t** d_ins = upload(ins);
  uint32_t** d_facs = upload(facs);
  uint32_t** d_omods = upload(omods);
  uint32_t** d_ratios = upload(ratios);
  uint32_t** d_bks = upload(bks);
  const size_t smem = ((I * O / 32 + 1) * 32 + 256 * I) * 4;  // evaluator.cpp:891-898
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(k_bco<I, O>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int it = 0; it < iters; it++)
    k_bco<I, O><<<dim3(GRID_DIM_X, n_conv), BLOCK_DIM_X, smem>>>(
        d_outs, d_ins, (const uint32_t**)d_facs, (const uint32_t**)d_omods, (const uint32_t**)d_ratios,
        (const uint32_t**)d_bks);
  cudaEventRecord(e1);
  cudaError_t err = cudaDeviceSynchronize();
  if (ms) cudaEventElapsedTime(ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(d_fac); cudaFree(d_omod); cudaFree(d_ratio); cudaFree(d_bk);
  cudaFree(d_outs); cudaFree(d_ins); cudaFree(d_facs); cudaFree(d_omods); cudaFree(d_ratios); cudaFree(d_bks);
  return err == cudaSuccess ? 0 : 2;
}

}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API int refcuda_create(void** out, const uint32_t* primes, int n_primes) {
  auto* h = new Harness();
  h->n_primes = n_primes;
  h->primes.assign(primes, primes + n_primes);
  const size_t n = LENGTH;
  const int logn = 16;
  std::vector<uint2> fwd(n * n_primes), inv(n * n_primes);
  std::vector<uint32_t> mod(n_primes), ratio(n_primes), bk(n_primes, 58);
  for (int r = 0; r < n_primes; r++) {
    const uint32_t q = primes[r];
    mod[r] = q;
    ratio[r] = (uint32_t)(((uint64_t)1 << 58) / q);
    const uint64_t psi = min_root(q, logn), ipsi = powmod(psi, q - 2, q), half = powmod(2, q - 2, q);
    std::vector<uint32_t> w(n), ws(n), wi(n), wis(n);
    uint64_t p = psi, pi = ipsi;
    for (size_t j = 1; j < n; j++) {
      const uint32_t at = brev((uint32_t)j, logn);
      w[at] = (uint32_t)p;
      ws[at] = shoup32((uint32_t)p, q);
      const uint32_t d2 = (uint32_t)mulmod(pi, half, q);
      wi[at] = d2;
      wis[at] = shoup32(d2, q);
      p = mulmod(p, psi, q);
      pi = mulmod(pi, ipsi, q);
    }
    w[0] = 1;
    ws[0] = shoup32(1, q);
    wi[0] = (uint32_t)half;
    wis[0] = shoup32((uint32_t)half, q);
    permute(w, 1, 256, 4);
    permute(ws, 1, 256, 4);
    permute(w, 256, n, 4);
    permute(ws, 256, n, 4);
    permute(wi, 128, n, 8);
    permute(wis, 128, n, 8);
    for (size_t j = 0; j < n; j++) {
      fwd[r * n + j] = make_uint2(w[j], ws[j]);
      inv[r * n + j] = make_uint2(wi[j], wis[j]);
    }
  }
  h->d_mod = upload(mod);
  h->d_ratio = upload(ratio);
  h->d_k = upload(bk);
  h->d_fwd = upload(fwd);
  h->d_inv = upload(inv);
  if (!h->d_mod || !h->d_ratio || !h->d_k || !h->d_fwd || !h->d_inv) return 2;
  *out = h;
  return 0;
}

REF_API void refcuda_destroy(void* hh) {
  auto* h = static_cast<Harness*>(hh);
  if (!h) return;
  cudaFree(h->d_mod); cudaFree(h->d_ratio); cudaFree(h->d_k); cudaFree(h->d_fwd); cudaFree(h->d_inv);
  delete h;
}

// Forward (inverse = 0) or inverse NTT of `count` contiguous limbs, in -> out (device pointers);
// limb i uses prime bases[i] (host array).  Runs `iters` times and reports the total milliseconds.
REF_API int refcuda_ntt(void* hh, uint32_t* out, const uint32_t* in, const uint32_t* bases, int count, int inverse,
                        int iters, float* ms) {
  auto* h = static_cast<Harness*>(hh);
  uint32_t** d_outs = limb_table(out, count);
  const uint32_t** d_ins = (const uint32_t**)limb_table(const_cast<uint32_t*>(in), count);
  uint32_t* d_bases = upload(std::vector<uint32_t>(bases, bases + count));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int it = 0; it < iters; it++) {
    if (!inverse) {
      k_ntt0<<<dim3(NTT0_GRID_DIM_X, count), NTT0_BLOCK_DIM_X>>>(d_outs, d_ins, d_bases, h->d_mod, h->d_fwd);
      k_ntt1<<<dim3(NTT1_GRID_DIM_X, count), NTT1_BLOCK_DIM_X>>>(d_outs, d_bases, h->d_mod, h->d_fwd);
    } else {
      k_int0<<<dim3(INT0_GRID_DIM_X, count), INT0_BLOCK_DIM_X>>>(d_outs, d_ins, d_bases, h->d_mod, h->d_inv);
      k_int1<<<dim3(INT1_GRID_DIM_X, count), INT1_BLOCK_DIM_X>>>(d_outs, d_bases, h->d_mod, h->d_inv);
    }
  }
  cudaEventRecord(e1);
  cudaError_t err = cudaDeviceSynchronize();
  if (ms) cudaEventElapsedTime(ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(d_outs); cudaFree(d_ins); cudaFree(d_bases);
  if (err != cudaSuccess) fprintf(stderr, "refcuda_ntt: %s\n", cudaGetErrorString(err));
  return err == cudaSuccess ? 0 : 2;
}

// SuD: out = (in1 + 4q - NTT(in2)) * factor[prime] mod q for `count` contiguous limbs.
// factors: host array with one entry per prime of the context (compute_sud_factors layout).
REF_API int refcuda_sud(void* hh, uint32_t* out, const uint32_t* in1, const uint32_t* in2, const uint32_t* bases,
                        int count, const uint32_t* factors, int iters, float* ms) {
  auto* h = static_cast<Harness*>(hh);
  uint32_t** d_outs = limb_table(out, count);
  const uint32_t** d_in1 = (const uint32_t**)limb_table(const_cast<uint32_t*>(in1), count);
  const uint32_t** d_in2 = (const uint32_t**)limb_table(const_cast<uint32_t*>(in2), count);
  uint32_t* d_bases = upload(std::vector<uint32_t>(bases, bases + count));
  uint32_t* d_fac = upload(std::vector<uint32_t>(factors, factors + h->n_primes));
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  cudaEventRecord(e0);
  for (int it = 0; it < iters; it++) {
    k_sud0<<<dim3(NTT0_GRID_DIM_X, count), NTT0_BLOCK_DIM_X>>>(d_outs, d_in2, d_bases, h->d_mod, h->d_fwd);
    k_sud1<<<dim3(NTT1_GRID_DIM_X, count), NTT1_BLOCK_DIM_X>>>(d_outs, d_in1, d_bases, h->d_mod, h->d_fwd, d_fac,
                                                               h->d_ratio, h->d_k);
  }
  cudaEventRecord(e1);
  cudaError_t err = cudaDeviceSynchronize();
  if (ms) cudaEventElapsedTime(ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(d_outs); cudaFree(d_in1); cudaFree(d_in2); cudaFree(d_bases); cudaFree(d_fac);
  if (err != cudaSuccess) fprintf(stderr, "refcuda_sud: %s\n", cudaGetErrorString(err));
  return err == cudaSuccess ? 0 : 2;
}

// Base conversion convert<I,O> for the instantiated shapes; n_conv independent conversions over
// contiguous [n_conv][I][N] -> [n_conv][O][N] with the same prime sets.
REF_API int refcuda_bconv(void* hh, uint32_t* out, const uint32_t* in, const uint32_t* in_idx, int I,
                          const uint32_t* out_idx, int O, int n_conv, int iters, float* ms) {
  auto* h = static_cast<Harness*>(hh);
#define SHAPE(i, o) \
  if (I == i && O == o) return run_bco<i, o>(h, out, in, in_idx, out_idx, n_conv, iters, ms);
  SHAPE(5, 35)
  SHAPE(5, 30)
  SHAPE(2, 6)
  SHAPE(3, 5)
  SHAPE(18, 12)
  SHAPE(32, 8)
#undef SHAPE
  return 3;
}
