// CPU check of the double-precision modular arithmetic of cerium_b200/csrc/modarith.cuh (the same
// source the kernels compile, built here with the CUDA stand-ins): fp_mulmod returns exactly
// y*w - c*q with |result| <= q*(1/2 + B/32) for |y| <= B*q <= 4q, fp_reduce returns a value
// congruent to x within q*(1/2 + 2^-40), and the word <-> double conversions are exact.
// TEST INFRASTRUCTURE ONLY.  Prints "OK <worst ratio>" or a line starting with "FAIL".
#include <cmath>
#include <cstdio>
#include <random>

#include "modarith.cuh"

typedef __int128 i128;
using namespace cerium;

int main() {
  std::mt19937_64 rng(12345);
  // 50-bit NTT primes (largest below 2^50 and a smaller one), a 28-bit and a 20-bit prime
  const int64_t qs[] = {1125899906826241LL, 1125899903827969LL, 268042241LL, 786433LL};
  double worst = 0;
  for (int64_t q : qs) {
    const double qd = (double)q, nq = -qd, qinv = 1.0 / qd;
    for (long it = 0; it < 4000000; it++) {
      int64_t w = (int64_t)(rng() % (uint64_t)q);
      if (w > q / 2) w -= q;
      const int64_t lim = 4 * q;
      int64_t y = (int64_t)(rng() % (uint64_t)(2 * lim + 1)) - lim;
      if (it % 7 == 0) y = (it & 8) ? lim : -lim;           // extreme operands
      if (it % 11 == 0) w = (it & 16) ? q / 2 : -(q / 2);   // extreme twiddles
      const double wd = (double)w, wq = wd / qd, yd = (double)y;
      const double r = fp_mulmod(yd, wd, wq, nq);
      if (r != std::floor(r)) { std::printf("FAIL not an integer q=%lld\n", (long long)q); return 1; }
      const i128 diff = (i128)y * w - (i128)(int64_t)r;
      if (diff % q != 0) { std::printf("FAIL mulmod not congruent q=%lld y=%lld w=%lld\n", (long long)q, (long long)y, (long long)w); return 1; }
      const double B = std::fabs(yd) / qd;
      if (std::fabs(r) > qd * (0.5 + B / 32.0) + 1.0) { std::printf("FAIL mulmod bound q=%lld y=%lld w=%lld r=%.0f\n", (long long)q, (long long)y, (long long)w, r); return 1; }
      worst = std::fmax(worst, std::fabs(r) / qd);
      // reduction of anything below 8q in magnitude
      int64_t x = (int64_t)(rng() % (uint64_t)(16 * q)) - 8 * q;
      if (it % 13 == 0) x = (it & 32) ? 8 * q - 1 : -(8 * q - 1);
      const double xr = fp_reduce((double)x, qinv, nq);
      if (((i128)x - (i128)(int64_t)xr) % q != 0 || std::fabs(xr) > qd * 0.5000001 + 1.0) {
        std::printf("FAIL reduce q=%lld x=%lld -> %.0f\n", (long long)q, (long long)x, xr);
        return 1;
      }
      // conversions
      const uint64_t u = rng() & 0x000fffffffffffffull;
      if (fp_to_u64(fp_from_u64(u)) != u) { std::printf("FAIL conversion %llu\n", (unsigned long long)u); return 1; }
    }
  }
  std::printf("OK %.6f\n", worst);
  return 0;
}
