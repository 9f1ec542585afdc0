// Host model check of the correctly rounded Float64 exp used by the kernels
// (knet.jl_b200/csrc/exp64.cuh compiles for the host with the same IEEE operations): compares it with
// the 113-bit libquadmath value rounded once, on pseudo-random arguments of several distributions.
// Usage: exp64_check <count> <seed>; prints "checked N mismatches M slow S".
#include <quadmath.h>

#include <cstdio>
#include <cstdlib>

static long g_slow = 0;
#define KN_EXP64_COUNT_SLOW (g_slow++)
#include "exp64.cuh"

static unsigned long long s_state;
static inline unsigned long long next() {
  s_state ^= s_state << 13;
  s_state ^= s_state >> 7;
  s_state ^= s_state << 17;
  return s_state;
}
static inline double unit() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }

int main(int argc, char** argv) {
  const long n = argc > 1 ? atol(argv[1]) : 1000000;
  s_state = argc > 2 ? strtoull(argv[2], nullptr, 10) * 2654435761ull + 88172645463325252ull : 88172645463325252ull;
  long bad = 0, checked = 0;
  for (long i = 0; i < n; i++) {
    double x;
    switch (i & 7) {
      case 0: x = -708.0 + unit() * 1417.0; break;                 // the whole range
      case 1: x = -unit() * 40.0; break;                           // sigm's arguments
      case 2: x = (unit() - 0.5) * 12.0; break;                    // N(0,1)-like magnitudes
      case 3: x = (unit() - 0.5) * 0x1p-20; break;                 // tiny
      case 4: x = (double)((long)(unit() * 1400) - 700) * 0x1.62e42fefa39efp-7; break;  // near multiples of ln2/64
      case 5: x = (double)((long)(unit() * 90000) - 45000) * KN_EXP64_L1; break;        // exact multiples of L1
      case 6: x = -unit() * unit() * 700.0; break;
      default: x = (double)(float)((unit() - 0.5) * 20.0); break;  // Float32-valued arguments
    }
    if (x < -708.0 || x > 709.0) continue;
    const double got = kn::x64::exp_cr64_inrange(x);
    const double want = (double)expq((__float128)x);
    checked++;
    if (got != want) {
      if (bad < 10) printf("x=%a got=%a want=%a\n", x, got, want);
      bad++;
    }
  }
  printf("checked %ld mismatches %ld slow %ld\n", checked, bad, g_slow);
  return bad ? 1 : 0;
}
