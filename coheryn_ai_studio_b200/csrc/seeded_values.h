// Seeded random weights as a pure function of (seed, tensor name, element index).
//
//   key        = seed XOR fnv1a64(tensor name)
//   draw(n)    = the n-th output (n >= 1) of the SplitMix64 stream whose state starts at key
//                (constants of crates/coheryn-engine/src/sampling.rs:123-130)
//   u1         = ((draw(2 i + 1) >> 11) + 1) / 2^53      in (0, 1]
//   u2         =  (draw(2 i + 2) >> 11)      / 2^53      in [0, 1)
//   z          = sqrt(-2 ln u1) * cos(2 pi u2)           (Box-Muller, the cosine branch)
//   value(i)   = float32(mean + deviation * z)
//
// The same bits come out of this header compiled for the host, of the CUDA kernel that
// includes it, and of a numpy restatement: ln and cos are evaluated here with IEEE double
// additions, multiplications, divisions and one square root only, in a fixed order, never
// fused (a library's ln or cos differs from another's in the last place, which would change
// a float32 now and then).  The polynomials are good to about 1e-16, far below the float32
// that is kept.
#pragma once
#include <stdint.h>

#if defined(__CUDA_ARCH__)
#define SV_FN __device__ __forceinline__
#define SV_MUL(a, b) __dmul_rn((a), (b))
#define SV_ADD(a, b) __dadd_rn((a), (b))
#define SV_DIV(a, b) __ddiv_rn((a), (b))
#define SV_SQRT(a) __dsqrt_rn((a))
#else
#include <math.h>
#define SV_FN static inline
// The host file is compiled with -ffp-contract=off, so these stay separate operations.
#define SV_MUL(a, b) ((a) * (b))
#define SV_ADD(a, b) ((a) + (b))
#define SV_DIV(a, b) ((a) / (b))
#define SV_SQRT(a) sqrt((a))
#endif

SV_FN uint64_t sv_draw(uint64_t key, uint64_t n) {
  uint64_t z = key + n * 0x9e3779b97f4a7c15ull;
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

// ln of k * 2^-53 for an integer 1 <= k <= 2^53.
SV_FN double sv_ln_unit(uint64_t k) {
  if (k >> 53) return 0.0;                                              // k = 2^53: u = 1
  // The position of the leading one gives the exponent exactly.
#if defined(__CUDA_ARCH__)
  const int lead = 63 - __clzll((long long)k);
#else
  const int lead = 63 - __builtin_clzll(k);
#endif
  double m = (double)(k << (52 - lead)) * (1.0 / 4503599627370496.0);   // in [1, 2), exact
  int e = lead - 53;                                                    // u = m * 2^e
  if (m > 1.4142135623730951) { m = SV_MUL(m, 0.5); e += 1; }
  const double s = SV_DIV(SV_ADD(m, -1.0), SV_ADD(m, 1.0));
  const double s2 = SV_MUL(s, s);
  double p = 1.0 / 23.0;
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 21.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 19.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 17.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 15.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 13.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 11.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 9.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 7.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 5.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0 / 3.0);
  p = SV_ADD(SV_MUL(p, s2), 1.0);
  const double ln_m = SV_MUL(SV_MUL(2.0, s), p);
  return SV_ADD(SV_MUL((double)e, 0.6931471805599453), ln_m);
}

// cos(2 pi j 2^-53) for an integer 0 <= j < 2^53.
SV_FN double sv_cos_turn(uint64_t j) {
  const int quarter = (int)(j >> 51);                                   // which quarter of the turn
  const double g = (double)(j & ((1ull << 51) - 1)) * (1.0 / 2251799813685248.0);   // place in it, [0, 1), exact
  // The angle inside the quarter is pi/4 + x with x = (g - 1/2) pi/2 in [-pi/4, pi/4).
  const double x = SV_MUL(SV_ADD(g, -0.5), 1.5707963267948966);
  const double x2 = SV_MUL(x, x);
  double c = 1.0 / 6402373705728000.0;            // 1/18!
  c = SV_ADD(SV_MUL(c, x2), -1.0 / 20922789888000.0);    // 16!
  c = SV_ADD(SV_MUL(c, x2), 1.0 / 87178291200.0);        // 14!
  c = SV_ADD(SV_MUL(c, x2), -1.0 / 479001600.0);         // 12!
  c = SV_ADD(SV_MUL(c, x2), 1.0 / 3628800.0);            // 10!
  c = SV_ADD(SV_MUL(c, x2), -1.0 / 40320.0);             // 8!
  c = SV_ADD(SV_MUL(c, x2), 1.0 / 720.0);
  c = SV_ADD(SV_MUL(c, x2), -1.0 / 24.0);
  c = SV_ADD(SV_MUL(c, x2), 0.5);
  c = SV_ADD(SV_MUL(SV_MUL(c, x2), -1.0), 1.0);          // cos x = 1 - x2 (1/2 - x2/24 + ...)
  double s = 1.0 / 121645100408832000.0;          // 1/19!
  s = SV_ADD(SV_MUL(s, x2), -1.0 / 355687428096000.0);   // 17!
  s = SV_ADD(SV_MUL(s, x2), 1.0 / 1307674368000.0);      // 15!
  s = SV_ADD(SV_MUL(s, x2), -1.0 / 6227020800.0);        // 13!
  s = SV_ADD(SV_MUL(s, x2), 1.0 / 39916800.0);           // 11!
  s = SV_ADD(SV_MUL(s, x2), -1.0 / 362880.0);            // 9!
  s = SV_ADD(SV_MUL(s, x2), 1.0 / 5040.0);
  s = SV_ADD(SV_MUL(s, x2), -1.0 / 120.0);
  s = SV_ADD(SV_MUL(s, x2), 1.0 / 6.0);
  s = SV_ADD(SV_MUL(SV_MUL(s, x2), -1.0), 1.0);
  s = SV_MUL(s, x);                                       // sin x
  const double r = 0.7071067811865476;
  const double cos_q = SV_MUL(SV_ADD(c, SV_MUL(s, -1.0)), r);   // cos(pi/4 + x)
  const double sin_q = SV_MUL(SV_ADD(s, c), r);                 // sin(pi/4 + x)
  switch (quarter) {
    case 0: return cos_q;
    case 1: return SV_MUL(sin_q, -1.0);
    case 2: return SV_MUL(cos_q, -1.0);
    default: return sin_q;
  }
}

SV_FN float sv_value(uint64_t key, uint64_t index, double mean, double deviation) {
  const uint64_t a = sv_draw(key, 2 * index + 1), b = sv_draw(key, 2 * index + 2);
  const double ln_u = sv_ln_unit((a >> 11) + 1);
  const double radius = SV_SQRT(SV_MUL(-2.0, ln_u));
  const double z = SV_MUL(radius, sv_cos_turn(b >> 11));
  return (float)SV_ADD(mean, SV_MUL(deviation, z));
}
