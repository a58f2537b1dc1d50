// Seeded random weights on the host: fills a float32 or bfloat16 buffer with the values of
// seeded_values.h, several threads each taking a stretch of the indices.  Compiled with
// -ffp-contract=off so that no multiplication and addition are fused (the CUDA kernel and the
// numpy restatement of the tests round after every operation, and so must this).
#include <stdint.h>

#include <thread>
#include <vector>

#include "seeded_values.h"

#define HOST_EXPORT extern "C" __attribute__((visibility("default")))

static inline uint16_t bf16_bits_rne(float f) {
  uint32_t u;
  __builtin_memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);      // finite values only: the generator makes no NaN or infinity
  return (uint16_t)(u >> 16);
}

// out_kind 0: float32, 1: bfloat16 (the float32 value rounded to nearest even).
// Elements first .. first + count - 1 of the tensor go to out[0 .. count - 1].
HOST_EXPORT int coheryn_seeded_fill_host(void* out, int out_kind, unsigned long long key, unsigned long long first,
                                         unsigned long long count, double mean, double deviation, int threads) {
  if (!out || (out_kind != 0 && out_kind != 1)) return 1;
  if (threads < 1) threads = 1;
  if ((unsigned long long)threads > count / 65536 + 1) threads = (int)(count / 65536 + 1);
  auto work = [=](unsigned long long lo, unsigned long long hi) {
    if (out_kind == 0) {
      float* o = (float*)out;
      for (unsigned long long i = lo; i < hi; ++i) o[i] = sv_value(key, first + i, mean, deviation);
    } else {
      uint16_t* o = (uint16_t*)out;
      for (unsigned long long i = lo; i < hi; ++i) o[i] = bf16_bits_rne(sv_value(key, first + i, mean, deviation));
    }
  };
  std::vector<std::thread> pool;
  const unsigned long long per = (count + threads - 1) / threads;
  for (int t = 1; t < threads; ++t) {
    const unsigned long long lo = per * t, hi = lo + per < count ? lo + per : count;
    if (lo < hi) pool.emplace_back(work, lo, hi);
  }
  work(0, per < count ? per : count);
  for (auto& th : pool) th.join();
  return 0;
}

HOST_EXPORT unsigned long long coheryn_seeded_key(unsigned long long seed, const char* name, int length) {
  unsigned long long h = 0xcbf29ce484222325ull;
  for (int i = 0; i < length; ++i) {
    h ^= (unsigned char)name[i];
    h *= 0x100000001b3ull;
  }
  return seed ^ h;
}
