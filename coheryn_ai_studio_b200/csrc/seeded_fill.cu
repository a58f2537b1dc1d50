// Seeded random weights made on the device: the values of seeded_values.h, one thread per
// element, written as float32 or as bfloat16 (the float32 value rounded to nearest even).
#include "common.cuh"
#include "seeded_values.h"

template <typename Out>
__global__ void seeded_fill_kernel(Out* __restrict__ out, unsigned long long key, unsigned long long first,
                                   unsigned long long count, double mean, double deviation) {
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
    const float v = sv_value(key, first + i, mean, deviation);
    if constexpr (sizeof(Out) == 4) out[i] = v;
    else out[i] = __float2bfloat16_rn(v);
  }
}

CO_EXPORT int coheryn_seeded_fill(void* out, int out_kind, unsigned long long key, unsigned long long first,
                                  unsigned long long count, double mean, double deviation, cudaStream_t stream) {
  if (!out) CO_FAIL("seeded_fill: no output buffer");
  if (count == 0) return 0;
  const int block = 256;
  unsigned long long blocks = (count + block - 1) / block;
  if (blocks > 148ull * 32) blocks = 148ull * 32;
  if (out_kind == CO_F32)
    seeded_fill_kernel<float><<<(unsigned)blocks, block, 0, stream>>>((float*)out, key, first, count, mean, deviation);
  else if (out_kind == CO_BF16)
    seeded_fill_kernel<__nv_bfloat16><<<(unsigned)blocks, block, 0, stream>>>((__nv_bfloat16*)out, key, first, count, mean,
                                                                             deviation);
  else
    CO_FAIL("seeded_fill: unknown output kind %d", out_kind);
  CO_CHECK_LAUNCH("seeded_fill");
  return 0;
}
