// Memory-bound kernels of a step: embedding gather, residual-add + RMSNorm, SiLU-gate,
// rotary position encoding fused with the write of keys and values into cache pages.
// The residual stream is float32 in every precision mode; norm statistics and rotation
// are computed in float32.
#include "common.cuh"

// ---------------------------------------------------------------------------------
// Embedding: out[t, :] = table[ids[t], :]  (float32 residual stream)
// ---------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int H, int V, int* __restrict__ status) {
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = co_to_float(row[j]);
}

CO_EXPORT int coheryn_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                                   int T, int H, int V, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == CO_F32)
    embed_gather_kernel<float><<<T, threads, 0, stream>>>((const float*)table, ids, out, H, V, status);
  else if (table_dtype == CO_BF16)
    embed_gather_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>((const __nv_bfloat16*)table, ids, out, H, V, status);
  else
    CO_FAIL("embed_gather: unknown table dtype %d", table_dtype);
  CO_CHECK_LAUNCH("embed_gather");
  return 0;
}

// ---------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   x = resid[src] (+ delta[src]);  if update: resid[src] = x
//   out[r] = (x * (1/sqrt(mean(x^2) + eps))) * w
// src = rows ? rows[r] : r.  One block per row; the sum of squares is reduced in a
// fixed order, so a row's result does not depend on what else is in the batch.
// ---------------------------------------------------------------------------------
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const void* __restrict__ weight,
                                   int wdtype, float eps, TO* __restrict__ out, int H, int update) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  const TD* d = delta ? delta + src * H : nullptr;
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = x[j];
    if (d) {
      v += co_to_float(d[j]);
      if (update) x[j] = v;
    }
    ss += v * v;
  }
  ss = co_block_sum(ss, scratch);
  const float mean = ss / (float)H;
  const float scale = 1.0f / sqrtf(mean + eps);
  TO* o = out + (size_t)r * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float v = x[j];
    if (d && !update) v += co_to_float(d[j]);
    o[j] = co_from_float<TO>((v * scale) * co_load_any(weight, wdtype, j));
  }
}

CO_EXPORT int coheryn_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const int* rows,
                                  const void* weight, int wdtype, float eps, void* out, int out_dtype,
                                  int n_rows, int H, int update, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (rows && update) CO_FAIL("add_rmsnorm: cannot update the residual through a row gather");
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define LAUNCH(TD, TO)                                                                         \
  add_rmsnorm_kernel<TD, TO><<<n_rows, threads, 0, stream>>>(resid, (const TD*)delta, rows, weight, \
                                                             wdtype, eps, (TO*)out, H, update)
  if (delta_dtype == CO_F32 && out_dtype == CO_F32) LAUNCH(float, float);
  else if (delta_dtype == CO_BF16 && out_dtype == CO_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == CO_F32 && out_dtype == CO_BF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == CO_BF16 && out_dtype == CO_F32) LAUNCH(__nv_bfloat16, float);
  else CO_FAIL("add_rmsnorm: unknown dtypes %d/%d", delta_dtype, out_dtype);
#undef LAUNCH
  CO_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------
// Gated activation over interleaved columns: out[m, j] = silu(in[m, 2j]) * in[m, 2j+1],
// in is [M, 2I] (column 2j = gate_j, column 2j+1 = up_j).
// silu(g) = g / (1 + exp(-g)) in float32.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int I, size_t total) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const size_t m = i / I, j = i % I;
    const float g = co_to_float(in[m * 2 * I + 2 * j]);
    const float u = co_to_float(in[m * 2 * I + 2 * j + 1]);
    out[i] = co_from_float<T>((g / (1.0f + expf(-g))) * u);
  }
}

CO_EXPORT int coheryn_silu_mul(const void* in, void* out, int dtype, int M, int I, cudaStream_t stream) {
  const size_t total = (size_t)M * I;
  if (total == 0) return 0;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == CO_F32) silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)in, (float*)out, I, total);
  else if (dtype == CO_BF16) silu_mul_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, I, total);
  else CO_FAIL("silu_mul: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("silu_mul");
  return 0;
}

// ---------------------------------------------------------------------------------
// Rotary position encoding (rotate-half pairing (i, i + rot/2)) of q and k, fused with
// the write of k and v into their cache pages.
//   qkv: [T, (nh + 2 nkv) * hd]; q is rotated in place; rotated k and plain v go to
//   k_cache / v_cache, laid out [page][kv head][slot in page][hd].
//   cos_sin: float2 [max_pos][rot/2] = (cos, sin) of the angle of pair i at a position.
//   slots[t] = page * page_size + offset, or < 0 to write nothing for token t.
// Rotation is done in float32: out_a = fma(a, cos, -(b sin)), out_b = fma(a, sin, b cos).
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const float2* __restrict__ cos_sin, const int* __restrict__ slots,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, int nh, int nkv,
                                     int hd, int rot, int page_size, int write_kv) {
  const int t = blockIdx.x;
  const int head = blockIdx.y;  // [0, nh): q   [nh, nh+nkv): k   [nh+nkv, nh+2nkv): v
  const int row_stride = (nh + 2 * nkv) * hd;
  T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;
  const int pos = positions[t];
  const int half = rot >> 1;
  T* dst = nullptr;
  if (head >= nh) {
    if (!write_kv) return;
    const int slot = slots[t];
    if (slot < 0) return;
    const int page = slot / page_size, off = slot % page_size;
    const int kvh = head < nh + nkv ? head - nh : head - nh - nkv;
    T* base = head < nh + nkv ? k_cache : v_cache;
    dst = base + (((size_t)page * nkv + kvh) * page_size + off) * hd;
  }
  if (head < nh + nkv) {
    const float2* cs = cos_sin + (size_t)pos * half;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float a = co_to_float(src[i]), b = co_to_float(src[i + half]);
      const float2 c = cs[i];
      const T ra = co_from_float<T>(fmaf(a, c.x, -(b * c.y)));
      const T rb = co_from_float<T>(fmaf(a, c.y, b * c.x));
      if (dst) { dst[i] = ra; dst[i + half] = rb; }
      else { src[i] = ra; src[i + half] = rb; }
    }
    if (dst)
      for (int i = rot + threadIdx.x; i < hd; i += blockDim.x) dst[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = src[i];
  }
}

CO_EXPORT int coheryn_rope_kv_write(void* qkv, int dtype, const int* positions, const float* cos_sin,
                                    const int* slots, void* k_cache, void* v_cache, int T, int nh, int nkv,
                                    int hd, int rot, int page_size, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1)) CO_FAIL("rope_kv_write: rotary size %d does not fit head size %d", rot, hd);
  dim3 grid(T, nh + 2 * nkv);
  const int threads = hd >= 128 ? 64 : 32;
  if (dtype == CO_F32)
    rope_kv_write_kernel<float><<<grid, threads, 0, stream>>>((float*)qkv, positions, (const float2*)cos_sin, slots,
                                                              (float*)k_cache, (float*)v_cache, nh, nkv, hd, rot, page_size, write_kv);
  else if (dtype == CO_BF16)
    rope_kv_write_kernel<__nv_bfloat16><<<grid, threads, 0, stream>>>((__nv_bfloat16*)qkv, positions, (const float2*)cos_sin, slots,
                                                                      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, hd, rot, page_size, write_kv);
  else CO_FAIL("rope_kv_write: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("rope_kv_write");
  return 0;
}
