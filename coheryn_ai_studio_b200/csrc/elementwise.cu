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
                                    float* __restrict__ out, int H, int V, int* __restrict__ status, float scale) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  if (id < 0 || id >= V) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * H;
  if (scale == 1.0f) {
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = co_to_float(row[j]);
  } else {   // an architecture that multiplies its embedding rows by a constant
    for (int j = threadIdx.x; j < H; j += blockDim.x) out[(size_t)t * H + j] = co_to_float(row[j]) * scale;
  }
}

CO_EXPORT int coheryn_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                                   int T, int H, int V, int* status, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  const int threads = H >= 1024 ? 256 : 128;
  if (table_dtype == CO_F32)
    co_launch(embed_gather_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, out, H, V, status, scale);
  else if (table_dtype == CO_BF16)
    co_launch(embed_gather_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)table, ids, out, H, V, status, scale);
  else
    CO_FAIL("embed_gather: unknown table dtype %d", table_dtype);
  CO_CHECK_LAUNCH("embed_gather");
  return 0;
}

// ---------------------------------------------------------------------------------
// Row gather: out[r, :] = src[rows[r], :] for rows of `row_bytes` bytes (any element type).
// ---------------------------------------------------------------------------------
template <typename Unit>
__global__ void gather_rows_kernel(const char* __restrict__ src, long src_stride, const int* __restrict__ rows,
                                   char* __restrict__ out, int units) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const Unit* from = (const Unit*)(src + (size_t)rows[blockIdx.x] * src_stride);
  Unit* to = (Unit*)(out + (size_t)blockIdx.x * units * sizeof(Unit));
  for (int j = threadIdx.x; j < units; j += blockDim.x) to[j] = from[j];
}

CO_EXPORT int coheryn_gather_rows(const void* src, long src_stride_bytes, const int* rows, void* out, int R,
                                  int row_bytes, cudaStream_t stream) {
  if (R <= 0 || row_bytes <= 0) return 0;
  const bool wide = row_bytes % 16 == 0 && src_stride_bytes % 16 == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)out % 16) == 0;
  const bool words = row_bytes % 4 == 0 && src_stride_bytes % 4 == 0 && ((uintptr_t)src % 4) == 0 && ((uintptr_t)out % 4) == 0;
  if (wide)
    co_launch(gather_rows_kernel<uint4>, dim3(R), dim3(128), 0, stream, (const char*)src, src_stride_bytes, rows, (char*)out, row_bytes / 16);
  else if (words)
    co_launch(gather_rows_kernel<uint32_t>, dim3(R), dim3(128), 0, stream, (const char*)src, src_stride_bytes, rows, (char*)out, row_bytes / 4);
  else
    co_launch(gather_rows_kernel<unsigned char>, dim3(R), dim3(128), 0, stream, (const char*)src, src_stride_bytes, rows, (char*)out, row_bytes);
  CO_CHECK_LAUNCH("gather_rows");
  return 0;
}

// out[rows[r]] = src[r] for 32-bit elements (the inverse of a gather of single words).
__global__ void scatter_words_kernel(const uint32_t* __restrict__ src, const int* __restrict__ rows, uint32_t* __restrict__ out, int R) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < R) out[rows[r]] = src[r];
}

CO_EXPORT int coheryn_scatter_words(const void* src, const int* rows, void* out, int R, cudaStream_t stream) {
  if (R <= 0) return 0;
  co_launch(scatter_words_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, (const uint32_t*)src, rows, (uint32_t*)out, R);
  CO_CHECK_LAUNCH("scatter_words");
  return 0;
}

// ---------------------------------------------------------------------------------
// Logits of an architecture that scales them or adds a bias: x[r, v] = x[r, v] * scale + bias[v].
// ---------------------------------------------------------------------------------
__global__ void scale_add_bias_kernel(float* __restrict__ x, long stride, int V, float scale, const void* __restrict__ bias,
                                      int bias_dtype) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  float* row = x + (size_t)blockIdx.y * stride;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < V; v += gridDim.x * blockDim.x)
    row[v] = row[v] * scale + (bias ? co_load_any(bias, bias_dtype, v) : 0.f);
}

CO_EXPORT int coheryn_scale_add_bias(float* x, long stride, int R, int V, float scale, const void* bias, int bias_dtype,
                                     cudaStream_t stream) {
  if (R <= 0 || V <= 0) return 0;
  if (R > 65535) CO_FAIL("scale_add_bias: at most 65535 rows, not %d", R);
  const int blocks = (V + 1023) / 1024 < 64 ? (V + 1023) / 1024 : 64;
  co_launch(scale_add_bias_kernel, dim3(blocks, R), dim3(256), 0, stream, x, stride, V, scale, bias, bias_dtype);
  CO_CHECK_LAUNCH("scale_add_bias");
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
  co_pdl_launch_dependents();
  co_pdl_wait();
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

// Vector variant for widths that are a multiple of 4 and at most 8192: the row stays in
// registers between the two passes (float4 per thread and step), the delta is read four at
// a time.  Same arithmetic and the same order of summation per thread count.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
  }
};

// Thread-block clusters: rank and size of this CTA's cluster (1 CTA when launched without one),
// and a sum over the cluster's CTAs: every CTA writes its term into slot `rank` of EVERY
// CTA's `slots` (distributed shared memory), the cluster meets at its hardware barrier, and
// each CTA adds its own copy of the slots in rank order.  No CTA reads a peer's memory, so
// none has to outlive the others.  `v` must be the same in all threads of the CTA.
__device__ __forceinline__ unsigned co_cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned co_cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ float co_cluster_sum(float v, float* slots /* >= cluster size floats, shared */) {
  const unsigned n = co_cluster_size(), rank = co_cluster_rank();
  if (n == 1) return v;
  if (threadIdx.x < n) {
    unsigned local = (unsigned)__cvta_generic_to_shared(slots + rank), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(threadIdx.x));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
  }
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  float total = 0.f;
  for (unsigned k = 0; k < n; ++k) total += slots[k];
  return total;
}

template <typename TD, typename TO, typename TW, int STEPS>
__global__ void __launch_bounds__(256)
add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const int* __restrict__ rows,
                       const TW* __restrict__ weight, float eps, TO* __restrict__ out, int H, int update) {
  __shared__ float scratch[33];
  __shared__ float cl_slots[8];
  co_pdl_launch_dependents();
  // The CTAs of a cluster share a row: CTA k of n takes the k-th run of columns.
  const int cl_n = (int)co_cluster_size(), cl_r = (int)co_cluster_rank();
  const int c_per = ((H / 4 + cl_n - 1) / cl_n) * 4;
  const int c_lo = cl_r * c_per, c_hi = min(H, c_lo + c_per);
  float4 wv[STEPS];   // the weights depend on no earlier kernel
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    wv[i] = j < c_hi ? Vec4<TW>::load(weight + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  co_pdl_wait();
  const int r = blockIdx.x / cl_n;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  const TD* d = delta ? delta + src * H : nullptr;
  float4 v[STEPS];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    if (j < c_hi) {
      v[i] = Vec4<float>::load(x + j);
      if (d) {
        const float4 dv = Vec4<TD>::load(d + j);
        v[i].x += dv.x; v[i].y += dv.y; v[i].z += dv.z; v[i].w += dv.w;
        if (update) Vec4<float>::store(x + j, v[i]);
      }
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = co_cluster_sum(co_block_sum(ss, scratch), cl_slots);
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    if (j < c_hi) {
      const float4 w = wv[i];
      Vec4<TO>::store(o + j, make_float4((v[i].x * scale) * w.x, (v[i].y * scale) * w.y, (v[i].z * scale) * w.z,
                                         (v[i].w * scale) * w.w));
    }
  }
}

// Many rows (prompt portions): W warps per row (1, 2, 4 or 8: at most 16 float4 per lane), eight warps
// per CTA, so that a few hundred CTAs hold every row of the step at once, each row's loads are all
// in flight together and a one-warp row is reduced by shuffles alone.
template <typename TD, typename TO, typename TW, int VPL, int W>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ resid, const TD* __restrict__ delta, const int* __restrict__ rows,
                        const TW* __restrict__ weight, float eps, TO* __restrict__ out, int H, int update, int n_rows) {
  __shared__ float partial[8];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.x * (8 / W) + warp / W, wsub = warp % W;
  const bool live = r < n_rows;
  const size_t src = live ? (rows ? (size_t)rows[r] : (size_t)r) : 0;
  float* x = resid + src * H;
  const TD* d = delta ? delta + src * H : nullptr;
  float4 v[VPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = ((i * W + wsub) * 32 + lane) * 4;
    v[i] = (live && j < H) ? Vec4<float>::load(x + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (d) {
    float4 dv[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int j = ((i * W + wsub) * 32 + lane) * 4;
      dv[i] = (live && j < H) ? Vec4<TD>::load(d + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int j = ((i * W + wsub) * 32 + lane) * 4;
      v[i].x += dv[i].x; v[i].y += dv[i].y; v[i].z += dv[i].z; v[i].w += dv[i].w;
      if (update && live && j < H) Vec4<float>::store(x + j, v[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
  ss = co_warp_sum(ss);
  if (W > 1) {
    if (lane == 0) partial[warp] = ss;
    __syncthreads();
    ss = 0.f;
#pragma unroll
    for (int k = 0; k < W; ++k) ss += partial[(warp / W) * W + k];
  }
  if (!live) return;
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = ((i * W + wsub) * 32 + lane) * 4;
    if (j < H) {
      const float4 w = Vec4<TW>::load(weight + j);
      Vec4<TO>::store(o + j, make_float4((v[i].x * scale) * w.x, (v[i].y * scale) * w.y, (v[i].z * scale) * w.z,
                                         (v[i].w * scale) * w.w));
    }
  }
}

// With few rows one CTA per row leaves the GPU idle and the row's latency long: a cluster of
// four CTAs shares each row (from 1024 columns on, up to 64 rows).
inline int norm_cluster(int n_rows, int H) { return (n_rows <= 64 && H >= 1024 && (H / 4) % 4 == 0) ? 4 : 1; }

template <typename TD, typename TO, typename TW>
void launch_rmsnorm_vec(float* resid, const void* delta, const int* rows, const void* weight, float eps, void* out,
                        int n_rows, int H, int update, cudaStream_t stream) {
  if (n_rows > 64) {
    // warps per row and float4 per lane: the fewest warps that keep a lane at 16 float4 or fewer
    int W = 1;
    while (W < 8 && (H / 4 + 32 * W - 1) / (32 * W) > 16) W *= 2;
    const int vpl = (H / 4 + 32 * W - 1) / (32 * W);
    const dim3 grid((n_rows + 8 / W - 1) / (8 / W));
#define ROWS(V, WW) co_launch(add_rmsnorm_rows_kernel<TD, TO, TW, V, WW>, grid, dim3(256), 0, stream, resid, (const TD*)delta, rows, \
                              (const TW*)weight, eps, (TO*)out, H, update, n_rows)
#define ROWS_W(WW) do { if (vpl <= 4) ROWS(4, WW); else if (vpl <= 8) ROWS(8, WW); else if (vpl <= 12) ROWS(12, WW); else ROWS(16, WW); } while (0)
    if (vpl <= 16) {
      if (W == 1) ROWS_W(1); else if (W == 2) ROWS_W(2); else if (W == 4) ROWS_W(4); else ROWS_W(8);
      return;
    }
#undef ROWS_W
#undef ROWS
  }
  const int cl = norm_cluster(n_rows, H);
  const int steps = (H / 4 / cl + 255) / 256;
#define GO(S) co_launch_cluster(cl, add_rmsnorm_vec_kernel<TD, TO, TW, S>, dim3(n_rows * cl), dim3(256), 0, stream, resid, \
                                (const TD*)delta, rows, (const TW*)weight, eps, (TO*)out, H, update)
  if (steps <= 1) GO(1); else if (steps <= 2) GO(2); else if (steps <= 4) GO(4); else GO(8);
#undef GO
}

CO_EXPORT int coheryn_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const int* rows,
                                  const void* weight, int wdtype, float eps, void* out, int out_dtype,
                                  int n_rows, int H, int update, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (rows && update) CO_FAIL("add_rmsnorm: cannot update the residual through a row gather");
  if (H % 4 == 0 && H <= 8192 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)delta & 7) == 0 &&
      ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0 && (!delta || delta_dtype == out_dtype)) {
    const bool bf = out_dtype == CO_BF16;
    if (bf && wdtype == CO_BF16) launch_rmsnorm_vec<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(resid, delta, rows, weight, eps, out, n_rows, H, update, stream);
    else if (bf) launch_rmsnorm_vec<__nv_bfloat16, __nv_bfloat16, float>(resid, delta, rows, weight, eps, out, n_rows, H, update, stream);
    else if (wdtype == CO_F32) launch_rmsnorm_vec<float, float, float>(resid, delta, rows, weight, eps, out, n_rows, H, update, stream);
    else launch_rmsnorm_vec<float, float, __nv_bfloat16>(resid, delta, rows, weight, eps, out, n_rows, H, update, stream);
    CO_CHECK_LAUNCH("add_rmsnorm");
    return 0;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define LAUNCH(TD, TO)                                                                              \
  co_launch(add_rmsnorm_kernel<TD, TO>, dim3(n_rows), dim3(threads), 0, stream, resid, (const TD*)delta, rows, \
            weight, wdtype, eps, (TO*)out, H, update)
  if (delta_dtype == CO_F32 && out_dtype == CO_F32) LAUNCH(float, float);
  else if (delta_dtype == CO_BF16 && out_dtype == CO_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == CO_F32 && out_dtype == CO_BF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == CO_BF16 && out_dtype == CO_F32) LAUNCH(__nv_bfloat16, float);
  else CO_FAIL("add_rmsnorm: unknown dtypes %d/%d", delta_dtype, out_dtype);
#undef LAUNCH
  CO_CHECK_LAUNCH("add_rmsnorm");
  return 0;
}

// The same with the delta given as a stack of float32 partial sums [splits][n][H] (a matrix
// product that split K over CTAs and left the addition to its consumer): the parts are added
// in order 0, 1, ... and then to the residual.  All of a thread's loads are independent.
template <typename TO, typename TW, int STEPS>
__global__ void __launch_bounds__(256)
add_parts_rmsnorm_vec_kernel(float* __restrict__ resid, const float* __restrict__ parts, int splits, size_t split_stride,
                             const int* __restrict__ rows, const TW* __restrict__ weight, float eps,
                             TO* __restrict__ out, int H, int update) {
  __shared__ float scratch[33];
  __shared__ float cl_slots[8];
  co_pdl_launch_dependents();
  // The CTAs of a cluster share a row: CTA k of n takes the k-th run of columns.
  const int cl_n = (int)co_cluster_size(), cl_r = (int)co_cluster_rank();
  const int c_per = ((H / 4 + cl_n - 1) / cl_n) * 4;
  const int c_lo = cl_r * c_per, c_hi = min(H, c_lo + c_per);
  float4 wv[STEPS];   // the weights depend on no earlier kernel
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    wv[i] = j < c_hi ? Vec4<TW>::load(weight + j) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  co_pdl_wait();
  const int r = blockIdx.x / cl_n;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  const float* d = parts + src * H;
  // Up to sixteen parts of every step are fetched before the first is added (the twelve heads of an
  // output projection, the twelve K slices of a down projection: one round trip); the additions
  // keep the order 0, 1, ...
  constexpr int ZB = STEPS == 1 ? 16 : 8;
  float4 v[STEPS], sum[STEPS];
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    v[i] = j < c_hi ? Vec4<float>::load(x + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int z0 = 0; z0 < splits; z0 += ZB) {
    float4 t[STEPS][ZB];
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      const int j = c_lo + (i * 256 + threadIdx.x) * 4;
#pragma unroll
      for (int u = 0; u < ZB; ++u)
        t[i][u] = (j < c_hi && z0 + u < splits) ? Vec4<float>::load(d + (size_t)(z0 + u) * split_stride + j)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int i = 0; i < STEPS; ++i)
#pragma unroll
      for (int u = 0; u < ZB; ++u) {
        sum[i].x += t[i][u].x; sum[i].y += t[i][u].y; sum[i].z += t[i][u].z; sum[i].w += t[i][u].w;
      }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    if (j < c_hi) {
      v[i].x += sum[i].x; v[i].y += sum[i].y; v[i].z += sum[i].z; v[i].w += sum[i].w;
      if (update) Vec4<float>::store(x + j, v[i]);
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = co_cluster_sum(co_block_sum(ss, scratch), cl_slots);
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    const int j = c_lo + (i * 256 + threadIdx.x) * 4;
    if (j < c_hi) {
      const float4 w = wv[i];
      Vec4<TO>::store(o + j, make_float4((v[i].x * scale) * w.x, (v[i].y * scale) * w.y, (v[i].z * scale) * w.z,
                                         (v[i].w * scale) * w.w));
    }
  }
}

template <typename TO>
__global__ void add_parts_rmsnorm_kernel(float* __restrict__ resid, const float* __restrict__ parts, int splits,
                                         size_t split_stride, const int* __restrict__ rows,
                                         const void* __restrict__ weight, int wdtype, float eps, TO* __restrict__ out,
                                         int H, int update) {
  __shared__ float scratch[33];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x;
  const size_t src = rows ? (size_t)rows[r] : (size_t)r;
  float* x = resid + src * H;
  const float* d = parts + src * H;
  auto value = [&](int j) {
    float sum = d[j];
    for (int z = 1; z < splits; ++z) sum += d[z * split_stride + j];
    return x[j] + sum;
  };
  float ss = 0.f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = value(j);
    ss += v * v;
  }
  ss = co_block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)H + eps);
  TO* o = out + (size_t)r * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    const float v = value(j);
    o[j] = co_from_float<TO>((v * scale) * co_load_any(weight, wdtype, j));
    if (update) x[j] = v;   // after the last read of x[j] by this thread, its only reader
  }
}

// parts: float32 [splits][n][H] with `split_stride` elements between splits (n = the rows of
// resid).  Otherwise as coheryn_add_rmsnorm.
CO_EXPORT int coheryn_add_parts_rmsnorm(float* resid, const float* parts, int splits, long split_stride,
                                        const int* rows, const void* weight, int wdtype, float eps, void* out,
                                        int out_dtype, int n_rows, int H, int update, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (splits < 1 || !parts) CO_FAIL("add_parts_rmsnorm: %d parts", splits);
  if (rows && update) CO_FAIL("add_parts_rmsnorm: cannot update the residual through a row gather");
  const bool bf = out_dtype == CO_BF16;
  if (!bf && out_dtype != CO_F32) CO_FAIL("add_parts_rmsnorm: unknown output dtype %d", out_dtype);
  if (H % 4 == 0 && H <= 8192 && (split_stride & 3) == 0 && ((uintptr_t)resid & 15) == 0 && ((uintptr_t)parts & 15) == 0 &&
      ((uintptr_t)weight & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    const int cl = norm_cluster(n_rows, H);
    const int steps = (H / 4 / cl + 255) / 256;
#define GO2(TO, TW, S) co_launch_cluster(cl, add_parts_rmsnorm_vec_kernel<TO, TW, S>, dim3(n_rows * cl), dim3(256), 0, stream, resid, parts, \
                                 splits, (size_t)split_stride, rows, (const TW*)weight, eps, (TO*)out, H, update)
#define GO(TO, TW) do { if (steps <= 1) GO2(TO, TW, 1); else if (steps <= 2) GO2(TO, TW, 2); else if (steps <= 4) GO2(TO, TW, 4); else GO2(TO, TW, 8); } while (0)
    if (bf && wdtype == CO_BF16) GO(__nv_bfloat16, __nv_bfloat16);
    else if (bf) GO(__nv_bfloat16, float);
    else if (wdtype == CO_F32) GO(float, float);
    else GO(float, __nv_bfloat16);
#undef GO
#undef GO2
    CO_CHECK_LAUNCH("add_parts_rmsnorm");
    return 0;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  if (bf) co_launch(add_parts_rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, stream, resid, parts, splits,
                    (size_t)split_stride, rows, weight, wdtype, eps, (__nv_bfloat16*)out, H, update);
  else co_launch(add_parts_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, stream, resid, parts, splits,
                 (size_t)split_stride, rows, weight, wdtype, eps, (float*)out, H, update);
  CO_CHECK_LAUNCH("add_parts_rmsnorm");
  return 0;
}

// ---------------------------------------------------------------------------------
// Gated activation over interleaved columns: out[m, j] = silu(in[m, 2j]) * in[m, 2j+1],
// in is [M, 2I] (column 2j = gate_j, column 2j+1 = up_j).
// silu(g) = g / (1 + exp(-g)) in float32.
// ---------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int I, size_t total) {
  co_pdl_launch_dependents();
  co_pdl_wait();
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
  if (dtype == CO_F32) co_launch(silu_mul_kernel<float>, dim3(blocks), dim3(threads), 0, stream, (const float*)in, (float*)out, I, total);
  else if (dtype == CO_BF16) co_launch(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, I, total);
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
  co_pdl_launch_dependents();
  co_pdl_wait();
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

// Vector variant: one block per token; an item is 16 bytes of a head's first half together
// with the matching 16 bytes of its second half (q and k heads), or 16 bytes of a v head.
// Needs rot == hd and hd/2 a multiple of the vector width.
template <typename T>
__global__ void __launch_bounds__(128)
rope_kv_write_vec_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const float2* __restrict__ cos_sin,
                         const int* __restrict__ slots, T* __restrict__ k_cache, T* __restrict__ v_cache, int nh,
                         int nkv, int hd, int page_size, int write_kv) {
  constexpr int VEC = 16 / sizeof(T);
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int t = blockIdx.x;
  const int half = hd >> 1, per_half = half / VEC, per_head = hd / VEC;
  T* row = qkv + (size_t)t * (nh + 2 * nkv) * hd;
  const int pos = positions[t];
  const float2* cs = cos_sin + (size_t)pos * half;
  const int slot = write_kv ? slots[t] : -1;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int rot_items = (nh + (write_kv ? nkv : 0)) * per_half;
  const int items = rot_items + (write_kv ? nkv * per_head : 0);
  for (int it = threadIdx.x; it < items; it += blockDim.x) {
    if (it < rot_items) {
      const int head = it / per_half, c = (it % per_half) * VEC;
      T* src = row + (size_t)head * hd;
      T a[VEC], b[VEC];
      *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(src + c);
      *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(src + half + c);
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float fa = co_to_float(a[i]), fb = co_to_float(b[i]);
        const float2 k = cs[c + i];
        a[i] = co_from_float<T>(fmaf(fa, k.x, -(fb * k.y)));
        b[i] = co_from_float<T>(fmaf(fa, k.y, fb * k.x));
      }
      T* dst = src;
      if (head >= nh) {
        if (slot < 0) continue;
        dst = k_cache + (((size_t)page * nkv + (head - nh)) * page_size + off) * hd;
      }
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(a);
      *reinterpret_cast<uint4*>(dst + half + c) = *reinterpret_cast<const uint4*>(b);
    } else {
      if (slot < 0) continue;
      const int j = it - rot_items;
      const int kvh = j / per_head, c = (j % per_head) * VEC;
      const T* src = row + (size_t)(nh + nkv + kvh) * hd;
      T* dst = v_cache + (((size_t)page * nkv + kvh) * page_size + off) * hd;
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
    }
  }
}

// The same for a q/k/v product whose K slices have not been added yet: value(t, col) = sum over
// the slices of parts[s][t][col] (in order, from zero) + bias[col], rounded to bfloat16 as the
// product's own output would be, then rotated; q goes to q_out [T, nh * hd], k and v to the cache.
__global__ void __launch_bounds__(32)
rope_kv_write_parts_kernel(const float* __restrict__ parts, int splits, size_t split_stride, const void* __restrict__ bias,
                           int bias_dtype, __nv_bfloat16* __restrict__ q_out, const int* __restrict__ positions,
                           const float2* __restrict__ cos_sin, const int* __restrict__ slots,
                           __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache, int nh, int nkv, int hd,
                           int page_size) {
  typedef __nv_bfloat16 T;
  constexpr int VEC = 8;
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int t = blockIdx.x;
  const int half = hd >> 1, per_half = half / VEC, per_head = hd / VEC;
  const size_t width = (size_t)(nh + 2 * nkv) * hd;
  const float* row = parts + (size_t)t * width;
  const int pos = positions[t];
  const float2* cs = cos_sin + (size_t)pos * half;
  const int slot = slots[t];
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  auto gather = [&](size_t col, float (&v)[VEC]) {      // eight columns from col, slices added in order, bias, rounding
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    for (int z = 0; z < splits; ++z) {
      const float4 a = *reinterpret_cast<const float4*>(row + (size_t)z * split_stride + col);
      const float4 b = *reinterpret_cast<const float4*>(row + (size_t)z * split_stride + col + 4);
      lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
      hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
    }
    v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (bias) v[i] += co_load_any(bias, bias_dtype, col + i);
      v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
    }
  };
  // One block per (token, head): heads 0 .. nh - 1 are queries, then the keys, then the values.
  const int head = blockIdx.y;
  if (head < nh + nkv) {
    for (int it = threadIdx.x; it < per_half; it += blockDim.x) {
      const int c = it * VEC;
      float fa[VEC], fb[VEC];
      gather((size_t)head * hd + c, fa);
      gather((size_t)head * hd + half + c, fb);
      T a[VEC], b[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float2 k = cs[c + i];
        a[i] = __float2bfloat16_rn(fmaf(fa[i], k.x, -(fb[i] * k.y)));
        b[i] = __float2bfloat16_rn(fmaf(fa[i], k.y, fb[i] * k.x));
      }
      T* dst;
      if (head < nh) dst = q_out + ((size_t)t * nh + head) * hd;
      else {
        if (slot < 0) continue;
        dst = k_cache + (((size_t)page * nkv + (head - nh)) * page_size + off) * hd;
      }
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(a);
      *reinterpret_cast<uint4*>(dst + half + c) = *reinterpret_cast<const uint4*>(b);
    }
  } else if (slot >= 0) {
    const int kvh = head - nh - nkv;
    for (int it = threadIdx.x; it < per_head; it += blockDim.x) {
      const int c = it * VEC;
      float fv[VEC];
      gather((size_t)head * hd + c, fv);
      T v[VEC];
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = __float2bfloat16_rn(fv[i]);
      T* dst = v_cache + (((size_t)page * nkv + kvh) * page_size + off) * hd;
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(v);
    }
  }
}

// parts: float32 [splits][T][(nh + 2 nkv) * hd]; the whole head is rotated (rotary size = hd, hd / 2 a
// multiple of 8); q_out: bfloat16 [T, nh * hd].
CO_EXPORT int coheryn_rope_kv_write_parts(const float* parts, int splits, long split_stride, const void* bias, int bias_dtype,
                                          void* q_out, const int* positions, const float* cos_sin, const int* slots,
                                          void* k_cache, void* v_cache, int T, int nh, int nkv, int hd, int page_size,
                                          cudaStream_t stream) {
  if (T <= 0) return 0;
  if (splits < 1 || (hd / 2) % 8 || (hd & 1)) CO_FAIL("rope_kv_write_parts: %d parts, head size %d", splits, hd);
  if (((uintptr_t)parts & 15) || (split_stride & 3) || ((uintptr_t)q_out & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    CO_FAIL("rope_kv_write_parts: operands must be 16-byte aligned");
  if (nh + 2 * nkv > 65535) CO_FAIL("rope_kv_write_parts: %d heads", nh + 2 * nkv);
  co_launch(rope_kv_write_parts_kernel, dim3(T, nh + 2 * nkv), dim3(32), 0, stream, parts, splits, (size_t)split_stride, bias, bias_dtype,
            (__nv_bfloat16*)q_out, positions, (const float2*)cos_sin, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh,
            nkv, hd, page_size);
  CO_CHECK_LAUNCH("rope_kv_write_parts");
  return 0;
}

CO_EXPORT int coheryn_rope_kv_write(void* qkv, int dtype, const int* positions, const float* cos_sin,
                                    const int* slots, void* k_cache, void* v_cache, int T, int nh, int nkv,
                                    int hd, int rot, int page_size, int write_kv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1)) CO_FAIL("rope_kv_write: rotary size %d does not fit head size %d", rot, hd);
  const int vec = dtype == CO_F32 ? 4 : 8;
  if (rot == hd && (hd / 2) % vec == 0 && ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 &&
      ((uintptr_t)v_cache & 15) == 0) {
    if (dtype == CO_F32)
      co_launch(rope_kv_write_vec_kernel<float>, dim3(T), dim3(128), 0, stream, (float*)qkv, positions,
                (const float2*)cos_sin, slots, (float*)k_cache, (float*)v_cache, nh, nkv, hd, page_size, write_kv);
    else if (dtype == CO_BF16)
      co_launch(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(T), dim3(128), 0, stream, (__nv_bfloat16*)qkv, positions,
                (const float2*)cos_sin, slots, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, hd, page_size,
                write_kv);
    else CO_FAIL("rope_kv_write: unknown dtype %d", dtype);
    CO_CHECK_LAUNCH("rope_kv_write");
    return 0;
  }
  dim3 grid(T, nh + 2 * nkv);
  const int threads = hd >= 128 ? 64 : 32;
  if (dtype == CO_F32)
    co_launch(rope_kv_write_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, positions, (const float2*)cos_sin, slots,
              (float*)k_cache, (float*)v_cache, nh, nkv, hd, rot, page_size, write_kv);
  else if (dtype == CO_BF16)
    co_launch(rope_kv_write_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (__nv_bfloat16*)qkv, positions, (const float2*)cos_sin, slots,
              (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nh, nkv, hd, rot, page_size, write_kv);
  else CO_FAIL("rope_kv_write: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("rope_kv_write");
  return 0;
}
