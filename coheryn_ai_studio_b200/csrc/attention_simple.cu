// Causal (optionally windowed) grouped-query attention over cache pages, written for
// clarity: one block per (token, query head), float32 arithmetic throughout.  It is
// the attention of the true 32-bit path and the any-shape reference of the bfloat16
// tensor-core kernels.
//
// For token t of request r at position p the keys are positions first..p of r's cache,
// first = max(0, p - window + 1) with a window, else 0; the cache already holds the
// keys that this step wrote.  Four warps each run an online softmax over the keys
// k = first + warp, first + warp + 4, ...; their (max, sum, accumulator) triples are
// merged in warp order.  The result therefore depends only on (p, first), never on
// how the step was cut or batched.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_PER_LANE = 8;  // head sizes up to 256

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simple_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ block_tables, int max_blocks,
                        const int* __restrict__ token_req, const int* __restrict__ positions, int nh,
                        int nkv, int hd, int page_size, int window, float scale) {
  extern __shared__ float smem[];
  float* qs = smem;                         // [hd]
  float* merge_acc = smem + hd;             // [WARPS][hd]
  __shared__ float merge_m[WARPS], merge_l[WARPS];

  const int t = blockIdx.x, h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int req = token_req[t];
  const int pos = positions[t];
  const int first = window > 0 ? max(0, pos - window + 1) : 0;
  const int kvh = h / (nh / nkv);
  const int* table = block_tables + (size_t)req * max_blocks;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = co_to_float(qrow[d]);
  __syncthreads();

  float m = -INFINITY, l = 0.f;
  float acc[MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) acc[i] = 0.f;

  for (int kp = first + warp; kp <= pos; kp += WARPS) {
    const int page = table[kp / page_size];
    const size_t base = (((size_t)page * nkv + kvh) * page_size + (kp % page_size)) * hd;
    const T* kr = k_cache + base;
    const T* vr = v_cache + base;
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) dot = fmaf(qs[d], co_to_float(kr[d]), dot);
    }
    dot = co_warp_sum(dot);
    const float s = dot * scale;
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first key
    const float p = expf(s - m_new);
    l = l * corr + p;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) acc[i] = acc[i] * corr + p * co_to_float(vr[d]);
    }
    m = m_new;
  }
  if (lane == 0) { merge_m[warp] = m; merge_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < MAX_PER_LANE; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) merge_acc[warp * hd + d] = acc[i];
  }
  __syncthreads();
  float M = -INFINITY;
#pragma unroll
  for (int w = 0; w < WARPS; ++w) M = fmaxf(M, merge_m[w]);
  float L = 0.f;
  float f[WARPS];
#pragma unroll
  for (int w = 0; w < WARPS; ++w) {
    f[w] = merge_m[w] == -INFINITY ? 0.f : expf(merge_m[w] - M);
    L += merge_l[w] * f[w];
  }
  const float inv = 1.0f / L;
  T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) o += merge_acc[w * hd + d] * f[w];
    orow[d] = co_from_float<T>(o * inv);
  }
}
}  // namespace

CO_EXPORT int coheryn_attention_simple(const void* q, long q_stride, void* out, long out_stride,
                                       const void* k_cache, const void* v_cache, int dtype,
                                       const int* block_tables, int max_blocks, const int* token_req,
                                       const int* positions, int T, int nh, int nkv, int hd, int page_size,
                                       int window, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hd > 32 * MAX_PER_LANE) CO_FAIL("attention_simple: head size %d exceeds %d", hd, 32 * MAX_PER_LANE);
  if (nkv <= 0 || nh % nkv != 0) CO_FAIL("attention_simple: %d heads do not group over %d kv heads", nh, nkv);
  dim3 grid(T, nh);
  const size_t smem = (size_t)(1 + WARPS) * hd * sizeof(float);
  if (dtype == CO_F32)
    attention_simple_kernel<float><<<grid, WARPS * 32, smem, stream>>>(
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_cache, (const float*)v_cache,
        block_tables, max_blocks, token_req, positions, nh, nkv, hd, page_size, window, scale);
  else if (dtype == CO_BF16)
    attention_simple_kernel<__nv_bfloat16><<<grid, WARPS * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_cache,
        (const __nv_bfloat16*)v_cache, block_tables, max_blocks, token_req, positions, nh, nkv, hd,
        page_size, window, scale);
  else CO_FAIL("attention_simple: unknown dtype %d", dtype);
  CO_CHECK_LAUNCH("attention_simple");
  return 0;
}
