// out[M, N] = x[M, K] . W[N, K]^T (+ bias[N]) with float32 FMA accumulation on the CUDA
// cores: the matrix product of the true 32-bit path (no reduced-precision tensor mode),
// and the slow, any-shape reference for the bfloat16 tensor-core kernels.
//
// Each output element is accumulated over k = 0..K-1 in ascending order by one thread,
// whatever M is, so a row's result does not depend on the other rows of the batch.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TX, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const void* __restrict__ bias,
                 int bias_dtype, TO* __restrict__ out, int M, int N, int K, long ldx, long ldo) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * TM, tn = (tid % 16) * TN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 x 16 elements per operand tile, 256 threads: 4 elements each.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, c = idx % BK;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? co_to_float(x[(size_t)gm * ldx + gk]) : 0.f;
      ws[c][r] = (gn < N && gk < K) ? co_to_float(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += co_load_any(bias, bias_dtype, gn);
      out[(size_t)gm * ldo + gn] = co_from_float<TO>(v);
    }
  }
}
}  // namespace

// x: [M, K] with row stride ldx; w: [N, K] contiguous; out: [M, N] with row stride ldo.
CO_EXPORT int coheryn_gemm_simt(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias,
                                int bias_dtype, void* out, int out_dtype, int M, int N, int K, long ldx,
                                long ldo, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) CO_FAIL("gemm_simt: K must be positive");
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
#define LAUNCH(TX, TW, TO)                                                                       \
  gemm_simt_kernel<TX, TW, TO><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, bias, bias_dtype, \
                                                         (TO*)out, M, N, K, ldx, ldo)
  if (x_dtype == CO_F32 && w_dtype == CO_F32 && out_dtype == CO_F32) LAUNCH(float, float, float);
  else if (x_dtype == CO_BF16 && w_dtype == CO_BF16 && out_dtype == CO_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == CO_BF16 && w_dtype == CO_BF16 && out_dtype == CO_F32) LAUNCH(__nv_bfloat16, __nv_bfloat16, float);
  else CO_FAIL("gemm_simt: unsupported dtypes x=%d w=%d out=%d", x_dtype, w_dtype, out_dtype);
#undef LAUNCH
  CO_CHECK_LAUNCH("gemm_simt");
  return 0;
}
