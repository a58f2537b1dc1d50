// out[M, N] = x[M, K] . W[N, K]^T (+ bias) for few rows (M <= 64), bfloat16 operands,
// float32 accumulation on the tensor cores (mma.sync m16n8k16).  This is the matrix
// product of decode steps: it is bound by reading W once from HBM, so the kernel is
// shaped around the weight stream, not around the arithmetic.
//
// A CTA owns NT*8 consecutive rows of W (output features) for ALL tokens; its warps
// split K in interleaved blocks of 64 (warp w takes blocks w, w+W, ...).  In a block a
// thread fetches 32 contiguous bytes of a W row with streaming loads, so the four
// threads that share a row cover one 128-byte line.  Tokens sit on the M axis of the MMA
// (tiles of 16, zero padded), features on the N axis (tiles of 8).  The k order inside a
// block is permuted identically for both operands so that a thread's 16 bytes feed two
// MMAs without a shuffle.  Per-warp partial sums are combined through shared memory in
// warp order.  An output element is therefore always summed in the same order, whatever
// M is: a row's result does not depend on the batch around it.
//
// The first batch of weight loads is issued BEFORE the kernel waits for its predecessor
// in the stream (programmatic dependent launch): weights depend on nothing, so the stream
// of the next matrix starts while the previous kernel drains.
//
// Epilogues: bias; or gated SiLU over interleaved rows (row 2j = gate_j, row 2j+1 = up_j:
// out[m, j] = silu(acc[2j]) * acc[2j+1]), which keeps a gate/up pair in one thread.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int EPI_GATED_SILU = 1;

template <int MT, int NT>
__global__ void __launch_bounds__(512)
gemm_small_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                  const void* __restrict__ bias, int bias_dtype, void* __restrict__ out, int out_dtype,
                  int M, int N, int K, long ldx, long ldo, int epilogue) {
  extern __shared__ float red[];  // [warps][MT][NT][4][32]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_base = blockIdx.x * NT * 8;

  const __nv_bfloat16* wrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) wrow[nt] = w + (size_t)min(n_base + nt * 8 + g, N - 1) * K;

  // Blocks of 64 k are taken in batches of U: all loads of a batch are issued before its
  // first MMA, so that a warp keeps U * NT * 1 KB of the weight stream in flight.
  constexpr int U = (MT * NT >= 8) ? 1 : ((MT * NT >= 4) ? 2 : 4);
  const int nblk = (K + 63) >> 6;
  uint4 wv[U][NT][2];
  auto load_w = [&](int blk0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((blk0 + u * warps) << 6) + (t << 4);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int p = 0; p < 2; ++p)   // K is a multiple of 8: a 16-byte piece is whole or absent
          wv[u][nt][p] = (k + 8 * p < K) ? ld_stream(wrow[nt] + k + 8 * p) : make_uint4(0, 0, 0, 0);
    }
  };
  load_w(warp);                  // weights depend on no earlier kernel
  co_pdl_launch_dependents();
  co_pdl_wait();                 // x is the predecessor's output

  const __nv_bfloat16* xrow[MT][2];
  bool xok[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = mt * 16 + h * 8 + g;
      xok[mt][h] = m < M;
      xrow[mt][h] = x + (size_t)min(m, M - 1) * ldx;
    }
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[mt][nt][i] = 0.f;

  for (int blk0 = warp; blk0 < nblk; blk0 += warps * U) {
    if (blk0 != warp) load_w(blk0);
    uint4 xa[U][MT][2], xb[U][MT][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((blk0 + u * warps) << 6) + (t << 4);
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const bool valid = k + 8 * p < K;
          xa[u][mt][p] = (valid && xok[mt][0]) ? __ldg((const uint4*)(xrow[mt][0] + k + 8 * p)) : make_uint4(0, 0, 0, 0);
          xb[u][mt][p] = (valid && xok[mt][1]) ? __ldg((const uint4*)(xrow[mt][1] + k + 8 * p)) : make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int p = 0; p < 2; ++p)
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 a = xa[u][mt][p], b = xb[u][mt][p], c = wv[u][nt][p];
            mma_bf16(acc[mt][nt], a.x, b.x, a.y, b.y, c.x, c.y);
            mma_bf16(acc[mt][nt], a.z, b.z, a.w, b.w, c.z, c.w);
          }
  }

  // Partial sums of every warp, laid out so that lanes write consecutive words.
  constexpr int E = MT * NT * 4 * 32;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp * E + ((mt * NT + nt) * 4 + i) * 32 + lane] = acc[mt][nt][i];
  __syncthreads();

  // One thread per pair of neighbouring features (i = 0,1 or 2,3 of a fragment).
  constexpr int PAIRS = MT * NT * 2 * 32;
  for (int e = threadIdx.x; e < PAIRS; e += blockDim.x) {
    const int l = e & 31, half = (e >> 5) & 1, tile = e >> 6;
    const int nt = tile % NT, mt = tile / NT;
    const int m = mt * 16 + half * 8 + (l >> 2);
    const int n = n_base + nt * 8 + (l & 3) * 2;
    if (m >= M || n >= N) continue;
    const int base = ((mt * NT + nt) * 4 + half * 2) * 32 + l;
    float v0 = 0.f, v1 = 0.f;
    for (int wi = 0; wi < warps; ++wi) {
      v0 += red[wi * E + base];
      v1 += red[wi * E + base + 32];
    }
    if (epilogue == EPI_GATED_SILU) {
      // rows (n, n+1) = (gate_j, up_j), j = n / 2
      const float r = (v0 / (1.0f + __expf(-v0))) * v1;
      const size_t o = (size_t)m * ldo + (n >> 1);
      if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(r);
      else ((float*)out)[o] = r;
      continue;
    }
    const bool has1 = n + 1 < N;
    if (bias) {
      v0 += co_load_any(bias, bias_dtype, n);
      if (has1) v1 += co_load_any(bias, bias_dtype, n + 1);
    }
    const size_t o = (size_t)m * ldo + n;
    if (out_dtype == CO_BF16) {
      __nv_bfloat16* p = (__nv_bfloat16*)out + o;
      if (has1 && ((o & 1) == 0)) *(__nv_bfloat162*)p = __floats2bfloat162_rn(v0, v1);
      else { p[0] = __float2bfloat16_rn(v0); if (has1) p[1] = __float2bfloat16_rn(v1); }
    } else {
      float* p = (float*)out + o;
      p[0] = v0;
      if (has1) p[1] = v1;
    }
  }
}

// The q/k/v product of a decode batch (at most 16 rows) with the rotation and the cache write
// in its epilogue, which saves the kernel that would otherwise re-read q/k/v.  A CTA owns 8
// features of a head's first half and the 8 that pair with them in the second half (two MMA
// tiles), so that both elements of every rotate-half pair meet in one thread:
//   q heads: rotated, to q_out[m, head * hd + ...];  k heads: rotated, to the cache slot of
//   token m;  v heads: as they are, to the cache.
// The sums (+ bias) are rounded to bfloat16 BEFORE the rotation, as the two-kernel path stores
// them, so both paths give the same bits.  Rotation in float32 from the (cos, sin) table:
// out_a = fma(a, cos, -(b sin)), out_b = fma(a, sin, b cos).
__global__ void __launch_bounds__(512)
gemm_small_rope_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const void* __restrict__ bias, int bias_dtype, __nv_bfloat16* __restrict__ q_out, long ldq,
                       const int* __restrict__ positions, const float2* __restrict__ cos_sin,
                       const int* __restrict__ slots, __nv_bfloat16* __restrict__ k_cache,
                       __nv_bfloat16* __restrict__ v_cache, int M, int K, long ldx, int nh, int nkv, int hd,
                       int page_size) {
  extern __shared__ float red[];  // [warps][2 tiles][4][32]
  constexpr int NT = 2, U = 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int blocks_per_head = hd >> 4, half = hd >> 1;
  const int head = blockIdx.x / blocks_per_head, jb = blockIdx.x % blocks_per_head;
  const int row0 = head * hd + jb * 8, row1 = row0 + half;
  const __nv_bfloat16* wrow[NT] = {w + (size_t)(row0 + g) * K, w + (size_t)(row1 + g) * K};
  const int nblk = (K + 63) >> 6;
  uint4 wv[U][NT][2];
  auto load_w = [&](int blk0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((blk0 + u * warps) << 6) + (t << 4);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int p = 0; p < 2; ++p)
          wv[u][nt][p] = (k + 8 * p < K) ? ld_stream(wrow[nt] + k + 8 * p) : make_uint4(0, 0, 0, 0);
    }
  };
  load_w(warp);                  // weights depend on no earlier kernel
  co_pdl_launch_dependents();
  co_pdl_wait();                 // x is the predecessor's output

  const bool xok0 = g < M, xok1 = g + 8 < M;
  const __nv_bfloat16* xr0 = x + (size_t)min(g, M - 1) * ldx;
  const __nv_bfloat16* xr1 = x + (size_t)min(g + 8, M - 1) * ldx;
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;
  for (int blk0 = warp; blk0 < nblk; blk0 += warps * U) {
    if (blk0 != warp) load_w(blk0);
    uint4 xa[U][2], xb[U][2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = ((blk0 + u * warps) << 6) + (t << 4);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const bool valid = k + 8 * p < K;
        xa[u][p] = (valid && xok0) ? __ldg((const uint4*)(xr0 + k + 8 * p)) : make_uint4(0, 0, 0, 0);
        xb[u][p] = (valid && xok1) ? __ldg((const uint4*)(xr1 + k + 8 * p)) : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int p = 0; p < 2; ++p)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4 a = xa[u][p], b = xb[u][p], c = wv[u][nt][p];
          mma_bf16(acc[nt], a.x, b.x, a.y, b.y, c.x, c.y);
          mma_bf16(acc[nt], a.z, b.z, a.w, b.w, c.z, c.w);
        }
  }
  constexpr int E = NT * 4 * 32;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp * E + (nt * 4 + i) * 32 + lane] = acc[nt][i];
  __syncthreads();

  // One thread per (token m, pair j of this CTA's eight): fragment element (row m, column j) of
  // tile nt sits in lane (m % 8) * 4 + j / 2, register (m / 8) * 2 + (j & 1).
  for (int e = threadIdx.x; e < M * 8; e += blockDim.x) {
    const int m = e >> 3, j = e & 7;
    const int src = ((m >> 3) * 2 + (j & 1)) * 32 + (m & 7) * 4 + (j >> 1);
    float a = 0.f, b = 0.f;
    for (int wi = 0; wi < warps; ++wi) {
      a += red[wi * E + src];
      b += red[wi * E + 4 * 32 + src];
    }
    if (bias) {
      a += co_load_any(bias, bias_dtype, row0 + j);
      b += co_load_any(bias, bias_dtype, row1 + j);
    }
    a = __bfloat162float(__float2bfloat16_rn(a));
    b = __bfloat162float(__float2bfloat16_rn(b));
    const int d = jb * 8 + j;
    __nv_bfloat16 ra, rb;
    if (head < nh + nkv) {
      const float2 c = cos_sin[(size_t)positions[m] * half + d];
      ra = __float2bfloat16_rn(fmaf(a, c.x, -(b * c.y)));
      rb = __float2bfloat16_rn(fmaf(a, c.y, b * c.x));
    } else {
      ra = __float2bfloat16_rn(a);
      rb = __float2bfloat16_rn(b);
    }
    __nv_bfloat16* dst;
    if (head < nh) {
      dst = q_out + (size_t)m * ldq + (size_t)head * hd;
    } else {
      const int slot = slots[m];
      if (slot < 0) continue;
      const int page = slot / page_size, off = slot - page * page_size;
      const int kvh = head < nh + nkv ? head - nh : head - nh - nkv;
      dst = (head < nh + nkv ? k_cache : v_cache) + (((size_t)page * nkv + kvh) * page_size + off) * hd;
    }
    dst[d] = ra;
    dst[d + half] = rb;
  }
}

template <int MT, int NT>
int launch_small(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                 int M, int N, int K, long ldx, long ldo, int epilogue, int warps, cudaStream_t stream) {
  const size_t smem = (size_t)warps * MT * NT * 4 * 32 * sizeof(float);
  auto kernel = gemm_small_kernel<MT, NT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) CO_FAIL("gemm_small: shared memory %zu: %s", smem, cudaGetErrorString(e));
  }
  const int grid = (N + NT * 8 - 1) / (NT * 8);
  cudaError_t e = co_launch_ex(true /* x is re-read through L1 */, kernel, dim3(grid), dim3(warps * 32), smem, stream, (const __nv_bfloat16*)x,
                            (const __nv_bfloat16*)w, bias, bias_dtype, out, out_dtype, M, N, K, ldx, ldo, epilogue);
  if (e != cudaSuccess) CO_FAIL("gemm_small: launch failed: %s", cudaGetErrorString(e));
  CO_CHECK_LAUNCH("gemm_small");
  return 0;
}
}  // namespace

// x: [M, K] bfloat16, row stride ldx (elements, a multiple of 8, base 16-byte aligned);
// w: [N, K] bfloat16 contiguous; K a multiple of 8; M <= 64.
// epilogue 0: out[M, N] (+ bias); 1: gated SiLU over interleaved rows, out[M, N/2].
CO_EXPORT int coheryn_gemm_bf16_small(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                                      int out_dtype, int M, int N, int K, long ldx, long ldo, int epilogue,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64) CO_FAIL("gemm_bf16_small: M = %d exceeds 64", M);
  if (K <= 0 || (K & 7) || (ldx & 7)) CO_FAIL("gemm_bf16_small: K = %d and the row stride %ld must be multiples of 8", K, ldx);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("gemm_bf16_small: operands must be 16-byte aligned");
  if (epilogue == 1 && (N & 1)) CO_FAIL("gemm_bf16_small: gated epilogue needs an even number of rows");
  if (epilogue != 0 && epilogue != 1) CO_FAIL("gemm_bf16_small: unknown epilogue %d", epilogue);
  // Rows per CTA: as many as keep at least ~2 CTAs per SM (148 SMs); more rows per CTA
  // mean fewer re-reads of x through L2.  The warps of a CTA split K (a function of K
  // alone, so the order of summation never depends on M or N).
  const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
  int nt = 8 / mt;  // MT * NT <= 8 bounds registers and the reduction buffer
  while (nt > 1 && (N + nt * 8 - 1) / (nt * 8) < 296) nt >>= 1;
  const int nblk = (K + 63) / 64;
  const int warps = nblk >= 64 ? 16 : (nblk >= 8 ? 8 : (nblk >= 4 ? 4 : (nblk >= 2 ? 2 : 1)));
#define GO(MT_, NT_) return launch_small<MT_, NT_>(x, w, bias, bias_dtype, out, out_dtype, M, N, K, ldx, ldo, epilogue, warps, stream)
  if (mt == 1) { if (nt == 8) GO(1, 8); if (nt == 4) GO(1, 4); if (nt == 2) GO(1, 2); GO(1, 1); }
  if (mt == 2) { if (nt == 4) GO(2, 4); if (nt == 2) GO(2, 2); GO(2, 1); }
  if (nt == 2) GO(4, 2);
  GO(4, 1);
#undef GO
}

// x: [M, K] bfloat16 rows of stride ldx, M <= 16; w: [(nh + 2 nkv) * hd, K] (q, k, v rows
// stacked); q_out: [M, nh * hd] rows of stride ldq; caches [page][kv head][slot][hd]; positions
// and slots per row (slot < 0: nothing is written for that row); cos_sin: float2
// [max_pos][hd / 2].  The whole head is rotated; hd a multiple of 16, K of 8.
CO_EXPORT int coheryn_qkv_rope_bf16_small(const void* x, const void* w, const void* bias, int bias_dtype, void* q_out,
                                          long ldq, const int* positions, const float* cos_sin, const int* slots,
                                          void* k_cache, void* v_cache, int M, int K, long ldx, int nh, int nkv,
                                          int hd, int page_size, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (M > 16) CO_FAIL("qkv_rope_bf16_small: M = %d exceeds 16", M);
  if (K <= 0 || (K & 7) || (ldx & 7)) CO_FAIL("qkv_rope_bf16_small: K = %d and the row stride %ld must be multiples of 8", K, ldx);
  if (hd <= 0 || (hd & 15) || nh <= 0 || nkv <= 0 || page_size <= 0)
    CO_FAIL("qkv_rope_bf16_small: head size %d must be a multiple of 16 (heads %d, kv heads %d, page %d)", hd, nh, nkv, page_size);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("qkv_rope_bf16_small: operands must be 16-byte aligned");
  const int nblk = (K + 63) / 64;
  const int warps = nblk >= 64 ? 16 : (nblk >= 8 ? 8 : (nblk >= 4 ? 4 : (nblk >= 2 ? 2 : 1)));
  const size_t smem = (size_t)warps * 2 * 4 * 32 * sizeof(float);
  const int grid = (nh + 2 * nkv) * (hd / 16);
  cudaError_t e = co_launch_ex(true /* x is re-read through L1 */, gemm_small_rope_kernel, dim3(grid), dim3(warps * 32), smem,
                               stream, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, bias, bias_dtype,
                               (__nv_bfloat16*)q_out, ldq, positions, (const float2*)cos_sin, slots,
                               (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, M, K, ldx, nh, nkv, hd, page_size);
  if (e != cudaSuccess) CO_FAIL("qkv_rope_bf16_small: launch failed: %s", cudaGetErrorString(e));
  CO_CHECK_LAUNCH("qkv_rope_small");
  return 0;
}
