// out[M, N] = x[M, K] . W[N, K]^T (+ bias | gated SiLU) for FEW rows (decode batches, short
// prompt portions: M <= 256) in bfloat16 on the 5th-generation tensor cores.  The product is
// bound by reading W once, so the operands swap places: the OUTPUT FEATURES sit on the 128
// lanes of the accumulator in tensor memory (W tile 128 x 64 = operand A) and the tokens on
// its BT columns (x tile BT x 64 = operand B, BT = 16, 32, 64, 128 or 256).  No lane is wasted on
// padding rows, and the weight stream is moved by TMA alone: 16 KB per copy, STAGES copies
// in flight per CTA, no thread computes an address.
//
// One CTA owns a tile of 128 features and, where the tiles are too few to occupy the GPU, a
// slice of K (grid.y splits; a function of N and K only, so a row's sum never depends on the
// batch).  Warp roles as in the kernel for many rows: warp 0 producer, warp 1 MMA issuer,
// warps 2-5 epilogue (thread = feature, registers = tokens; a warp stores 32 consecutive
// features of a token).  With splits every CTA leaves its float32 tile in a workspace and
// bumps the tile's counter; the CTA that arrives last adds the splits IN ORDER 0, 1, ... and
// runs the epilogue, then resets the counter.  The counters must be zero before the first call.
//
// The W tiles of the first STAGES steps are requested BEFORE the kernel waits for its
// predecessor in the stream (programmatic dependent launch): weights depend on nothing.
// Every wait is bounded: on expiry the kernel records an error code and winds down.
#include "tc_common.cuh"

namespace {

constexpr int BF = 128;          // features per tile = TMEM lanes
constexpr int EPI_GATED_SILU = 1;

template <int BT, int STAGES>
struct SmemFew {
  static constexpr int W_BYTES = BF * BK * 2;
  static constexpr int X_BYTES = BT * BK * 2;
  static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers, flags */;
};

template <int BT, int STAGES>
__global__ void __launch_bounds__(192)
gemm_tc_few_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const void* __restrict__ bias, int bias_dtype, void* __restrict__ out, int out_dtype, int M, int N,
                   int K, long ldo, int epilogue, int* __restrict__ status, float* __restrict__ partial,
                   int* __restrict__ counters, int k_per_split, int defer) {
  using S = SmemFew<BT, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = (unsigned long long*)(tiles + STAGES * S::STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* accum_full = empty + STAGES;
  unsigned* tmem_slot = (unsigned*)(accum_full + 1);
  int* last_flag = (int*)(tmem_slot + 1);
  static_assert(2 * STAGES * 8 + 8 + 8 <= 256, "barriers fit their slot");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BF;
  const int splits = gridDim.y;
  const int kt_begin = blockIdx.y * k_per_split;
  const int k_tiles = min(k_per_split, (K + BK - 1) / BK - kt_begin);
  constexpr int TMEM_COLS = BT < 32 ? 32 : BT;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  co_pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // The first steps' weights do not wait for the predecessor; their x tiles do.
      const int head = k_tiles < STAGES ? k_tiles : STAGES;
      for (int kt = 0; kt < head; ++kt) {
        mbar_expect_tx(&full[kt], S::STAGE_BYTES);
        tma_load_2d(tiles + kt * S::STAGE_BYTES, &map_w, (kt_begin + kt) * BK, n0, &full[kt]);
      }
      co_pdl_wait();
      for (int kt = 0; kt < head; ++kt)
        tma_load_2d(tiles + kt * S::STAGE_BYTES + S::W_BYTES, &map_x, (kt_begin + kt) * BK, 0, &full[kt]);
      for (int kt = head; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(&empty[s], ((kt / STAGES) - 1) & 1)) { atomicExch(status, 11); break; }
        unsigned char* a = tiles + s * S::STAGE_BYTES;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        tma_load_2d(a, &map_w, (kt_begin + kt) * BK, n0, &full[s]);
        tma_load_2d(a + S::W_BYTES, &map_x, (kt_begin + kt) * BK, 0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = umma_idesc(BF, BT);
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(&full[s], (kt / STAGES) & 1)) { atomicExch(status, 12); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char* a = tiles + s * S::STAGE_BYTES;
        const unsigned long long da = umma_desc(a), db = umma_desc(a + S::W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
        umma_commit(&empty[s]);
      }
      umma_commit(accum_full);
    }
  } else {
    // Epilogue warps 2..5: TMEM lane quarter = warp % 4; this thread's feature:
    const int quarter = warp & 3;
    const int f = quarter * 32 + lane, n = n0 + f;
    co_pdl_wait();   // out and the workspace may still be read by the predecessor
    const bool waited = mbar_wait(accum_full, 0);
    if (!waited && lane == 0) atomicExch(status, 13);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if constexpr (BT > 64) {
      // Many token columns: sixteen at a time from tensor memory straight to their destination.  K
      // slices are always left to the consumer here (the host refuses anything else).
      const int n_out = N >> 1;
      const float bv = (n < N && bias && (splits == 1 || blockIdx.y == 0)) ? co_load_any(bias, bias_dtype, n) : 0.f;
      float* mine = (float*)out + (size_t)blockIdx.y * M * N + n;
      for (int c0 = 0; c0 < BT && c0 < M && waited; c0 += 16) {
        unsigned r[16];
        tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
        if (splits > 1) {
          if (n < N)
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < M) mine[(size_t)(c0 + j) * N] = __uint_as_float(r[j]) + bv;
        } else if (epilogue == EPI_GATED_SILU) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(r[j]);
            const float other = __shfl_xor_sync(0xffffffffu, g, 1);
            if (c0 + j < M && !(lane & 1) && n + 1 < N && (n >> 1) < n_out) {
              const float y = __fdividef(g, 1.0f + __expf(-g)) * other;
              const size_t o = (size_t)(c0 + j) * ldo + (n >> 1);
              if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(y);
              else ((float*)out)[o] = y;
            }
          }
        } else if (n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < M) {
              const size_t o = (size_t)(c0 + j) * ldo + n;
              if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(__uint_as_float(r[j]) + bv);
              else ((float*)out)[o] = __uint_as_float(r[j]) + bv;
            }
        }
      }
    } else {
    float v[BT];
    if (waited) {
#pragma unroll
      for (int c0 = 0; c0 < BT; c0 += 16) {
        unsigned r[16];
        tmem_ld16(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[c0 + j] = __uint_as_float(r[j]);
      }
    }
    bool finish = waited;
    if (splits > 1 && defer) {
      // The consumer adds the splits: out is float32 [splits][M][N]; the bias rides in split 0.
      finish = false;
      if (waited && n < N) {
        const float bv = (bias && blockIdx.y == 0) ? co_load_any(bias, bias_dtype, n) : 0.f;
        float* mine = (float*)out + (size_t)blockIdx.y * M * N + n;
#pragma unroll
        for (int j = 0; j < BT; ++j)
          if (j < M) mine[(size_t)j * N] = v[j] + bv;
      }
    } else if (splits > 1) {
      // partial[tile][split][token][feature]: a warp writes 32 consecutive floats per token.
      float* mine = partial + (((size_t)blockIdx.x * splits + blockIdx.y) * BT) * BF + f;
      if (waited) {
#pragma unroll
        for (int j = 0; j < BT; ++j)
          if (j < M) __stcg(mine + (size_t)j * BF, v[j]);
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (threadIdx.x == 64) *last_flag = atomicAdd(&counters[blockIdx.x], 1) == splits - 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      finish = *last_flag != 0;
      if (finish) {
        __threadfence();
        const float* all = partial + ((size_t)blockIdx.x * splits * BT) * BF + f;
#pragma unroll
        for (int j = 0; j < BT; ++j) v[j] = 0.f;
        // Four splits' loads are in flight at once; the additions keep the order 0, 1, 2, ...
        for (int z0 = 0; z0 < splits; z0 += 4) {
          float t[4][BT];
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < BT; ++j)
              t[u][j] = (z0 + u < splits && j < M) ? __ldcg(all + ((size_t)(z0 + u) * BT + j) * BF) : 0.f;
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < BT; ++j) v[j] += t[u][j];
        }
        if (threadIdx.x == 64) counters[blockIdx.x] = 0;   // ready for the next product
      }
    }
    if (finish) {
      if (epilogue == EPI_GATED_SILU) {
        // features (2i, 2i+1) = (gate_i, up_i) sit in neighbouring lanes
        const int n_out = N >> 1;
#pragma unroll
        for (int j = 0; j < BT; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          if (j < M && !(lane & 1) && n + 1 < N) {
            const float r = __fdividef(v[j], 1.0f + __expf(-v[j])) * other;
            const size_t o = (size_t)j * ldo + (n >> 1);
            if ((n >> 1) < n_out) {
              if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(r);
              else ((float*)out)[o] = r;
            }
          }
        }
      } else if (n < N) {
        const float bv = bias ? co_load_any(bias, bias_dtype, n) : 0.f;
#pragma unroll
        for (int j = 0; j < BT; ++j) {
          if (j >= M) break;
          const size_t o = (size_t)j * ldo + n;
          if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v[j] + bv);
          else ((float*)out)[o] = v[j] + bv;
        }
      }
    }
    }   // BT <= 64
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

// K splits of a product with few feature tiles: about one CTA per SM, at least two k-steps each.
// A function of N and K alone.
int few_splits(int N, int K) {
  const int tiles = (N + BF - 1) / BF;
  const int k_tiles = (K + BK - 1) / BK;
  if (tiles >= 100 || k_tiles < 4) return 1;
  int s = (148 + tiles / 2) / tiles;
  if (s > k_tiles / 2) s = k_tiles / 2;
  if (s < 2) return 1;
  const int per = (k_tiles + s - 1) / s;
  return (k_tiles + per - 1) / per;    // no split is left empty
}

template <int BT, int STAGES>
int launch_few(const CUtensorMap& mw, const CUtensorMap& mx, const void* bias, int bias_dtype, void* out, int out_dtype,
               int M, int N, int K, long ldo, int epilogue, int* status, float* workspace, int splits, int defer,
               cudaStream_t stream) {
  auto kernel = gemm_tc_few_kernel<BT, STAGES>;
  constexpr int smem = SmemFew<BT, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) CO_FAIL("gemm_tc_few: %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int tiles = (N + BF - 1) / BF;
  const int k_tiles = (K + BK - 1) / BK;
  const int k_per_split = (k_tiles + splits - 1) / splits;
  // Workspace: one counter per tile (padded to a multiple of 64 ints), then the partial tiles.
  int* counters = (int*)workspace;
  float* partial = workspace ? workspace + ((tiles + 63) / 64) * 64 : nullptr;
  cudaError_t le = co_launch(kernel, dim3(tiles, splits), dim3(192), (size_t)smem, stream, mw, mx, bias, bias_dtype, out,
                             out_dtype, M, N, K, ldo, epilogue, status, partial, counters, k_per_split, defer);
  if (le != cudaSuccess) CO_FAIL("gemm_tc_few: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("gemm_tc_few");
  return 0;
}
}  // namespace

// Floats of zero-initialised workspace that coheryn_gemm_bf16_tc_few needs for this shape (0:
// none).  The kernel leaves the counters at its head zero again, so one workspace serves
// every product that runs in stream order.
CO_EXPORT long coheryn_gemm_tc_few_workspace_floats(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int s = few_splits(N, K);
  if (s <= 1) return 0;
  const long tiles = (N + BF - 1) / BF;
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  return ((tiles + 63) / 64) * 64 + tiles * s * bt * BF;
}

// The number of K splits of this shape (1: none).
CO_EXPORT int coheryn_gemm_tc_few_splits(int N, int K) { return (N <= 0 || K <= 0) ? 1 : few_splits(N, K); }

// x: [M, K] bfloat16 with row stride ldx, M <= 256 (above 64 rows a product whose K is cut needs defer = 1); w: [N, K] bfloat16 contiguous; K and ldx
// multiples of 8, bases 16-byte aligned.  epilogue 0: out[M, N] (+ bias); 1: gated SiLU over
// interleaved rows of w, out[M, N/2].  status: device word that receives 11/12/13 if a
// bounded wait of the producer / the MMA issuer / the epilogue ran out.  workspace: see above.
// defer = 1 (epilogue 0 only) leaves the addition of the K splits to the consumer: out is then
// float32 [splits][M][N], contiguous, the bias added to split 0, and no workspace is used.
CO_EXPORT int coheryn_gemm_bf16_tc_few(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                                       int out_dtype, int M, int N, int K, long ldx, long ldo, int epilogue,
                                       int* status, float* workspace, long workspace_floats, int defer,
                                       cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 256) CO_FAIL("gemm_bf16_tc_few: M = %d exceeds 256", M);
  if (K <= 0 || (K & 7) || (ldx & 7)) CO_FAIL("gemm_bf16_tc_few: K = %d and the row stride %ld must be multiples of 8", K, ldx);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("gemm_bf16_tc_few: operands must be 16-byte aligned");
  if (epilogue == 1 && (N & 1)) CO_FAIL("gemm_bf16_tc_few: gated epilogue needs an even number of rows");
  if (epilogue != 0 && epilogue != 1) CO_FAIL("gemm_bf16_tc_few: unknown epilogue %d", epilogue);
  const int splits = few_splits(N, K);
  if (defer && (epilogue != 0 || out_dtype != CO_F32)) CO_FAIL("gemm_bf16_tc_few: deferred splits are float32 and take no gate");
  if (splits > 1 && !defer && (!workspace || workspace_floats < coheryn_gemm_tc_few_workspace_floats(M, N, K)))
    CO_FAIL("gemm_bf16_tc_few: the workspace of %ld floats is too small for M=%d N=%d K=%d", workspace_floats, M, N, K);
  const int bt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : (M <= 128 ? 128 : 256)));
  if (bt > 64 && splits > 1 && !defer)
    CO_FAIL("gemm_bf16_tc_few: with more than 64 rows the K slices of N=%d K=%d have to be left to the consumer", N, K);
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, K, BF) || !make_map(&mx, x, M, K, ldx, bt))
    CO_FAIL("gemm_bf16_tc_few: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%ld)", M, N, K, ldx);
#define GO(BT_, ST_) return launch_few<BT_, ST_>(mw, mx, bias, bias_dtype, out, out_dtype, M, N, K, ldo, epilogue, status, workspace, splits, defer, stream)
  // One CTA per SM at most: a deeper ring keeps more of the stream in flight.  Six stages
  // (111 KB) leave room on the SM for a CTA of the NEXT few-rows product, which then fetches
  // its first tiles while this one still runs (gate/up followed by down).
  const bool one_wave = (long)((N + BF - 1) / BF) * splits <= 148;
  if (bt == 16 && one_wave) GO(16, 6);
  if (bt == 16) GO(16, 5);
  if (bt == 32 && one_wave) GO(32, 7);
  if (bt == 32) GO(32, 5);
  if (bt == 64 && one_wave) GO(64, 7);
  if (bt == 64) GO(64, 4);
  if (bt == 128) GO(128, 6);     // 32 KB per stage
  GO(256, 4);                    // 48 KB per stage
#undef GO
}
