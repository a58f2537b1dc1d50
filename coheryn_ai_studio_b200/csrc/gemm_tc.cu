// out[M, N] = x[M, K] . W[N, K]^T (+ bias | gated SiLU) for many rows (prompt portions), in
// bfloat16 on the 5th-generation tensor cores: TMA (cp.async.bulk.tensor) stages 128-byte
// swizzled tiles of both operands in shared memory, one thread issues tcgen05.mma with the
// accumulator in tensor memory, and the epilogue reads it back with tcgen05.ld.
//
// One CTA computes a 128 x BN tile of the output (tokens on the 128 TMEM lanes, output
// features on BN columns) over all of K in steps of 64:
//   warp 0   producer: waits for a free stage, arms its mbarrier with the byte count and
//            issues the two TMA loads (x tile 128 x 64, W tile BN x 64);
//   warp 1   MMA issuer: waits for a full stage, issues four m128 nBN k16 MMAs, and lets
//            tcgen05.commit release the stage (and, after the last step, signal the epilogue);
//   warps 2-5 epilogue: each reads its 32 lanes of the accumulator, applies bias or the gate
//            and converts.  bfloat16 output goes 64 columns at a time into a swizzled 4 KB
//            staging buffer in shared memory (the stages are free by then) and leaves as a
//            32 x 64 box through a TMA store, two boxes in flight per warp; float32 output
//            and split-K partial sums are stored from registers, 32 columns at a time.
// Rows and columns beyond M, N and the K tail are zero filled by TMA and masked on store.
// Every wait is bounded: on expiry the kernel records an error code and winds down.
#include <cuda.h>
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;          // tokens per tile = TMEM lanes
constexpr int EPI_PLAIN = 0, EPI_GATED_SILU = 1;

template <int BN, int STAGES>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + 2 * BN * 4 /* bias */;
};

// Sixty-four bfloat16 output columns of a warp's 32 rows (lane = row) through shared memory and
// one TMA store: the accumulator columns come from tensor memory (64 of them, or 128 gate/up
// columns in the gated case), bias or gate is applied, the 128 bytes of a row go to `stage`
// (4 KB, 1024-byte aligned) in the 128-byte swizzle of the output tensor map, and lane 0 sends
// the 32 x 64 box.  Rows and columns beyond the tensor are clipped by the copy.
// bias_chunk: the bias of the chunk's first accumulator column (or null).
__device__ __forceinline__ void store_chunk_tma(unsigned tmem_chunk, const float* bias_chunk, bool gated,
                                                unsigned char* stage, const CUtensorMap* map_out, int out_col,
                                                int out_row, int lane) {
  uint4 pk[8];
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(pk);
  if (gated) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      unsigned r[32];
      tmem_ld32(tmem_chunk + 32 * q, r);
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const float g0 = __uint_as_float(r[2 * j]), u0 = __uint_as_float(r[2 * j + 1]);
        const float g1 = __uint_as_float(r[2 * j + 2]), u1 = __uint_as_float(r[2 * j + 3]);
        h[q * 8 + (j >> 1)] = __floats2bfloat162_rn(__fdividef(g0, 1.0f + __expf(-g0)) * u0,
                                                    __fdividef(g1, 1.0f + __expf(-g1)) * u1);
      }
    }
  } else {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      unsigned r[32];
      tmem_ld32(tmem_chunk + 32 * q, r);
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        float a = __uint_as_float(r[j]), b = __uint_as_float(r[j + 1]);
        if (bias_chunk) { a += bias_chunk[32 * q + j]; b += bias_chunk[32 * q + j + 1]; }
        h[q * 16 + (j >> 1)] = __floats2bfloat162_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4)) = pk[c];
  fence_proxy_async();
  __syncwarp();
  if (lane == 0) {
    tma_store_2d(map_out, stage, out_col, out_row);
    tma_store_commit();
  }
}
constexpr int STAGING_BYTES = 4 * 2 * 4096;   // four epilogue warps, two chunks each

template <int BN, int STAGES>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               const __grid_constant__ CUtensorMap map_out, int tma_out,
               const void* __restrict__ bias, int bias_dtype, void* __restrict__ out, int out_dtype, int M, int N,
               int K, long ldo, int epilogue, int* __restrict__ status, float* __restrict__ partial, int k_per_split) {
  using S = Smem<BN, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  // 128-byte swizzled tiles must start on a 1024-byte boundary.
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = (unsigned long long*)(tiles + STAGES * S::STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* accum_full = empty + STAGES;
  unsigned* tmem_slot = (unsigned*)(accum_full + 1);
  float* bias_s = (float*)(tiles + STAGES * S::STAGE_BYTES + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  // Split K: CTA z of the grid sums the k-steps [kt_begin, kt_begin + k_tiles) and leaves its raw
  // float32 tile in partial[z]; splitk_reduce_kernel adds the splits in order and finishes.
  const int kt_begin = partial ? blockIdx.z * k_per_split : 0;
  const int k_tiles = partial ? min(k_per_split, (K + BK - 1) / BK - kt_begin) : (K + BK - 1) / BK;
  constexpr int TMEM_COLS = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));     // a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(accum_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {   // one warp allocates the accumulator columns (and frees them at the end)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  co_pdl_launch_dependents();
  // Barriers and tensor memory are set up.  W depends on no earlier kernel: the producer asks
  // for the first stages' W tiles before it waits for the predecessor, whose output x is.
  if (warp == 0) {
    if (lane == 0) {
      const int head = k_tiles < STAGES ? k_tiles : STAGES;
      for (int kt = 0; kt < head; ++kt) {
        mbar_expect_tx(&full[kt], S::STAGE_BYTES);
        tma_load_2d(tiles + kt * S::STAGE_BYTES + S::A_BYTES, &map_w, (kt_begin + kt) * BK, n0, &full[kt]);
      }
      co_pdl_wait();
      for (int kt = 0; kt < head; ++kt)
        tma_load_2d(tiles + kt * S::STAGE_BYTES, &map_x, (kt_begin + kt) * BK, m0, &full[kt]);
      for (int kt = head; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(&empty[s], ((kt / STAGES) - 1) & 1)) { atomicExch(status, 11); break; }
        unsigned char* a = tiles + s * S::STAGE_BYTES;
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        tma_load_2d(a, &map_x, (kt_begin + kt) * BK, m0, &full[s]);
        tma_load_2d(a + S::A_BYTES, &map_w, (kt_begin + kt) * BK, n0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = umma_idesc(BM, BN);
      bool ok = true;
      for (int kt = 0; kt < k_tiles && ok; ++kt) {
        const int s = kt % STAGES;
        if (!mbar_wait(&full[s], (kt / STAGES) & 1)) { atomicExch(status, 12); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned char* a = tiles + s * S::STAGE_BYTES;
        const unsigned long long da = umma_desc(a), db = umma_desc(a + S::A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)   // 32 bytes (>> 4 = 2) further along the swizzled row per step
          umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
        umma_commit(&empty[s]);                 // arrives when these MMAs have read the stage
      }
      umma_commit(accum_full);                  // arrives when every MMA issued so far is complete
    }
  } else {
    // Epilogue warps 2..5: TMEM lane quarter = warp % 4.
    const int quarter = warp & 3;
    const int row = m0 + quarter * 32 + lane;
    if (bias) {   // the tile's slice of the bias, once, while the main loop runs
      for (int i = threadIdx.x - 64; i < BN; i += 128) bias_s[i] = n0 + i < N ? co_load_any(bias, bias_dtype, n0 + i) : 0.f;
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    co_pdl_wait();   // out (and the split workspace) may still be in use by the predecessor
    const bool waited = mbar_wait(accum_full, 0);
    if (!waited && lane == 0) atomicExch(status, 13);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (waited && tma_out && !partial) {
      // bfloat16 output through shared memory and TMA stores: every MMA is complete, so the
      // stages are free and serve as the staging area (two 4 KB chunks per warp).
      const bool gated = epilogue == EPI_GATED_SILU;
      const int step = gated ? 128 : 64;
      unsigned char* stage = tiles + quarter * 8192;
      int chunk = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += step, ++chunk) {
        if (n0 + c0 >= N) break;
        if (chunk >= 2) {
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
        }
        store_chunk_tma(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, bias && !gated ? bias_s + c0 : nullptr,
                        gated, stage + (chunk & 1) * 4096, &map_out, gated ? (n0 + c0) >> 1 : n0 + c0, m0 + quarter * 32, lane);
      }
      if (lane == 0) tma_store_wait_all();
    } else if (waited) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= N) break;
        unsigned r[32];
        tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)c0, r);
        if (row >= M) continue;
        if (partial) {
          float* p = partial + ((size_t)blockIdx.z * M + row) * N + n0 + c0;
          if (n0 + c0 + 32 <= N && (((uintptr_t)p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ((uint4*)p)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          } else {
            for (int j = 0; j < 32 && n0 + c0 + j < N; ++j) p[j] = __uint_as_float(r[j]);
          }
          continue;
        }
        if (epilogue == EPI_GATED_SILU) {
          // columns (2j, 2j+1) = (gate_j, up_j): 16 outputs per 32 columns
          const int oc = (n0 + c0) >> 1;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g = __uint_as_float(r[2 * j]), u = __uint_as_float(r[2 * j + 1]);
            v[j] = __fdividef(g, 1.0f + __expf(-g)) * u;
          }
          const int n_out = N >> 1;
          if (out_dtype == CO_BF16) {
            __nv_bfloat16* p = (__nv_bfloat16*)out + (size_t)row * ldo + oc;
            if (oc + 16 <= n_out && (((uintptr_t)p) & 15) == 0) {
              uint4 q[2];
              __nv_bfloat162* h = (__nv_bfloat162*)q;
#pragma unroll
              for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              ((uint4*)p)[0] = q[0]; ((uint4*)p)[1] = q[1];
            } else {
              for (int j = 0; j < 16 && oc + j < n_out; ++j) p[j] = __float2bfloat16_rn(v[j]);
            }
          } else {
            float* p = (float*)out + (size_t)row * ldo + oc;
            for (int j = 0; j < 16 && oc + j < n_out; ++j) p[j] = v[j];
          }
          continue;
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] += bias_s[c0 + j];
        }
        const int nc = n0 + c0;
        if (out_dtype == CO_BF16) {
          __nv_bfloat16* p = (__nv_bfloat16*)out + (size_t)row * ldo + nc;
          if (nc + 32 <= N && (((uintptr_t)p) & 15) == 0) {
            uint4 q[4];
            __nv_bfloat162* h = (__nv_bfloat162*)q;
#pragma unroll
            for (int j = 0; j < 16; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
#pragma unroll
            for (int j = 0; j < 4; ++j) ((uint4*)p)[j] = q[j];
          } else {
            for (int j = 0; j < 32 && nc + j < N; ++j) p[j] = __float2bfloat16_rn(v[j]);
          }
        } else {
          float* p = (float*)out + (size_t)row * ldo + nc;
          if (nc + 32 <= N && (((uintptr_t)p) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) ((float4*)p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
            for (int j = 0; j < 32 && nc + j < N; ++j) p[j] = v[j];
          }
        }
      }
    }
  }

  // Wind down: everybody meets, then the allocating warp frees the accumulator columns.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

// One 32-column piece of an accumulator row: bias or gate, conversion, store.
__device__ __forceinline__ void store_piece(const unsigned (&r)[32], int row, int nc, const float* bias_piece,
                                            void* __restrict__ out, int out_dtype, int N, long ldo, int epilogue) {
  if (epilogue == EPI_GATED_SILU) {
    // columns (2j, 2j+1) = (gate_j, up_j): 16 outputs per 32 columns
    const int oc = nc >> 1, n_out = N >> 1;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float g = __uint_as_float(r[2 * j]), u = __uint_as_float(r[2 * j + 1]);
      v[j] = __fdividef(g, 1.0f + __expf(-g)) * u;
    }
    if (out_dtype == CO_BF16) {
      __nv_bfloat16* p = (__nv_bfloat16*)out + (size_t)row * ldo + oc;
      if (oc + 16 <= n_out && (((uintptr_t)p) & 15) == 0) {
        uint4 q[2];
        __nv_bfloat162* h = (__nv_bfloat162*)q;
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        ((uint4*)p)[0] = q[0]; ((uint4*)p)[1] = q[1];
      } else {
        for (int j = 0; j < 16 && oc + j < n_out; ++j) p[j] = __float2bfloat16_rn(v[j]);
      }
    } else {
      float* p = (float*)out + (size_t)row * ldo + oc;
      for (int j = 0; j < 16 && oc + j < n_out; ++j) p[j] = v[j];
    }
    return;
  }
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
  if (bias_piece) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] += bias_piece[j];
  }
  if (out_dtype == CO_BF16) {
    __nv_bfloat16* p = (__nv_bfloat16*)out + (size_t)row * ldo + nc;
    if (nc + 32 <= N && (((uintptr_t)p) & 15) == 0) {
      uint4 q[4];
      __nv_bfloat162* h = (__nv_bfloat162*)q;
#pragma unroll
      for (int j = 0; j < 16; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) ((uint4*)p)[j] = q[j];
    } else {
      for (int j = 0; j < 32 && nc + j < N; ++j) p[j] = __float2bfloat16_rn(v[j]);
    }
  } else {
    float* p = (float*)out + (size_t)row * ldo + nc;
    if (nc + 32 <= N && (((uintptr_t)p) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) ((float4*)p)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
      for (int j = 0; j < 32 && nc + j < N; ++j) p[j] = v[j];
    }
  }
}

// Adds the float32 tiles of the K splits in ascending order and applies the epilogue.  One
// thread per pair of neighbouring columns (a gate/up pair in the gated case).
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                     const void* __restrict__ bias, int bias_dtype, void* __restrict__ out,
                                     int out_dtype, long ldo, int epilogue) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const long pairs_per_row = (N + 1) / 2;
  const long total = (long)M * pairs_per_row;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long)gridDim.x * blockDim.x) {
    const long m = e / pairs_per_row;
    const int n = (int)(e % pairs_per_row) * 2;
    const bool has1 = n + 1 < N;
    float v0 = 0.f, v1 = 0.f;
    for (int z = 0; z < splits; ++z) {
      const float* p = partial + ((size_t)z * M + m) * N + n;
      v0 += p[0];
      if (has1) v1 += p[1];
    }
    if (epilogue == EPI_GATED_SILU) {
      const float r = __fdividef(v0, 1.0f + __expf(-v0)) * v1;
      const size_t o = (size_t)m * ldo + (n >> 1);
      if (out_dtype == CO_BF16) ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(r);
      else ((float*)out)[o] = r;
      continue;
    }
    if (bias) {
      v0 += co_load_any(bias, bias_dtype, n);
      if (has1) v1 += co_load_any(bias, bias_dtype, n + 1);
    }
    const size_t o = (size_t)m * ldo + n;
    if (out_dtype == CO_BF16) {
      ((__nv_bfloat16*)out)[o] = __float2bfloat16_rn(v0);
      if (has1) ((__nv_bfloat16*)out)[o + 1] = __float2bfloat16_rn(v1);
    } else {
      ((float*)out)[o] = v0;
      if (has1) ((float*)out)[o + 1] = v1;
    }
  }
}

// ------------------------------------------------------------------------------------
// Persistent variant for products of many tiles: one CTA per SM walks the tiles
// t = blockIdx.x, blockIdx.x + gridDim.x, ... (row tiles fastest, so the CTAs that run at the
// same time share W tiles through L2).  Two accumulators in tensor memory (2 x BN columns)
// let the epilogue of one tile run while the MMAs of the next are issued; the shared-memory
// stages and their barriers simply keep cycling across tiles.
template <int BN, int STAGES>
__global__ void __launch_bounds__(192)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                          const void* __restrict__ bias, int bias_dtype, void* __restrict__ out, int out_dtype,
                          int M, int N, int K, long ldo, int epilogue, int* __restrict__ status) {
  using S = Smem<BN, STAGES>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = (unsigned long long*)(tiles + STAGES * S::STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;      // [2]
  unsigned long long* acc_empty = acc_full + 2;       // [2]
  unsigned* tmem_slot = (unsigned*)(acc_empty + 2);
  float* bias_s = (float*)(tiles + STAGES * S::STAGE_BYTES + 256);   // [2][BN]
  static_assert(2 * STAGES * 8 + 4 * 8 + 4 <= 256, "barriers fit their slot");
  static_assert(2 * BN <= 512, "two accumulators fit tensor memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_tiles = (K + BK - 1) / BK;
  constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 4); }
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
      long it = 0;   // k-steps issued so far, across tiles
      bool ok = true;
      // The first tile's first stages: W (which depends on no earlier kernel) before the wait
      // for the predecessor, x (its output) after it.
      const int head = k_tiles < STAGES ? k_tiles : STAGES;
      if (blockIdx.x < num_tiles) {
        const int m0 = (blockIdx.x % tiles_m) * BM, n0 = (blockIdx.x / tiles_m) * BN;
        for (int kt = 0; kt < head; ++kt) {
          mbar_expect_tx(&full[kt], S::STAGE_BYTES);
          tma_load_2d(tiles + kt * S::STAGE_BYTES + S::A_BYTES, &map_w, kt * BK, n0, &full[kt]);
        }
        co_pdl_wait();
        for (int kt = 0; kt < head; ++kt) tma_load_2d(tiles + kt * S::STAGE_BYTES, &map_x, kt * BK, m0, &full[kt]);
        it = head;
      }
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kt = tile == (int)blockIdx.x ? head : 0; kt < k_tiles; ++kt, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES && !mbar_wait(&empty[s], (unsigned)((it / STAGES) - 1) & 1)) { atomicExch(status, 11); ok = false; break; }
          unsigned char* a = tiles + s * S::STAGE_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(a, &map_x, kt * BK, m0, &full[s]);
          tma_load_2d(a + S::A_BYTES, &map_w, kt * BK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr unsigned idesc = umma_idesc(BM, BN);
      long it = 0;
      int j = 0;     // tiles done by this CTA
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++j) {
        const int acc = j & 1;
        if (j >= 2 && !mbar_wait(&acc_empty[acc], (unsigned)((j >> 1) - 1) & 1)) { atomicExch(status, 14); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + (unsigned)(acc * BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = (int)(it % STAGES);
          if (!mbar_wait(&full[s], (unsigned)(it / STAGES) & 1)) { atomicExch(status, 12); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned char* a = tiles + s * S::STAGE_BYTES;
          const unsigned long long da = umma_desc(a), db = umma_desc(a + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int j = 0;
    co_pdl_wait();   // out may still be in use by the predecessor
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++j) {
      const int acc = j & 1;
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      const int row = m0 + quarter * 32 + lane;
      float* bias_t = bias_s + acc * BN;
      if (bias) {
        for (int i = threadIdx.x - 64; i < BN; i += 128) bias_t[i] = n0 + i < N ? co_load_any(bias, bias_dtype, n0 + i) : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!mbar_wait(&acc_full[acc], (unsigned)(j >> 1) & 1)) {
        if (lane == 0) atomicExch(status, 13);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= N) break;
        unsigned r[32];
        tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), r);
        if (row < M) store_piece(r, row, n0 + c0, bias ? bias_t + c0 : nullptr, out, out_dtype, N, ldo, epilogue);
      }
      // This warp has read its quarter of the accumulator: hand it back to the MMA issuer.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------------------
// Pair variant: two CTAs of a cluster (two SMs) share one 256 x BN tile.  CTA r of the pair
// stages rows [128 r, 128 r + 128) of the x tile and rows [BN/2 r, BN/2 (r + 1)) of the W tile,
// so each SM pulls 128 + BN/2 rows of 128 bytes per k-step from L2 instead of 128 + BN for the
// same number of MMA cycles; the leader (rank 0) issues tcgen05.mma.cta_group::2, which reads
// both CTAs' shared memory and writes rows [128 r, ..) of the accumulator into CTA r's tensor
// memory.  Barriers:
//   full[s]       in the leader: armed by the leader's producer with the bytes of BOTH CTAs;
//                 the peer's TMA loads complete on it (cp.async.bulk.tensor ... cta_group::2);
//   empty[s]      in each CTA: the leader's tcgen05.commit arrives on both (multicast);
//   acc_full[a]   in each CTA: likewise, after a tile's last MMA;
//   acc_empty[a]  in the leader: the eight epilogue warps of both CTAs arrive on it.
// The pair walks the tiles t = pair, pair + pairs, ... (row tiles fastest) with two accumulators.
__device__ __forceinline__ unsigned cluster_ctarank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned map_to_cta(const void* local, unsigned rank) {
  unsigned ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
  return ra;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion is counted on a barrier of the pair's leader (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, unsigned bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                               unsigned idesc, unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives, once the MMAs issued so far are complete, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(unsigned long long* bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

template <int BN, int STAGES, int ACCS>
struct PairSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // Staging chunks per epilogue warp: two where shared memory allows, else one.
  static constexpr int SBUF = STAGES * STAGE_BYTES + STAGING_BYTES + 1024 + 256 + ACCS * BN * 4 <= 227 * 1024 ? 2 : 1;
  static constexpr int STAGING = SBUF * 4 * 4096;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + STAGING + 1024 /* alignment slack */ + 256 /* barriers */ + ACCS * BN * 4 /* bias */;
  static_assert(TOTAL <= 227 * 1024, "stages, staging area and barriers fit shared memory");
};

template <int BN, int STAGES, int ACCS>
__global__ void __launch_bounds__(192)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_out, int tma_out,
                    const void* __restrict__ bias, int bias_dtype, void* __restrict__ out, int out_dtype,
                    int M, int N, int K, long ldo, int epilogue, int* __restrict__ status) {
  using S = PairSmem<BN, STAGES, ACCS>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* staging = tiles + STAGES * S::STAGE_BYTES;      // [4 warps][SBUF][4 KB], 1024-byte aligned
  unsigned long long* full = (unsigned long long*)(staging + S::STAGING);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;      // [ACCS]
  unsigned long long* acc_empty = acc_full + ACCS;    // [ACCS]
  unsigned* tmem_slot = (unsigned*)(acc_empty + ACCS);
  float* bias_s = (float*)(staging + S::STAGING + 256);   // [ACCS][BN]
  static_assert(2 * STAGES * 8 + 2 * ACCS * 8 + 4 <= 256, "barriers fit their slot");
  static_assert(ACCS * BN <= 512 && BN % 128 == 0 && BN <= 256, "accumulators fit tensor memory, chunks of 128 divide them");
  static_assert(S::STAGE_BYTES % 1024 == 0, "the staging area stays 1024-byte aligned");
  constexpr int TMEM_COLS = ACCS * BN <= 32 ? 32 : (ACCS * BN <= 64 ? 64 : (ACCS * BN <= 128 ? 128 : (ACCS * BN <= 256 ? 256 : 512)));
  constexpr int PM = 2 * BM;   // rows of a pair's tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned rank = cluster_ctarank();   // 0: the leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int tiles_m = (M + PM - 1) / PM, tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int k_tiles = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < ACCS; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 8); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {   // the same warp of both CTAs allocates (and frees) the pair's columns
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // the peer's barriers are initialised before anything is counted on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  co_pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      long it = 0;
      bool ok = true;
      const int head = k_tiles < STAGES ? k_tiles : STAGES;
      // W of the first tile's first stages before the wait for the predecessor, x after it.
      if (pair < num_tiles) {
        const int m0 = (pair % tiles_m) * PM + (int)rank * BM, n0 = (pair / tiles_m) * BN + (int)rank * (BN / 2);
        for (int kt = 0; kt < head; ++kt) {
          if (rank == 0) mbar_expect_tx(&full[kt], 2 * S::STAGE_BYTES);
          tma_load_2d_pair(tiles + kt * S::STAGE_BYTES + S::A_BYTES, &map_w, kt * BK, n0, map_to_cta(&full[kt], 0));
        }
        co_pdl_wait();
        for (int kt = 0; kt < head; ++kt)
          tma_load_2d_pair(tiles + kt * S::STAGE_BYTES, &map_x, kt * BK, m0, map_to_cta(&full[kt], 0));
        it = head;
      }
      for (int tile = pair; tile < num_tiles && ok; tile += pairs) {
        const int m0 = (tile % tiles_m) * PM + (int)rank * BM, n0 = (tile / tiles_m) * BN + (int)rank * (BN / 2);
        for (int kt = tile == pair ? head : 0; kt < k_tiles; ++kt, ++it) {
          const int s = (int)(it % STAGES);
          if (it >= STAGES && !mbar_wait(&empty[s], (unsigned)((it / STAGES) - 1) & 1)) { atomicExch(status, 11); ok = false; break; }
          unsigned char* a = tiles + s * S::STAGE_BYTES;
          const unsigned bar = map_to_cta(&full[s], 0);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);
          tma_load_2d_pair(a, &map_x, kt * BK, m0, bar);
          tma_load_2d_pair(a + S::A_BYTES, &map_w, kt * BK, n0, bar);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      constexpr unsigned idesc = umma_idesc(PM, BN);
      long it = 0;
      int j = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += pairs, ++j) {
        const int acc = j % ACCS;
        if (j >= ACCS && !mbar_wait(&acc_empty[acc], (unsigned)((j / ACCS) - 1) & 1)) { atomicExch(status, 14); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned d = tmem_base + (unsigned)(acc * BN);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = (int)(it % STAGES);
          if (!mbar_wait(&full[s], (unsigned)(it / STAGES) & 1)) { atomicExch(status, 12); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          unsigned char* a = tiles + s * S::STAGE_BYTES;
          const unsigned long long da = umma_desc(a), db = umma_desc(a + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16_pair(d, da + 2 * k, db + 2 * k, idesc, (kt | k) != 0);
          umma_commit_pair(&empty[s]);
        }
        if (ok) umma_commit_pair(&acc_full[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    int j = 0, chunk = 0;
    co_pdl_wait();   // out may still be in use by the predecessor
    for (int tile = pair; tile < num_tiles; tile += pairs, ++j) {
      const int acc = j % ACCS;
      const int m0 = (tile % tiles_m) * PM + (int)rank * BM, n0 = (tile / tiles_m) * BN;
      const int row = m0 + quarter * 32 + lane;
      float* bias_t = bias_s + acc * BN;
      if (bias) {
        for (int i = threadIdx.x - 64; i < BN; i += 128) bias_t[i] = n0 + i < N ? co_load_any(bias, bias_dtype, n0 + i) : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!mbar_wait(&acc_full[acc], (unsigned)(j / ACCS) & 1)) {
        if (lane == 0) atomicExch(status, 13);
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (tma_out) {
        const bool gated = epilogue == EPI_GATED_SILU;
        const int step = gated ? 128 : 64;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += step, ++chunk) {
          if (n0 + c0 >= N) break;
          if (chunk >= S::SBUF) {   // the chunk that used this staging buffer has left it
            if (lane == 0) tma_store_wait_read<S::SBUF - 1>();
            __syncwarp();
          }
          store_chunk_tma(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0),
                          bias && !gated ? bias_t + c0 : nullptr, gated,
                          staging + (quarter * S::SBUF + chunk % S::SBUF) * 4096, &map_out,
                          gated ? (n0 + c0) >> 1 : n0 + c0, m0 + quarter * 32, lane);
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= N) break;
          unsigned r[32];
          tmem_ld32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * BN + c0), r);
          if (row < M) store_piece(r, row, n0 + c0, bias ? bias_t + c0 : nullptr, out, out_dtype, N, ldo, epilogue);
        }
      }
      // This warp has read its part of the accumulator: tell the leader's MMA issuer.
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
    }
    if (tma_out && lane == 0) tma_store_wait_all();
  }

  // Wind down: both CTAs meet (nothing of the pair is in flight any more), then free the columns.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

// The tensor map of a bfloat16 output [M, n_out] with row stride ldo for the TMA-store epilogue
// (boxes of 32 rows x 64 columns); false if the output does not qualify (another dtype, a base
// or a row pitch off the 16-byte grid) or COHERYN_TMA_STORE=0 is in the environment.
bool make_out_map(CUtensorMap* map, const void* out, int out_dtype, int M, int n_out, long ldo) {
  static const bool enabled = !(getenv("COHERYN_TMA_STORE") && getenv("COHERYN_TMA_STORE")[0] == '0');
  if (!enabled || out_dtype != CO_BF16 || !out || ((uintptr_t)out & 15) || (ldo & 7) || n_out <= 0) return false;
  return make_map(map, out, M, n_out, ldo, 32);
}

template <int BN, int STAGES>
int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, const void* bias, int bias_dtype, void* out,
              int out_dtype, int M, int N, int K, long ldo, int epilogue, int* status, cudaStream_t stream,
              float* partial = nullptr, int splits = 1, bool leave_parts = false) {
  // bfloat16 output leaves through shared memory and TMA stores where whole chunks of 64 output
  // columns divide the tile.
  CUtensorMap mo = mx;
  const int tma_out = !(partial && splits > 1) && BN % (epilogue == EPI_GATED_SILU ? 128 : 64) == 0 &&
                      make_out_map(&mo, out, out_dtype, M, epilogue == EPI_GATED_SILU ? N / 2 : N, ldo) ? 1 : 0;
  auto kernel = gemm_tc_kernel<BN, STAGES>;
  constexpr int smem = Smem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) CO_FAIL("gemm_tc: %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int k_tiles = (K + BK - 1) / BK;
  const int k_per_split = partial ? (k_tiles + splits - 1) / splits : k_tiles;
  const int used = partial ? (k_tiles + k_per_split - 1) / k_per_split : 1;    // no split is left empty
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, used);
  cudaError_t le = co_launch(kernel, grid, dim3(192), (size_t)smem, stream, mx, mw, mo, tma_out, bias, bias_dtype, out, out_dtype, M, N,
                             K, ldo, epilogue, status, used > 1 ? partial : (float*)nullptr, k_per_split);
  if (le != cudaSuccess) CO_FAIL("gemm_tc: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("gemm_tc");
  if (used > 1 && !leave_parts) {
    const long pairs = (long)M * ((N + 1) / 2);
    const int blocks = (int)((pairs + 255) / 256 < 148 * 8 ? (pairs + 255) / 256 : 148 * 8);
    le = co_launch(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)partial, used, M, N, bias,
                   bias_dtype, out, out_dtype, ldo, epilogue);
    if (le != cudaSuccess) CO_FAIL("gemm_tc: launch failed: %s", cudaGetErrorString(le));
    CO_CHECK_LAUNCH("splitk_reduce");
  }
  return 0;
}
template <int BN, int STAGES>
int launch_tc_persistent(const CUtensorMap& mx, const CUtensorMap& mw, const void* bias, int bias_dtype, void* out,
                         int out_dtype, int M, int N, int K, long ldo, int epilogue, int* status,
                         cudaStream_t stream) {
  auto kernel = gemm_tc_persistent_kernel<BN, STAGES>;
  constexpr int smem = Smem<BN, STAGES>::TOTAL;
  static int sms = 0;
  if (!sms) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) CO_FAIL("gemm_tc: %d bytes of shared memory: %s", smem, cudaGetErrorString(e));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  const long tiles = (long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
  const int grid = (int)(tiles < sms ? tiles : sms);
  cudaError_t le = co_launch(kernel, dim3(grid), dim3(192), (size_t)smem, stream, mx, mw, bias, bias_dtype, out,
                             out_dtype, M, N, K, ldo, epilogue, status);
  if (le != cudaSuccess) CO_FAIL("gemm_tc: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("gemm_tc_persistent");
  return 0;
}
// Pairs that can be resident at once (a cluster needs two free SMs of one GPC); 0 if unknown.
template <int BN, int STAGES, int ACCS>
int pair_slots() {
  static int slots = -1;
  if (slots < 0) {
    auto kernel = gemm_tc_pair_kernel<BN, STAGES, ACCS>;
    constexpr int smem = PairSmem<BN, STAGES, ACCS>::TOTAL;
    slots = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return slots;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms > 1 ? (sms & ~1) : 2);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, (void*)kernel, &cfg) == cudaSuccess && clusters > 0) slots = clusters;
    else (void)cudaGetLastError();
    if (slots > sms / 2) slots = sms / 2;
  }
  return slots;
}

template <int BN, int STAGES, int ACCS>
int launch_tc_pair(const CUtensorMap& mx, const CUtensorMap& mw, const void* bias, int bias_dtype, void* out,
                   int out_dtype, int M, int N, int K, long ldo, int epilogue, int* status, cudaStream_t stream) {
  auto kernel = gemm_tc_pair_kernel<BN, STAGES, ACCS>;
  constexpr int smem = PairSmem<BN, STAGES, ACCS>::TOTAL;
  const int slots = pair_slots<BN, STAGES, ACCS>();
  if (slots <= 0) CO_FAIL("gemm_tc_pair: no pair of CTAs with %d bytes of shared memory fits the device", smem);
  const long tiles = (long)((N + BN - 1) / BN) * ((M + 2 * BM - 1) / (2 * BM));
  const int pairs = (int)(tiles < slots ? tiles : slots);
  CUtensorMap mo = mx;
  const int tma_out = make_out_map(&mo, out, out_dtype, M, epilogue == EPI_GATED_SILU ? N / 2 : N, ldo) ? 1 : 0;
  cudaError_t le = co_launch_cluster(2, kernel, dim3(2 * pairs), dim3(192), (size_t)smem, stream, mx, mw, mo, tma_out, bias, bias_dtype,
                                     out, out_dtype, M, N, K, ldo, epilogue, status);
  if (le != cudaSuccess) CO_FAIL("gemm_tc_pair: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("gemm_tc_pair");
  return 0;
}

// Whether pairs with 256 x 256 tiles suit an [M, N] output: if its tiles fill whole rounds of the
// resident pairs to three quarters or more (COHERYN_GEMM_PAIR=0 in the environment: never).
int g_pairs = -1;   // -1: not decided yet; coheryn_gemm_tc_set_pairs overrides the environment
bool pair_enabled() {
  if (g_pairs < 0) {
    const char* e = getenv("COHERYN_GEMM_PAIR");
    g_pairs = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pairs == 1;
}
bool pair_suits(int M, int N) {
  if (!pair_enabled() || M <= BM) return false;
  const int slots = pair_slots<256, 6, 2>();
  if (slots <= 0) return false;
  const long tiles = (long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
  const long rounds = (tiles + slots - 1) / slots;
  // useful rows and columns over those the rounds pay for
  return (double)M * N / ((double)rounds * slots * 2 * BM * 256) >= 0.75;
}
}  // namespace

// Tuning knobs for experiments: tile width (0 = by shape, 128 caps it) and stage count
// (0 = the default of the tile width).
static int g_bn = 0, g_stages = 0;
CO_EXPORT void coheryn_gemm_tc_tune(int bn, int stages) { g_bn = bn; g_stages = stages; }
// Whether coheryn_gemm_bf16_tc may hand suitable shapes to pairs of CTAs (default: yes).
CO_EXPORT void coheryn_gemm_tc_set_pairs(int on) { g_pairs = on ? 1 : 0; }

// Tile width by shape: 256 columns where the output is wide; with a single row tile (a decode
// batch, a short portion) narrower tiles put more CTAs on the weight stream.
static int tile_width(int M, int N) {
  int bn = N >= 192 ? 256 : (N >= 96 ? 128 : (N >= 48 ? 64 : 32));
  const long tiles_m = (M + BM - 1) / BM;
  // A single wave of 256-wide tiles that leaves SMs idle: 192-wide tiles if they still fit one wave.
  if (bn == 256 && tiles_m > 1 && tiles_m * ((N + 255) / 256) < 148 && tiles_m * ((N + 191) / 192) <= 148 &&
      tiles_m * ((N + 191) / 192) > tiles_m * ((N + 255) / 256))
    bn = 192;
  while (tiles_m == 1 && bn > 128 && (N + bn - 1) / bn < 74) bn >>= 1;
  if (g_bn == 128 && bn > 128) bn = 128;
  return bn;
}
// K splits for outputs of too few tiles to occupy the GPU (1 = none).
static int splits_for(int M, int N, int K, int bn) {
  const long tiles = (long)((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  const int k_tiles = (K + BK - 1) / BK;
  if (tiles >= 74 || k_tiles < 8) return 1;
  int s = (int)(148 / tiles);
  if (s > 8) s = 8;
  if (s > k_tiles / 4) s = k_tiles / 4;     // at least four k-steps per split
  return s < 2 ? 1 : s;
}

// Floats of workspace with which coheryn_gemm_bf16_tc splits K over several CTAs (0: this
// shape is not split).  Without the workspace the product runs unsplit.
CO_EXPORT long coheryn_gemm_tc_workspace_floats(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (pair_suits(M, N)) return 0;
  const int s = splits_for(M, N, K, tile_width(M, N));
  return s > 1 ? (long)s * M * N : 0;
}

CO_EXPORT int coheryn_gemm_bf16_tc_pair(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                                        int out_dtype, int M, int N, int K, long ldx, long ldo, int epilogue,
                                        int* status, cudaStream_t stream);

// x: [M, K] bfloat16 with row stride ldx; w: [N, K] bfloat16 contiguous; K and ldx multiples
// of 8, bases 16-byte aligned.  epilogue 0: out[M, N] (+ bias); 1: gated SiLU over
// interleaved rows of w, out[M, N/2].  status: device word that receives 11/12/13 if a
// bounded wait of the producer / the MMA issuer / the epilogue ran out (14: the issuer waiting
// for a free accumulator in the persistent variant).  workspace: see above, may be null.
CO_EXPORT int coheryn_gemm_bf16_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                                   int out_dtype, int M, int N, int K, long ldx, long ldo, int epilogue,
                                   int* status, float* workspace, long workspace_floats, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7)) CO_FAIL("gemm_bf16_tc: K = %d and the row stride %ld must be multiples of 8", K, ldx);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("gemm_bf16_tc: operands must be 16-byte aligned");
  if (epilogue == 1 && (N & 1)) CO_FAIL("gemm_bf16_tc: gated epilogue needs an even number of rows");
  if (epilogue != 0 && epilogue != 1) CO_FAIL("gemm_bf16_tc: unknown epilogue %d", epilogue);
  if (status && pair_suits(M, N))
    return coheryn_gemm_bf16_tc_pair(x, w, bias, bias_dtype, out, out_dtype, M, N, K, ldx, ldo, epilogue, status, stream);
  const int bn = tile_width(M, N);
  const long tiles_m = (M + BM - 1) / BM;
  int splits = splits_for(M, N, K, bn);
  if (splits > 1 && (!workspace || workspace_floats < (long)splits * M * N)) splits = 1;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, ldx, BM) || !make_map(&mw, w, N, K, K, bn))
    CO_FAIL("gemm_bf16_tc: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%ld)", M, N, K, ldx);
#define GO(BN_, ST_) return launch_tc<BN_, ST_>(mx, mw, bias, bias_dtype, out, out_dtype, M, N, K, ldo, epilogue, status, stream, workspace, splits)
  if (bn == 256 && g_stages != 1 && tiles_m * ((N + 255) / 256) > 148)
    return launch_tc_persistent<256, 4>(mx, mw, bias, bias_dtype, out, out_dtype, M, N, K, ldo, epilogue, status, stream);
  if (bn == 256 && g_stages == 2) GO(256, 2);
  if (bn == 256 && g_stages == 3) GO(256, 3);
  if (bn == 128 && g_stages == 3) GO(128, 3);
  if (bn == 256) GO(256, 4);
  if (bn == 192) GO(192, 4);
  if (bn == 128) GO(128, 6);
  if (bn == 64) GO(64, 8);
  GO(32, 8);
#undef GO
}

// How many K slices coheryn_gemm_bf16_tc_parts leaves for this shape (0 or 1: the shape is not split,
// use the ordinary entry).
CO_EXPORT int coheryn_gemm_tc_parts_count(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || pair_suits(M, N)) return 0;
  const int bn = tile_width(M, N);
  if (bn == 256 && (long)((M + BM - 1) / BM) * ((N + 255) / 256) > 148) return 0;
  const int s = splits_for(M, N, K, bn);
  if (s < 2) return 0;
  const int k_tiles = (K + BK - 1) / BK, per = (k_tiles + s - 1) / s;
  return (k_tiles + per - 1) / per;
}

// The product of a shape whose K is split, with the addition of the slices left to the consumer:
// parts receives float32 [count][M][N] (count = coheryn_gemm_tc_parts_count), no bias, no epilogue.
CO_EXPORT int coheryn_gemm_bf16_tc_parts(const void* x, const void* w, float* parts, int M, int N, int K, long ldx,
                                         int* status, cudaStream_t stream) {
  const int count = coheryn_gemm_tc_parts_count(M, N, K);
  if (count < 2) CO_FAIL("gemm_bf16_tc_parts: the shape M=%d N=%d K=%d is not split over K", M, N, K);
  if ((K & 7) || (ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("gemm_bf16_tc_parts: misaligned operands");
  const int bn = tile_width(M, N);
  const int splits = splits_for(M, N, K, bn);
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, ldx, BM) || !make_map(&mw, w, N, K, K, bn))
    CO_FAIL("gemm_bf16_tc_parts: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%ld)", M, N, K, ldx);
#define GO(BN_, ST_) return launch_tc<BN_, ST_>(mx, mw, nullptr, CO_F32, parts, CO_F32, M, N, K, (long)N, 0, status, stream, parts, splits, true)
  if (bn == 256) GO(256, 4);
  if (bn == 192) GO(192, 4);
  if (bn == 128) GO(128, 6);
  if (bn == 64) GO(64, 8);
  GO(32, 8);
#undef GO
}

// The same product by pairs of CTAs (see gemm_tc_pair_kernel): 256 x 256 tiles, for many rows.
// status receives 11 / 12 / 13 / 14 as above.
CO_EXPORT int coheryn_gemm_bf16_tc_pair(const void* x, const void* w, const void* bias, int bias_dtype, void* out,
                                        int out_dtype, int M, int N, int K, long ldx, long ldo, int epilogue,
                                        int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7)) CO_FAIL("gemm_bf16_tc_pair: K = %d and the row stride %ld must be multiples of 8", K, ldx);
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) CO_FAIL("gemm_bf16_tc_pair: operands must be 16-byte aligned");
  if (epilogue == 1 && (N & 1)) CO_FAIL("gemm_bf16_tc_pair: gated epilogue needs an even number of rows");
  if (epilogue != 0 && epilogue != 1) CO_FAIL("gemm_bf16_tc_pair: unknown epilogue %d", epilogue);
  if (!status) CO_FAIL("gemm_bf16_tc_pair: a status word is required");
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, ldx, BM) || !make_map(&mw, w, N, K, K, 128))
    CO_FAIL("gemm_bf16_tc_pair: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d ldx=%ld)", M, N, K, ldx);
  return launch_tc_pair<256, 6, 2>(mx, mw, bias, bias_dtype, out, out_dtype, M, N, K, ldo, epilogue, status, stream);
}
