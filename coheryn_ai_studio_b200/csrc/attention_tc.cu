// Causal (optionally windowed) grouped-query attention over cache pages for prompt portions
// on the 5th-generation tensor cores, compiled for one head size (CO_HEAD_DIM, a multiple of
// 64 up to 256).
//
// One CTA owns a tile of query rows of one (request, kv head): TOK = 128 / G whole tokens
// times the G heads of the group (row r = token * G + head), at most 128 rows = the lanes of
// tensor memory.  It walks the key positions the tile can see in tiles of 128:
//   warp 0     producer: the Q tile once (one 3-D TMA box per 64 columns), then per key tile
//              the K and V pages (2-D TMA boxes of one page, or of 128 rows of a larger page),
//              two stages deep;
//   warp 1     MMA issuer: S = Q K^T into tensor memory (tcgen05.mma, both operands K-major in
//              shared memory), and O += P V with P read from tensor memory and V in shared
//              memory as it lies in the cache (positions x head dim: operand B MN-major);
//   warps 2-9  softmax: two threads per row, each with half of the tile's key columns.  They
//              read their part of S, agree on the row's maximum, turn the scores into
//              probabilities (float32, log2 domain), write them as bfloat16 pairs into tensor
//              memory for the next MMA, and rescale their half of the row of O when the
//              reference maximum moved.  At the end they divide by the sum and store the row.
// S for the next key tile is issued as soon as the softmax threads hold the current one in
// registers, so the exponentials overlap the next Q K^T.
//
// A short portion over a long context makes few row tiles with many key tiles each.  The kernel
// then runs as clusters of 2, 4 or 8 CTAs along x that share a row tile: CTA r takes the key
// tiles [N r / C, N (r + 1) / C), all but the last publish their (reference maximum, sum,
// accumulator) in their own shared memory, and the last one, which always holds the diagonal
// tile, adds the parts in rank order through distributed shared memory and stores the rows.
//
// Slots of a page beyond the request's length, and pages a window has given back (table
// entry -1, fetched as an out-of-range box = zeros), are masked by position; the cache pool
// must hold finite numbers everywhere (it is zeroed when made).
// Every wait is bounded: on expiry the kernel records a code in `status` and winds down.
#include <cuda_bf16.h>

#include "attention_tc.h"
#include "tc_common.cuh"

#ifndef CO_HEAD_DIM
#define CO_HEAD_DIM 128
#endif

namespace {

typedef __nv_bfloat16 bf16;
constexpr int HD = CO_HEAD_DIM;
constexpr bool SUPPORTED = HD % 64 == 0 && HD <= 256;
constexpr int BN = 128;                          // key positions per tile
constexpr int KCH = SUPPORTED ? HD / 64 : 1;     // 64-column chunks of the head dim
constexpr int CHUNK_BYTES = 128 * 128;           // 128 rows of 128 bytes
constexpr int NST = HD <= 128 ? 3 : 1;           // K/V stages
constexpr int Q_BYTES = KCH * CHUNK_BYTES, KV_BYTES = KCH * CHUNK_BYTES;
constexpr int SMEM_BYTES = Q_BYTES + NST * 2 * KV_BYTES + 1024 /* alignment slack */ + 256 /* barriers */ + 1024 /* row_ex */;
constexpr int COL_S = 0, COL_O = 128, COL_P = 128 + HD;
constexpr int TMEM_COLS = COL_P + 64 <= 256 ? 256 : 512;
static_assert(!SUPPORTED || SMEM_BYTES <= 227 * 1024, "the stages fit shared memory");

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // ex2(-inf) = +0
  return y;
}

__device__ __forceinline__ unsigned cluster_rank() { unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ unsigned cluster_size() { unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Four floats from the same place in the shared memory of CTA `rank` of the cluster.
__device__ __forceinline__ float4 ld_cluster4(const float* local, unsigned rank) {
  unsigned ra;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(ra) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cluster1(const float* local, unsigned rank) {
  unsigned ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}
constexpr int XLD = HD + 4;                       // row stride (floats) of a CTA's published accumulator
constexpr int MAX_CLUSTER = 8;
static_assert(!SUPPORTED || (size_t)(128 * XLD + 256) * 4 <= (size_t)Q_BYTES + (size_t)NST * 2 * KV_BYTES, "a published accumulator fits the tiles");

__global__ void __launch_bounds__(320, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long out_stride,
               const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
               const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int cache_rows, int window,
               float scale_log2, int skip_small, int rows_per_box, int* __restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = tiles;                                   // [KCH][128 rows][128 B]
  unsigned char* kv_s = tiles + Q_BYTES;                        // [NST][K, V][KCH][128 rows][128 B]
  unsigned long long* bars = (unsigned long long*)(kv_s + NST * 2 * KV_BYTES);
  unsigned long long* q_full = bars;                // 1
  unsigned long long* k_full = bars + 1;            // [NST]
  unsigned long long* v_full = k_full + NST;        // [NST]
  unsigned long long* kv_empty = v_full + NST;      // [NST]
  unsigned long long* s_full = kv_empty + NST;      // MMA -> softmax: S is complete
  unsigned long long* s_free = s_full + 1;          // softmax -> MMA: S is in registers (256 arrivals)
  unsigned long long* p_full = s_free + 1;          // softmax -> MMA: P written, O rescaled (256 arrivals)
  unsigned long long* pv_done = p_full + 1;         // MMA -> softmax: O += P V is complete
  unsigned* tmem_slot = (unsigned*)(pv_done + 1);
  float (*row_ex)[128] = (float (*)[128])((unsigned char*)bars + 256);   // [half][row]: the two threads of a row meet here
  static_assert((5 + 3 * NST) * 8 + 4 <= 256, "barriers fit their slot");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1); mbar_init(s_free, 256); mbar_init(p_full, 256); mbar_init(pv_done, 1);
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
  co_pdl_wait();

  // Late row tiles see the most keys: they are started first.  The CTAs of a cluster (along x)
  // share a row tile and split its key tiles among them; the last one merges.
  const int csize = (int)cluster_size(), crank = (int)cluster_rank();
  const int b = blockIdx.z, kvh = blockIdx.y, rt = (int)(gridDim.x / csize) - 1 - (int)(blockIdx.x / csize);
  const int G = nh / nkv, TOK = 128 / G, RT = TOK * G;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  const bool active = rt * RT < rows && !(skip_small && rows <= 16);
  const int base_pos = kv_len - q_len;
  const int row_first = rt * RT, row_last = min(rows, row_first + RT) - 1;
  const int pos_lo = base_pos + row_first / G, pos_hi = base_pos + row_last / G;
  const int key_first = window > 0 ? max(0, pos_lo - window + 1) : 0;
  const int all_tiles = active ? pos_hi / BN - key_first / BN + 1 : 0;        // of the row tile
  const int my_first = all_tiles * crank / csize;                             // rank r: tiles [N r / C, N (r + 1) / C)
  const int n_tiles = all_tiles * (crank + 1) / csize - my_first;             // of this CTA (0 only below the last rank)
  const int tile_first = key_first / BN + my_first;                           // this CTA's first key tile
  const bool merger = crank == csize - 1;
  float* xfer = reinterpret_cast<float*>(q_s);                                // [128][XLD] accumulator, then m[128], l[128]: over the tiles
  // softmax threads' state, finished after the cluster has met
  float m = -INFINITY, l = 0.f;
  bool ok = true;

  if (warp == 0) {
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, (unsigned)(KCH * RT * 128));
        for (int c = 0; c < KCH; ++c) tma_load_3d(q_s + c * CHUNK_BYTES, &map_q, c * 64, kvh * G, tok0 + rt * TOK, q_full);
      }
      const int* table = block_tables + (size_t)b * max_blocks;
      const int boxes = BN / rows_per_box;       // lane i < boxes fetches box i of every tile
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % NST;
        if (j >= NST) {
          if (lane == 0 && !mbar_wait(&kv_empty[s], (unsigned)((j / NST) - 1) & 1)) { atomicExch(status, 31); ok = false; }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
        }
        unsigned char* k_dst = kv_s + (size_t)s * 2 * KV_BYTES;
        unsigned char* v_dst = k_dst + KV_BYTES;
        if (lane == 0) {
          mbar_expect_tx(&k_full[s], (unsigned)KV_BYTES);
          mbar_expect_tx(&v_full[s], (unsigned)KV_BYTES);
        }
        __syncwarp();
        for (int i = lane; i < boxes; i += 32) {
          const int pos = (tile_first + j) * BN + i * rows_per_box;
          const int blk = pos / page_size;
          const int page = blk < max_blocks ? table[blk] : -1;
          // a page that is not there: a box beyond the tensor, fetched as zeros
          const int row = page >= 0 ? (page * nkv + kvh) * page_size + (pos - blk * page_size) : cache_rows;
          for (int c = 0; c < KCH; ++c)
            tma_load_2d(k_dst + c * CHUNK_BYTES + i * rows_per_box * 128, &map_k, c * 64, row, &k_full[s]);
          for (int c = 0; c < KCH; ++c)
            tma_load_2d(v_dst + c * CHUNK_BYTES + i * rows_per_box * 128, &map_v, c * 64, row, &v_full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr unsigned idesc_qk = umma_idesc(128, BN);
      constexpr unsigned idesc_pv = umma_idesc_b_mn(128, HD);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, 32);
      auto issue_qk = [&](int j) {
        const int s = j % NST;
        if (!mbar_wait(&k_full[s], (unsigned)(j / NST) & 1)) { atomicExch(status, 33); return false; }
        if (j > 0 && !mbar_wait(s_free, (unsigned)(j - 1) & 1)) { atomicExch(status, 34); return false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* k_src = kv_s + (size_t)s * 2 * KV_BYTES;
#pragma unroll
        for (int c = 0; c < KCH; ++c) {
          const unsigned long long dq = umma_desc(q_s + c * CHUNK_BYTES), dk = umma_desc(k_src + c * CHUNK_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + COL_S, dq + 2 * k, dk + 2 * k, idesc_qk, (c | k) != 0);
        }
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        // With two stages the next S is issued before this tile's P V (its keys are there
        // already); with one, the next keys only arrive after P V has released the stage.
        if (NST > 1 && j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const int s = j % NST;
        if (!mbar_wait(p_full, (unsigned)j & 1)) { atomicExch(status, 35); break; }
        if (!mbar_wait(&v_full[s], (unsigned)(j / NST) & 1)) { atomicExch(status, 36); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned char* v_src = kv_s + (size_t)s * 2 * KV_BYTES + KV_BYTES;
        // One MMA per 16 positions over the whole head dim: operand B MN-major, its 64-column
        // chunks CHUNK_BYTES apart (the leading offset), groups of eight positions 1024 bytes
        // apart (the stride offset).
        const unsigned long long dv = umma_desc_offsets(v_src, CHUNK_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk)   // 16 positions = 16 rows of 128 bytes further per step
          umma_bf16_a_tmem(tmem_base + COL_O, tmem_base + COL_P + kk * 8, dv + (unsigned long long)(kk * 128), idesc_pv,
                           (j | kk) != 0);
        umma_commit(&kv_empty[s]);
        umma_commit(pv_done);
        if (NST == 1 && j + 1 < n_tiles) ok = issue_qk(j + 1);
      }
    }
  } else if (n_tiles > 0) {
    // Softmax warps 2..9: TMEM lane quarter = warp % 4; two threads share a row, warps 2..5
    // taking key columns 0..63 of every tile (and the first half of the head dim of O), warps
    // 6..9 the rest.  The pair sits on one scheduler, so one's latencies hide behind the other.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    const bool valid = row < RT && row_first + row < rows;
    const int pos = base_pos + (row_first + row) / G;
    const int hi = valid ? pos : -1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(s_full, (unsigned)j & 1)) { if (lane == 0) atomicExch(status, 37); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      unsigned sr[2][32];
      tmem_ld32_nowait(lane_addr + COL_S + half * 64, sr[0]);
      tmem_ld32_nowait(lane_addr + COL_S + half * 64 + 32, sr[1]);
      tmem_wait_ld();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(s_free);
      const int key0 = (tile_first + j) * BN + half * 64;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (key0 >= lo && key0 + 63 <= hi) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[i][c]));
      } else {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = key0 + i * 32 + c;
            if (key < lo || key > hi) sr[i][c] = __float_as_uint(-INFINITY);
            mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[i][c]));
          }
      }
      // The row's maximum over both halves, through shared memory: the pair of warps meets
      // once to publish and once more before the slots are written again.
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      row_ex[half][row] = mx;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      mx = fmaxf(mx, row_ex[half ^ 1][row]);
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      // The exponent's reference point m follows the running maximum LAZILY: it moves only when
      // some row of the warp has outgrown it by more than 2^8 (p then stays below 256, far inside
      // bfloat16's range), because moving it costs a pass over the row of O in tensor memory.
      // Both threads of a row see the same numbers and decide alike.
      const float m_row = fmaxf(m, mx * scale_log2);            // scale > 0 keeps the order
      const bool move = m == -INFINITY ? m_row != -INFINITY : m_row - m > 8.0f;
      const bool moved = __any_sync(0xffffffffu, move);
      const float m_new = moved ? m_row : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;    // everything masked so far: every p is zero
      const float corr = ex2_approx(m - m_use);
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned pr[32];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          sr[i][c] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(sr[i][c]), scale_log2, -m_use)));
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float p0 = __uint_as_float(sr[i][c]), p1 = __uint_as_float(sr[i][c + 1]);
          sum4[(c >> 1) & 3] += p0 + p1;
          __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
          pr[i * 16 + (c >> 1)] = *reinterpret_cast<unsigned*>(&h);
        }
      }
      l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m = m_new;
      if (j > 0) {
        if (!mbar_wait(pv_done, (unsigned)(j - 1) & 1)) { if (lane == 0) atomicExch(status, 38); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (moved) {
#pragma unroll 1
          for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
            unsigned o[32];
            tmem_ld32(lane_addr + COL_O + c0, o);
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
            tmem_st32(lane_addr + COL_O + c0, o);
          }
        }
      }
      tmem_st32(lane_addr + COL_P + half * 32, pr);
      tmem_wait_st();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(p_full);
    }
    if (ok) {
      if (!mbar_wait(pv_done, (unsigned)(n_tiles - 1) & 1)) { if (lane == 0) atomicExch(status, 39); ok = false; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    // The row's sum: the first half's plus the second's.
    row_ex[half][row] = l;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
    l = row_ex[0][row] + row_ex[1][row];
    if (!merger) {
      // Publish (reference maximum, sum, accumulator) over the Q and K/V tiles, which nothing reads
      // any more: the last MMA is complete.
      if (half == 0) { xfer[128 * XLD + row] = m; xfer[128 * XLD + 128 + row] = l; }
#pragma unroll 1
      for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
        unsigned o[32];
        tmem_ld32(lane_addr + COL_O + c0, o);
#pragma unroll
        for (int c = 0; c < 32; c += 4)
          *reinterpret_cast<float4*>(xfer + row * XLD + c0 + c) =
              make_float4(__uint_as_float(o[c]), __uint_as_float(o[c + 1]), __uint_as_float(o[c + 2]), __uint_as_float(o[c + 3]));
      }
    }
  }

  // The cluster meets: the parts are published.  (Every thread of every CTA comes here, whatever
  // happened in its role, so nobody waits for a CTA that gave up.)
  const bool clustered = csize > 1 && all_tiles > 0;
  if (clustered) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_barrier();
  }
  if (warp >= 2 && merger && n_tiles > 0 && ok) {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
    const bool valid = row < RT && row_first + row < rows;
    // Parts of the other CTAs that had key tiles, in rank order; factors relative to the largest
    // reference maximum.
    float pm[MAX_CLUSTER], pl[MAX_CLUSTER];
    float M = m;
#pragma unroll
    for (int p = 0; p < MAX_CLUSTER - 1; ++p) {
      pm[p] = -INFINITY; pl[p] = 0.f;
      if (p < csize - 1 && all_tiles * (p + 1) / csize - all_tiles * p / csize > 0) {
        pm[p] = ld_cluster1(xfer + 128 * XLD + row, (unsigned)p);
        pl[p] = ld_cluster1(xfer + 128 * XLD + 128 + row, (unsigned)p);
        M = fmaxf(M, pm[p]);
      }
    }
    const float M_use = M == -INFINITY ? 0.f : M;
    const float f_own = ex2_approx(m - M_use);
    float den = l * f_own;
#pragma unroll
    for (int p = 0; p < MAX_CLUSTER - 1; ++p) {
      pm[p] = ex2_approx(pm[p] - M_use);           // now the part's factor (0 for a part without tiles)
      den += pl[p] * pm[p];
    }
    const float inv = 1.0f / den;
    const int rr = row_first + row;
    bf16* orow = out + (size_t)(tok0 + rr / G) * out_stride + (size_t)(kvh * G + rr % G) * HD;
#pragma unroll 1
    for (int c0 = half * (HD / 2); c0 < (half + 1) * (HD / 2); c0 += 32) {
      unsigned o[32];
      tmem_ld32(lane_addr + COL_O + c0, o);     // warp-collective: invalid rows read too, and skip the store
      float v[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(o[c]) * f_own;
#pragma unroll 1
      for (int p = 0; p < csize - 1; ++p) {
        if (pm[p] == 0.f) continue;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 x = ld_cluster4(xfer + row * XLD + c0 + c, (unsigned)p);
          v[c] += x.x * pm[p]; v[c + 1] += x.y * pm[p]; v[c + 2] += x.z * pm[p]; v[c + 3] += x.w * pm[p];
        }
      }
      if (valid) {
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          __nv_bfloat162 a = __floats2bfloat162_rn(v[c] * inv, v[c + 1] * inv);
          __nv_bfloat162 d = __floats2bfloat162_rn(v[c + 2] * inv, v[c + 3] * inv);
          uint2 raw;
          raw.x = *reinterpret_cast<unsigned*>(&a);
          raw.y = *reinterpret_cast<unsigned*>(&d);
          *reinterpret_cast<uint2*>(orow + c0 + c) = raw;
        }
      }
    }
  }
  if (clustered) cluster_barrier();   // nobody leaves while its published part may still be read

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(TMEM_COLS) : "memory");
  }
}

}  // namespace

static int g_forced_cluster = -1;   // -1: the environment decides at the first launch; 0: by shape
void coheryn_attention_tc_set_cluster(int cluster) { g_forced_cluster = cluster; }

bool coheryn_attention_tc_takes(int nh, int nkv, int page_size) {
  if (!SUPPORTED || nkv <= 0 || nh % nkv) return false;
  const int G = nh / nkv;
  if (G > 128) return false;
  const char* e = getenv("COHERYN_ATTN_TC");
  if (e && e[0] == '0') return false;
  return page_size >= 8 && (BN % page_size == 0 || page_size % BN == 0);   // a box is whole pages of >= 1024 bytes
}

int coheryn_attention_tc_launch(const void* q, long q_stride, int total_tokens, void* out, long out_stride,
                                const void* k_cache, const void* v_cache, int num_pages, const int* block_tables,
                                int max_blocks, const int* cu_q, const int* kv_lens, int B, int nh, int nkv,
                                int page_size, int window, float scale_log2, int max_rows, int max_kv_len, int skip_small,
                                int* status, cudaStream_t stream) {
  if (!SUPPORTED) CO_FAIL("attention_tc: head size %d is not a multiple of 64 up to 256", HD);
  const int G = nh / nkv, TOK = 128 / G, RT = TOK * G;
  const int rows_per_box = page_size < BN ? page_size : BN;
  const long cache_rows = (long)num_pages * nkv * page_size;
  if (cache_rows >= (1L << 31)) CO_FAIL("attention_tc: the cache holds %ld rows per tensor, beyond 2^31", cache_rows);
  CUtensorMap mq, mk, mv;
  {
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)total_tokens};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_stride * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)TOK};
    if (!make_map_nd(&mq, q, 3, dims, strides, box)) CO_FAIL("attention_tc: the query tensor map was refused");
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)cache_rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)rows_per_box};
    if (!make_map_nd(&mk, k_cache, 2, dims, strides, box) || !make_map_nd(&mv, v_cache, 2, dims, strides, box))
      CO_FAIL("attention_tc: the cache tensor map was refused");
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) CO_FAIL("attention_tc: %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
    configured = true;
  }
  // CTAs per row tile (a cluster that splits the tile's keys): more while even the split leaves SMs
  // idle (a short portion over a long context) and every CTA still gets eight key tiles or more; a
  // CTA's fixed cost is several key tiles' worth, so a batch that fills the GPU stays unsplit.
  // COHERYN_ATTN_TC_CLUSTER in the environment or coheryn_attention_tc_set_cluster fixes it.
  const int row_tiles = (max_rows + RT - 1) / RT;
  const long ctas = (long)row_tiles * nkv * B;
  const int key_tiles = (max_kv_len + BN - 1) / BN;
  if (g_forced_cluster < 0) g_forced_cluster = getenv("COHERYN_ATTN_TC_CLUSTER") ? atoi(getenv("COHERYN_ATTN_TC_CLUSTER")) : 0;
  const int forced = g_forced_cluster;
  int cluster = 1;
  while (cluster < MAX_CLUSTER && ctas * cluster * 2 <= 148L && key_tiles >= 16 * cluster) cluster *= 2;
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) cluster = forced;
  dim3 grid(row_tiles * cluster, nkv, B);
  cudaError_t le = co_launch_cluster(cluster, attn_tc_kernel, grid, dim3(320), (size_t)SMEM_BYTES, stream, mq, mk, mv, (bf16*)out,
                                     out_stride, block_tables, max_blocks, cu_q, kv_lens, nh, nkv, page_size, (int)cache_rows,
                                     window, scale_log2, skip_small, rows_per_box, status);
  if (le != cudaSuccess) CO_FAIL("attention_tc: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("attn_tc");
  return 0;
}
