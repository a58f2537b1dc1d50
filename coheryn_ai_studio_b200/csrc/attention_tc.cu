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
// registers, so the exponentials overlap the next Q K^T.  (attn_tc2_kernel further down gives a
// CTA two row tiles that share every fetched key tile; it takes long prompts.)
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
// The rows of a query tile beyond its RT = TOK * G whole tokens are not fetched; they are zeroed (by the
// thread that issues the MMAs, once the tile has landed) so that their scores are 0 and their softmax
// threads, whose results nobody reads, walk the same path as the others.
__device__ __forceinline__ void zero_spare_rows(unsigned char* q_tile, int RT) {
  for (int c = 0; c < KCH; ++c)
    for (int r = RT; r < 128; ++r)
      for (int piece = 0; piece < 8; ++piece)
        *reinterpret_cast<uint4*>(q_tile + c * CHUNK_BYTES + r * 128 + piece * 16) = make_uint4(0, 0, 0, 0);
  fence_proxy_async();
}
constexpr int XLD = HD + 4;                       // row stride (floats) of a CTA's published accumulator
constexpr int MAX_CLUSTER = 8;
static_assert(!SUPPORTED || (size_t)(128 * XLD + 256) * 4 <= (size_t)Q_BYTES + (size_t)NST * 2 * KV_BYTES, "a published accumulator fits the tiles");

__global__ void __launch_bounds__(320, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long out_stride,
               const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
               const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int cache_rows, int window,
               float scale_log2, int skip_small, int rows_per_box, int* __restrict__ status, int n_req, int n_units) {
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
  unsigned long long* s_free = s_full + 1;          // softmax -> MMA: S is in registers (one arrival per warp)
  unsigned long long* p_full = s_free + 1;          // softmax -> MMA: P written, O rescaled (one arrival per warp)
  unsigned long long* pv_done = p_full + 1;         // MMA -> softmax: O += P V is complete
  unsigned* tmem_slot = (unsigned*)(pv_done + 1);
  float (*row_ex)[128] = (float (*)[128])((unsigned char*)bars + 256);   // [half][row]: the two threads of a row meet here
  static_assert((5 + 3 * NST) * 8 + 4 <= 256, "barriers fit their slot");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < NST; ++s) { mbar_init(&k_full[s], 1); mbar_init(&v_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1); mbar_init(s_free, 8); mbar_init(p_full, 8); mbar_init(pv_done, 1);
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

  // Late row tiles see the most keys: they are started first, for ALL (request, kv head) pairs before
  // any earlier row tile (the grid is one-dimensional and the row tile its slowest index; CTAs start
  // in the order of their index).  The CTAs of a cluster (consecutive indices) share a row tile and
  // split its key tiles among them; the last one merges.
  const int csize = (int)cluster_size(), crank = (int)cluster_rank();
  const int unit = (int)(blockIdx.x / csize), heads_reqs = nkv * n_req;
  const int b = (unit % heads_reqs) / nkv, kvh = unit % nkv, rt = n_units - 1 - unit / heads_reqs;
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
      zero_spare_rows(q_s, RT);
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
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      const int key0 = (tile_first + j) * BN + half * 64;
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (!valid || (key0 >= lo && key0 + 63 <= hi)) {
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
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
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


// ------------------------------------------------------------------------------------------
// Two query tiles per CTA.  Every CTA of a (request, kv head) streams the same keys and values
// out of L2, and with one tile of 128 rows per CTA that stream, not the tensor pipe or the
// softmax, bounds the kernel (8.4 MFLOP per 64 KB).  Here a CTA owns two consecutive row tiles
// A and B (256 rows) and fetches every key tile once for both: S_A, S_B, O_A, O_B fill the 512
// columns of tensor memory.  A tile's chain S -> softmax -> P -> P V is kept from being serial:
//   * one softmax thread per row (warps 2-5 tile A, 6-9 tile B; one of each per scheduler) takes
//     the row's 128 scores into registers and hands the score buffer back at once, so the next
//     Q K^T of the tile runs while the exponentials are computed;
//   * the probabilities go to SHARED memory (128 x 128 bfloat16 per row tile, written row by row
//     in the 128-byte swizzle) and P V reads both operands from there;
//   * the MMA thread issues Q K_A^T(j+1), Q K_B^T(j+1), P V_A(j), P V_B(j): the products of one
//     tile run while the other tile's softmax works.
// Key tiles are 128 positions (an MMA instruction takes about 70 cycles however narrow it is).
// Two K stages and one V stage, released separately; K runs one tile ahead of V.  Tile A sees
// fewer keys than tile B by at most one key tile and stops early.  Head sizes up to 128.
constexpr bool TWO_OK = SUPPORTED && HD <= 128;
constexpr int NKS2 = 2;                           // K stages (V has one)
constexpr int P2_BYTES = 2 * CHUNK_BYTES;         // 128 rows x 128 bfloat16, as two 64-column chunks
constexpr int SMEM2_BYTES = 2 * Q_BYTES + (NKS2 + 1) * KV_BYTES + 2 * P2_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
static_assert(!TWO_OK || SMEM2_BYTES <= 227 * 1024, "two query tiles, the stages and the probabilities fit shared memory");

__global__ void __launch_bounds__(320, 1)
attn_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long out_stride,
                const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int cache_rows, int window,
                float scale_log2, int skip_small, int rows_per_box, int* __restrict__ status, int n_req, int n_units) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_s = tiles;                                   // [tile][KCH][128 rows][128 B]
  unsigned char* k_s = q_s + 2 * Q_BYTES;                       // [NKS2][KCH][128 rows][128 B]
  unsigned char* v_s = k_s + NKS2 * KV_BYTES;                   // [KCH][128 rows][128 B]
  unsigned char* p_s = v_s + KV_BYTES;                          // [tile][2][128 rows][128 B]
  unsigned long long* bars = (unsigned long long*)(p_s + 2 * P2_BYTES);
  unsigned long long* q_full = bars;                // 1
  unsigned long long* k_full = bars + 1;            // [NKS2]
  unsigned long long* k_empty = k_full + NKS2;      // [NKS2] both tiles' Q K^T have read the stage
  unsigned long long* v_full = k_empty + NKS2;      // 1
  unsigned long long* v_empty = v_full + 1;         // 1: both tiles' P V have read the stage
  unsigned long long* s_full = v_empty + 1;         // [tile] MMA -> softmax: S is complete
  unsigned long long* s_free = s_full + 2;          // [tile] softmax -> MMA: S is in registers (one arrival per warp)
  unsigned long long* p_full = s_free + 2;          // [tile] softmax -> MMA: P written, O rescaled (one arrival per warp)
  unsigned long long* pv_done = p_full + 2;         // [tile] MMA -> softmax: O += P V is complete
  unsigned* tmem_slot = (unsigned*)(pv_done + 2);
  static_assert((3 + 2 * NKS2 + 8) * 8 + 4 <= 256, "barriers fit their slot");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    for (int s = 0; s < NKS2; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&s_free[t], 4); mbar_init(&p_full[t], 4); mbar_init(&pv_done[t], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem_base = *tmem_slot;
  co_pdl_launch_dependents();
  co_pdl_wait();

  // Late rows see the most keys: their pairs of tiles are started first, for all (request, kv head)
  // pairs before any earlier pair of tiles (one-dimensional grid, the pair of tiles its slowest index).
  const int unit = (int)blockIdx.x, heads_reqs = nkv * n_req;
  const int b = (unit % heads_reqs) / nkv, kvh = unit % nkv, pair = n_units - 1 - unit / heads_reqs;
  const int G = nh / nkv, TOK = 128 / G, RT = TOK * G;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  const bool active_a = 2 * pair * RT < rows && !(skip_small && rows <= 16);
  const bool active_b = active_a && (2 * pair + 1) * RT < rows;
  const int base_pos = kv_len - q_len;
  const int first_a = 2 * pair * RT, first_b = first_a + RT;
  const int last_a = min(rows, first_a + RT) - 1, last_b = min(rows, first_b + RT) - 1;
  const int pos_lo = base_pos + first_a / G;                                  // the pair's first position
  const int pos_hi_a = base_pos + last_a / G, pos_hi_b = base_pos + last_b / G;
  const int key_first = window > 0 ? max(0, pos_lo - window + 1) : 0;
  const int tile_first = key_first / BN;
  const int n_a = active_a ? pos_hi_a / BN - tile_first + 1 : 0;              // key tiles of tile A, of tile B
  const int n_b = active_b ? pos_hi_b / BN - tile_first + 1 : 0;
  const int n_tiles = n_b > n_a ? n_b : n_a;

  if (warp == 0) {
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(q_full, (unsigned)(KCH * RT * 128 * (active_b ? 2 : 1)));
        for (int t = 0; t < (active_b ? 2 : 1); ++t)
          for (int c = 0; c < KCH; ++c)
            tma_load_3d(q_s + t * Q_BYTES + c * CHUNK_BYTES, &map_q, c * 64, kvh * G, tok0 + (2 * pair + t) * TOK, q_full);
      }
      const int* table = block_tables + (size_t)b * max_blocks;
      const int boxes = BN / rows_per_box;       // lane i < boxes fetches box i of every tile
      // The first row of this lane's box of key tile j in the cache tensors.  A page that is not
      // there: a box beyond the tensor, fetched as zeros.
      auto box_row = [&](int j) {
        if (lane >= boxes || j >= n_tiles) return 0;
        const int pos = (tile_first + j) * BN + lane * rows_per_box;
        const int blk = pos / page_size;
        const int page = blk < max_blocks ? table[blk] : -1;
        return page >= 0 ? (page * nkv + kvh) * page_size + (pos - blk * page_size) : cache_rows;
      };
      auto fetch = [&](const CUtensorMap* map, unsigned char* dst, int row, unsigned long long* full) {
        if (lane == 0) mbar_expect_tx(full, (unsigned)KV_BYTES);
        __syncwarp();
        if (lane < boxes)
          for (int c = 0; c < KCH; ++c) tma_load_2d(dst + c * CHUNK_BYTES + lane * rows_per_box * 128, map, c * 64, row, full);
      };
      auto wait_for = [&](unsigned long long* bar, unsigned parity) {
        int ok = 1;
        if (lane == 0 && !mbar_wait(bar, parity)) { atomicExch(status, 31); ok = 0; }
        return __shfl_sync(0xffffffffu, ok, 0) != 0;
      };
      // K runs one tile ahead of V: K(0), then K(i + 1) and V(i).  The table entries of a tile are
      // read one step before they are needed.
      int row_v = box_row(0), row_k = box_row(1);
      fetch(&map_k, k_s, row_v, &k_full[0]);
      bool ok = true;
      for (int i = 0; i < n_tiles && ok; ++i) {
        const int row_next = box_row(i + 2);
        if (i + 1 < n_tiles) {
          const int s = (i + 1) % NKS2;
          if (i + 1 >= NKS2) ok = wait_for(&k_empty[s], (unsigned)(((i + 1) / NKS2) - 1) & 1);
          if (!ok) break;
          fetch(&map_k, k_s + (size_t)s * KV_BYTES, row_k, &k_full[s]);
        }
        if (i >= 1) ok = wait_for(v_empty, (unsigned)(i - 1) & 1);
        if (!ok) break;
        fetch(&map_v, v_s, row_v, v_full);
        row_v = row_k; row_k = row_next;
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr unsigned idesc_qk = umma_idesc(128, BN);
      constexpr unsigned idesc_pv = umma_idesc_b_mn(128, HD);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicExch(status, 32);
      zero_spare_rows(q_s, RT);
      zero_spare_rows(q_s + Q_BYTES, RT);
      auto issue_qk = [&](int t, int j) {        // S_t = Q_t K(j)^T; K(j) has landed and S_t is free
        const unsigned char* k_src = k_s + (size_t)(j % NKS2) * KV_BYTES;
#pragma unroll
        for (int c = 0; c < KCH; ++c) {
          const unsigned long long dq = umma_desc(q_s + t * Q_BYTES + c * CHUNK_BYTES), dk = umma_desc(k_src + c * CHUNK_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_base + 128 * t, dq + 2 * k, dk + 2 * k, idesc_qk, (c | k) != 0);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int j) {        // O_t += P_t V(j); P and V(j) have been waited for
        const unsigned long long dv = umma_desc_offsets(v_s, CHUNK_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {   // 16 positions: 32 bytes along a row of P (64 per chunk), 16 rows of V further
          const unsigned long long dp = umma_desc(p_s + t * P2_BYTES + (kk >> 2) * CHUNK_BYTES) + 2 * (kk & 3);
          umma_bf16(tmem_base + 256 + 128 * t, dp, dv + (unsigned long long)(kk * 128), idesc_pv, (j | kk) != 0);
        }
        umma_commit(&pv_done[t]);
      };
      if (ok && !mbar_wait(&k_full[0], 0)) { atomicExch(status, 33); ok = false; }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_qk(0, 0);
        if (n_b > 0) issue_qk(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        // The next scores first: they wait only for the softmax threads to hold S(j) in registers.
        if (j + 1 < n_tiles) {
          if (!mbar_wait(&k_full[(j + 1) % NKS2], (unsigned)((j + 1) / NKS2) & 1)) { atomicExch(status, 33); ok = false; break; }
          for (int t = 0; t < 2 && ok; ++t)
            if (j + 1 < (t ? n_b : n_a)) {
              if (!mbar_wait(&s_free[t], (unsigned)j & 1)) { atomicExch(status, 34); ok = false; break; }
              asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
              issue_qk(t, j + 1);
            }
          if (!ok) break;
          umma_commit(&k_empty[(j + 1) % NKS2]);
        }
        for (int t = 0; t < 2 && ok; ++t)
          if (j < (t ? n_b : n_a)) {
            if (!mbar_wait(&p_full[t], (unsigned)j & 1)) { atomicExch(status, 35); ok = false; break; }
            if (!mbar_wait(v_full, (unsigned)j & 1)) { atomicExch(status, 36); ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_pv(t, j);
          }
        if (!ok) break;
        umma_commit(v_empty);
      }
    }
  } else {
    // Softmax warps: 2..5 for tile A, 6..9 for tile B; TMEM lane quarter = warp % 4; one thread per row.
    const int t = warp >= 6 ? 1 : 0;
    const int quarter = warp & 3;
    const int my_tiles = t ? n_b : n_a;
    if (my_tiles > 0) {
      const int row = quarter * 32 + lane;
      const int row_first = t ? first_b : first_a;
      const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);
      const unsigned col_s = 128 * t, col_o = 256 + 128 * t;
      unsigned char* p_row = p_s + t * P2_BYTES + row * 128;
      const bool valid = row < RT && row_first + row < rows;
      const int pos = base_pos + (row_first + row) / G;
      const int hi = valid ? pos : -1;
      const int lo = window > 0 ? max(0, pos - window + 1) : 0;
      float m = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j < my_tiles; ++j) {
        if (!mbar_wait(&s_full[t], (unsigned)j & 1)) { if (lane == 0) atomicExch(status, 37); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        unsigned sr[4][32];
#pragma unroll
        for (int i = 0; i < 4; ++i) tmem_ld32_nowait(lane_addr + col_s + 32 * i, sr[i]);
        tmem_wait_ld();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[t]);
        const int key0 = (tile_first + j) * BN;
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (!valid || (key0 >= lo && key0 + BN - 1 <= hi)) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[i][c]));
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int key = key0 + i * 32 + c;
              if (key < lo || key > hi) sr[i][c] = __float_as_uint(-INFINITY);
              mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[i][c]));
            }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // The reference point m follows the running maximum lazily (see attn_tc_kernel); the warp
        // decides together, because rescaling O is a warp-wide access to tensor memory.
        const float m_row = fmaxf(m, mx * scale_log2);
        const bool move = m == -INFINITY ? m_row != -INFINITY : m_row - m > 8.0f;
        const bool moved = __any_sync(0xffffffffu, move);
        const float m_new = moved ? m_row : m;
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        const float corr = ex2_approx(m - m_use);
        if (j > 0) {
          // P V(j - 1) has read the P tile that is about to be overwritten, and O is whole again
          if (!mbar_wait(&pv_done[t], (unsigned)(j - 1) & 1)) { if (lane == 0) atomicExch(status, 38); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (moved) {
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
              unsigned o[32];
              tmem_ld32(lane_addr + col_o + c0, o);
#pragma unroll
              for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * corr);
              tmem_st32(lane_addr + col_o + c0, o);
            }
            tmem_wait_st();
          }
        }
        // Exponentials, 32 columns at a time, each group packed and stored at once: row `row` of
        // chunk i / 2 of the P tile, 16-byte piece c at c ^ (row % 8).
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          unsigned pr[16];
#pragma unroll
          for (int c = 0; c < 32; ++c)
            sr[i][c] = __float_as_uint(ex2_approx(fmaf(__uint_as_float(sr[i][c]), scale_log2, -m_use)));
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = __uint_as_float(sr[i][c]), p1 = __uint_as_float(sr[i][c + 1]);
            sum4[(c >> 1) & 3] += p0 + p1;
            __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
            pr[c >> 1] = *reinterpret_cast<unsigned*>(&h);
          }
          unsigned char* dst = p_row + (i >> 1) * CHUNK_BYTES;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(dst + ((((i & 1) * 4 + c) ^ (row & 7)) << 4)) = make_uint4(pr[4 * c], pr[4 * c + 1], pr[4 * c + 2], pr[4 * c + 3]);
        }
        l = l * corr + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
        m = m_new;
        fence_proxy_async();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      if (ok) {
        if (!mbar_wait(&pv_done[t], (unsigned)(my_tiles - 1) & 1)) { if (lane == 0) atomicExch(status, 39); ok = false; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (ok) {
        const float inv = 1.0f / l;
        const int rr = row_first + row;
        bf16* orow = out + (size_t)(tok0 + rr / G) * out_stride + (size_t)(kvh * G + rr % G) * HD;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          unsigned o[32];
          tmem_ld32(lane_addr + col_o + c0, o);     // warp-collective: invalid rows read too, and skip the store
          if (valid) {
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
              __nv_bfloat162 d = __floats2bfloat162_rn(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
              uint2 raw;
              raw.x = *reinterpret_cast<unsigned*>(&a);
              raw.y = *reinterpret_cast<unsigned*>(&d);
              *reinterpret_cast<uint2*>(orow + c0 + c) = raw;
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(512) : "memory");
  }
}

}  // namespace

static int g_forced_cluster = -1;   // -1: the environment decides at the first launch; 0: by shape
void coheryn_attention_tc_set_cluster(int cluster) { g_forced_cluster = cluster; }
static int g_two_tiles = -1;        // -1: the environment decides at the first launch; 0 never, 1 always, 2 by the number of CTAs
void coheryn_attention_tc_set_two_tiles(int mode) { g_two_tiles = mode < 0 || mode > 2 ? 2 : mode; }

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
  if (g_two_tiles < 0) { const char* e = getenv("COHERYN_ATTN_TC_TWO"); g_two_tiles = e ? (e[0] == '0' ? 0 : e[0] == '1' ? 1 : 2) : 2; }
  // Two row tiles per CTA (every key tile fetched once for 256 rows) once the pairs still fill the
  // GPU with a quarter to spare: measured at 12 query heads in 2 groups, 4,096 tokens (196 CTAs)
  // 96 against 109 us, 16,384 tokens 0.91 against 1.25 ms, but 2,048 tokens (98 CTAs) 53 against 37.
  // A portion at the end of a long context has few row tiles and many key tiles each; there the pairs
  // pay from somewhat over half the SMs on (2,048 tokens after 14,336: 98 CTAs, 331 against 405 us;
  // 40 heads in 8 groups, 512 tokens after 15,872: 88 CTAs, 326 against 448; but 60 CTAs: 317 against 227).
  const long pair_ctas = (long)((row_tiles + 1) / 2) * nkv * B;
  const bool pairs_pay = pair_ctas >= 185 || (pair_ctas >= 84 && key_tiles >= 48);
  if (TWO_OK && cluster == 1 && row_tiles >= 2 && (g_two_tiles == 1 || (g_two_tiles == 2 && pairs_pay))) {
    static bool configured2 = false;
    if (!configured2) {
      cudaError_t e = cudaFuncSetAttribute(attn_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM2_BYTES);
      if (e != cudaSuccess) CO_FAIL("attention_tc: %d bytes of shared memory: %s", SMEM2_BYTES, cudaGetErrorString(e));
      configured2 = true;
    }
    const int pairs = (row_tiles + 1) / 2;
    if (pair_ctas >= (1L << 31)) CO_FAIL("attention_tc: %ld CTAs", pair_ctas);
    dim3 grid2((unsigned)pair_ctas);
    cudaError_t le2 = co_launch(attn_tc2_kernel, grid2, dim3(320), (size_t)SMEM2_BYTES, stream, mq, mk, mv, (bf16*)out, out_stride,
                                block_tables, max_blocks, cu_q, kv_lens, nh, nkv, page_size, (int)cache_rows, window, scale_log2,
                                skip_small, rows_per_box, status, B, pairs);
    if (le2 != cudaSuccess) CO_FAIL("attention_tc: launch failed: %s", cudaGetErrorString(le2));
    CO_CHECK_LAUNCH("attn_tc2");
    return 0;
  }
  if (ctas * cluster >= (1L << 31)) CO_FAIL("attention_tc: %ld CTAs", ctas * cluster);
  dim3 grid((unsigned)(ctas * cluster));
  cudaError_t le = co_launch_cluster(cluster, attn_tc_kernel, grid, dim3(320), (size_t)SMEM_BYTES, stream, mq, mk, mv, (bf16*)out,
                                     out_stride, block_tables, max_blocks, cu_q, kv_lens, nh, nkv, page_size, (int)cache_rows,
                                     window, scale_log2, skip_small, rows_per_box, status, B, row_tiles);
  if (le != cudaSuccess) CO_FAIL("attention_tc: launch failed: %s", cudaGetErrorString(le));
  CO_CHECK_LAUNCH("attn_tc");
  return 0;
}
