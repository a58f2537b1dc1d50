// Causal (optionally windowed) grouped-query attention over cache pages in bfloat16 on the
// tensor cores (mma.sync m16n8k16, float32 accumulation and float32 softmax), compiled for
// one head size (CO_HEAD_DIM, a multiple of 16 up to 256).
//
// The query rows of a request and kv head are numbered r = token * G + head_in_group
// (G = heads / kv_heads), so that all G query heads of a group share each key/value tile
// that is read.  Two kernels:
//
//  * attn_tiles:  one CTA per (request, kv head, tile of 64 rows); key/value tiles of 64
//    positions are copied from the pages into shared memory with cp.async (double
//    buffered); eight warps = four row tiles of 16 x two halves of each key tile, the
//    halves merged at the end.  Used for prompt portions.
//  * attn_stream: for requests with at most 16 rows per kv head (decoding).  The key range
//    is cut into splits of 128, 256 or 512 positions at ABSOLUTE multiples of the split; one
//    CTA per (request, kv head, split) streams its positions through a three-stage ring of
//    64-position tiles, each of its four warps taking 16 positions of every tile.  The warps'
//    (max, sum, accumulator) triples are merged in warp order and written to scratch;
//    attn_combine merges the splits of a row.
//
// Tiles start at absolute multiples of their size and splits likewise.  The split size is
// chosen from the batch's size, so a row's result may differ between batches by rounding
// (another order of merging), never by more.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "attention_tc.h"
#include "common.cuh"

#ifndef CO_HEAD_DIM
#define CO_HEAD_DIM 128
#endif

namespace {
constexpr int HD = CO_HEAD_DIM;
constexpr int LDS = HD + 8;       // shared-memory row stride: 16 bytes of padding keep ldmatrix conflict-free
constexpr int SPLIT_MIN = 128;    // positions per CTA of attn_stream: a power of two from 128 to 2048
constexpr int SPLIT_MAX = 2048;
constexpr int SPLIT_PAGES = 258;  // block-table entries a CTA keeps: a split spans at most 256 pages (+ 2)
constexpr int CHUNKS = HD / 8;    // 16-byte pieces per row
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 in 16..256");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0 fills the 16 bytes with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// The pages that hold positions [key0, key0 + TB): each lane of a warp fetches up to two
// block-table entries once per tile (entries lane and lane + 32 of the tile's page run);
// page_of() then hands them out by shuffle, so that the copies below wait on no load.
struct TilePages {
  int e0, e1, first_block;
};
template <int TB>
__device__ __forceinline__ TilePages tile_pages(const int* __restrict__ table, int page_size, int key0,
                                                int kv_begin, int kv_end) {
  const int lane = threadIdx.x & 31;
  TilePages tp;
  const int lo = max(key0, kv_begin), hi = min(key0 + TB, kv_end) - 1;   // positions really read
  tp.first_block = lo / page_size;
  const int last_block = hi >= lo ? hi / page_size : tp.first_block - 1;
  tp.e0 = tp.first_block + lane <= last_block ? table[tp.first_block + lane] : 0;
  tp.e1 = tp.first_block + lane + 32 <= last_block ? table[tp.first_block + lane + 32] : 0;
  return tp;
}
__device__ __forceinline__ int page_of(const TilePages& tp, int block) {
  const int i = block - tp.first_block;   // 0..63 for pages of at least one position
  const int a = __shfl_sync(0xffffffffu, tp.e0, i & 31);
  const int b = __shfl_sync(0xffffffffu, tp.e1, i & 31);
  return i < 32 ? a : b;
}

// Copies key or value rows of positions [key0, key0 + TB) of one kv head from the pages
// into a [TB][LDS] tile; positions outside [kv_begin, kv_end) are zero filled and their
// pages are not touched (a window may already have given them back).  NT threads with ids
// `tid` cooperate (whole warps, NT = 32 or 128): a thread owns TB / NT rows or, with more
// threads than rows, a share of one row; the row's address is worked out once.
__host__ __device__ constexpr int largest_divisor_up_to(int n, int cap) {
  int best = 1;
  for (int d = 1; d <= cap; ++d)
    if (n % d == 0) best = d;
  return best;
}

template <int NT, int TB>
__device__ __forceinline__ void load_tile(bf16* tile, const bf16* __restrict__ cache, const TilePages& tp,
                                          int kvh, int nkv, int page_size, int key0, int kv_begin, int kv_end,
                                          int tid) {
  constexpr int SLOTS = NT >= TB ? NT / TB : 1;                  // threads that sit on one row
  constexpr int TPR = largest_divisor_up_to(CHUNKS, SLOTS);      // of which this many copy
  constexpr int RPT = NT >= TB ? 1 : TB / NT;                    // rows per thread
  constexpr int PIECES = CHUNKS / TPR;                           // 16-byte pieces per thread and row
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int row = NT >= TB ? tid / SLOTS : i * NT + tid;
    const int sub = NT >= TB ? tid % SLOTS : 0;
    const int piece0 = sub * PIECES;
    const int pos = key0 + row;
    const bool valid = pos >= kv_begin && pos < kv_end;
    const int block = valid ? pos / page_size : tp.first_block;
    const int page = page_of(tp, block);                         // a shuffle: every lane takes part
    if (sub >= TPR) continue;
    const bf16* src = valid ? cache + (((size_t)page * nkv + kvh) * page_size + (pos - block * page_size)) * HD + piece0 * 8
                            : cache;
    bf16* dst = tile + row * LDS + piece0 * 8;
#pragma unroll
    for (int c = 0; c < PIECES; ++c) cp_async16(dst + c * 8, valid ? src + c * 8 : src, valid);
  }
}

struct RowState {
  float m[2];   // running maximum of the scaled scores (log2 domain), rows g and g+8
  float l[2];   // this thread's share of the running sum
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // ex2(-inf) = +0
  return y;
}

// One warp, MT tiles of 16 query rows against one tile of TB key positions in shared memory:
// S = Q K^T, masking, online softmax, O += P V.  Key and value fragments are fetched once and
// used for all MT row tiles.
//   Q fragments: registers (qf) when MT == 1 and QSMEM is false, else read from the warp's
//   rows in shared memory (Qs, [16 * MT][LDS]).
//   Ks/Vs: [TB][KVS] tiles; key0: position of the tile's row 0; lo/hi[mi][h]: first and last
//   visible key of the thread's rows g (h = 0) and g + 8 (h = 1) of row tile mi.  MASK false
//   promises that every key of the tile is visible to every row.
template <int MT, int TB, bool QSMEM, bool MASK, int KVS = LDS>
__device__ __forceinline__ void attend_tile(const unsigned (*qf)[4], const bf16* Qs, const bf16* Ks, const bf16* Vs,
                                            float (&o)[MT][HD / 8][4], RowState (&st)[MT], int key0,
                                            const int (&lo)[MT][2], const int (&hi)[MT][2], float scale_log2) {
  const int lane = threadIdx.x & 31;
  const int t = lane & 3;
  const int id = lane >> 3, r = lane & 7;
  float s[MT][TB / 8][4];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi)
#pragma unroll
    for (int j = 0; j < TB / 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[mi][j][i] = 0.f;

  // S = Q K^T.  ldmatrix.x4 on K rows yields the B fragments of two neighbouring key tiles.
#pragma unroll
  for (int kd = 0; kd < HD / 16; ++kd) {
    unsigned a[MT][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi) {
      if (QSMEM) ldmatrix_x4(a[mi], Qs + (mi * 16 + (id & 1) * 8 + r) * LDS + kd * 16 + (id >> 1) * 8);
      else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[mi][i] = qf[kd][i];
      }
    }
#pragma unroll
    for (int jp = 0; jp < TB / 16; ++jp) {
      unsigned b[4];
      ldmatrix_x4(b, Ks + (jp * 16 + (id >> 1) * 8 + r) * KVS + kd * 16 + (id & 1) * 8);
#pragma unroll
      for (int mi = 0; mi < MT; ++mi) {
        mma_bf16(s[mi][2 * jp], a[mi], b[0], b[1]);
        mma_bf16(s[mi][2 * jp + 1], a[mi], b[2], b[3]);
      }
    }
  }
  // Online softmax.  A thread holds, for rows g (i = 0,1) and g+8 (i = 2,3), the key
  // columns key0 + 8 j + 2 t + (i & 1).  The maximum is tracked in the log2 domain of the
  // scaled scores; p = 2^(s * scale_log2 - m) is one fused multiply-add and one ex2.
  bool rescale = false;
  float corr[MT][2];
#pragma unroll
  for (int mi = 0; mi < MT; ++mi)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < TB / 8; ++j)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (MASK) {
            const int key = key0 + j * 8 + 2 * t + i;
            if (key < lo[mi][h] || key > hi[mi][h]) s[mi][j][2 * h + i] = -INFINITY;
          }
          mx = fmaxf(mx, s[mi][j][2 * h + i]);
        }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(st[mi].m[h], mx * scale_log2);   // scale > 0 keeps the order
      // Everything masked so far: keep the state and let every p be zero.
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float c = ex2_approx(st[mi].m[h] - m_use);
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < TB / 8; ++j)
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float p = ex2_approx(fmaf(s[mi][j][2 * h + i], scale_log2, -m_use));
          s[mi][j][2 * h + i] = p;
          part += p;
        }
      st[mi].l[h] = st[mi].l[h] * c + part;
      st[mi].m[h] = m_new;
      corr[mi][h] = c;
      rescale |= c != 1.f;
    }
  if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
    for (int mi = 0; mi < MT; ++mi)
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        o[mi][dt][0] *= corr[mi][0]; o[mi][dt][1] *= corr[mi][0];
        o[mi][dt][2] *= corr[mi][1]; o[mi][dt][3] *= corr[mi][1];
      }
  }

  // O += P V.  The S accumulators of two neighbouring key tiles are the A fragment of one
  // 16-position step; ldmatrix.x4.trans on V rows yields B fragments of two head-dim tiles.
#pragma unroll
  for (int kt = 0; kt < TB / 16; ++kt) {
    unsigned a[MT][4];
#pragma unroll
    for (int mi = 0; mi < MT; ++mi) {
      a[mi][0] = pack_bf16(s[mi][2 * kt][0], s[mi][2 * kt][1]);
      a[mi][1] = pack_bf16(s[mi][2 * kt][2], s[mi][2 * kt][3]);
      a[mi][2] = pack_bf16(s[mi][2 * kt + 1][0], s[mi][2 * kt + 1][1]);
      a[mi][3] = pack_bf16(s[mi][2 * kt + 1][2], s[mi][2 * kt + 1][3]);
    }
#pragma unroll
    for (int dp = 0; dp < HD / 16; ++dp) {
      unsigned b[4];
      ldmatrix_x4_trans(b, Vs + (kt * 16 + (id & 1) * 8 + r) * KVS + dp * 16 + (id >> 1) * 8);
#pragma unroll
      for (int mi = 0; mi < MT; ++mi) {
        mma_bf16(o[mi][2 * dp], a[mi], b[0], b[1]);
        mma_bf16(o[mi][2 * dp + 1], a[mi], b[2], b[3]);
      }
    }
  }
}

// Copies query rows [row0, row0 + nrows) of (request, kv head) into shared memory; rows at
// or beyond `rows` are zero.
__device__ __forceinline__ void load_q_rows(bf16* Qs, const bf16* __restrict__ q, long q_stride, int tok0, int kvh,
                                            int G, int row0, int nrows, int rows, int tid, int nthreads) {
  for (int c = tid; c < nrows * CHUNKS; c += nthreads) {
    const int rr = c / CHUNKS, piece = c % CHUNKS;
    const int r = row0 + rr;
    const bool valid = r < rows;
    const bf16* src = q;
    if (valid) src = q + (size_t)(tok0 + r / G) * q_stride + (size_t)(kvh * G + r % G) * HD + piece * 8;
    cp_async16(Qs + rr * LDS + piece * 8, src, valid);
  }
}

// ------------------------------------------------------------------------------------
// attn_tiles: 64 query rows per CTA and key tiles of 64 positions, eight warps: warp w owns
// rows 16 * (w & 3) .. + 15 and the key half (w >> 2) of every tile, so two warps share a row
// tile and meet once at the end (the second half's (max, sum, accumulator) is merged into
// the first's through shared memory).  Twice the warps per row than a warp-per-row-tile
// layout, half the steps per warp: the kernel is bound by dependent latencies, not by
// arithmetic.  Two stages of (K tile, V tile); the copy of a row costs its thread one
// block-table entry (fetched a tile ahead) and a handful of integer operations.
#ifndef CO_ATTN_KGROUPS
#define CO_ATTN_KGROUPS 2
#endif
constexpr int KG = CO_ATTN_KGROUPS;   // key groups: warps that share a row tile
constexpr int TBN = 32;           // key positions per warp and step
constexpr int TILE = KG * TBN;    // key positions per CTA step
constexpr int BM = 64;            // query rows per CTA

__global__ void __launch_bounds__(128 * KG, HD <= 128 ? (KG == 2 ? 2 : 1) : 1)
attn_tiles_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                  const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window,
                  float scale_log2, int skip_small) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [BM][LDS]
  bf16* stages = Qs + BM * LDS;                                 // [2][K: TILE rows, V: TILE rows][LDS]
  constexpr int STAGE = 2 * TILE * LDS;

  co_pdl_launch_dependents();
  co_pdl_wait();
  // Late row tiles see the most keys: they are started first.
  const int b = blockIdx.z, kvh = blockIdx.y, rt = gridDim.x - 1 - blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rt * BM >= rows) return;
  if (skip_small && rows <= 16) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int rw = warp & 3, kg = warp >> 2;
  const int* table = block_tables + (size_t)b * max_blocks;
  const int base_pos = kv_len - q_len;   // position of the request's first token in this step

  // Key range needed by this tile of rows.
  const int row_first = rt * BM, row_last = min(rows, row_first + BM) - 1;
  const int pos_lo = base_pos + row_first / G, pos_hi = base_pos + row_last / G;
  const int key_first = window > 0 ? max(0, pos_lo - window + 1) : 0;
  const int tile_first = key_first / TILE, tile_last = pos_hi / TILE;
  const int kv_end = pos_hi + 1;

  // Copies: thread -> (row tid / 4 of the tile, a quarter of the row's 16-byte pieces).
  constexpr int TPR = largest_divisor_up_to(CHUNKS, 4);
  constexpr int PIECES = CHUNKS / TPR;
  const int c_row = tid >> 2, c_sub = tid & 3;
  auto page_for = [&](int tile) -> int {     // block-table entry of this thread's row in a tile
    const int pos = tile * TILE + c_row;
    return (tile <= tile_last && pos >= key_first && pos < kv_end) ? table[pos / page_size] : -1;
  };
  auto issue = [&](int tile, int page) {     // one commit group per call, possibly empty
    if (tile <= tile_last && c_sub < TPR) {
      bf16* st = stages + ((tile - tile_first) & 1) * STAGE + c_row * LDS + c_sub * PIECES * 8;
      const bool valid = page >= 0;
      const int pos = tile * TILE + c_row;
      const size_t off = valid ? (((size_t)page * nkv + kvh) * page_size + pos % page_size) * HD + c_sub * PIECES * 8 : 0;
#pragma unroll
      for (int c = 0; c < PIECES; ++c) {
        cp_async16(st + c * 8, k_cache + off + (valid ? c * 8 : 0), valid);
        cp_async16(st + TILE * LDS + c * 8, v_cache + off + (valid ? c * 8 : 0), valid);
      }
    }
    cp_async_commit();
  };
  load_q_rows(Qs, q, q_stride, tok0, kvh, G, row_first, BM, rows, tid, 128 * KG);
  issue(tile_first, page_for(tile_first));   // group 0: the query rows and the first tile
  int page_next = page_for(tile_first + 1);

  // Visible key range of the thread's rows, and of the warp's rows as a whole.
  int lo[1][2], hi[1][2];
  const int w_row_first = row_first + rw * 16;
  const int w_row_last = min(rows - 1, w_row_first + 15);
  const bool w_active = w_row_first < rows;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = w_row_first + h * 8 + g;
    if (r < rows) {
      hi[0][h] = base_pos + r / G;
      lo[0][h] = window > 0 ? max(0, hi[0][h] - window + 1) : 0;
    } else {
      hi[0][h] = -1; lo[0][h] = 0;
    }
  }
  const int w_hi_max = w_active ? base_pos + w_row_last / G : -1;           // last key any row sees
  const int w_hi_min = w_active ? base_pos + w_row_first / G : -1;          // last key EVERY row sees
  const int w_lo_min = w_active && window > 0 ? max(0, base_pos + w_row_first / G - window + 1) : 0;
  const int w_lo_max = w_active && window > 0 ? max(0, base_pos + w_row_last / G - window + 1) : 0;
  const bool w_full = w_row_first + 16 <= rows;                             // no padding rows

  float o[1][HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[0][dt][i] = 0.f;
  RowState st[1];
  st[0].m[0] = st[0].m[1] = -INFINITY;
  st[0].l[0] = st[0].l[1] = 0.f;
  const bf16* Qw = Qs + rw * 16 * LDS;

  for (int tile = tile_first; tile <= tile_last; ++tile) {
    issue(tile + 1, page_next);   // into the stage that tile - 1 used (all warps are past it)
    page_next = page_for(tile + 2);
    cp_async_wait<1>();           // this tile's group has landed; the next one may be in flight
    __syncthreads();
    const bf16* st_k = stages + ((tile - tile_first) & 1) * STAGE + kg * TBN * LDS;
    const int key0 = tile * TILE + kg * TBN;
    if (w_active && key0 <= w_hi_max && key0 + TBN > w_lo_min) {
      const bool all_visible = w_full && key0 + TBN - 1 <= w_hi_min && key0 >= w_lo_max;
      if (all_visible)
        attend_tile<1, TBN, true, false>(nullptr, Qw, st_k, st_k + TILE * LDS, o, st, key0, lo, hi, scale_log2);
      else
        attend_tile<1, TBN, true, true>(nullptr, Qw, st_k, st_k + TILE * LDS, o, st, key0, lo, hi, scale_log2);
    }
    __syncthreads();
  }

  // The key groups of a row tile meet: groups 1.. write their state, group 0 merges them
  // in ascending order.
  float* merge = reinterpret_cast<float*>(stages);              // [KG - 1][4 row warps][16 rows][HD + 2]
  constexpr int MS = HD + 2;
  float l2[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float l = st[0].l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    l2[h] = l;
  }
  if (kg >= 1) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* dst = merge + ((size_t)((kg - 1) * 4 + rw) * 16 + h * 8 + g) * MS;
      if (t == 0) { dst[0] = st[0].m[h]; dst[1] = l2[h]; }
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        dst[2 + dt * 8 + 2 * t] = o[0][dt][2 * h];
        dst[2 + dt * 8 + 2 * t + 1] = o[0][dt][2 * h + 1];
      }
    }
  }
  __syncthreads();
  if (kg == 0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = w_row_first + h * 8 + g;
      if (r >= rows) continue;
      float M = st[0].m[h];
#pragma unroll
      for (int k = 1; k < KG; ++k) M = fmaxf(M, merge[((size_t)((k - 1) * 4 + rw) * 16 + h * 8 + g) * MS]);
      float f[KG];                                      // M is finite: a row always sees its own key
      f[0] = st[0].m[h] == -INFINITY ? 0.f : exp2f(st[0].m[h] - M);
      float den = l2[h] * f[0];
#pragma unroll
      for (int k = 1; k < KG; ++k) {
        const float* src = merge + ((size_t)((k - 1) * 4 + rw) * 16 + h * 8 + g) * MS;
        f[k] = src[0] == -INFINITY ? 0.f : exp2f(src[0] - M);
        den += src[1] * f[k];
      }
      const float inv = 1.0f / den;
      bf16* orow = out + (size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * HD;
#pragma unroll
      for (int dt = 0; dt < HD / 8; ++dt) {
        float a = o[0][dt][2 * h] * f[0], c = o[0][dt][2 * h + 1] * f[0];
#pragma unroll
        for (int k = 1; k < KG; ++k) {
          const float* src = merge + ((size_t)((k - 1) * 4 + rw) * 16 + h * 8 + g) * MS;
          a += src[2 + dt * 8 + 2 * t] * f[k];
          c += src[2 + dt * 8 + 2 * t + 1] * f[k];
        }
        *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + 2 * t) = __floats2bfloat162_rn(a * inv, c * inv);
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// Scratch per (request, kv head, split): 16 x HD floats of unnormalised accumulators (row r at
// r * HD, 16-byte aligned), then 16 pairs (max in the log2 domain, sum).  In shared memory the
// warps' triples are laid out as rows of PART floats: [0] = max, [1] = sum, [2..] = accumulator.
constexpr int PART = HD + 2;
constexpr int SPLIT_FLOATS = 16 * HD + 32;

// attn_stream: decoding is bound by reading each key and value once, so the kernel is a
// copy pipeline with a little arithmetic attached.  A CTA owns `split` consecutive
// positions (a multiple of 64, at absolute multiples of `split`) of one (request, kv head)
// and streams them through a ring of SSTAGES tiles of 64 positions, keys and values, with
// cp.async: while the warps work on tile i, the next SSTAGES-1 tiles are in flight.  Warp w
// takes positions 16 w .. 16 w + 15 of every tile for the request's <= 16 rows, keeps its
// own running (max, sum, accumulator), and the four warps merge once at the end in warp
// order.  About 110 KB of shared memory at head size 128: two CTAs per SM, so one CTA's
// prologue and merge hide behind the other's stream.
//
// What the step's earlier kernels do not write is fetched BEFORE the kernel waits for its
// predecessor (programmatic dependent launch): the lengths and block tables (inputs of the
// step) and every tile whose positions all precede the request's new tokens (written by
// earlier steps; the predecessor writes only the new tokens' slots).  With a split of 128
// positions the whole split is in flight while the q/k/v projection still runs; after the
// wait only the queries and the tile with the new tokens are read.
//
// A tile's copies are planned one iteration ahead: threads 0..63 turn the tile's positions
// into element offsets (one division and one block-table entry from shared memory per row),
// and the copy loop then moves consecutive 16-byte pieces with consecutive lanes, so a warp
// instruction covers whole 128-byte lines.
// Two ring depths are built: three stages (two CTAs per SM at head size 128: the deepest
// prefetch, for batches whose CTAs all fit the GPU at once) and two stages (three CTAs per SM:
// more warps to hide each other's latencies, for batches whose CTAs queue up).
constexpr int STILE = 64;
constexpr size_t stream_smem(int stages) { return (size_t)(16 + stages * 2 * STILE) * LDS * sizeof(bf16); }
static_assert((size_t)4 * 16 * PART * sizeof(float) <= (size_t)2 * 2 * STILE * LDS * sizeof(bf16),
              "the merge area fits the ring");
static_assert(stream_smem(3) + 6 * 1024 <= 227 * 1024, "the ring fits shared memory at every head size");

template <int SSTAGES, bool PER_WARP = false>
__global__ void __launch_bounds__(128)
attn_stream_kernel(const bf16* __restrict__ q, long q_stride, float* __restrict__ scratch, int max_splits,
                   const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                   const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                   const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window, float scale_log2,
                   int split, int settled) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ long long rowoff[SSTAGES][STILE];   // element offset of a tile's rows in a cache tensor, -1: not read
  __shared__ int pages_s[SPLIT_PAGES];           // block-table entries of the split's pages
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][LDS]
  bf16* ring = Qs + 16 * LDS;                                   // [SSTAGES][K, V][STILE][LDS]
  float* merge = reinterpret_cast<float*>(ring);               // reused after the tiles: [4][16][PART]

  co_pdl_launch_dependents();
  // Inputs of the step: written before its first kernel started.
  const int b = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rows > 16 || rows <= 0) return;
  const int base_pos = kv_len - q_len;   // the first new position: everything before it is an earlier step's
  const int pos_hi = kv_len - 1;
  const int key_first = window > 0 ? max(0, base_pos - window + 1) : 0;
  const int c0 = (key_first / split + sp) * split;   // the split's first position
  if (c0 > pos_hi) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_tables + (size_t)b * max_blocks;
  const int lo_key = max(c0, key_first), hi_key = min(c0 + split, pos_hi + 1);   // positions [lo_key, hi_key) are read
  const int t_first = (lo_key - c0) / STILE;                  // a window hides earlier tiles
  const int t_end = (hi_key - c0 + STILE - 1) / STILE;        // tiles [t_first, t_end)
  const int blk0 = lo_key / page_size;
  for (int j = tid; j <= (hi_key - 1) / page_size - blk0; j += 128) pages_s[j] = table[blk0 + j];
  __syncthreads();

  auto stage_of = [&](int i) { return ring + (size_t)((i - t_first) % SSTAGES) * 2 * STILE * LDS; };
  auto plan = [&](int i) {
    if (tid < STILE && i < t_end) {
      const int pos = c0 + i * STILE + tid;
      long long off = -1;
      if (pos >= lo_key && pos < hi_key) {
        const int blk = pos / page_size;
        off = (((long long)pages_s[blk - blk0] * nkv + kvh) * page_size + (pos - blk * page_size)) * HD;
      }
      rowoff[(i - t_first) % SSTAGES][tid] = off;
    }
  };
  auto issue = [&](int i) {   // one group per call, with or without copies
    if (i < t_end) {
      bf16* Ks = stage_of(i);
      const long long* ro = rowoff[(i - t_first) % SSTAGES];
#pragma unroll
      for (int c = tid; c < STILE * CHUNKS; c += 128) {
        const int row = c / CHUNKS, piece = c % CHUNKS;
        const long long off = ro[row];
        const bool valid = off >= 0;
        const size_t src = valid ? (size_t)off + piece * 8 : 0;
        cp_async16(Ks + row * LDS + piece * 8, k_cache + src, valid);
        cp_async16(Ks + (STILE + row) * LDS + piece * 8, v_cache + src, valid);
      }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int s = 0; s < SSTAGES; ++s) plan(t_first + s);
  __syncthreads();
  // `settled` = 0: the positions before the request's new tokens may have been written by this very
  // step (the wanted rows of a portion, run as one-token requests after the portion's keys and values
  // went to the cache): nothing of the cache is read before the wait then.
  int issued = 0;
  while (settled && issued < SSTAGES && (t_first + issued >= t_end || c0 + (t_first + issued + 1) * STILE <= base_pos)) {
    issue(t_first + issued);
    ++issued;
  }
  co_pdl_wait();   // the queries and the new tokens' keys and values are the predecessor's output
  for (int c = tid; c < 16 * CHUNKS; c += 128) {
    const int rr = c / CHUNKS, piece = c % CHUNKS;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < rows)
      v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + rr / G) * q_stride + (size_t)(kvh * G + rr % G) * HD + piece * 8);
    *reinterpret_cast<uint4*>(Qs + rr * LDS + piece * 8) = v;
  }
  for (; issued < SSTAGES; ++issued) issue(t_first + issued);
  __syncthreads();
  unsigned qf[HD / 16][4];
#pragma unroll
  for (int kd = 0; kd < HD / 16; ++kd)
    ldmatrix_x4(qf[kd], Qs + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + kd * 16 + (lane >> 4) * 8);

  int lo[1][2], hi[1][2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    if (r < rows) {
      hi[0][h] = base_pos + r / G;
      lo[0][h] = window > 0 ? max(0, hi[0][h] - window + 1) : 0;
    } else {
      hi[0][h] = -1; lo[0][h] = 0;
    }
  }
  // Positions [all_lo, all_hi] are visible to every valid row: tiles inside need no mask.
  const int all_lo = window > 0 ? max(0, pos_hi - window + 1) : 0, all_hi = base_pos;
  float o[1][HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[0][dt][i] = 0.f;
  RowState st[1];
  st[0].m[0] = st[0].m[1] = -INFINITY;
  st[0].l[0] = st[0].l[1] = 0.f;

  if constexpr (PER_WARP) {
    // At most SSTAGES tiles, all of them requested by now: every warp takes a whole tile of its own (eight
    // independent accumulators in Q K^T instead of two), so the tiles are worked on side by side.
    cp_async_wait<0>();
    __syncthreads();
    const int i = t_first + warp;
    const int key0 = c0 + i * STILE;
    if (i < t_end && key0 < hi_key && key0 + STILE > lo_key) {
      const bf16* Ks = stage_of(i);
      if (key0 >= all_lo && key0 + STILE - 1 <= all_hi)
        attend_tile<1, STILE, false, false>(qf, nullptr, Ks, Ks + STILE * LDS, o, st, key0, lo, hi, scale_log2);
      else
        attend_tile<1, STILE, false, true>(qf, nullptr, Ks, Ks + STILE * LDS, o, st, key0, lo, hi, scale_log2);
    }
  } else {
#pragma unroll 1
  for (int i = t_first; i < t_end; ++i) {
    // Tile i is group i - t_first; groups complete in order.
    if (i == t_first) cp_async_wait<SSTAGES - 1>(); else cp_async_wait<SSTAGES - 2>();
    __syncthreads();                // landed for all threads; every warp is done with tile i - 1
    if (i > t_first) issue(i + SSTAGES - 1);   // into the stage that tile i - 1 used
    plan(i + SSTAGES);              // for the next iteration's issue; its slot was last read when tile i was issued
    const int key0 = c0 + i * STILE + warp * 16;
    if (key0 < hi_key && key0 + 16 > lo_key) {
      const bf16* Ks = stage_of(i) + warp * 16 * LDS;
      if (key0 >= all_lo && key0 + 15 <= all_hi)
        attend_tile<1, 16, false, false>(qf, nullptr, Ks, Ks + STILE * LDS, o, st, key0, lo, hi, scale_log2);
      else
        attend_tile<1, 16, false, true>(qf, nullptr, Ks, Ks + STILE * LDS, o, st, key0, lo, hi, scale_log2);
    }
  }
  }
  cp_async_wait<0>();
  __syncthreads();   // all warps are done with their tiles: the ring becomes the merge area

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    float l = st[0].l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (r >= rows) continue;            // rows without a query are not merged
    float* dst = merge + ((size_t)warp * 16 + r) * PART;
    if (t == 0) *reinterpret_cast<float2*>(dst) = make_float2(st[0].m[h], l);
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt)
      *reinterpret_cast<float2*>(dst + 2 + dt * 8 + 2 * t) = make_float2(o[0][dt][2 * h], o[0][dt][2 * h + 1]);
  }
  __syncthreads();
  // Merge the four warps in warp order; write the valid rows.
  float* dst_base = scratch + (((size_t)b * nkv + kvh) * max_splits + sp) * SPLIT_FLOATS;
  for (int e = tid; e < rows * (HD + 1); e += 128) {
    const int r = e / (HD + 1), c = e % (HD + 1);   // c == HD: the (max, sum) pair
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, merge[(w * 16 + r) * PART]);
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = merge[(w * 16 + r) * PART];
      const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
      acc += f * (c == HD ? merge[(w * 16 + r) * PART + 1] : merge[(w * 16 + r) * PART + 2 + c]);
    }
    if (c == HD) { dst_base[16 * HD + 2 * r] = M; dst_base[16 * HD + 2 * r + 1] = acc; }
    else dst_base[r * HD + c] = acc;
  }
}

// One CTA per (request, kv head), one warp per row and no shared memory.  A lane reads the
// (max, sum) pair of one split (32 splits at a time), the warp agrees on the maximum, and the
// lanes then add the splits' accumulators, four columns per lane and up to sixteen independent
// loads at a time, in ascending order of the splits.
__global__ void __launch_bounds__(512)
attn_combine_kernel(const float* __restrict__ scratch, int max_splits, bf16* __restrict__ out, long out_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, int nh, int nkv, int window,
                    int split) {
  constexpr int UB = HD > 128 ? 8 : 16;   // splits whose loads are in flight together
  co_pdl_launch_dependents();
  // The lengths are inputs of the step: a warp without a row leaves before it waits.
  const int b = blockIdx.y, kvh = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rows > 16 || warp >= rows) return;
  co_pdl_wait();
  const int base_pos = kv_len - q_len;
  const int key_first = window > 0 ? max(0, base_pos - window + 1) : 0;
  const int nsplits = (kv_len - 1) / split - key_first / split + 1;
  const float* base = scratch + ((size_t)b * nkv + kvh) * max_splits * SPLIT_FLOATS;
  for (int r = warp; r < rows; r += nwarps) {
    float M = -INFINITY;
    for (int s = lane; s < nsplits; s += 32) M = fmaxf(M, base[(size_t)s * SPLIT_FLOATS + 16 * HD + 2 * r]);
    M = co_warp_max(M);
    float den = 0.f;
    float4 acc[(HD + 127) / 128];
#pragma unroll
    for (int q = 0; q < (HD + 127) / 128; ++q) acc[q] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsplits; s0 += 32) {
      float f = 0.f, l = 0.f;
      if (s0 + lane < nsplits) {
        const float2 ml = *reinterpret_cast<const float2*>(base + (size_t)(s0 + lane) * SPLIT_FLOATS + 16 * HD + 2 * r);
        f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
        l = ml.y;
      }
      den += f * l;
      const int n = min(32, nsplits - s0);
      for (int u0 = 0; u0 < n; u0 += UB) {
        float4 t[UB][(HD + 127) / 128];
#pragma unroll
        for (int u = 0; u < UB; ++u)
#pragma unroll
          for (int q = 0; q < (HD + 127) / 128; ++q) {
            const int c = q * 128 + lane * 4;
            t[u][q] = (u0 + u < n && c < HD)
                          ? *reinterpret_cast<const float4*>(base + (size_t)(s0 + u0 + u) * SPLIT_FLOATS + r * HD + c)
                          : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
        for (int u = 0; u < UB; ++u) {
          const float fu = __shfl_sync(0xffffffffu, f, (u0 + u) & 31);
#pragma unroll
          for (int q = 0; q < (HD + 127) / 128; ++q) {
            acc[q].x += fu * t[u][q].x; acc[q].y += fu * t[u][q].y; acc[q].z += fu * t[u][q].z; acc[q].w += fu * t[u][q].w;
          }
        }
      }
    }
    den = co_warp_sum(den);
    const float inv = 1.0f / den;
    bf16* orow = out + (size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * HD;
#pragma unroll
    for (int q = 0; q < (HD + 127) / 128; ++q) {
      const int c = q * 128 + lane * 4;
      if (c < HD) {
        __nv_bfloat162 lo2 = __floats2bfloat162_rn(acc[q].x * inv, acc[q].y * inv);
        __nv_bfloat162 hi2 = __floats2bfloat162_rn(acc[q].z * inv, acc[q].w * inv);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&lo2);
        raw.y = *reinterpret_cast<unsigned*>(&hi2);
        *reinterpret_cast<uint2*>(orow + c) = raw;
      }
    }
  }
}

constexpr size_t TILES_SMEM = (size_t)(BM + 4 * TILE) * LDS * sizeof(bf16);
static_assert((size_t)(KG - 1) * 4 * 16 * (HD + 2) * sizeof(float) <= (size_t)4 * TILE * LDS * sizeof(bf16), "the merge area fits the stages");

// Positions per CTA of attn_stream.  coheryn_attn_set_split (or COHERYN_ATTN_SPLIT = 128 |
// 256 | 512 in the environment, read at first use) fixes it; otherwise the largest of the
// three whose grid still fills the GPU (two CTAs per SM), else the smallest.
// COHERYN_ATTN_PER_WARP=0 switches the tile-per-warp variant (and the split of 192 positions chosen for it) off.
bool per_warp_on() {
  static int on = -1;
  if (on < 0) { const char* e = getenv("COHERYN_ATTN_PER_WARP"); on = (e && e[0] == '0') ? 0 : 1; }
  return on != 0;
}

int g_forced_split = -1;
int split_keys(int B, int nkv, int max_kv_len, int page_size) {
  if (g_forced_split < 0) {
    const char* e = getenv("COHERYN_ATTN_SPLIT");
    const int v = e ? atoi(e) : 0;
    g_forced_split = (v == 128 || v == 192 || v == 256 || v == 512 || v == 1024 || v == 2048) ? v : 0;
  }
  int cap = SPLIT_MAX;                                    // the kernel keeps split / page_size + 2 table entries
  while (cap > SPLIT_MIN && cap / page_size + 2 > SPLIT_PAGES) cap >>= 1;
  if (g_forced_split) return g_forced_split < cap ? g_forced_split : cap;
  // Measured at batch 4 to 256 with contexts of 4,096 to 32,768 (lengths uniform up to the bound, so about
  // two thirds of the counted CTAs have keys).  1,024 positions per CTA pay where those CTAs either all fit
  // the three resident slots per SM of the shallow ring at once or queue up four deep and more (batch 64 at
  // 4,096: 2.59 -> 2.48 ms per step; batch 16 at 16,384: 2.28 -> 2.11; batch 256: 5.74 -> 5.59), not in
  // between, where the second round is half empty (batch 128: 3.45 -> 3.56), and not below (batch 4 at
  // 32,768: 1.72 -> 1.87); 2,048 never paid.  512 when they fill the two slots per SM of the deep ring; 256
  // already at four fifths of those (batch 8: half as many partial results to merge beat 128 by 2.4 %).
  const long slots = (stream_smem(3) + 4 * 1024 <= 227 * 1024 / 2 ? 2 : 1) * 148L;
  if (cap >= 1024) {
    const long wide = (long)B * nkv * ((max_kv_len + 1023) / 1024);
    if ((wide >= 3 * 148L && wide <= 640) || wide >= 12 * 148L) return 1024;
  }
  for (int s = cap < 512 ? cap : 512; s > SPLIT_MIN; s >>= 1)
    if ((long)B * nkv * ((max_kv_len + s - 1) / s) >= (s >= 512 ? slots : slots * 4 / 5)) {
      // Where 256 positions would be chosen, 192 are three tiles that three warps work on side by side
      // (see attn_stream_kernel), as long as the CTAs counted from the context bound still about fit the
      // resident slots: batch 8 with contexts uniform up to 4,096: 1.345 -> 1.29 ms per step; every context
      // at 2,000: 1.330 -> 1.285; every context at 3,900 (more CTAs than slots): 1.405 -> 1.442.
      if (s == 256 && cap >= 192 && per_warp_on() && (long)B * nkv * ((max_kv_len + 191) / 192) <= slots * 6 / 5) return 192;
      return s;
    }
  return SPLIT_MIN;
}

template <int SSTAGES, bool PER_WARP = false>
int launch_stream_kernel(dim3 grid, cudaStream_t stream, const void* q, long q_stride, float* scratch, int max_splits,
                         const void* k_cache, const void* v_cache, const int* block_tables, int max_blocks,
                         const int* cu_q, const int* kv_lens, int nh, int nkv, int page_size, int window,
                         float scale_log2, int split, int settled) {
  constexpr size_t SMEM = stream_smem(SSTAGES);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_stream_kernel<SSTAGES, PER_WARP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
    configured = true;
  }
  co_launch(attn_stream_kernel<SSTAGES, PER_WARP>, grid, dim3(128), SMEM, stream, (const bf16*)q, q_stride, scratch, max_splits,
            (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks, cu_q, kv_lens, nh, nkv, page_size,
            window, scale_log2, split, settled);
  CO_CHECK_LAUNCH("attn_stream");
  return 0;
}

// ------------------------------------------------------------------------------------
// attn_merge_oproj: decoding with one token per request.  Instead of attn_combine writing the merged
// rows and a separate product reading them back, a CTA per (query head h, tile of 128 output
// features) merges the splits of head h for every request (as attn_combine does, in ascending order),
// rounds the rows to bfloat16 as the combine would, and multiplies them with its tile of the output
// matrix: out_h[b, n] = sum_k o_h[b, k] W[n, h HD + k].  The heads' contributions are left as a
// float32 stack parts[h][b][n] for the norm that follows, which adds them in order anyway.  The W
// tile (a constant) is fetched before the kernel waits for the splits.
// ------------------------------------------------------------------------------------
constexpr int MO_TILE = 128;
constexpr int MO_THREADS = 256;
constexpr size_t MO_SMEM_TILES = (size_t)(MO_TILE + 16) * LDS * sizeof(bf16);
// plus, per request and split, the split's maximum (then its factor) and its sum
inline size_t mo_smem(int max_splits) { return MO_SMEM_TILES + (size_t)2 * 16 * max_splits * sizeof(float); }

__global__ void __launch_bounds__(MO_THREADS)
attn_merge_oproj_kernel(const float* __restrict__ scratch, int max_splits, const int* __restrict__ kv_lens, int B,
                        int nh, int nkv, int window, int split, const bf16* __restrict__ w, long ldw, int H,
                        const void* __restrict__ bias, int bias_dtype, float* __restrict__ parts) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Ws = reinterpret_cast<bf16*>(smem_raw);      // [MO_TILE][LDS]: W[n0 + i, h HD ..]
  bf16* As = Ws + MO_TILE * LDS;                     // [16][LDS]: the merged rows of head h
  float* fs = reinterpret_cast<float*>(As + 16 * LDS);   // [16][max_splits]: maximum, then factor, of a split
  float* ls = fs + 16 * max_splits;                      // [16][max_splits]: sum of a split
  __shared__ int nsp[16];
  __shared__ float inv_den[16];
  co_pdl_launch_dependents();
  const int n0 = blockIdx.x * MO_TILE, h = blockIdx.y;
  const int G = nh / nkv, kvh = h / G, r = h % G;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  for (int c = tid; c < MO_TILE * CHUNKS; c += MO_THREADS) {
    const int row = c / CHUNKS, piece = c % CHUNKS;
    const bool valid = n0 + row < H;
    cp_async16(Ws + row * LDS + piece * 8, w + (valid ? (size_t)(n0 + row) * ldw + (size_t)h * HD + piece * 8 : 0), valid);
  }
  cp_async_commit();
  for (int c = tid; c < 16 * CHUNKS; c += MO_THREADS)    // rows without a request stay zero
    *reinterpret_cast<uint4*>(As + (c / CHUNKS) * LDS + (c % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
  if (tid < 16) {                                        // the lengths are inputs of the step
    int n = 0;
    if (tid < B) {
      const int kv_len = kv_lens[tid];
      const int key_first = window > 0 ? max(0, kv_len - window) : 0;
      n = (kv_len - 1) / split - key_first / split + 1;
    }
    nsp[tid] = n;
  }
  __syncthreads();
  co_pdl_wait();
  // One round trip for everything: a thread owns (request, four columns) and asks for the first
  // sixteen splits' accumulators at once; the (maximum, sum) pairs of all splits go to shared memory
  // beside them, and the factors are worked out while the accumulators are still on their way.
  constexpr int PRE = 16;
  const int item = tid;                                   // items beyond B * HD / 4 own nothing
  const int ib = item / (HD / 4), ic = (item - ib * (HD / 4)) * 4;
  const bool owns = item < B * (HD / 4);
  const int in = owns ? nsp[ib] : 0;
  const float* ibase = scratch + ((size_t)(owns ? ib : 0) * nkv + kvh) * max_splits * SPLIT_FLOATS + r * HD + ic;
  float4 pre[PRE];
#pragma unroll
  for (int u = 0; u < PRE; ++u)
    pre[u] = u < in ? *reinterpret_cast<const float4*>(ibase + (size_t)u * SPLIT_FLOATS) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = tid; i < B * max_splits; i += MO_THREADS) {
    const int b = i / max_splits, sp = i - b * max_splits;
    if (sp < nsp[b]) {
      const float2 ml = *reinterpret_cast<const float2*>(scratch + (((size_t)b * nkv + kvh) * max_splits + sp) * SPLIT_FLOATS +
                                                         16 * HD + 2 * r);
      fs[i] = ml.x;
      ls[i] = ml.y;
    }
  }
  __syncthreads();
  for (int b = warp; b < B; b += MO_THREADS / 32) {      // a warp per request: the factors and the denominator
    const int n = nsp[b];
    float* f = fs + b * max_splits;
    const float* l = ls + b * max_splits;
    float M = -INFINITY;
    for (int sp = lane; sp < n; sp += 32) M = fmaxf(M, f[sp]);
    M = co_warp_max(M);
    float den = 0.f;
    for (int sp = lane; sp < n; sp += 32) {
      const float fac = f[sp] == -INFINITY ? 0.f : exp2f(f[sp] - M);
      f[sp] = fac;
      den += fac * l[sp];
    }
    den = co_warp_sum(den);
    if (lane == 0) inv_den[b] = 1.0f / den;
  }
  __syncthreads();
  // The splits' accumulators added in ascending order: the first sixteen from registers, the rest
  // (long contexts) eight loads at a time; then further items of a head size above 128 or B * HD / 4 > 256.
  for (int i = tid; i < B * (HD / 4); i += MO_THREADS) {
    const int b = i / (HD / 4), c = (i - b * (HD / 4)) * 4;
    const int n = nsp[b];
    const float* f = fs + b * max_splits;
    const float* base = scratch + ((size_t)b * nkv + kvh) * max_splits * SPLIT_FLOATS + r * HD + c;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int s0 = 0;
    if (i == tid) {
#pragma unroll
      for (int u = 0; u < PRE; ++u) {
        const float fu = u < n ? f[u] : 0.f;
        acc.x += fu * pre[u].x; acc.y += fu * pre[u].y; acc.z += fu * pre[u].z; acc.w += fu * pre[u].w;
      }
      s0 = PRE;
    }
    for (; s0 < n; s0 += 8) {
      float4 tv[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        tv[u] = s0 + u < n ? *reinterpret_cast<const float4*>(base + (size_t)(s0 + u) * SPLIT_FLOATS) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float fu = s0 + u < n ? f[s0 + u] : 0.f;
        acc.x += fu * tv[u].x; acc.y += fu * tv[u].y; acc.z += fu * tv[u].z; acc.w += fu * tv[u].w;
      }
    }
    const float inv = inv_den[b];
    uint2 raw;
    raw.x = pack_bf16(acc.x * inv, acc.y * inv);
    raw.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(As + b * LDS + c) = raw;
  }
  cp_async_wait<0>();
  __syncthreads();
  // out[16 requests, 128 features]: warp w owns features 16 w .. 16 w + 15
  float o[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
#pragma unroll
  for (int kd = 0; kd < HD / 16; ++kd) {
    unsigned a[4];
    ldmatrix_x4(a, As + (((lane >> 3) & 1) * 8 + (lane & 7)) * LDS + kd * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const bf16* wr = Ws + (warp * 16 + nt * 8 + g) * LDS + kd * 16 + 2 * t;
      mma_bf16(o[nt], a, *reinterpret_cast<const unsigned*>(wr), *reinterpret_cast<const unsigned*>(wr + 8));
    }
  }
  float* dst = parts + (size_t)h * B * H;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int n = n0 + warp * 16 + nt * 8 + 2 * t;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int b = g + half * 8;
      if (b >= B) continue;
#pragma unroll
      for (int e = 0; e < 2; ++e)
        if (n + e < H) {
          float v = o[nt][half * 2 + e];
          if (bias && h == 0) v += co_load_any(bias, bias_dtype, n + e);
          dst[(size_t)b * H + n + e] = v;
        }
    }
  }
}

// The stream kernel over every request with at most 16 rows; the splits' partial results stay in
// scratch.  Returns the positions per split through *split_out (and the slots per request and kv head).
int launch_stream_splits(const void* q, long q_stride, const void* k_cache, const void* v_cache, const int* block_tables,
                         int max_blocks, const int* cu_q, const int* kv_lens, int B, int nh, int nkv, int page_size,
                         int window, float scale_log2, int max_kv_len, float* scratch, long scratch_floats, int settled,
                         cudaStream_t stream, int* split_out, int* max_splits_out) {
  const int split = split_keys(B, nkv, max_kv_len, page_size);
  const int max_splits = (max_kv_len + split - 1) / split + 1;
  if (!scratch || scratch_floats < (long)B * nkv * max_splits * SPLIT_FLOATS)
    CO_FAIL("attention_bf16: scratch of %ld floats is too small", scratch_floats);
  const dim3 grid(max_splits, nkv, B);
  // CTAs that queue up (more than two per SM): the shallower ring, three CTAs per SM.
  static int forced_stages = -1;
  if (forced_stages < 0) {
    const char* e = getenv("COHERYN_ATTN_STAGES");
    forced_stages = e ? atoi(e) : 0;
  }
  const bool shallow = forced_stages ? forced_stages == 2 : (long)B * nkv * ((max_kv_len + split - 1) / split) > 3 * 148L;
  *split_out = split;
  *max_splits_out = max_splits;
  // Splits of three tiles: a tile per warp, all three resident in the deep ring (two CTAs per SM).
  if (split == 3 * STILE && !forced_stages && per_warp_on())
    return launch_stream_kernel<3, true>(grid, stream, q, q_stride, scratch, max_splits, k_cache, v_cache, block_tables,
                                         max_blocks, cu_q, kv_lens, nh, nkv, page_size, window, scale_log2, split, settled);
  return shallow ? launch_stream_kernel<2>(grid, stream, q, q_stride, scratch, max_splits, k_cache, v_cache, block_tables,
                                           max_blocks, cu_q, kv_lens, nh, nkv, page_size, window, scale_log2, split, settled)
                 : launch_stream_kernel<3>(grid, stream, q, q_stride, scratch, max_splits, k_cache, v_cache, block_tables,
                                           max_blocks, cu_q, kv_lens, nh, nkv, page_size, window, scale_log2, split, settled);
}

int launch_stream(const void* q, long q_stride, void* out, long out_stride, const void* k_cache, const void* v_cache,
                  const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int B, int nh, int nkv,
                  int page_size, int window, float scale_log2, int max_kv_len, int max_rows, float* scratch,
                  long scratch_floats, int settled, cudaStream_t stream) {
  int split = 0, max_splits = 0;
  const int rc = launch_stream_splits(q, q_stride, k_cache, v_cache, block_tables, max_blocks, cu_q, kv_lens, B, nh, nkv,
                                      page_size, window, scale_log2, max_kv_len, scratch, scratch_floats, settled, stream,
                                      &split, &max_splits);
  if (rc) return rc;
  const int threads = 32 * (max_rows < 16 ? max_rows : 16);
  co_launch(attn_combine_kernel, dim3(nkv, B), dim3(threads), 0, stream, (const float*)scratch, max_splits,
            (bf16*)out, out_stride, cu_q, kv_lens, nh, nkv, window, split);
  CO_CHECK_LAUNCH("attn_combine");
  return 0;
}
}  // namespace

CO_EXPORT int coheryn_attn_head_dim() { return HD; }
CO_EXPORT int coheryn_attn_split_keys() { return SPLIT_MIN; }
// keys = 128, 256 or 512 fixes the positions per CTA of the decode kernel; 0 restores the choice by batch size.
CO_EXPORT void coheryn_attn_set_tc_cluster(int cluster) { coheryn_attention_tc_set_cluster(cluster); }
CO_EXPORT void coheryn_attn_set_tc_two_tiles(int mode) { coheryn_attention_tc_set_two_tiles(mode); }
CO_EXPORT void coheryn_attn_set_split(int keys) {
  g_forced_split = (keys == 128 || keys == 256 || keys == 512 || keys == 1024 || keys == 2048) ? keys : 0;
}

// Floats of scratch that coheryn_attention_bf16 needs for B requests of at most
// max_kv_len positions when some request takes the split path.
CO_EXPORT long coheryn_attn_scratch_floats(int B, int nkv, int max_kv_len) {
  const long max_splits = (max_kv_len + SPLIT_MIN - 1) / SPLIT_MIN + 1;   // the smallest split needs the most
  return (long)B * nkv * max_splits * SPLIT_FLOATS;
}

// q: [T, nh*HD] rows of stride q_stride; out likewise.  Caches: [page][kv head][slot][HD].
// cu_q [B+1], kv_lens [B] on the device.  Host hints: max_rows = the largest q_len*G of the
// batch, any_small / any_large = whether some request has <= 16 / > 16 rows, max_kv_len,
// total_tokens = T, num_pages = pages per cache tensor; settled = whether the positions before each
// request's new tokens were written by EARLIER steps (the decode kernel then reads them ahead of time).
CO_EXPORT int coheryn_attention_bf16(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks, const int* cu_q,
                                     const int* kv_lens, int B, int nh, int nkv, int page_size, int window,
                                     float scale, int max_rows, int any_small, int any_large, int max_kv_len,
                                     float* scratch, long scratch_floats, int* status, int total_tokens,
                                     int num_pages, int settled, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh % nkv) CO_FAIL("attention_bf16: %d heads do not group over %d kv heads", nh, nkv);
  if ((q_stride & 7) || (out_stride & 3) || ((uintptr_t)out & 7))
    CO_FAIL("attention_bf16: q rows must keep 16-byte and out rows 8-byte alignment");
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    CO_FAIL("attention_bf16: operands must be 16-byte aligned");
  const float scale_log2 = scale * 1.4426950408889634f;
  const int G = nh / nkv;
  // Requests with at most 16 rows per kv head stream their keys through attn_stream.
  (void)status;
  const bool split_path = any_small && G <= 16 &&
                          (max_kv_len + SPLIT_MIN - 1) / SPLIT_MIN + 1 <= 512;   // attn_combine keeps 512 factors
  if (any_large || (any_small && !split_path)) {
    // Prompt portions: the tcgen05 kernel where it takes the shape, else the mma.sync one.
    if (status && coheryn_attention_tc_takes(nh, nkv, page_size) && ((uintptr_t)out & 7) == 0) {
      if (coheryn_attention_tc_launch(q, q_stride, total_tokens, out, out_stride, k_cache, v_cache, num_pages, block_tables,
                                      max_blocks, cu_q, kv_lens, B, nh, nkv, page_size, window, scale_log2, max_rows, max_kv_len,
                                      split_path ? 1 : 0, status, stream))
        return -1;
    } else {
      static bool configured = false;
      if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILES_SMEM);
        if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", TILES_SMEM, cudaGetErrorString(e));
        configured = true;
      }
      dim3 grid((max_rows + BM - 1) / BM, nkv, B);
      co_launch(attn_tiles_kernel, grid, dim3(128 * KG), TILES_SMEM, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,
                (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks, cu_q, kv_lens, nh, nkv, page_size,
                window, scale_log2, split_path ? 1 : 0);
      CO_CHECK_LAUNCH("attn_tiles");
    }
  }
  if (split_path)
    return launch_stream(q, q_stride, out, out_stride, k_cache, v_cache, block_tables, max_blocks, cu_q, kv_lens, B, nh,
                         nkv, page_size, window, scale_log2, max_kv_len, max_rows, scratch, scratch_floats, settled, stream);
  return 0;
}

// Decoding, one token per request (B <= 16 requests, at most 16 heads per kv head): attention over the
// cache pages and the output projection in two kernels.  q: [B, nh*HD]; w: [H, nh*HD] bfloat16 rows of
// stride ldw; parts: float32 [nh][B][H], the heads' contributions to q_attended @ w.T (+ bias in part
// 0), whose sum over the heads is the projection's output.  cu_q must be 0, 1, .., B.
CO_EXPORT int coheryn_attention_oproj_bf16(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                                           const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens,
                                           int B, int nh, int nkv, int page_size, int window, float scale, int max_kv_len,
                                           float* scratch, long scratch_floats, const void* w, long ldw, int H,
                                           const void* bias, int bias_dtype, float* parts, int settled, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (B > 16) CO_FAIL("attention_oproj: at most 16 requests, not %d", B);
  if (nkv <= 0 || nh % nkv || nh / nkv > 16) CO_FAIL("attention_oproj: %d heads over %d kv heads", nh, nkv);
  if ((q_stride & 7) || ((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)w & 15) ||
      (ldw & 7))
    CO_FAIL("attention_oproj: operands must be 16-byte aligned");
  if ((max_kv_len + SPLIT_MIN - 1) / SPLIT_MIN + 1 > 512) CO_FAIL("attention_oproj: %d positions are too many splits", max_kv_len);
  int split = 0, max_splits = 0;
  const int rc = launch_stream_splits(q, q_stride, k_cache, v_cache, block_tables, max_blocks, cu_q, kv_lens, B, nh, nkv,
                                      page_size, window, scale * 1.4426950408889634f, max_kv_len, scratch, scratch_floats,
                                      settled, stream, &split, &max_splits);
  if (rc) return rc;
  static size_t configured = 0;
  const size_t smem = mo_smem(max_splits);
  if (smem > configured) {
    if (smem > 200 * 1024) CO_FAIL("attention_oproj: %d splits need %zu bytes of shared memory", max_splits, smem);
    cudaError_t e = cudaFuncSetAttribute(attn_merge_oproj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) CO_FAIL("attention_oproj: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  co_launch(attn_merge_oproj_kernel, dim3((H + MO_TILE - 1) / MO_TILE, nh), dim3(MO_THREADS), smem, stream, (const float*)scratch,
            max_splits, kv_lens, B, nh, nkv, window, split, (const bf16*)w, ldw, H, bias, bias_dtype, parts);
  CO_CHECK_LAUNCH("attn_merge_oproj");
  return 0;
}
