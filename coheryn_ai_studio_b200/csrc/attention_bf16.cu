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
//  * attn_split:  for requests with at most 16 rows per kv head (decoding).  The key range
//    is cut into splits of 128 positions at ABSOLUTE multiples of 128; one CTA per
//    (request, kv head, split), each of its four warps taking tiles of 32 positions.
//    The warps' (max, sum, accumulator) triples are merged in warp order and written to
//    scratch; attn_combine merges the splits of a row in ascending order.
//
// Tiles start at absolute multiples of their size and splits likewise, so a
// row's result depends only on its own position and window, never on the batch.
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"

#ifndef CO_HEAD_DIM
#define CO_HEAD_DIM 128
#endif

namespace {
constexpr int HD = CO_HEAD_DIM;
constexpr int LDS = HD + 8;       // shared-memory row stride: 16 bytes of padding keep ldmatrix conflict-free
constexpr int SPLIT_MIN = 128;    // the smaller of the two split sizes of attn_split
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
// Scratch layout per (request, kv head, split): 16 rows x (HD + 2) floats:
// [0] = max (log2 domain), [1] = sum, [2..] = unnormalised accumulator.
constexpr int PART = HD + 2;

// Key positions per warp step in attn_split: a warp owns one buffer of SBN keys and SBN
// values and walks its share of the split (positions w*SBN, (w+4)*SBN, ... of the split)
// through it.  About 74 KB per CTA at head size 128: three CTAs, twelve warps per SM,
// each with its own copies in flight.
//
// Two shapes are built: <64, 256> (one CTA per SM, eight tiles of 64 in flight: best when
// the whole grid fits the GPU at once) and <32, 128> (three CTAs per SM: best when CTAs
// queue up).  Which one runs depends only on the batch's size, and a row's result depends
// on the shape (rounding), so a request may see either across steps.
template <int SBN, int SPLIT>
__global__ void __launch_bounds__(128)
attn_split_kernel(const bf16* __restrict__ q, long q_stride, float* __restrict__ scratch, int max_splits,
                  const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window, float scale_log2) {
  constexpr int SPLIT_TILES = SPLIT / (4 * SBN);   // tiles per warp
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][LDS]
  bf16* KVs = Qs + 16 * LDS;                                   // [4 warps][2][SBN][LDS]
  float* merge = reinterpret_cast<float*>(KVs);                // reused after the tiles: [4][16][PART]

  co_pdl_launch_dependents();
  co_pdl_wait();
  const int b = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rows > 16 || rows <= 0) return;
  const int base_pos = kv_len - q_len;
  const int pos_hi = kv_len - 1;
  const int key_first = window > 0 ? max(0, base_pos - window + 1) : 0;
  const int split = key_first / SPLIT + sp;      // absolute split index
  if (split * SPLIT > pos_hi) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_tables + (size_t)b * max_blocks;
  const int kv_end = pos_hi + 1;

  bf16* Kw = KVs + (size_t)warp * 2 * SBN * LDS;
  bf16* Vw = Kw + SBN * LDS;
  auto tile_key0 = [&](int i) { return split * SPLIT + (i * 4 + warp) * SBN; };
  // The warp's first tile that reaches into the visible range (a window hides earlier ones).
  int i0 = 0;
  while (i0 < SPLIT_TILES && tile_key0(i0) + SBN <= key_first) ++i0;
  load_q_rows(Qs, q, q_stride, tok0, kvh, G, 0, 16, rows, tid, 128);
  if (i0 < SPLIT_TILES && tile_key0(i0) <= pos_hi) {
    const TilePages tp = tile_pages<SBN>(table, page_size, tile_key0(i0), key_first, kv_end);
    load_tile<32, SBN>(Kw, k_cache, tp, kvh, nkv, page_size, tile_key0(i0), key_first, kv_end, lane);
    load_tile<32, SBN>(Vw, v_cache, tp, kvh, nkv, page_size, tile_key0(i0), key_first, kv_end, lane);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

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
  float o[1][HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[0][dt][i] = 0.f;
  RowState st[1];
  st[0].m[0] = st[0].m[1] = -INFINITY;
  st[0].l[0] = st[0].l[1] = 0.f;
#pragma unroll 1
  for (int i = i0; i < SPLIT_TILES; ++i) {
    if (tile_key0(i) > pos_hi) break;     // tiles of a warp ascend: nothing further is visible
    if (i > i0) {
      __syncwarp();                       // every lane is done reading the buffer
      const TilePages tp = tile_pages<SBN>(table, page_size, tile_key0(i), key_first, kv_end);
      load_tile<32, SBN>(Kw, k_cache, tp, kvh, nkv, page_size, tile_key0(i), key_first, kv_end, lane);
      load_tile<32, SBN>(Vw, v_cache, tp, kvh, nkv, page_size, tile_key0(i), key_first, kv_end, lane);
      cp_async_commit();
      cp_async_wait<0>();
      __syncwarp();
    }
    attend_tile<1, SBN, true, true>(nullptr, Qs, Kw, Vw, o, st, tile_key0(i), lo, hi, scale_log2);
  }
  __syncthreads();   // all warps are done with their tiles: the buffer becomes the merge area

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    float l = st[0].l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float* dst = merge + ((size_t)warp * 16 + r) * PART;
    if (t == 0) { dst[0] = st[0].m[h]; dst[1] = l; }
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
      dst[2 + dt * 8 + 2 * t] = o[0][dt][2 * h];
      dst[2 + dt * 8 + 2 * t + 1] = o[0][dt][2 * h + 1];
    }
  }
  __syncthreads();
  // Merge the four warps in warp order; write the valid rows.
  float* dst_base = scratch + (((size_t)b * nkv + kvh) * max_splits + sp) * 16 * PART;
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
    if (c == HD) { dst_base[r * PART] = M; dst_base[r * PART + 1] = acc; }
    else dst_base[r * PART + 2 + c] = acc;
  }
}

// One CTA per (request, kv head, row): the splits' (max, sum) pairs are read once into
// shared memory, then every thread merges its head-dim columns over the splits in
// ascending order with independent loads.
template <int SPLIT>
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* __restrict__ scratch, int max_splits, bf16* __restrict__ out, long out_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, int nh, int nkv, int window) {
  __shared__ float factor[512];
  __shared__ float s_den;
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int b = blockIdx.z, kvh = blockIdx.y, r = blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rows > 16 || r >= rows) return;
  const int base_pos = kv_len - q_len;
  const int key_first = window > 0 ? max(0, base_pos - window + 1) : 0;
  const int nsplits = min((kv_len - 1) / SPLIT - key_first / SPLIT + 1, 512);
  const float* src = scratch + (((size_t)b * nkv + kvh) * max_splits * 16 + r) * PART;
  const size_t stride = (size_t)16 * PART;
  for (int s = threadIdx.x; s < nsplits; s += blockDim.x) factor[s] = src[s * stride];
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = -INFINITY;
    for (int s = 0; s < nsplits; ++s) M = fmaxf(M, factor[s]);
    float den = 0.f;
    for (int s = 0; s < nsplits; ++s) {
      const float f = factor[s] == -INFINITY ? 0.f : exp2f(factor[s] - M);
      factor[s] = f;
      den += f * src[s * stride + 1];
    }
    s_den = den;
  }
  __syncthreads();
  const float inv = 1.0f / s_den;
  bf16* orow = out + (size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * HD;
  for (int c = threadIdx.x; c < HD; c += blockDim.x) {
    float num = 0.f;
#pragma unroll 4
    for (int s = 0; s < nsplits; ++s) num += factor[s] * src[s * stride + 2 + c];
    orow[c] = __float2bfloat16_rn(num * inv);
  }
}

// ------------------------------------------------------------------------------------
// attn_split with bulk copies.  Within a page the rows of a kv head are contiguous, so a
// warp's tile of 32 positions is fetched by a few cp.async.bulk copies (one per page it
// touches, per tensor) that ONE lane issues and an mbarrier counts in; no lane computes
// addresses of 16-byte pieces.  The tiles are unpadded in shared memory (ldmatrix then
// meets bank conflicts, which do not matter here: the kernel waits for memory, not for
// arithmetic).  One tile per warp, splits of 128 positions, three CTAs per SM.
// The wait on the mbarrier is bounded; if it runs out, `status` receives 21.
constexpr int BSBN = 32;
constexpr int BSPLIT = 4 * BSBN;

__device__ __forceinline__ void bulk_copy(void* dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}

__global__ void __launch_bounds__(128)
attn_split_bulk_kernel(const bf16* __restrict__ q, long q_stride, float* __restrict__ scratch, int max_splits,
                       const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                       const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                       const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window, float scale_log2,
                       int* __restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* KVs = reinterpret_cast<bf16*>(smem_raw);                // [4 warps][K: BSBN rows, V: BSBN rows][HD]
  bf16* Qs = KVs + 4 * 2 * BSBN * HD;                           // [16][LDS]
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(Qs + 16 * LDS);   // [4]
  float* merge = reinterpret_cast<float*>(smem_raw);            // reused after the tiles: [4][16][PART]

  co_pdl_launch_dependents();
  co_pdl_wait();
  const int b = blockIdx.z, kvh = blockIdx.y, sp = blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rows > 16 || rows <= 0) return;
  const int base_pos = kv_len - q_len;
  const int pos_hi = kv_len - 1;
  const int key_first = window > 0 ? max(0, base_pos - window + 1) : 0;
  const int split = key_first / BSPLIT + sp;      // absolute split index
  if (split * BSPLIT > pos_hi) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_tables + (size_t)b * max_blocks;
  const int kv_end = pos_hi + 1;

  bf16* Kw = KVs + (size_t)warp * 2 * BSBN * HD;
  bf16* Vw = Kw + BSBN * HD;
  const int key0 = split * BSPLIT + warp * BSBN;
  const int c_lo = max(key0, key_first), c_hi = min(key0 + BSBN, kv_end);   // positions to copy: [c_lo, c_hi)
  const bool w_active = c_lo < c_hi;
  load_q_rows(Qs, q, q_stride, tok0, kvh, G, 0, 16, rows, tid, 128);
  cp_async_commit();
  if (w_active) {
    if (lane == 0) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&bars[warp])));
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Rows of the tile that are not copied must still be finite for P V: zero them.
    for (int i = lane; i < BSBN * CHUNKS; i += 32) {
      const int row = i / CHUNKS;
      if (key0 + row < c_lo || key0 + row >= c_hi) {
        *reinterpret_cast<uint4*>(Kw + row * HD + (i % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(Vw + row * HD + (i % CHUNKS) * 8) = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes before the async copies
    __syncwarp();
    const TilePages tp = tile_pages<BSBN>(table, page_size, key0, key_first, kv_end);
    if (lane == 0) {
      const unsigned bytes = (unsigned)(c_hi - c_lo) * HD * 2 * 2;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(&bars[warp])), "r"(bytes) : "memory");
    }
    for (int pos = c_lo; pos < c_hi;) {
      const int block = pos / page_size;
      const int n = min(c_hi, (block + 1) * page_size) - pos;
      const int page = page_of(tp, block);                      // a shuffle: every lane takes part
      if (lane == 0) {
        const size_t off = (((size_t)page * nkv + kvh) * page_size + (pos - block * page_size)) * HD;
        bulk_copy(Kw + (pos - key0) * HD, k_cache + off, (unsigned)n * HD * 2, &bars[warp]);
        bulk_copy(Vw + (pos - key0) * HD, v_cache + off, (unsigned)n * HD * 2, &bars[warp]);
      }
      pos += n;
    }
  }
  cp_async_wait<0>();
  __syncthreads();              // the query rows are visible to every warp

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
  float o[1][HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[0][dt][i] = 0.f;
  RowState st[1];
  st[0].m[0] = st[0].m[1] = -INFINITY;
  st[0].l[0] = st[0].l[1] = 0.f;
  if (w_active) {
    bool landed = false;
    for (unsigned i = 0; i < (1u << 24) && !landed; ++i) {
      unsigned done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done) : "r"(smem_addr(&bars[warp])) : "memory");
      landed = done != 0;
    }
    if (landed) attend_tile<1, BSBN, true, true, HD>(nullptr, Qs, Kw, Vw, o, st, key0, lo, hi, scale_log2);
    else if (lane == 0) atomicExch(status, 21);
  }
  __syncthreads();   // all warps are done with their tiles: the buffer becomes the merge area

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    float l = st[0].l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float* dst = merge + ((size_t)warp * 16 + r) * PART;
    if (t == 0) { dst[0] = st[0].m[h]; dst[1] = l; }
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
      dst[2 + dt * 8 + 2 * t] = o[0][dt][2 * h];
      dst[2 + dt * 8 + 2 * t + 1] = o[0][dt][2 * h + 1];
    }
  }
  __syncthreads();
  // Merge the four warps in warp order; write the valid rows.
  float* dst_base = scratch + (((size_t)b * nkv + kvh) * max_splits + sp) * 16 * PART;
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
    if (c == HD) { dst_base[r * PART] = M; dst_base[r * PART + 1] = acc; }
    else dst_base[r * PART + 2 + c] = acc;
  }
}

constexpr size_t bulk_smem() {
  const size_t tiles = (size_t)4 * 2 * BSBN * HD * sizeof(bf16) + (size_t)16 * LDS * sizeof(bf16) + 4 * sizeof(unsigned long long);
  const size_t merge = (size_t)4 * 16 * PART * sizeof(float);
  return (tiles > merge ? tiles : merge) + 128;
}

constexpr size_t TILES_SMEM = (size_t)(BM + 4 * TILE) * LDS * sizeof(bf16);
static_assert((size_t)(KG - 1) * 4 * 16 * (HD + 2) * sizeof(float) <= (size_t)4 * TILE * LDS * sizeof(bf16), "the merge area fits the stages");
constexpr size_t split_smem(int sbn) {
  const size_t tiles = (size_t)(16 + 4 * 2 * sbn) * LDS * sizeof(bf16);
  const size_t merge = (size_t)16 * LDS * sizeof(bf16) + (size_t)4 * 16 * PART * sizeof(float);
  return tiles > merge ? tiles : merge;
}

template <int SBN, int SPLIT>
int launch_split(const void* q, long q_stride, void* out, long out_stride, const void* k_cache, const void* v_cache,
                 const int* block_tables, int max_blocks, const int* cu_q, const int* kv_lens, int B, int nh, int nkv,
                 int page_size, int window, float scale_log2, int max_kv_len, float* scratch, long scratch_floats,
                 cudaStream_t stream) {
  constexpr size_t SMEM = split_smem(SBN);
  const int max_splits = (max_kv_len + SPLIT - 1) / SPLIT + 1;
  if (!scratch || scratch_floats < (long)B * nkv * max_splits * 16 * PART)
    CO_FAIL("attention_bf16: scratch of %ld floats is too small", scratch_floats);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_split_kernel<SBN, SPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
    configured = true;
  }
  co_launch(attn_split_kernel<SBN, SPLIT>, dim3(max_splits, nkv, B), dim3(128), SMEM, stream, (const bf16*)q, q_stride,
            scratch, max_splits, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks, cu_q, kv_lens,
            nh, nkv, page_size, window, scale_log2);
  CO_CHECK_LAUNCH("attn_split");
  co_launch(attn_combine_kernel<SPLIT>, dim3(16, nkv, B), dim3(HD >= 128 ? 128 : 64), 0, stream, (const float*)scratch,
            max_splits, (bf16*)out, out_stride, cu_q, kv_lens, nh, nkv, window);
  CO_CHECK_LAUNCH("attn_combine");
  return 0;
}
int launch_split_bulk(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                      const void* v_cache, const int* block_tables, int max_blocks, const int* cu_q,
                      const int* kv_lens, int B, int nh, int nkv, int page_size, int window, float scale_log2,
                      int max_kv_len, float* scratch, long scratch_floats, int* status, cudaStream_t stream) {
  constexpr size_t SMEM = bulk_smem();
  const int max_splits = (max_kv_len + BSPLIT - 1) / BSPLIT + 1;
  if (!scratch || scratch_floats < (long)B * nkv * max_splits * 16 * PART)
    CO_FAIL("attention_bf16: scratch of %ld floats is too small", scratch_floats);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_split_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", SMEM, cudaGetErrorString(e));
    configured = true;
  }
  co_launch(attn_split_bulk_kernel, dim3(max_splits, nkv, B), dim3(128), SMEM, stream, (const bf16*)q, q_stride, scratch,
            max_splits, (const bf16*)k_cache, (const bf16*)v_cache, block_tables, max_blocks, cu_q, kv_lens, nh, nkv,
            page_size, window, scale_log2, status);
  CO_CHECK_LAUNCH("attn_split_bulk");
  co_launch(attn_combine_kernel<BSPLIT>, dim3(16, nkv, B), dim3(HD >= 128 ? 128 : 64), 0, stream, (const float*)scratch,
            max_splits, (bf16*)out, out_stride, cu_q, kv_lens, nh, nkv, window);
  CO_CHECK_LAUNCH("attn_combine");
  return 0;
}

// Which decode kernel runs: COHERYN_ATTN_SPLIT = auto | wide | narrow | bulk (experiments).
int split_choice() {
  static int choice = -1;
  if (choice < 0) {
    const char* e = getenv("COHERYN_ATTN_SPLIT");
    choice = !e ? 0 : (e[0] == 'w' ? 1 : (e[0] == 'n' ? 2 : (e[0] == 'b' ? 3 : 0)));
  }
  return choice;
}
}  // namespace

CO_EXPORT int coheryn_attn_head_dim() { return HD; }
CO_EXPORT int coheryn_attn_split_keys() { return SPLIT_MIN; }

// Floats of scratch that coheryn_attention_bf16 needs for B requests of at most
// max_kv_len positions when some request takes the split path.
CO_EXPORT long coheryn_attn_scratch_floats(int B, int nkv, int max_kv_len) {
  const long max_splits = (max_kv_len + SPLIT_MIN - 1) / SPLIT_MIN + 1;   // covers both split sizes
  return (long)B * nkv * max_splits * 16 * PART;
}

// q: [T, nh*HD] rows of stride q_stride; out likewise.  Caches: [page][kv head][slot][HD].
// cu_q [B+1], kv_lens [B] on the device.  Host hints: max_rows = the largest q_len*G of the
// batch, any_small / any_large = whether some request has <= 16 / > 16 rows, max_kv_len.
CO_EXPORT int coheryn_attention_bf16(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks, const int* cu_q,
                                     const int* kv_lens, int B, int nh, int nkv, int page_size, int window,
                                     float scale, int max_rows, int any_small, int any_large, int max_kv_len,
                                     float* scratch, long scratch_floats, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh % nkv) CO_FAIL("attention_bf16: %d heads do not group over %d kv heads", nh, nkv);
  if ((q_stride & 7) || (out_stride & 1)) CO_FAIL("attention_bf16: row strides must keep 16-byte alignment");
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    CO_FAIL("attention_bf16: operands must be 16-byte aligned");
  const float scale_log2 = scale * 1.4426950408889634f;
  const int G = nh / nkv;
  // The split kernel keeps eight tiles in shared memory; beyond 227 KB every request takes
  // the tile kernel instead.
  const bool split_path = any_small && G <= 16 && split_smem(32) <= 227 * 1024 &&
                          (max_kv_len + SPLIT_MIN - 1) / SPLIT_MIN + 1 <= 512;   // attn_combine keeps 512 factors
  if (any_large || (any_small && !split_path)) {
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
  if (split_path) {
    // All CTAs of the wide shape resident at once (one per SM, with a little queueing)?
    const long wide_ctas = (long)B * nkv * ((max_kv_len + 255) / 256 + 1);
    const int choice = split_choice();
    // Measured on a B200 inside whole decode steps (cold cache): the wide shape wins while its
    // grid fits the GPU about twice over, the narrow one beyond.
    const bool wide = choice == 1 || (choice == 0 && wide_ctas <= 2 * 148);
    if (wide && split_smem(64) <= 227 * 1024)
      return launch_split<64, 256>(q, q_stride, out, out_stride, k_cache, v_cache, block_tables, max_blocks, cu_q,
                                   kv_lens, B, nh, nkv, page_size, window, scale_log2, max_kv_len, scratch,
                                   scratch_floats, stream);
    if (choice != 3 || !status)   // measured: the bulk-copy shape is no faster than the cp.async one
      return launch_split<32, 128>(q, q_stride, out, out_stride, k_cache, v_cache, block_tables, max_blocks, cu_q,
                                   kv_lens, B, nh, nkv, page_size, window, scale_log2, max_kv_len, scratch,
                                   scratch_floats, stream);
    return launch_split_bulk(q, q_stride, out, out_stride, k_cache, v_cache, block_tables, max_blocks, cu_q, kv_lens, B,
                             nh, nkv, page_size, window, scale_log2, max_kv_len, scratch, scratch_floats, status, stream);
  }
  return 0;
}
