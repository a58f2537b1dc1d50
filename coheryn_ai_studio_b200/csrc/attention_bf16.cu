// Causal (optionally windowed) grouped-query attention over cache pages in bfloat16 on the
// tensor cores (mma.sync m16n8k16, float32 accumulation and float32 softmax), compiled for
// one head size (CO_HEAD_DIM, a multiple of 16 up to 256).
//
// The query rows of a request and kv head are numbered r = token * G + head_in_group
// (G = heads / kv_heads), so that all G query heads of a group share each key/value tile
// that is read.  Two kernels:
//
//  * attn_tiles:  one CTA per (request, kv head, tile of 64 rows); four warps of 16 rows
//    share key/value tiles of 64 positions that are copied from the pages into shared
//    memory with cp.async (double buffered).  Used for prompt portions.
//  * attn_split:  for requests with at most 16 rows per kv head (decoding).  The key range
//    is cut into splits of 256 positions at ABSOLUTE multiples of 256; one CTA per
//    (request, kv head, split), each of its four warps taking one tile of 64 positions.
//    The warps' (max, sum, accumulator) triples are merged in warp order and written to
//    scratch; attn_combine merges the splits of a row in ascending order.
//
// Tiles start at absolute multiples of 64 and splits at absolute multiples of 256, so a
// row's result depends only on its own position and window, never on the batch.
#include <cuda_bf16.h>

#include "common.cuh"

#ifndef CO_HEAD_DIM
#define CO_HEAD_DIM 128
#endif

namespace {
constexpr int HD = CO_HEAD_DIM;
constexpr int BN = 64;            // key positions per tile
constexpr int BM = 64;            // query rows per CTA in attn_tiles
constexpr int LDS = HD + 8;       // shared-memory row stride: 16 bytes of padding keep ldmatrix conflict-free
constexpr int SPLIT = 256;        // key positions per split in attn_split
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

// The pages that hold positions [key0, key0 + BN): each lane of a warp fetches up to two
// block-table entries once per tile (entries lane and lane + 32 of the tile's page run);
// page_of() then hands them out by shuffle, so that the copies below wait on no load.
struct TilePages {
  int e0, e1, first_block;
};
__device__ __forceinline__ TilePages tile_pages(const int* __restrict__ table, int page_size, int key0,
                                                int kv_begin, int kv_end) {
  const int lane = threadIdx.x & 31;
  TilePages tp;
  const int lo = max(key0, kv_begin), hi = min(key0 + BN, kv_end) - 1;   // positions really read
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

// Copies key or value rows of positions [key0, key0 + BN) of one kv head from the pages
// into a [BN][LDS] tile; positions outside [kv_begin, kv_end) are zero filled and their
// pages are not touched (a window may already have given them back).  `nthreads` threads
// with ids `tid` cooperate (whole warps; every lane runs every iteration).
__device__ __forceinline__ void load_tile(bf16* tile, const bf16* __restrict__ cache, const TilePages& tp,
                                          int kvh, int nkv, int page_size, int key0, int kv_begin, int kv_end,
                                          int tid, int nthreads) {
  constexpr int TOTAL = BN * CHUNKS;
  for (int c0 = 0; c0 < TOTAL; c0 += nthreads) {
    const int c = c0 + tid;
    const int row = c / CHUNKS, piece = c % CHUNKS;
    const int pos = key0 + row;
    const bool valid = c < TOTAL && pos >= kv_begin && pos < kv_end;
    const int block = valid ? pos / page_size : tp.first_block;
    const int page = page_of(tp, block);
    if (c < TOTAL) {
      const bf16* src = valid ? cache + (((size_t)page * nkv + kvh) * page_size + (pos - block * page_size)) * HD + piece * 8
                              : cache;
      cp_async16(tile + row * LDS + piece * 8, src, valid);
    }
  }
}

struct RowState {
  float m[2];   // running maximum of the scaled scores (log2 domain), rows g and g+8
  float l[2];   // this thread's share of the running sum
};

// One warp, 16 query rows against one tile of BN key positions in shared memory:
// S = Q K^T, masking, online softmax, O += P V.
//   qf: the warp's Q fragments; Ks/Vs: [BN][LDS] tiles; key0: position of the tile's row 0;
//   lo[h], hi[h]: first and last visible key position of the thread's rows g (h=0), g+8 (h=1).
__device__ __forceinline__ void attend_tile(const unsigned (&qf)[HD / 16][4], const bf16* Ks, const bf16* Vs,
                                            float (&o)[HD / 8][4], RowState& st, int key0, const int (&lo)[2],
                                            const int (&hi)[2], float scale_log2) {
  const int lane = threadIdx.x & 31;
  const int t = lane & 3;
  float s[BN / 8][4];
#pragma unroll
  for (int j = 0; j < BN / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[j][i] = 0.f;

  // S = Q K^T.  ldmatrix.x4 on K rows yields the B fragments of two neighbouring key tiles.
  {
    const int id = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kd = 0; kd < HD / 16; ++kd) {
#pragma unroll
      for (int jp = 0; jp < BN / 16; ++jp) {
        unsigned b[4];
        ldmatrix_x4(b, Ks + (jp * 16 + (id >> 1) * 8 + r) * LDS + kd * 16 + (id & 1) * 8);
        mma_bf16(s[2 * jp], qf[kd], b[0], b[1]);
        mma_bf16(s[2 * jp + 1], qf[kd], b[2], b[3]);
      }
    }
  }

  // Mask and online softmax.  Thread holds, for rows g (i = 0,1) and g+8 (i = 2,3), the
  // key columns key0 + 8 j + 2 t + (i & 1).
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int key = key0 + j * 8 + 2 * t + i;
        float v = s[j][2 * h + i] * scale_log2;
        if (key < lo[h] || key > hi[h]) v = -INFINITY;
        s[j][2 * h + i] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(st.m[h], mx);
    // Everything masked so far: keep the state untouched and let p be zero.
    const float m_use = m_new == -INFINITY ? 0.f : m_new;
    const float corr = st.m[h] == -INFINITY ? 0.f : exp2f(st.m[h] - m_use);
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float p = exp2f(s[j][2 * h + i] - m_use);  // exp2(-inf) = 0 for masked keys
        s[j][2 * h + i] = p;
        part += p;
      }
    st.l[h] = st.l[h] * corr + part;
    st.m[h] = m_new;
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
      o[dt][2 * h] *= corr;
      o[dt][2 * h + 1] *= corr;
    }
  }

  // O += P V.  The S accumulators of two neighbouring key tiles are the A fragment of one
  // 16-position step; ldmatrix.x4.trans on V rows yields B fragments of two head-dim tiles.
  {
    const int id = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kt = 0; kt < BN / 16; ++kt) {
      unsigned a[4];
      a[0] = pack_bf16(s[2 * kt][0], s[2 * kt][1]);
      a[1] = pack_bf16(s[2 * kt][2], s[2 * kt][3]);
      a[2] = pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]);
      a[3] = pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3]);
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        unsigned b[4];
        ldmatrix_x4_trans(b, Vs + (kt * 16 + (id & 1) * 8 + r) * LDS + dp * 16 + (id >> 1) * 8);
        mma_bf16(o[2 * dp], a, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
  }
}

// Loads the warp's 16 query rows (already in shared memory, [16][LDS]) as A fragments.
__device__ __forceinline__ void load_q_frags(unsigned (&qf)[HD / 16][4], const bf16* Qs) {
  const int lane = threadIdx.x & 31;
  const int id = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kd = 0; kd < HD / 16; ++kd) ldmatrix_x4(qf[kd], Qs + ((id & 1) * 8 + r) * LDS + kd * 16 + (id >> 1) * 8);
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
__global__ void __launch_bounds__(128)
attn_tiles_kernel(const bf16* __restrict__ q, long q_stride, bf16* __restrict__ out, long out_stride,
                  const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window,
                  float scale_log2, int skip_small) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [BM][LDS]
  bf16* Ks = Qs + BM * LDS;                                    // [2][BN][LDS]
  bf16* Vs = Ks + 2 * BN * LDS;                                // [2][BN][LDS]

  const int b = blockIdx.z, kvh = blockIdx.y, rt = blockIdx.x;
  const int G = nh / nkv;
  const int tok0 = cu_q[b], q_len = cu_q[b + 1] - tok0, kv_len = kv_lens[b];
  const int rows = q_len * G;
  if (rt * BM >= rows) return;
  if (skip_small && rows <= 16) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int* table = block_tables + (size_t)b * max_blocks;
  const int base_pos = kv_len - q_len;   // position of the request's first token in this step

  // Key range needed by this tile of rows.
  const int row_first = rt * BM, row_last = min(rows, row_first + BM) - 1;
  const int pos_lo = base_pos + row_first / G, pos_hi = base_pos + row_last / G;
  const int key_first = window > 0 ? max(0, pos_lo - window + 1) : 0;
  const int tile_first = key_first / BN, tile_last = pos_hi / BN;
  const int kv_end = pos_hi + 1;

  load_q_rows(Qs, q, q_stride, tok0, kvh, G, row_first, BM, rows, tid, 128);
  {
    const TilePages tp = tile_pages(table, page_size, tile_first * BN, key_first, kv_end);
    load_tile(Ks, k_cache, tp, kvh, nkv, page_size, tile_first * BN, key_first, kv_end, tid, 128);
    load_tile(Vs, v_cache, tp, kvh, nkv, page_size, tile_first * BN, key_first, kv_end, tid, 128);
  }
  cp_async_commit();

  int lo[2], hi[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_first + warp * 16 + h * 8 + g;
    if (r < rows) {
      hi[h] = base_pos + r / G;
      lo[h] = window > 0 ? max(0, hi[h] - window + 1) : 0;
    } else {
      hi[h] = -1; lo[h] = 0;
    }
  }
  // The warp's own key range (skip tiles in which none of its 16 rows sees a key).
  const int w_row_first = row_first + warp * 16;
  const int w_row_last = min(rows - 1, w_row_first + 15);
  const bool w_active = w_row_first < rows;
  const int w_hi = w_active ? base_pos + w_row_last / G : -1;
  const int w_lo = w_active ? (window > 0 ? max(0, base_pos + w_row_first / G - window + 1) : 0) : 0;

  float o[HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;
  RowState st;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
  unsigned qf[HD / 16][4];

  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int buf = (tile - tile_first) & 1;
    if (tile < tile_last) {
      const TilePages tp = tile_pages(table, page_size, (tile + 1) * BN, key_first, kv_end);
      load_tile(Ks + (buf ^ 1) * BN * LDS, k_cache, tp, kvh, nkv, page_size, (tile + 1) * BN, key_first, kv_end, tid, 128);
      load_tile(Vs + (buf ^ 1) * BN * LDS, v_cache, tp, kvh, nkv, page_size, (tile + 1) * BN, key_first, kv_end, tid, 128);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (tile == tile_first) load_q_frags(qf, Qs + warp * 16 * LDS);
    const int key0 = tile * BN;
    if (w_active && key0 <= w_hi && key0 + BN > w_lo)
      attend_tile(qf, Ks + buf * BN * LDS, Vs + buf * BN * LDS, o, st, key0, lo, hi, scale_log2);
    __syncthreads();
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_first + warp * 16 + h * 8 + g;
    float l = st.l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (r >= rows) continue;
    const float inv = 1.0f / l;
    bf16* orow = out + (size_t)(tok0 + r / G) * out_stride + (size_t)(kvh * G + r % G) * HD;
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt)
      *reinterpret_cast<__nv_bfloat162*>(orow + dt * 8 + 2 * t) =
          __floats2bfloat162_rn(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
  }
}

// ------------------------------------------------------------------------------------
// Scratch layout per (request, kv head, split): 16 rows x (HD + 2) floats:
// [0] = max (log2 domain), [1] = sum, [2..] = unnormalised accumulator.
constexpr int PART = HD + 2;

__global__ void __launch_bounds__(128)
attn_split_kernel(const bf16* __restrict__ q, long q_stride, float* __restrict__ scratch, int max_splits,
                  const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                  const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ cu_q,
                  const int* __restrict__ kv_lens, int nh, int nkv, int page_size, int window, float scale_log2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);                 // [16][LDS]
  bf16* KVs = Qs + 16 * LDS;                                   // [4 warps][2][BN][LDS]
  float* merge = reinterpret_cast<float*>(KVs);                // reused after the tiles: [4][16][PART]

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

  // Each warp takes one tile of the split.
  const int key0 = split * SPLIT + warp * BN;
  bf16* Kw = KVs + (size_t)warp * 2 * BN * LDS;
  bf16* Vw = Kw + BN * LDS;
  const bool w_active = key0 <= pos_hi && key0 + BN > key_first;
  load_q_rows(Qs, q, q_stride, tok0, kvh, G, 0, 16, rows, tid, 128);
  if (w_active) {
    const TilePages tp = tile_pages(table, page_size, key0, key_first, kv_end);
    load_tile(Kw, k_cache, tp, kvh, nkv, page_size, key0, key_first, kv_end, lane, 32);
    load_tile(Vw, v_cache, tp, kvh, nkv, page_size, key0, key_first, kv_end, lane, 32);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();

  int lo[2], hi[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    if (r < rows) {
      hi[h] = base_pos + r / G;
      lo[h] = window > 0 ? max(0, hi[h] - window + 1) : 0;
    } else {
      hi[h] = -1; lo[h] = 0;
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int dt = 0; dt < HD / 8; ++dt)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[dt][i] = 0.f;
  RowState st;
  st.m[0] = st.m[1] = -INFINITY;
  st.l[0] = st.l[1] = 0.f;
  if (w_active) {
    unsigned qf[HD / 16][4];
    load_q_frags(qf, Qs);
    attend_tile(qf, Kw, Vw, o, st, key0, lo, hi, scale_log2);
  }
  __syncthreads();   // all warps are done with their tiles: the buffer becomes the merge area

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = h * 8 + g;
    float l = st.l[h];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    float* dst = merge + ((size_t)warp * 16 + r) * PART;
    if (t == 0) { dst[0] = st.m[h]; dst[1] = l; }
#pragma unroll
    for (int dt = 0; dt < HD / 8; ++dt) {
      dst[2 + dt * 8 + 2 * t] = o[dt][2 * h];
      dst[2 + dt * 8 + 2 * t + 1] = o[dt][2 * h + 1];
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
__global__ void __launch_bounds__(128)
attn_combine_kernel(const float* __restrict__ scratch, int max_splits, bf16* __restrict__ out, long out_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, int nh, int nkv, int window) {
  __shared__ float factor[512];
  __shared__ float s_den;
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

constexpr size_t TILES_SMEM = (size_t)(BM + 4 * BN) * LDS * sizeof(bf16);
constexpr size_t SPLIT_TILE_SMEM = (size_t)(16 + 4 * 2 * BN) * LDS * sizeof(bf16);
constexpr size_t SPLIT_MERGE_SMEM = (size_t)16 * LDS * sizeof(bf16) + (size_t)4 * 16 * PART * sizeof(float);
constexpr size_t SPLIT_SMEM = SPLIT_TILE_SMEM > SPLIT_MERGE_SMEM ? SPLIT_TILE_SMEM : SPLIT_MERGE_SMEM;
}  // namespace

CO_EXPORT int coheryn_attn_head_dim() { return HD; }
CO_EXPORT int coheryn_attn_split_keys() { return SPLIT; }

// Floats of scratch that coheryn_attention_bf16 needs for B requests of at most
// max_kv_len positions when some request takes the split path.
CO_EXPORT long coheryn_attn_scratch_floats(int B, int nkv, int max_kv_len) {
  const long max_splits = (max_kv_len + SPLIT - 1) / SPLIT + 1;
  return (long)B * nkv * max_splits * 16 * PART;
}

// q: [T, nh*HD] rows of stride q_stride; out likewise.  Caches: [page][kv head][slot][HD].
// cu_q [B+1], kv_lens [B] on the device.  Host hints: max_rows = the largest q_len*G of the
// batch, any_small / any_large = whether some request has <= 16 / > 16 rows, max_kv_len.
CO_EXPORT int coheryn_attention_bf16(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                                     const void* v_cache, const int* block_tables, int max_blocks, const int* cu_q,
                                     const int* kv_lens, int B, int nh, int nkv, int page_size, int window,
                                     float scale, int max_rows, int any_small, int any_large, int max_kv_len,
                                     float* scratch, long scratch_floats, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh % nkv) CO_FAIL("attention_bf16: %d heads do not group over %d kv heads", nh, nkv);
  if ((q_stride & 7) || (out_stride & 1)) CO_FAIL("attention_bf16: row strides must keep 16-byte alignment");
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15))
    CO_FAIL("attention_bf16: operands must be 16-byte aligned");
  const float scale_log2 = scale * 1.4426950408889634f;
  const int G = nh / nkv;
  // The split kernel keeps eight tiles in shared memory; beyond 227 KB every request takes
  // the tile kernel instead.
  const bool split_path = any_small && G <= 16 && SPLIT_SMEM <= 227 * 1024;
  if (any_large || (any_small && !split_path)) {
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_tiles_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TILES_SMEM);
      if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", TILES_SMEM, cudaGetErrorString(e));
      configured = true;
    }
    dim3 grid((max_rows + BM - 1) / BM, nkv, B);
    attn_tiles_kernel<<<grid, 128, TILES_SMEM, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_tables,
        max_blocks, cu_q, kv_lens, nh, nkv, page_size, window, scale_log2, split_path ? 1 : 0);
    CO_CHECK_LAUNCH("attn_tiles");
  }
  if (split_path) {
    const int max_splits = (max_kv_len + SPLIT - 1) / SPLIT + 1;
    if (!scratch || scratch_floats < (long)B * nkv * max_splits * 16 * PART)
      CO_FAIL("attention_bf16: scratch of %ld floats is too small", scratch_floats);
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SPLIT_SMEM);
      if (e != cudaSuccess) CO_FAIL("attention_bf16: %zu bytes of shared memory: %s", SPLIT_SMEM, cudaGetErrorString(e));
      configured = true;
    }
    dim3 grid(max_splits, nkv, B);
    attn_split_kernel<<<grid, 128, SPLIT_SMEM, stream>>>(
        (const bf16*)q, q_stride, scratch, max_splits, (const bf16*)k_cache, (const bf16*)v_cache, block_tables,
        max_blocks, cu_q, kv_lens, nh, nkv, page_size, window, scale_log2);
    CO_CHECK_LAUNCH("attn_split");
    attn_combine_kernel<<<dim3(16, nkv, B), HD >= 128 ? 128 : 64, 0, stream>>>(scratch, max_splits, (bf16*)out, out_stride, cu_q, kv_lens,
                                                          nh, nkv, window);
    CO_CHECK_LAUNCH("attn_combine");
  }
  return 0;
}
