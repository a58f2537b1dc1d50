// Token selection on the device.
//
// argmax: greedy decoding, first index of the maximum (ties go to the lowest id), as
// crates/coheryn-engine/src/sampling.rs:160-173 scans with a strict '>'.
//
// sample: temperature sampling with optional top-k and top-p, in the reference's order
// of operations (sampling.rs:186-222): candidates are ranked by (value descending, id
// ascending); p_i = exp((v_i - v_max) / T); top-k keeps the first k; top-p keeps the
// shortest prefix whose normalised cumulative mass reaches top_p; the draw u in [0,1)
// (made on the host by the request's SplitMix64 stream) picks the first candidate whose
// cumulative mass exceeds u * (kept mass).  No sort is materialised: the rank order is
// walked by radix descent over the order-preserving 32-bit image of the logits, 8 bits
// a level, with per-bucket counts and masses accumulated in float64.
#include "common.cuh"

namespace {

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, long stride, int V, int* __restrict__ out,
              int* __restrict__ status) {
  __shared__ float sv[32];
  __shared__ int si[32];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const float* row = logits + (size_t)blockIdx.x * stride;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  bool bad = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if (bad) atomicExch(status, 2);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    bv = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Two-stage variant for wide rows: stage 1 lets many CTAs scan pieces of a row, stage 2
// (argmax_kernel over the partial values with their indices) picks among the pieces.
constexpr int ARGMAX_PIECE = 4096;

__global__ void __launch_bounds__(256)
argmax_pieces_kernel(const float* __restrict__ logits, long stride, int V, float* __restrict__ part_val,
                     int* __restrict__ part_idx, int pieces, int* __restrict__ status) {
  __shared__ float sv[8];
  __shared__ int si[8];
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.y, piece = blockIdx.x;
  const float* row = logits + (size_t)r * stride;
  const int lo = piece * ARGMAX_PIECE, hi = min(V, lo + ARGMAX_PIECE);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  bool bad = false;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  if (bad) atomicExch(status, 2);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
    part_val[(size_t)r * pieces + piece] = bv;
    part_idx[(size_t)r * pieces + piece] = bi;
  }
}

__global__ void __launch_bounds__(64)
argmax_final_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int pieces,
                    int* __restrict__ out) {
  co_pdl_launch_dependents();
  co_pdl_wait();
  const int r = blockIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    const float v = part_val[(size_t)r * pieces + i];
    const int idx = part_idx[(size_t)r * pieces + i];
    if (better(v, idx, bv, bi)) { bv = v; bi = idx; }
  }
  __shared__ float sv[2];
  __shared__ int si[2];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (better(sv[1], si[1], bv, bi)) { bv = sv[1]; bi = si[1]; }
    out[r] = bi == 0x7fffffff ? 0 : bi;
  }
}

// Order-preserving map: larger float -> SMALLER key, so ascending keys walk the
// candidates from the largest logit down.
__device__ __forceinline__ unsigned desc_key(float v) {
  unsigned u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);  // ascending image
  return ~u;                                        // descending
}

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ float key_value(unsigned key) {
  const unsigned asc = ~key;
  const unsigned bits = (asc & 0x80000000u) ? (asc & 0x7fffffffu) : ~asc;
  return __uint_as_float(bits);
}

// Histogram of the next 8-bit digit among the elements whose higher digits equal those
// of prefix: per bucket the number of candidates and their mass.  A thread keeps the
// bucket it is adding to in registers and only touches shared memory when the digit
// changes, because neighbouring logits mostly share their high digits.
__device__ void histogram(const float* row, int V, float vmax, float inv_t, unsigned prefix, int level,
                          double* h_mass, unsigned* h_count) {
  for (int b = threadIdx.x; b < 256; b += blockDim.x) { h_mass[b] = 0.0; h_count[b] = 0u; }
  __syncthreads();
  const int shift = 24 - 8 * level;
  int cur = -1;
  double cur_mass = 0.0;
  unsigned cur_count = 0u;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    const unsigned key = desc_key(v);
    if (level != 0 && (key >> (shift + 8)) != (prefix >> (shift + 8))) continue;
    const int digit = (int)((key >> shift) & 255u);
    if (digit != cur) {
      if (cur >= 0) { atomicAdd(&h_mass[cur], cur_mass); atomicAdd(&h_count[cur], cur_count); }
      cur = digit; cur_mass = 0.0; cur_count = 0u;
    }
    cur_mass += exp(((double)v - (double)vmax) * (double)inv_t);
    cur_count += 1u;
  }
  if (cur >= 0) { atomicAdd(&h_mass[cur], cur_mass); atomicAdd(&h_count[cur], cur_count); }
  __syncthreads();
}

struct SampleShared {
  double h_mass[256];
  unsigned h_count[256];
  double before_mass;      // mass of the candidates ranked before the current bucket
  long long before_count;  // their number
  unsigned prefix;         // key digits fixed so far
  unsigned bucket_count;   // candidates in the bucket picked last
  double result_mass;
  long long result_rank;
};

enum { BY_COUNT = 0, BY_FRACTION = 1, BY_MASS = 2 };

// Walks the rank order (value descending, id ascending) down to one key, one 8-bit digit a
// level, looking for the first rank r that satisfies
//   BY_COUNT:    r >= target_count            (result_mass = mass of ranks 1..r)
//   BY_FRACTION: mass(1..r) / total >= frac   (result_rank = r)
//   BY_MASS:     threshold < mass(1..r)       (prefix = its key, result_rank = rank among
//                                              the candidates of that key, 1-based)
// After four levels the bucket holds n candidates of ONE value, ranked by id, so the rank
// inside it follows from arithmetic on n equal masses.  If rounding leaves the target
// past the last candidate, the last one is taken.
__device__ void descend(SampleShared& sh, const float* row, int V, float vmax, float inv_t, int mode,
                        long long target_count, double total, double frac, double threshold) {
  if (threadIdx.x == 0) { sh.prefix = 0u; sh.before_mass = 0.0; sh.before_count = 0; }
  __syncthreads();
  for (int level = 0; level < 4; ++level) {
    histogram(row, V, vmax, inv_t, sh.prefix, level, sh.h_mass, sh.h_count);
    if (threadIdx.x == 0) {
      double cm = sh.before_mass;
      long long cc = sh.before_count;
      int pick = -1;
      double pick_cm = cm;
      long long pick_cc = cc;
      for (int b = 0; b < 256; ++b) {
        if (sh.h_count[b] == 0u) continue;
        const double nm = cm + sh.h_mass[b];
        const long long nc = cc + sh.h_count[b];
        bool inside;
        if (mode == BY_COUNT) inside = nc >= target_count;
        else if (mode == BY_FRACTION) inside = nm / total >= frac;
        else inside = threshold < nm;
        pick = b; pick_cm = cm; pick_cc = cc;
        if (inside) break;
        cm = nm; cc = nc;
      }
      sh.before_mass = pick_cm;
      sh.before_count = pick_cc;
      sh.prefix |= (unsigned)pick << (24 - 8 * level);
      sh.bucket_count = sh.h_count[pick];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const long long n = (long long)sh.bucket_count;
    const double p = exp(((double)key_value(sh.prefix) - (double)vmax) * (double)inv_t);
    const double cm = sh.before_mass;
    const long long cc = sh.before_count;
    long long j = 1;
    if (mode == BY_COUNT) {
      j = target_count - cc;
      if (j > n) j = n;
      if (j < 1) j = 1;
    } else if (mode == BY_FRACTION) {
      while (j < n && !((cm + (double)j * p) / total >= frac)) ++j;
    } else {
      while (j < n && !(threshold < cm + (double)j * p)) ++j;
    }
    sh.result_mass = cm + (double)j * p;
    sh.result_rank = mode == BY_MASS ? j : cc + j;
  }
  __syncthreads();
}

// One row per block.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const double* __restrict__ uniform, int* __restrict__ out, int* __restrict__ status) {
  __shared__ SampleShared sh;
  __shared__ float s_red[33];
  __shared__ int s_scan[SAMPLE_THREADS];
  __shared__ int s_owner;
  __shared__ long long s_rank;

  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * stride;
  const float inv_t = 1.0f / temperature[r];
  const double p_keep = (double)top_p[r];
  long long K = top_k[r];
  if (K <= 0 || K > V) K = V;

  float vmax = -INFINITY;
  bool bad = false;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (!isfinite(v)) bad = true;
    vmax = fmaxf(vmax, v);
  }
  if (bad) atomicExch(status, 2);
  vmax = co_warp_max(vmax);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = vmax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s_red[threadIdx.x] : -INFINITY;
    t = co_warp_max(t);
    if (threadIdx.x == 0) s_red[32] = t;
  }
  __syncthreads();
  vmax = s_red[32];

  // 1. total = mass of the K best candidates (top-k is applied first; K = V without it)
  descend(sh, row, V, vmax, inv_t, BY_COUNT, K, 0.0, 0.0, 0.0);
  const double total = sh.result_mass;
  // 2. keep = first rank whose normalised cumulative mass reaches top_p (never beyond K)
  long long keep = K;
  if (p_keep < 1.0) {
    descend(sh, row, V, vmax, inv_t, BY_FRACTION, 0, total, p_keep, 0.0);
    keep = sh.result_rank < K ? sh.result_rank : K;
  }
  // 3. kept = mass of ranks 1..keep; the draw lands at u * kept
  double kept = total;
  if (keep < K) {
    descend(sh, row, V, vmax, inv_t, BY_COUNT, keep, 0.0, 0.0, 0.0);
    kept = sh.result_mass;
  }
  // 4. the first candidate whose cumulative mass exceeds the threshold
  descend(sh, row, V, vmax, inv_t, BY_MASS, 0, 0.0, 0.0, uniform[r] * kept);
  if (threadIdx.x == 0) {
    long long j = sh.result_rank;
    if (sh.before_count + j > keep) j = keep - sh.before_count;   // never outside the kept prefix
    if (j < 1) j = 1;
    s_rank = j;
  }
  __syncthreads();

  // The s_rank-th id (ascending) whose key equals the final key: blocked partition,
  // count, scan, then the owning thread walks its chunk.
  const unsigned key = sh.prefix;
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(V, (int)threadIdx.x * chunk), hi = min(V, lo + chunk);
  int mine = 0;
  for (int i = lo; i < hi; ++i) mine += desc_key(row[i]) == key;
  s_scan[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long want = s_rank;
    long long acc = 0;
    int owner = -1, last_owner = 0;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {
      if (s_scan[t] > 0) last_owner = t;
      if (owner < 0 && acc + s_scan[t] >= want) { owner = t; s_rank = want - acc; }
      acc += s_scan[t];
    }
    if (owner < 0) { owner = last_owner; s_rank = s_scan[last_owner]; }
    s_owner = owner;
  }
  __syncthreads();
  if ((int)threadIdx.x == s_owner) {
    long long seen = 0;
    int choice = lo;
    for (int i = lo; i < hi; ++i)
      if (desc_key(row[i]) == key) { choice = i; if (++seen == s_rank) break; }
    out[r] = choice;
  }
}

// Penalties over the ids a request has seen (sampling.rs:131-143): for item i,
// v = logits[rows[i], ids[i]]; v = v < 0 ? v * rep : v / rep; v -= presence + count * frequency.
__global__ void apply_penalties_kernel(float* __restrict__ logits, long stride, int n,
                                       const int* __restrict__ rows, const int* __restrict__ ids,
                                       const int* __restrict__ counts, const float* __restrict__ rep,
                                       const float* __restrict__ freq, const float* __restrict__ pres) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float* p = logits + (size_t)rows[i] * stride + ids[i];
  float v = *p;
  v = v < 0.f ? v * rep[i] : v / rep[i];
  v -= pres[i] + (float)counts[i] * freq[i];
  *p = v;
}
}  // namespace

// Each (row, id) pair must appear at most once.
CO_EXPORT int coheryn_apply_penalties(float* logits, long stride, int n, const int* rows, const int* ids,
                                      const int* counts, const float* rep, const float* freq,
                                      const float* pres, cudaStream_t stream) {
  if (n <= 0) return 0;
  apply_penalties_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, stride, n, rows, ids, counts, rep, freq, pres);
  CO_CHECK_LAUNCH("apply_penalties");
  return 0;
}

// The two-stage path puts the rows on the grid's y dimension, which ends at 65,535.
constexpr int ARGMAX_MAX_ROWS = 65535;

// Number of 8-byte scratch slots coheryn_argmax wants for R rows of V logits (0: none).
CO_EXPORT long coheryn_argmax_scratch_slots(int R, int V) {
  const int pieces = (V + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
  return pieces >= 4 ? (long)R * pieces : 0;
}

// scratch: 8 bytes per slot (see above), or null for the single-kernel path.
CO_EXPORT int coheryn_argmax(const float* logits, long stride, int R, int V, int* out, int* status,
                             void* scratch, long scratch_slots, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) CO_FAIL("argmax: empty vocabulary");
  const int pieces = (V + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
  if (pieces >= 4 && R <= ARGMAX_MAX_ROWS && scratch && scratch_slots >= (long)R * pieces) {
    float* pv = (float*)scratch;
    int* pi = (int*)scratch + (size_t)R * pieces;
    co_launch(argmax_pieces_kernel, dim3(pieces, R), dim3(256), 0, stream, logits, stride, V, pv, pi, pieces, status);
    CO_CHECK_LAUNCH("argmax_pieces");
    co_launch(argmax_final_kernel, dim3(R), dim3(64), 0, stream, (const float*)pv, (const int*)pi, pieces, out);
    CO_CHECK_LAUNCH("argmax_final");
    return 0;
  }
  co_launch(argmax_kernel, dim3(R), dim3(1024), 0, stream, logits, stride, V, out, status);
  CO_CHECK_LAUNCH("argmax");
  return 0;
}

// temperature[r] > 0, top_k[r] (0 = off), top_p[r] in (0, 1], uniform[r] in [0, 1).
CO_EXPORT int coheryn_sample(const float* logits, long stride, int R, int V, const float* temperature,
                             const int* top_k, const float* top_p, const double* uniform, int* out,
                             int* status, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) CO_FAIL("sample: empty vocabulary");
  sample_kernel<<<R, SAMPLE_THREADS, 0, stream>>>(logits, stride, V, temperature, top_k, top_p, uniform,
                                                  out, status);
  CO_CHECK_LAUNCH("sample");
  return 0;
}

// ------------------------------------------------------------------------------------
// Allocation-free greedy selection; see no_alloc.h for who needs it and for its limits.
// ------------------------------------------------------------------------------------
#include "no_alloc.h"

// The piece buffers: values (float) for all rows first, then indices (int).  Device code
// could name this array directly; host code may only use its address as looked up below.
static __device__ __align__(256) unsigned char g_argmax_static_scratch[(size_t)COHERYN_ARGMAX_STATIC_SLOTS * 8];

namespace {
constexpr int MAX_DEVICES = 64;
void* g_static_scratch_ptr[MAX_DEVICES];   // per device: the array's device address, once looked up
}  // namespace

CO_EXPORT int coheryn_argmax_static(const float* logits, long stride, int rows, int vocab, int* out, int* status,
                                    cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) CO_FAIL("argmax_static: empty vocabulary");
  if (rows > ARGMAX_MAX_ROWS)
    CO_FAIL("argmax_static: at most %d rows per call (one grid row each), not %d", ARGMAX_MAX_ROWS, rows);
  const long pieces = ((long)vocab + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
  if ((long)rows * pieces > COHERYN_ARGMAX_STATIC_SLOTS)
    CO_FAIL("argmax_static: %d rows of %d logits need %ld piece slots; the static scratch holds %d "
            "(use coheryn_argmax with a caller-provided buffer)", rows, vocab, (long)rows * pieces,
            COHERYN_ARGMAX_STATIC_SLOTS);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
    CO_FAIL("argmax_static: no usable current device (%s)", cudaGetErrorString(e));
  void* base = __atomic_load_n(&g_static_scratch_ptr[dev], __ATOMIC_ACQUIRE);
  if (!base) {
    // Set-up, once per device, with that device current: the symbol's name is a host-side
    // stand-in, the kernels need the device address.
    e = cudaGetSymbolAddress(&base, g_argmax_static_scratch);
    if (e != cudaSuccess || !base) CO_FAIL("argmax_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    __atomic_store_n(&g_static_scratch_ptr[dev], base, __ATOMIC_RELEASE);
  }
  float* pv = (float*)base;
  int* pi = (int*)base + (size_t)rows * pieces;
  co_launch(argmax_pieces_kernel, dim3((unsigned)pieces, rows), dim3(256), 0, stream, logits, stride, vocab, pv, pi,
            (int)pieces, status);
  CO_CHECK_LAUNCH("argmax_static pieces");
  co_launch(argmax_final_kernel, dim3(rows), dim3(64), 0, stream, (const float*)pv, (const int*)pi, (int)pieces, out);
  CO_CHECK_LAUNCH("argmax_static final");
  return 0;
}
