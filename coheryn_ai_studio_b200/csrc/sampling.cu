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

// One row per block.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long stride, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const double* __restrict__ uniform, int* __restrict__ out, int* __restrict__ status) {
  __shared__ double h_mass[256];
  __shared__ unsigned h_count[256];
  __shared__ float s_red[33];
  __shared__ int s_scan[SAMPLE_THREADS];
  __shared__ double s_total, s_threshold, s_before_mass;
  __shared__ long long s_keep_count, s_before_count;
  __shared__ unsigned s_prefix, s_neq;
  __shared__ long long s_rank;  // 1-based rank, among the candidates of the final key, of the chosen one

  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * stride;
  const float inv_t = 1.0f / temperature[r];
  const int k = top_k[r];
  const double p_keep = (double)top_p[r];

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

  // Three descents over the rank order (value descending, id ascending):
  //  phase 0: the number of candidates that top-p keeps = the first rank whose
  //           cumulative mass / total mass >= top_p; then top-k caps it;
  //  phase 1: the mass of the kept prefix; the threshold is u * that mass;
  //  phase 2: the first candidate whose cumulative mass exceeds the threshold.
  // A descent narrows (key prefix, mass before, count before) by one digit a level.
  // After four levels the bucket holds candidates of ONE value (n of them, ranked by
  // id), so the rank inside it follows from arithmetic on n equal masses.
  for (int phase = 0; phase < 3; ++phase) {
    if (threadIdx.x == 0) { s_prefix = 0u; s_before_mass = 0.0; s_before_count = 0; }
    __syncthreads();
    for (int level = 0; level < 4; ++level) {
      histogram(row, V, vmax, inv_t, s_prefix, level, h_mass, h_count);
      if (threadIdx.x == 0) {
        if (phase == 0 && level == 0) {
          double tot = 0.0;
          for (int b = 0; b < 256; ++b) tot += h_mass[b];
          s_total = tot;
        }
        double cm = s_before_mass;
        long long cc = s_before_count;
        int pick = -1, last = -1;
        double last_cm = cm;
        long long last_cc = cc;
        for (int b = 0; b < 256; ++b) {
          if (h_count[b] == 0u) continue;
          const double nm = cm + h_mass[b];
          const long long nc = cc + h_count[b];
          bool inside;
          if (phase == 0) inside = nm / s_total >= p_keep;
          else if (phase == 1) inside = nc >= s_keep_count;
          else inside = s_threshold < nm;
          last = b; last_cm = cm; last_cc = cc;
          if (inside) { pick = b; break; }
          cm = nm; cc = nc;
        }
        if (pick < 0) { pick = last; cm = last_cm; cc = last_cc; }  // rounding: take the last bucket
        s_before_mass = cm;
        s_before_count = cc;
        s_prefix |= (unsigned)pick << (24 - 8 * level);
        s_neq = h_count[pick];
      }
      __syncthreads();
    }
    if (threadIdx.x == 0) {
      const long long n = (long long)s_neq;
      const double p = exp(((double)key_value(s_prefix) - (double)vmax) * (double)inv_t);
      const double cm = s_before_mass;
      const long long cc = s_before_count;
      if (phase == 0) {
        long long j = 1;
        while (j < n && !((cm + (double)j * p) / s_total >= p_keep)) ++j;
        long long keep = cc + j;
        if (k > 0 && k < keep) keep = k;
        s_keep_count = keep;
      } else if (phase == 1) {
        long long j = s_keep_count - cc;
        if (j < 1) j = 1;
        if (j > n) j = n;
        s_threshold = uniform[r] * (cm + (double)j * p);
      } else {
        long long j = 1;
        while (j < n && !(s_threshold < cm + (double)j * p)) ++j;
        // Never step outside the kept prefix.
        if (cc + j > s_keep_count) j = s_keep_count - cc;
        if (j < 1) j = 1;
        s_rank = j;
      }
    }
    __syncthreads();
  }
  // The s_rank-th id (ascending) whose key equals s_prefix: blocked partition, count,
  // scan, then the owning thread walks its chunk.
  const unsigned key = s_prefix;
  const int chunk = (V + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
  int mine = 0;
  for (int i = lo; i < hi; ++i) mine += desc_key(row[i]) == key;
  s_scan[threadIdx.x] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long want = s_rank;
    int acc = 0, owner = -1, last_owner = -1;
    for (int t = 0; t < SAMPLE_THREADS; ++t) {
      if (s_scan[t] > 0) last_owner = t;
      if (owner < 0 && acc + s_scan[t] >= want) { owner = t; s_rank = want - acc; }
      acc += s_scan[t];
    }
    if (owner < 0) { owner = last_owner; s_rank = s_scan[last_owner]; }
    s_neq = (unsigned)owner;
  }
  __syncthreads();
  if (threadIdx.x == (int)s_neq) {
    long long seen = 0;
    int choice = lo;
    for (int i = lo; i < hi; ++i)
      if (desc_key(row[i]) == key) { choice = i; if (++seen == s_rank) break; }
    out[r] = choice;
  }
}
}  // namespace

CO_EXPORT int coheryn_argmax(const float* logits, long stride, int R, int V, int* out, int* status,
                             cudaStream_t stream) {
  if (R <= 0) return 0;
  if (V <= 0) CO_FAIL("argmax: empty vocabulary");
  argmax_kernel<<<R, 1024, 0, stream>>>(logits, stride, V, out, status);
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
